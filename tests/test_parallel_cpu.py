"""Partition arithmetic and collective wiring of the tensor-parallel layer on CPU ranks (gloo,
world size 2).  The local linear is the CPU oracle, injected through ``local_linear``: what is under
test is the sharding, the all-gather / all-reduce composition and the failure behaviour."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import seeded
from oracle import mlp as omlp
from oracle import w4a16 as oracle
from xqt_b200 import quantize
from xqt_b200.errors import XQTBackendError
from xqt_b200.parallel import (ColumnParallelLinear, RowParallelLinear,
                               shard_packed_weight)


def _oracle_linear(x, weight, *, out_dtype=None, bias=None):
    meta = weight.metadata
    return oracle.gemm(x, weight.qweight, weight.scales, weight.zero_points, group_size=meta.group_size,
                       signed=meta.nibble_signed, bias=bias, out_dtype=out_dtype)


def _layers():
    hidden, inter = 256, 512
    mk = lambda n, k, s: quantize.quantize_w4_asymmetric(torch.randn((n, k), generator=seeded(s)) * 0.02, group_size=128)
    return mk(inter, hidden, 20), mk(inter, hidden, 21), mk(hidden, inter, 22)


def test_shards_are_slices_and_cover_the_weight():
    gate, _, down = _layers()
    parts = [shard_packed_weight(gate, world=4, rank=r, axis=0) for r in range(4)]
    assert torch.equal(torch.cat([p.qweight for p in parts]), gate.qweight)
    assert torch.equal(torch.cat([p.scales for p in parts]), gate.scales)
    assert all(p.metadata.shard_axis == 0 and p.metadata.local_shape == (128, 256) for p in parts)
    kparts = [shard_packed_weight(down, world=2, rank=r, axis=1) for r in range(2)]
    assert torch.equal(torch.cat([p.qweight for p in kparts], dim=1), down.qweight)
    assert torch.equal(torch.cat([p.zero_points for p in kparts], dim=1), down.zero_points)
    assert kparts[0].metadata.logical_shape == (256, 256) and kparts[0].metadata.shard_axis == 1
    with pytest.raises(XQTBackendError):
        shard_packed_weight(down, world=3, rank=0, axis=1)       # 512 / 3 is not a whole number of groups
    with pytest.raises(XQTBackendError):
        shard_packed_weight(gate, world=5, rank=0, axis=0)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results, fail_rank):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        gate, up, down = _layers()
        x = torch.randn((5, 256), generator=seeded(1)).to(torch.bfloat16)
        col = ColumnParallelLinear(shard_packed_weight(gate, world=world, rank=rank, axis=0), local_linear=_oracle_linear)
        y_col = col(x)
        h = torch.randn((5, 512), generator=seeded(2)).to(torch.bfloat16)
        row = RowParallelLinear(shard_packed_weight(down, world=world, rank=rank, axis=1), local_linear=_oracle_linear)
        cols = 512 // world
        y_row = row(h[:, rank * cols:(rank + 1) * cols].contiguous())
        # the product's MLP block itself (it shards the canonical weights), its kernels replaced by the oracle
        from xqt_b200.ops.mlp import W4A16SwiGLUMLP

        mlp = W4A16SwiGLUMLP(gate, up, down, device=torch.device("cpu"), rank=rank, world=world, local_linear=_oracle_linear,
                             swiglu_fn=lambda gu: omlp.swiglu(gu[:, : gu.shape[1] // 2], gu[:, gu.shape[1] // 2:]))
        if rank == fail_rank:
            raise XQTBackendError("injected backend failure on this rank")
        y_mlp = mlp(x)
        results[rank] = (y_col, y_row, y_mlp)
    except XQTBackendError as exc:
        results[rank] = str(exc)
    finally:
        dist.destroy_process_group()


def _run(world, fail_rank=-1):
    manager = mp.Manager()
    results = manager.dict()
    port = _free_port()
    procs = [mp.Process(target=_worker, args=(r, world, port, results, fail_rank)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert not p.is_alive()
    return dict(results)


def test_two_rank_column_row_and_mlp_match_the_oracle():
    results = _run(2)
    gate, up, down = _layers()
    x = torch.randn((5, 256), generator=seeded(1)).to(torch.bfloat16)
    h = torch.randn((5, 512), generator=seeded(2)).to(torch.bfloat16)
    w = lambda pw: (pw.qweight, pw.scales, pw.zero_points)
    ref_col = oracle.gemm(x, *w(gate), group_size=128, signed=False)
    ref_row = oracle.gemm(h, *w(down), group_size=128, signed=False)
    ref_mlp = omlp.forward(x, w(gate), w(up), w(down), group_size=128)
    ref_mlp_sharded = omlp.forward_sharded(x, w(gate), w(up), w(down), group_size=128, world=2)
    for rank in range(2):
        y_col, y_row, y_mlp = results[rank]
        assert torch.equal(y_col, ref_col)                       # concatenation of exact slices
        assert oracle.rel_l2(y_row, ref_row) <= 1e-3             # different summation order across K shards
        assert torch.equal(y_mlp, ref_mlp_sharded)               # same order as the sharded oracle: bit-exact
        assert oracle.rel_l2(y_mlp, ref_mlp) <= 2e-3
    assert torch.equal(results[0][2], results[1][2])             # all ranks hold the same result


def test_a_failing_rank_surfaces_as_an_error_not_a_hang():
    # the rank that fails raises before its first collective of the MLP; the other rank's all-reduce
    # then fails or times out inside gloo and the process exits: nobody hangs (join has a deadline)
    results = _run(2, fail_rank=1)
    assert isinstance(results.get(1), str) and "injected" in results[1]
