"""W4A16 SwiGLU MLP block (hidden 4096, intermediate 14336 and a small shape) against the CPU oracle,
single GPU and, when two GPUs are visible, column/row partitioned over two NCCL ranks."""

from __future__ import annotations

import os
import socket
import subprocess
import sys

import pytest
import torch

from conftest import ROOT, seeded
from oracle import mlp as omlp
from oracle import w4a16 as oracle
from xqt_b200 import quantize

pytestmark = pytest.mark.gpu


def _weights(hidden, inter, seed):
    mk = lambda n, k, s: quantize.quantize_w4_asymmetric(torch.randn((n, k), generator=seeded(s)) * 0.02, group_size=128)
    return mk(inter, hidden, seed), mk(inter, hidden, seed + 1), mk(hidden, inter, seed + 2)


def test_swiglu_kernel_matches_oracle():
    from xqt_b200.ops.mlp import swiglu
    gu = torch.randn((7, 2 * 384), generator=seeded(1)).to(torch.bfloat16)
    out = swiglu(gu.cuda()).cpu()
    assert torch.equal(out, omlp.swiglu(gu[:, :384], gu[:, 384:]))


@pytest.mark.parametrize("hidden,inter,m", [(512, 1024, 1), (512, 1024, 16), (512, 1024, 100), (4096, 14336, 1),
                                             (4096, 14336, 16), (4096, 14336, 512)])
def test_mlp_single_gpu(hidden, inter, m):
    from xqt_b200.ops.mlp import W4A16SwiGLUMLP
    gate, up, down = _weights(hidden, inter, 20)
    x = torch.randn((m, hidden), generator=seeded(m)).to(torch.bfloat16)
    block = W4A16SwiGLUMLP(gate, up, down, device=torch.device("cuda", 0))
    out = block(x.cuda()).cpu()
    w = lambda pw: (pw.qweight, pw.scales, pw.zero_points)
    torch.set_num_threads(16)
    ref = omlp.forward(x, w(gate), w(up), w(down), group_size=128)
    # three chained bf16 roundings (gate/up, gating, down): the intermediate differs from the oracle's by isolated
    # ulps, which the down projection averages out
    assert oracle.rel_l2(out, ref) <= 2e-3
    assert block.execution_metadata()["decode_layout"] == "lanes"


_RANK_SCRIPT = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["XQT_ROOT"]); sys.path.insert(0, os.path.join(os.environ["XQT_ROOT"], "tests"))
from conftest import seeded
from xqt_b200 import quantize
from xqt_b200.ops.mlp import W4A16SwiGLUMLP
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dev = torch.device("cuda", rank); torch.cuda.set_device(dev)
dist.init_process_group("nccl", device_id=dev)
mk = lambda n, k, s: quantize.quantize_w4_asymmetric(torch.randn((n, k), generator=seeded(s)) * 0.02, group_size=128)
gate, up, down = mk(2048, 1024, 20), mk(2048, 1024, 21), mk(1024, 2048, 22)
block = W4A16SwiGLUMLP(gate, up, down, device=dev, rank=rank, world=world)            # peer-memory reduction at M <= 16
nccl_block = W4A16SwiGLUMLP(gate, up, down, device=dev, rank=rank, world=world, peer_reduce=False)
assert block.execution_metadata()["reduction"].startswith("peer_allreduce_kernel")
from xqt_b200 import native
for m in (4, 64, 300):
    x = torch.randn((m, 1024), generator=seeded(m)).to(torch.bfloat16).to(dev)
    y = block(x)
    torch.cuda.synchronize()
    if rank == 0:
        torch.save(y.cpu(), os.path.join(os.environ["XQT_OUT"], f"y{m}.pt"))
# the peer-memory reduction over several calls (alternating slots), against NCCL on the same partials
for step in range(5):
    x = torch.randn((1 + 3 * step, 1024), generator=seeded(100 + step)).to(torch.bfloat16).to(dev)
    a, b = block(x), nccl_block(x)
    torch.cuda.synchronize()
    assert native.workspace_status(dev) == 0
    err = ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert err <= 4e-3, (step, err)      # two bf16 roundings of sums added in different orders
    gathered = [torch.empty_like(a) for _ in range(world)]
    dist.all_gather(gathered, a)
    assert all(torch.equal(g, gathered[0]) for g in gathered)      # every rank holds the same bits
# the same block as one CUDA graph: the reduction's call number lives on the device, so replays hand-shake correctly,
# also with eager calls in between
replay = block.capture(4)
for step in range(4):
    x = torch.randn((4, 1024), generator=seeded(200 + step)).to(torch.bfloat16).to(dev)
    replay.input.copy_(x)
    a = replay().clone()
    if step == 2:
        assert torch.equal(block(x), a)
    b = nccl_block(x)
    torch.cuda.synchronize()
    block._peer.check()
    err = ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert err <= 4e-3, ("graph", step, err)
    gathered = [torch.empty_like(a) for _ in range(world)]
    dist.all_gather(gathered, a)
    assert all(torch.equal(g, gathered[0]) for g in gathered)
# peer-memory all-gather (counted form) of bytes written through a device-selected slot, eagerly and from a graph
from xqt_b200.parallel import PeerAllGather
from xqt_b200.ops.w4a16 import bind_w4a16_decode, prepare_decode
rows, n_local = 4, 512
gatherer = PeerAllGather(dev, rows * n_local * 2)
layer = mk(n_local, 1024, 50 + rank)
tiled = prepare_decode(layer.qweight.to(dev), layer.scales.to(dev), layer.zero_points.to(dev), group_size=128, nibble_signed=False)
run = bind_w4a16_decode(tiled, rows=rows, dtype=torch.bfloat16, out_select=gatherer.out_select)
plain = bind_w4a16_decode(tiled, rows=rows, dtype=torch.bfloat16)
local = gatherer.slot0.view(torch.bfloat16)[: rows * n_local].view(rows, n_local)
everything = torch.empty((world, rows, n_local), device=dev, dtype=torch.bfloat16)
def gathered_step(x):
    run(x, local)
    gatherer.gather(everything, rows * n_local * 2)
xs = [torch.randn((rows, 1024), generator=seeded(300 + i)).to(torch.bfloat16).to(dev) for i in range(6)]
static_x = xs[0].clone()
for i in range(3):
    gathered_step(xs[i])
    want = [torch.empty((rows, n_local), device=dev, dtype=torch.bfloat16) for _ in range(world)]
    dist.all_gather(want, plain(xs[i]))
    torch.cuda.synchronize()
    gatherer.check()
    assert all(torch.equal(everything[r], want[r]) for r in range(world)), ("gather", i)
side = torch.cuda.Stream(dev)
side.wait_stream(torch.cuda.current_stream(dev))
with torch.cuda.stream(side):
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        gathered_step(static_x)
torch.cuda.current_stream(dev).wait_stream(side)
for i in range(3, 6):
    static_x.copy_(xs[i])
    graph.replay()
    want = [torch.empty((rows, n_local), device=dev, dtype=torch.bfloat16) for _ in range(world)]
    dist.all_gather(want, plain(xs[i]))
    torch.cuda.synchronize()
    gatherer.check()
    assert all(torch.equal(everything[r], want[r]) for r in range(world)), ("gather graph", i)
dist.destroy_process_group()
'''


def test_mlp_two_ranks_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT)
    env = dict(os.environ, XQT_ROOT=str(ROOT), XQT_OUT=str(tmp_path), NCCL_NVLS_ENABLE="0", XQT_B200_REDUCE_BLOCKS="2")
    subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                    "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)], env=env, check=True,
                   timeout=300)
    gate, up, down = _weights(1024, 2048, 20)
    w = lambda pw: (pw.qweight, pw.scales, pw.zero_points)
    for m in (4, 64, 300):       # 300 rows: the reduction runs in column blocks overlapped with the down projection
        x = torch.randn((m, 1024), generator=seeded(m)).to(torch.bfloat16)
        ref = omlp.forward(x, w(gate), w(up), w(down), group_size=128)
        y = torch.load(tmp_path / f"y{m}.pt", weights_only=True)
        assert oracle.rel_l2(y, ref) <= 2e-3


def test_peer_allreduce_bounded_wait_reports_timeout_and_returns():
    """One GPU plays rank 0 of two; "rank 1" never launches, so its flag stays unset.  With a short
    poll limit the kernel must give up, store 128 to the (pinned host) status word and finish through
    its normal path; once the flag is set a second call produces the sum."""

    import ctypes

    from xqt_b200 import native

    lib = native.library()
    dev = torch.device("cuda", 0)
    count = n = 256
    partial = [torch.full((count,), 1.0, device=dev), torch.full((count,), 2.0, device=dev)]
    flags = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(2)]
    out = torch.zeros(count, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(16, dtype=torch.int32).pin_memory()
    array = ctypes.c_void_p * 2
    partials, flag_ptrs = array(*(t.data_ptr() for t in partial)), array(*(t.data_ptr() for t in flags))
    stream = native.stream_handle(dev)

    def call(number, limit):
        code = lib.xqt_b200_peer_allreduce(partials, flag_ptrs, 0, 2, number, count, n, None, out.data_ptr(),
                                           native.BF16, limit, status.data_ptr(), stream)
        assert code == 0
        torch.cuda.synchronize()

    call(1, 2000)                                   # about a millisecond of polling, then it gives up
    assert int(status[0]) == 128
    assert int(flags[1][0].item()) == 1             # rank 0 did signal its peer
    status.zero_()
    flags[0][1] = 2                                 # "rank 1" signals call 2
    torch.cuda.synchronize()
    call(2, 2000)
    assert int(status[0]) == 0
    assert torch.equal(out.float().cpu(), torch.full((count,), 3.0))


def test_peer_allreduce_refuses_graph_capture_and_surfaces_timeouts():
    """Host-side guards of PeerAllReduce that need no peer: a recorded timeout raises on the next
    use, and a captured call is refused (the call number is a host counter)."""

    from xqt_b200.errors import XQTBackendError
    from xqt_b200.parallel import PeerAllReduce

    obj = PeerAllReduce.__new__(PeerAllReduce)
    obj._host_status = torch.zeros(16, dtype=torch.int32).pin_memory()
    obj._host_status[0] = 128
    with pytest.raises(XQTBackendError):
        obj.check()
    assert int(obj._host_status[0]) == 0            # reported once, then cleared
    obj.check()


def test_static_decode_status_is_readable():
    import ctypes

    from xqt_b200 import native

    value = ctypes.c_uint(77)
    with torch.cuda.device(0):
        code = native.library().xqt_b200_w4a16_decode_static_status(ctypes.byref(value), native.stream_handle(torch.device("cuda", 0)))
    assert code == 0 and value.value == 0


def test_mlp_block_as_cuda_graph_matches_eager_calls():
    """`capture(rows)` replays the block from one CUDA graph: same bits as the eager call, for new inputs too."""

    from xqt_b200 import native
    from xqt_b200.ops.mlp import W4A16SwiGLUMLP
    dev = torch.device("cuda", 0)
    gate, up, down = _weights(1024, 2048, 20)
    block = W4A16SwiGLUMLP(gate, up, down, device=dev)
    replay = block.capture(4)
    for seed in (1, 2):
        x = torch.randn((4, 1024), generator=seeded(seed)).to(torch.bfloat16).to(dev)
        replay.input.copy_(x)
        got = replay().clone()
        assert torch.equal(got, block(x))
    assert native.workspace_status(dev) == 0


@pytest.mark.parametrize("m", [1, 16, 24])
def test_fused_swiglu_decode_epilogue_has_the_bits_of_the_unfused_form(m, monkeypatch):
    """gate/up + SwiGLU as one decode launch (interleaved tiles, gating in the kernel's epilogue) against the same
    block built with the fusion off: identical outputs."""

    from xqt_b200 import native
    from xqt_b200.ops.mlp import W4A16SwiGLUMLP
    dev = torch.device("cuda", 0)
    gate, up, down = _weights(1024, 2048 + 128, 30)         # 34 tiles of 64 + 64 rows
    x = torch.randn((m, 1024), generator=seeded(m + 7)).to(torch.bfloat16).to(dev)
    fused = W4A16SwiGLUMLP(gate, up, down, device=dev)
    assert fused.gate_up.glu
    monkeypatch.setenv("XQT_B200_FUSED_SWIGLU", "0")
    plain = W4A16SwiGLUMLP(gate, up, down, device=dev)
    assert not plain.gate_up.glu
    assert torch.equal(fused(x), plain(x))
    assert torch.equal(fused.gate_up.gated(x), plain._swiglu(plain.gate_up(x)))
    assert native.workspace_status(dev) == 0


def test_counted_peer_kernels_on_one_gpu():
    """The graph-safe (counted) reduction and gather with one GPU playing rank 0 of two: "rank 1" is a local buffer whose
    flag already carries a large call number, so no wait runs.  Three calls, eagerly and from one captured graph: the
    kernels take the call number from device memory, alternate between the two slots of every buffer and publish the
    count; the decode kernel writes its partial through the same word."""

    import ctypes

    from xqt_b200 import native, quantize
    from xqt_b200.ops.w4a16 import bind_w4a16_decode, prepare_decode

    lib = native.library()
    dev = torch.device("cuda", 0)
    stream = native.stream_handle(dev)
    array = ctypes.c_void_p * 2
    rows, n, k = 4, 256, 512
    count, stride = rows * n, 2048                      # elements per partial, elements between the two slots
    mine = torch.zeros(2 * stride, device=dev)          # rank 0: written by the decode kernel
    peer = torch.zeros(2 * stride, device=dev)
    peer[:count] = 10.0                                 # slot 0
    peer[stride:stride + count] = 20.0                  # slot 1
    flags = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(2)]
    flags[0][1] = 1 << 20                               # "rank 1" has signalled every call we are going to make
    counter = torch.zeros(4, dtype=torch.int32, device=dev)
    status = torch.zeros(16, dtype=torch.int32).pin_memory()
    out = torch.zeros(count, dtype=torch.bfloat16, device=dev)
    layer = quantize.quantize_w4_asymmetric(torch.randn((n, k), generator=seeded(3)) * 0.02, group_size=128)
    tiled = prepare_decode(layer.qweight.to(dev), layer.scales.to(dev), layer.zero_points.to(dev), group_size=128, nibble_signed=False)
    run = bind_w4a16_decode(tiled, rows=rows, dtype=torch.bfloat16, out_dtype=torch.float32,
                            out_select=(counter.data_ptr(), stride * 4))
    plain = bind_w4a16_decode(tiled, rows=rows, dtype=torch.bfloat16, out_dtype=torch.float32)
    x = torch.randn((rows, k), generator=seeded(4)).to(torch.bfloat16).to(dev)
    partials, flag_ptrs = array(mine.data_ptr(), peer.data_ptr()), array(*(t.data_ptr() for t in flags))

    def step():
        run(x, mine[:count].view(rows, n))
        assert lib.xqt_b200_peer_allreduce_counted(partials, flag_ptrs, 0, 2, counter.data_ptr(), stride, count, n, None,
                                                   out.data_ptr(), native.BF16, 1000, status.data_ptr(), native.stream_handle(dev)) == 0

    want = plain(x).reshape(-1)
    for call in (1, 2, 3):                              # slots 1, 0, 1
        step()
        torch.cuda.synchronize()
        assert int(counter[0].item()) == call and int(counter[1].item()) == 0 and int(status[0]) == 0
        assert int(flags[1][0].item()) == call          # rank 0 signalled its peer with the device-side call number
        addend = 20.0 if call & 1 else 10.0
        assert torch.equal(out.float(), (want + addend).to(torch.bfloat16).float())
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
    torch.cuda.current_stream(dev).wait_stream(side)
    for call in (4, 5):
        graph.replay()
        torch.cuda.synchronize()
        assert int(counter[0].item()) == call and int(status[0]) == 0
        assert torch.equal(out.float(), (want + (20.0 if call & 1 else 10.0)).to(torch.bfloat16).float())
    # the gather: rank 0's bytes are whatever the decode kernel wrote into the slot in use, rank 1's the constants
    gathered = torch.zeros((2, count), device=dev)
    gcounter = torch.zeros(4, dtype=torch.int32, device=dev)
    gflags = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(2)]
    gflags[0][1] = 1 << 20
    gflag_ptrs = array(*(t.data_ptr() for t in gflags))
    mine.zero_()
    mine[:count] = 1.0
    mine[stride:stride + count] = 2.0
    for call in (1, 2):
        assert lib.xqt_b200_peer_allgather_counted(partials, gflag_ptrs, 0, 2, gcounter.data_ptr(), stride * 4, count * 4,
                                                   gathered.data_ptr(), 1000, status.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert int(gcounter[0].item()) == call and int(status[0]) == 0
        assert torch.equal(gathered[0], torch.full((count,), 2.0 if call & 1 else 1.0, device=dev))
        assert torch.equal(gathered[1], torch.full((count,), 20.0 if call & 1 else 10.0, device=dev))
