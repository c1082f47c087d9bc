"""The tensor-parallel exchange kernel (all-reduce of the row-parallel partial results fused with the residual
update, over peer memory), through the C ABI.

On one GPU the kernel runs with a world of one rank: same code path minus the peers, checked bit for bit
against torch's addcmul.  With two or more GPUs a worker per GPU (tests/tp_exchange_worker.py, launched with
torch.distributed.run) checks the kernel against NCCL all-reduce + addcmul and the DiT stack's peer-exchange
forward (one CUDA graph, exchange kernels inside) against its NCCL forward.  Ranks never share a GPU."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_rank_equals_addcmul_and_replays_in_a_graph():
    from comfy_kitchen.tp_exchange import PeerExchange

    rows, cols, split = 777, 3072, 130
    g = torch.Generator(device="cuda").manual_seed(5)
    ex = PeerExchange(None, "cuda", rows, cols, torch.bfloat16)
    x0 = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    y = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    g0 = torch.randn(1, cols, device="cuda", generator=g).bfloat16()
    g1 = torch.randn(1, cols, device="cuda", generator=g).bfloat16()
    ex.residual.copy_(x0)
    ex.partial.copy_(y)
    want = x0.clone()
    for _ in range(2):   # two calls in a row: the epoch advances, the residual accumulates
        ex.exchange(g0, g1, split)
        want[:split] = torch.addcmul(want[:split], g0, y[:split])
        want[split:] = torch.addcmul(want[split:], g1, y[split:])
        assert torch.equal(ex.residual, want)
    ex.exchange(g0)      # one gate for all rows
    want = torch.addcmul(want, g0, y)
    assert torch.equal(ex.residual, want)
    # recorded into a CUDA graph and replayed: the kernel advances its own epoch, nothing is baked in
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        ex.exchange(g0, g1, split)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        graph.replay()
        want[:split] = torch.addcmul(want[:split], g0, y[:split])
        want[split:] = torch.addcmul(want[split:], g1, y[split:])
    assert torch.equal(ex.residual, want)
    assert ex.status() == 0


def test_argument_errors():
    import ctypes
    from comfy_kitchen import _native

    lib = _native.load()
    assert lib.ck_tp_pad_bytes() >= 4 * (2 * 512 * 8 + 512)
    arr = (ctypes.c_void_p * 1)(0)
    rc = lib.launch_tp_exchange_kernel(arr, arr, arr, None, None, 1, 0, None, None, 0, 16, 64, 2, 0, None)
    assert rc == -4
    rc = lib.launch_tp_exchange_kernel(arr, arr, arr, None, None, 9, 0, ctypes.c_void_p(256), None, 0, 16, 64, 2, 0, None)
    assert rc == -2 and b"ranks" in lib.ck_last_error()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs (ranks never share one)")
def test_two_ranks_against_nccl():
    n = 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29731", os.path.join(ROOT, "tests", "tp_exchange_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_EXCHANGE_WORKER_OK" in r.stdout


def test_row_range_front_end_and_single_rank_sequence_parallel_pieces():
    """The pieces of the sequence-parallel front end on one GPU: the fused norm -> NVFP4 kernel restricted to row
    ranges writes the same bytes at the same places as the whole-tensor call (ranges on 128-row boundaries, the last
    one carrying the scale buffer's padding rows), and the reduce-my-rows / gather kernels with a world of one rank
    reduce to the residual update."""
    from comfy_kitchen.backends import cuda as ck
    from comfy_kitchen.tp_exchange import PeerExchange

    n, d = 1000, 3072
    g = torch.Generator(device="cuda").manual_seed(31)
    x = torch.randn(1, n, d, device="cuda", generator=g).bfloat16()
    sc = (0.1 * torch.randn(1, 1, d, device="cuda", generator=g)).bfloat16()
    sh = (0.1 * torch.randn(1, 1, d, device="cuda", generator=g)).bfloat16()
    gs = torch.tensor([5.0 / (6 * 448)], device="cuda")
    q_ref, s_ref = ck.adaln_quantize_nvfp4(x, sc, sh, gs, 1e-6)
    q = torch.full_like(q_ref, 0xAA)
    s = torch.full((1024, 192), 0xAA, dtype=torch.uint8, device="cuda")
    for lo, hi in ((0, 256), (256, 256), (256, 768), (768, 1000)):
        ck.adaln_quantize_nvfp4_rows(x, sc, sh, gs, q, s, lo, hi, 1e-6)
    assert torch.equal(q, q_ref)
    assert torch.equal(s, s_ref.view(torch.uint8))
    assert ck.norm_device_status() == 0

    ex = PeerExchange(None, "cuda", n, d, torch.bfloat16)
    assert ex.row_bounds == [0, n] and (ex.row_lo, ex.row_hi) == (0, n)
    x0 = torch.randn(n, d, device="cuda", generator=g).bfloat16()
    y = torch.randn(n, d, device="cuda", generator=g).bfloat16()
    gate = torch.randn(d, device="cuda", generator=g).bfloat16()
    ex.residual.copy_(x0)
    ex.partial.copy_(y)
    ex.reduce_rows(gate)
    ex.qx.fill_(7)
    ex.gather_quantized()      # one rank: nothing to push, the barrier passes
    ex.gather_residual()
    assert torch.equal(ex.residual, torch.addcmul(x0, gate, y))
    assert int(ex.qx.min()) == 7
    assert ex.status() == 0
