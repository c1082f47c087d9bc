"""The allocation-free entry point, through the C ABI (collected last on purpose: a run that stops at the first
failure has then already run every other test).

launch_tp_exchange_noalloc_kernel is for hosts that cannot allocate device memory when they call the library (a
runtime with a fixed arena, a plugin in a pipeline where cudaMalloc would stall the device): the flag pad the
exchange kernel needs sits in a device array inside the library.  Its result must equal the ordinary entry
point's, which takes the pad from the caller -- checked on two calls in a row, since the second call finds the
epochs the first one left in the shared pad."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def test_noalloc_exchange_equals_the_ordinary_entry_point_twice():
    from comfy_kitchen import _native
    from comfy_kitchen.tp_exchange import PeerExchange

    rows, cols, split = 555, 3072, 200
    g = torch.Generator(device="cuda").manual_seed(17)
    x0 = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    g0 = torch.randn(cols, device="cuda", generator=g).bfloat16()
    g1 = torch.randn(cols, device="cuda", generator=g).bfloat16()
    ref = PeerExchange(None, "cuda", rows, cols, torch.bfloat16)     # ordinary path: pad allocated by the caller
    ref.residual.copy_(x0)
    mine = x0.clone()
    part = torch.empty(rows, cols, device="cuda", dtype=torch.bfloat16)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        part.copy_(torch.randn(rows, cols, device="cuda", generator=g).bfloat16())
        ref.partial.copy_(part)
        ref.exchange(g0, g1, split)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        _native.call("launch_tp_exchange_noalloc_kernel", _p(part), _p(mine), _p(g0), _p(g1), split, rows, cols, 2, 0, stream)
        torch.cuda.synchronize()
        if call == 1:   # (the first call may still load the kernel's code; the second takes no device memory at all)
            assert torch.cuda.mem_get_info()[0] >= free_before
        assert torch.equal(mine, ref.residual), f"call {call}: results differ"   # same kernel: bit equality
    assert ref.status() == 0
    # a grid the built-in pad cannot serve is refused, with a message that says why
    lib = _native.load()
    rc = lib.launch_tp_exchange_noalloc_kernel(_p(part), _p(mine), _p(g0), _p(g1), split, rows, cols, 2, 513, stream)
    assert rc == -2 and b"at most 512" in lib.ck_last_error()
