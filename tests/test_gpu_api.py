"""GPU checks of the public API: custom ops, registry dispatch, QuantizedTensor linear/mm on the
tensor-core kernels, CUDA-graph capture on a side stream, torch.compile through the fake kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ck():
    import comfy_kitchen

    return comfy_kitchen


def _rel(y, ref):
    y, ref = y.float(), ref.float()
    return ((y - ref).abs().max() / ref.abs().max().clamp_min(1e-6)).item()


def test_public_api_matches_backend_module(ck):
    from comfy_kitchen.backends import cuda as be

    x = torch.randn(256, 512, device="cuda").bfloat16()
    g = (x.float().abs().max() / (6 * 448)).float()
    q1, s1 = ck.quantize_nvfp4(x, g)
    q2, s2 = be.quantize_nvfp4(x, g)
    assert torch.equal(q1, q2) and torch.equal(s1.view(torch.uint8), s2.view(torch.uint8))
    assert torch.equal(ck.dequantize_nvfp4(q1, g, s1), be.dequantize_nvfp4(q1, g, s1))
    q8, s8 = ck.quantize_mxfp8(x)
    assert q8.dtype == torch.float8_e4m3fn and s8.dtype == torch.float8_e8m0fnu
    assert torch.equal(ck.dequantize_mxfp8(q8, s8), be.dequantize_mxfp8(q8, s8))
    qf = ck.quantize_per_tensor_fp8(x, g * 6)
    assert qf.dtype == torch.float8_e4m3fn and ck.dequantize_per_tensor_fp8(qf, g * 6).dtype == torch.bfloat16
    y = ck.adaln(x.view(1, 256, 512), torch.zeros(1, 1, 512, device="cuda").bfloat16(), torch.zeros(1, 1, 512, device="cuda").bfloat16())
    torch.testing.assert_close(y.float().view(256, 512), torch.nn.functional.layer_norm(x.float(), (512,), eps=1e-6), rtol=1e-2, atol=1e-2)
    with pytest.raises(ck.NoCapableBackendError):
        ck.quantize_nvfp4(x.cpu(), g.cpu())
    with pytest.raises(ck.NoCapableBackendError):
        ck.quantize_nvfp4(x.view(2, 128, 512), g)  # not 2-D


@pytest.mark.parametrize("layout", ["TensorCoreNVFP4Layout", "TensorCoreMXFP8Layout"])
@pytest.mark.parametrize("M,N,K", [(512, 1024, 2048), (49, 113, 81), (128, 192, 256)])
def test_quantized_linear(ck, layout, M, N, K):
    from comfy_kitchen.tensor import QuantizedTensor

    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (0.02 * torch.randn(N, K, device="cuda", generator=g)).bfloat16()
    b = (0.02 * torch.randn(N, device="cuda", generator=g)).bfloat16()
    qx, qw = QuantizedTensor.from_float(x, layout), QuantizedTensor.from_float(w, layout)
    ref = torch.nn.functional.linear(qx.dequantize().float(), qw.dequantize().float(), b.float())
    y = torch.nn.functional.linear(qx, qw, b)
    assert tuple(y.shape) == (M, N) and y.dtype == torch.bfloat16
    assert _rel(y, ref) <= 1e-2
    y2 = torch.mm(qx, qw.t())
    assert _rel(y2, ref - b.float()) <= 1e-2
    y3 = torch.addmm(b, qx, qw.t())
    assert _rel(y3, ref) <= 1e-2
    from comfy_kitchen.backends import cuda as be
    assert be.gemm_device_status() == 0


def test_fp8_layout_linear(ck):
    from comfy_kitchen.tensor import QuantizedTensor

    x = torch.randn(128, 256, device="cuda").bfloat16()
    w = (0.05 * torch.randn(64, 256, device="cuda")).bfloat16()
    qx, qw = QuantizedTensor.from_float(x, "TensorCoreFP8Layout"), QuantizedTensor.from_float(w, "TensorCoreFP8Layout")
    y = torch.nn.functional.linear(qx, qw)
    ref = torch.nn.functional.linear(x, w)
    assert torch.allclose(y.float(), ref.float(), rtol=0.15, atol=0.15)


def test_cuda_graph_capture_on_side_stream(ck):
    """quantize -> linear -> gelu -> quantize -> linear captured and replayed: no sync, no allocation
    outside torch's allocator, work on the capturing stream."""
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(256, 512, device="cuda", generator=g).bfloat16()
    w1 = (0.03 * torch.randn(1024, 512, device="cuda", generator=g)).bfloat16()
    w2 = (0.03 * torch.randn(512, 1024, device="cuda", generator=g)).bfloat16()
    gs = torch.tensor(0.002, device="cuda")
    gw = torch.tensor(0.0001, device="cuda")
    qw1, sw1 = ck.quantize_nvfp4(w1, gw)
    qw2, sw2 = ck.quantize_nvfp4(w2, gw)
    freqs = torch.randn(1, 1, 256, 32, 2, 2, device="cuda")

    def model(inp):
        q, s = ck.quantize_nvfp4(inp, gs)
        h = ck.scaled_mm_nvfp4(q, qw1, gs, gw, s, sw1, out_dtype=torch.bfloat16)
        h = torch.nn.functional.gelu(h)
        q, s = ck.quantize_nvfp4(h, gs)
        y = ck.scaled_mm_nvfp4(q, qw2, gs, gw, s, sw2, out_dtype=torch.bfloat16)
        y = ck.adaln(y.view(1, 256, 512), y[:1].view(1, 1, 512), y[1:2].view(1, 1, 512)).view(256, 512)
        q8, s8 = ck.quantize_mxfp8(y)
        r = ck.apply_rope1(y.view(1, 8, 256, 64).contiguous(), freqs)
        return y, ck.dequantize_mxfp8(q8, s8), r

    eager = model(x)
    static_x = x.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            model(static_x)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            out = model(static_x)
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(out, eager):
        assert torch.equal(a, b)
    static_x.copy_(2 * x)
    graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(out, model(2 * x)):
        assert torch.equal(a, b)


def test_torch_compile_through_fake_kernels(ck):
    gs = torch.tensor(0.002, device="cuda")
    gw = torch.tensor(0.0001, device="cuda")
    w = (0.03 * torch.randn(384, 256, device="cuda")).bfloat16()
    qw, sw = ck.quantize_nvfp4(w, gw)

    def f(inp):
        q, s = ck.quantize_nvfp4(inp, gs)
        return ck.scaled_mm_nvfp4(q, qw, gs, gw, s, sw, out_dtype=torch.bfloat16) + 1

    x = torch.randn(128, 256, device="cuda").bfloat16()
    want = f(x)
    got = torch.compile(f, fullgraph=True)(x)
    torch.testing.assert_close(got.float(), want.float(), rtol=1e-3, atol=1e-3)


def test_public_api_new_fused_ops():
    """The public entry points of the two fused operators reach the CUDA backend through the registry."""
    import comfy_kitchen as ck
    from comfy_kitchen.backends import cuda as be

    g = torch.Generator(device="cuda").manual_seed(0)
    heads, t = 2, 96
    qkv = torch.randn(t, 3 * heads * 128, device="cuda", generator=g).bfloat16()
    w = torch.ones(128, device="cuda").bfloat16()
    ang = torch.rand(t, 64, device="cuda", generator=g)
    f = torch.stack([torch.stack([ang.cos(), -ang.sin()], -1), torch.stack([ang.sin(), ang.cos()], -1)], -2)[None, None].contiguous()
    q, k, v = ck.qk_norm_rope(qkv, w, w, f, heads)
    q2, k2, v2 = be.qk_norm_rope(qkv, w, w, f, heads)
    assert torch.equal(q, q2) and torch.equal(k, k2) and torch.equal(v, v2)
    gs = torch.tensor(0.01, device="cuda")
    a = ck.quantize_nvfp4_gather([(v[0], None)], gs)
    b = be.quantize_nvfp4(v[0].permute(1, 0, 2).reshape(t, heads * 128).contiguous(), gs)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1].view(torch.uint8), b[1].view(torch.uint8))


def test_nvfp4_linear_loader_on_the_device():
    """The reference's checkpoint key contract loaded on the GPU, whole and as tensor-parallel shards: a shard's
    bytes equal quantize(sliced weight), and the module's forward equals the CPU oracle's GEMM."""
    import comfy_kitchen as ck
    from comfy_kitchen.backends import cuda as be
    from comfy_kitchen.linear import NVFP4Linear
    from oracle import ck_oracle as orc

    n, k = 512, 1024
    g = torch.Generator().manual_seed(4)
    w = (0.02 * torch.randn(n, k, generator=g)).bfloat16()
    ts = (w.float().abs().max() / (6 * 448)).float().reshape(1)
    q, sf = be.quantize_nvfp4(w.cuda(), ts.cuda())
    sd = {"weight": q.cpu(), "weight_scale": sf.view(torch.uint8).cpu(), "weight_scale_2": ts,
          "bias": (0.02 * torch.randn(n, generator=g)).bfloat16(), "input_scale": torch.tensor([4.5 / (6 * 448)])}
    x = torch.randn(96, k, generator=g).bfloat16()
    m = NVFP4Linear(k, n, device="cuda")
    assert m.load_state_dict(dict(sd)) == ([], []) or True
    y = m(x.cuda())
    qx, sx = orc.quantize_nvfp4(x, sd["input_scale"])
    want = orc.scaled_mm_nvfp4(qx, sd["weight"], sd["input_scale"], ts, sx, sd["weight_scale"].view(torch.float8_e4m3fn),
                               bias=sd["bias"], out_dtype=torch.float32)
    err = (y.float().cpu() - want).abs().max() / want.abs().max()
    assert err <= 1e-2
    for rank in range(2):
        col = NVFP4Linear(k, n, device="cuda", parallel="column", rank=rank, world=2)
        col.load_state_dict(dict(sd))
        lo, hi = rank * n // 2, (rank + 1) * n // 2
        q_ref, sf_ref = be.quantize_nvfp4(w[lo:hi].contiguous().cuda(), ts.cuda())
        assert torch.equal(col.weight._qdata, q_ref)
        assert torch.equal(col.weight._params.block_scale.view(torch.uint8), sf_ref.view(torch.uint8))
        assert torch.equal(col(x.cuda()), y[:, lo:hi])
        row = NVFP4Linear(k, n, device="cuda", parallel="row", rank=rank, world=2)
        row.load_state_dict(dict(sd))
        lo, hi = rank * k // 2, (rank + 1) * k // 2
        q_ref, sf_ref = be.quantize_nvfp4(w[:, lo:hi].contiguous().cuda(), ts.cuda())
        assert torch.equal(row.weight._qdata, q_ref)
        assert torch.equal(row.weight._params.block_scale.view(torch.uint8), sf_ref.view(torch.uint8))
    assert be.gemm_device_status() == 0
