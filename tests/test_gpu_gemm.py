"""GPU parity of the block-scaled GEMMs, through the C ABI.

Oracle: dequantize both operands to fp32, multiply in fp32, apply alpha and bias
(the comparison the reference's own GEMM tests use, tests/test_qdq.py:452-509).
Tolerance: max |y - ref| <= 1e-2 * max(|ref|, rms(ref)) on bf16 outputs; the
products themselves are exact in the tensor core (4-bit x 4-bit codes with 8-bit
scales), so the only differences are fp32 accumulation order and the bf16 cast.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ck():
    from comfy_kitchen.backends import cuda

    return cuda


@pytest.fixture(scope="module")
def orc():
    from oracle import ck_oracle

    return ck_oracle


def _rel_err(y, ref):
    y, ref = y.float().cpu(), ref.float().cpu()
    denom = torch.maximum(ref.abs(), ref.pow(2).mean().sqrt().expand_as(ref))
    return ((y - ref).abs() / denom).max().item()


def _operands(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (0.02 * torch.randn(N, K, generator=g)).bfloat16()
    bias = (0.02 * torch.randn(N, generator=g)).float()
    return x, w, bias


NVFP4_SHAPES = [(128, 192, 256), (256, 384, 512), (128, 192, 64), (200, 264, 320), (129, 200, 96), (512, 1024, 2048),
                (77, 8, 32), (1024, 3072, 3072), (300, 520, 192), (513, 264, 3104), (257, 256, 288)]


@pytest.mark.parametrize("M,N,K", NVFP4_SHAPES)
def test_scaled_mm_nvfp4_vs_oracle(ck, orc, M, N, K):
    x, w, bias = _operands(M, N, K, 0)
    gx = (x.float().abs().max() / (6 * 448)).float()
    gw = (w.float().abs().max() / (6 * 448)).float()
    pad = (K % 16 != 0)
    qx, sx = ck.quantize_nvfp4(x.cuda(), gx.cuda(), pad_16x=pad)
    qw, sw = ck.quantize_nvfp4(w.cuda(), gw.cuda(), pad_16x=pad)
    y = ck.scaled_mm_nvfp4(qx, qw, gx.cuda(), gw.cuda(), sx, sw, bias=bias.cuda(), out_dtype=torch.bfloat16)
    assert ck.gemm_device_status() == 0
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    if M * N * K <= 512 * 1024 * 2048:
        ref = orc.scaled_mm_nvfp4(qx.cpu(), qw.cpu(), gx, gw, sx.cpu(), sw.cpu(), bias=bias, out_dtype=torch.float32)
    else:
        a = ck.dequantize_nvfp4(qx, gx.cuda(), sx, torch.float32)
        b = ck.dequantize_nvfp4(qw, gw.cuda(), sw, torch.float32)
        ref = (a.double() @ b.double().t()).float() + bias.cuda()
    err = _rel_err(y, ref)
    assert err <= 1e-2, f"max rel err {err}"


def test_scaled_mm_nvfp4_options(ck, orc):
    M, N, K = 256, 384, 512
    x, w, bias = _operands(M, N, K, 1)
    gx = (x.float().abs().max() / (6 * 448)).float().cuda()
    gw = (w.float().abs().max() / (6 * 448)).float().cuda()
    qx, sx = ck.quantize_nvfp4(x.cuda(), gx)
    qw, sw = ck.quantize_nvfp4(w.cuda(), gw)
    ref = orc.scaled_mm_nvfp4(qx.cpu(), qw.cpu(), gx.cpu(), gw.cpu(), sx.cpu(), sw.cpu(), out_dtype=torch.float32)
    y32 = ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, out_dtype=torch.float32)
    assert _rel_err(y32, ref) <= 1e-4  # fp32 output: only the accumulation order differs
    y16 = ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, out_dtype=torch.float16)
    assert _rel_err(y16, ref) <= 2e-3
    # explicit alpha overrides the product of the tensor scales
    y2 = ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, out_dtype=torch.float32, alpha=(2 * gx * gw))
    assert _rel_err(y2, 2 * ref) <= 1e-4
    # bias dtypes
    for bdt in (torch.bfloat16, torch.float16, torch.float32):
        b = bias.to(bdt)
        yb = ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, bias=b.cuda(), out_dtype=torch.float32)
        assert _rel_err(yb, ref + b.float()) <= 1e-4
    # run twice: identical bits (deterministic accumulation order)
    assert torch.equal(y32, ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, out_dtype=torch.float32))
    assert ck.gemm_device_status() == 0


def test_scaled_mm_nvfp4_exact_small_integers(ck):
    # all products are small integers -> the fp32 result is exact whatever the order
    M, N, K = 128, 192, 256
    g = torch.Generator().manual_seed(5)
    codes = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, -1.0, -2.0])
    x = codes[torch.randint(0, 8, (M, K), generator=g)]
    w = codes[torch.randint(0, 8, (N, K), generator=g)]
    x[:, ::16] = 6.0  # every block has amax 6 -> block scale exactly 64 with g = 1/64
    w[:, ::16] = 6.0
    gs = torch.tensor(1.0 / 64, device="cuda")
    qx, sx = ck.quantize_nvfp4(x.cuda(), gs)
    qw, sw = ck.quantize_nvfp4(w.cuda(), gs)
    y = ck.scaled_mm_nvfp4(qx, qw, gs, gs, sx, sw, out_dtype=torch.float32)
    assert ck.gemm_device_status() == 0
    assert torch.equal(y.cpu(), x @ w.t())


def test_linearity_at_full_size(ck):
    # config-sized GEMM (4608 x 3072 x 3072): scaling one operand's tensor scale scales the output,
    # and the result matches an fp64 product of the dequantized operands
    M, N, K = 4608, 3072, 3072
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (0.02 * torch.randn(N, K, device="cuda", generator=g)).bfloat16()
    gx = (x.float().abs().max() / (6 * 448)).float()
    gw = (w.float().abs().max() / (6 * 448)).float()
    qx, sx = ck.quantize_nvfp4(x, gx)
    qw, sw = ck.quantize_nvfp4(w, gw)
    y = ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, out_dtype=torch.float32)
    y2 = ck.scaled_mm_nvfp4(qx, qw, 2 * gx, gw, sx, sw, out_dtype=torch.float32)
    assert ck.gemm_device_status() == 0
    assert torch.equal(y2, 2 * y)
    a = ck.dequantize_nvfp4(qx, gx, sx, torch.float32)
    b = ck.dequantize_nvfp4(qw, gw, sw, torch.float32)
    ref = (a[:512].double() @ b.double().t()).float()
    assert _rel_err(y[:512], ref) <= 1e-4
    ref = (a[-256:].double() @ b.double().t()).float()
    assert _rel_err(y[-256:], ref) <= 1e-4


MXFP8_SHAPES = [(128, 192, 128), (256, 384, 512), (128, 192, 32), (200, 264, 160), (129, 200, 96), (512, 1024, 2048),
                (1024, 3072, 3072), (300, 520, 160), (513, 264, 3104), (257, 256, 288)]


@pytest.mark.parametrize("M,N,K", MXFP8_SHAPES)
def test_scaled_mm_mxfp8_vs_oracle(ck, orc, M, N, K):
    x, w, bias = _operands(M, N, K, 2)
    qx, sx = ck.quantize_mxfp8(x.cuda())
    qw, sw = ck.quantize_mxfp8(w.cuda())
    y = ck.scaled_mm_mxfp8(qx, qw, sx, sw, bias=bias.cuda(), out_dtype=torch.bfloat16)
    assert ck.gemm_device_status() == 0
    if M * N * K <= 512 * 1024 * 2048:
        ref = orc.scaled_mm_mxfp8(qx.cpu(), qw.cpu(), sx.cpu(), sw.cpu(), bias=bias, out_dtype=torch.float32)
    else:
        a = ck.dequantize_mxfp8(qx, sx, torch.float32)
        b = ck.dequantize_mxfp8(qw, sw, torch.float32)
        ref = (a.double() @ b.double().t()).float() + bias.cuda()
    err = _rel_err(y, ref)
    assert err <= 1e-2, f"max rel err {err}"
    y32 = ck.scaled_mm_mxfp8(qx, qw, sx, sw, bias=bias.cuda(), out_dtype=torch.float32)
    assert _rel_err(y32, ref) <= 1e-4


def test_reference_argument_order_entry_point(ck):
    # launch_cublas_gemm_blockwise_fp4_kernel: weights first, bias in the output dtype
    import ctypes
    from comfy_kitchen import _native
    M, N, K = 128, 192, 256
    x, w, bias = _operands(M, N, K, 3)
    gx = (x.float().abs().max() / (6 * 448)).float().cuda()
    gw = (w.float().abs().max() / (6 * 448)).float().cuda()
    qx, sx = ck.quantize_nvfp4(x.cuda(), gx)
    qw, sw = ck.quantize_nvfp4(w.cuda(), gw)
    b16 = bias.bfloat16().cuda()
    want = ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, bias=b16, out_dtype=torch.bfloat16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    alpha = (gx * gw).reshape(1)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    _native.call("launch_cublas_gemm_blockwise_fp4_kernel", P(qw), P(sw), P(qx), P(sx), P(out), P(b16), M, N, K,
                 P(alpha), 2, ctypes.c_void_p(0), False, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert torch.equal(out, want)
    assert ck.gemm_device_status() == 0


@pytest.mark.parametrize("M,N,K", [(300, 520, 192), (1024, 3072, 3072), (4608, 3072, 12288)])
@pytest.mark.parametrize("odt", [torch.bfloat16, torch.float16])
def test_fused_residual_epilogue_equals_gemm_then_addcmul(ck, M, N, K, odt):
    """scaled_mm_nvfp4(residual=x, gate=g) must return the bytes of torch.addcmul(x, g, scaled_mm_nvfp4(...)), written
    to a fresh tensor or over the residual itself."""
    x, w, bias = _operands(M, N, K, 6)
    g = torch.Generator().manual_seed(7)
    res = torch.randn(M, N, generator=g).to(odt).cuda()
    gate = torch.randn(1, N, generator=g).to(odt).cuda()
    gx = (x.float().abs().max() / (6 * 448)).float().cuda()
    gw = (w.float().abs().max() / (6 * 448)).float().cuda()
    qx, sx = ck.quantize_nvfp4(x.cuda(), gx)
    qw, sw = ck.quantize_nvfp4(w.cuda(), gw)
    y = ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, bias=bias.cuda(), out_dtype=odt)
    want = torch.addcmul(res, gate, y)
    got = ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, bias=bias.cuda(), out_dtype=odt, residual=res, gate=gate)
    assert torch.equal(got, want)
    inplace = res.clone()
    ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, bias=bias.cuda(), out_dtype=odt, out=inplace, residual=inplace, gate=gate)
    assert torch.equal(inplace, want)
    assert ck.gemm_device_status() == 0


def test_tensor_map_cache_is_transparent(ck):
    """Encoded tensor maps are cached per (pointer, shape): a buffer that is freed and reallocated with another
    shape at the same address, and the cache switched off, must give the same results."""
    outs = []
    for use_cache in (1, 0, 1):
        ck.set_option("gemm_map_cache", use_cache)
        for (M, N, K) in [(256, 384, 512), (384, 256, 512), (256, 384, 512)]:
            x, w, bias = _operands(M, N, K, 8)
            gx = (x.float().abs().max() / (6 * 448)).float().cuda()
            gw = (w.float().abs().max() / (6 * 448)).float().cuda()
            qx, sx = ck.quantize_nvfp4(x.cuda(), gx)
            qw, sw = ck.quantize_nvfp4(w.cuda(), gw)
            outs.append((use_cache, M, N, ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, out_dtype=torch.float32).cpu()))
            del qx, sx, qw, sw
    ck.set_option("gemm_map_cache", 1)
    base = {(m, n): o for c, m, n, o in outs[:3]}
    for c, m, n, o in outs:
        assert torch.equal(o, base[(m, n)])


@pytest.mark.parametrize("M,N,K", [(128, 192, 256), (300, 520, 192), (513, 264, 3104), (1024, 3072, 3072), (4608, 3072, 12288),
                                   (2344, 1160, 6176)])
def test_pipeline_variants_agree(ck, M, N, K):
    """The two pipelines of the GEMM kernel (scales moved into TMEM by dedicated warps, or by tcgen05.cp from the MMA
    issuer with all copies signalling the pair leader's barrier; the launcher picks one per format and K) issue the
    same MMAs: one tile or many per CTA pair, ragged edges, partial last k-tile.  NVFP4 results are identical.  With
    MXFP8 the k-tiles of the two issuing warps can reach the tensor pipe in either order, with both pipelines, so
    fp32 sums may differ in the last bit even between two launches of the same pipeline (1e-6 relative allowed)."""
    x, w, bias = _operands(M, N, K, 9)
    gx = (x.float().abs().max() / (6 * 448)).float().cuda()
    gw = (w.float().abs().max() / (6 * 448)).float().cuda()
    qx, sx = ck.quantize_nvfp4(x.cuda(), gx)
    qw, sw = ck.quantize_nvfp4(w.cuda(), gw)
    q8x, s8x = ck.quantize_mxfp8(x.cuda())
    q8w, s8w = ck.quantize_mxfp8(w.cuda())
    outs = {}
    try:
        for variant in (1, 2):
            ck.set_option("gemm_tile", variant)
            outs[variant] = (ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, bias=bias.cuda(), out_dtype=torch.bfloat16),
                             ck.scaled_mm_mxfp8(q8x, q8w, s8x, s8w, bias=bias.cuda(), out_dtype=torch.float32))
            assert ck.gemm_device_status() == 0
    finally:
        ck.set_option("gemm_tile", 0)
    assert torch.equal(outs[1][0], outs[2][0])
    assert (outs[1][1] - outs[2][1]).abs().max() <= 1e-6 * outs[1][1].abs().max()


def test_scattered_output_single_gpu(ck):
    """The GEMM whose epilogue scatters its tile rows over the ranks of a tensor-parallel group, exercised on one GPU
    with three "ranks" whose buffers are separate local tensors: rows [bounds[d], bounds[d+1]) of the (offset) output
    must land in buffer d, counted from bounds[d], with the bytes of the ordinary GEMM."""
    import ctypes

    M, N, K = 608, 520, 512
    x, w, bias = _operands(M, N, K, 12)
    gx = (x.float().abs().max() / (6 * 448)).float().cuda()
    gw = (w.float().abs().max() / (6 * 448)).float().cuda()
    qx, sx = ck.quantize_nvfp4(x.cuda(), gx)
    qw, sw = ck.quantize_nvfp4(w.cuda(), gw)
    want = ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, bias=bias.cuda(), out_dtype=torch.bfloat16)
    bounds = [0, 256, 768, 1000]          # the group's matrix has 1000 rows; this GEMM supplies rows 128 .. 735
    row_offset = 128
    bufs = [torch.full((bounds[d + 1] - bounds[d], N), 7.0, dtype=torch.bfloat16, device="cuda") for d in range(3)]
    dests = (ctypes.c_void_p * 3)(*[b.data_ptr() for b in bufs])
    cb = (ctypes.c_int64 * 4)(*bounds)
    ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, bias=bias.cuda(), out_dtype=torch.bfloat16, scatter=(dests, cb, 3, row_offset))
    assert ck.gemm_device_status() == 0
    whole = torch.cat(bufs)                # rows of the group's matrix
    assert torch.equal(whole[row_offset:row_offset + M], want)
    assert bool((whole[:row_offset] == 7.0).all()) and bool((whole[row_offset + M:] == 7.0).all())   # nothing else touched
