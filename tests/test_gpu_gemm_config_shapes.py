"""GPU parity of the block-scaled GEMMs on the benchmark's own shapes, through the C ABI.

Shapes: M = 4608 * {1, 2, 4} tokens x (N, K) in {(9216, 3072), (3072, 3072), (12288, 3072),
(3072, 12288)}, fp32 bias, bf16 output, for NVFP4 and MXFP8 operands.  These are the sizes at which
the persistent kernel gives every CTA pair several output tiles (barrier phases, operand ring and
scale buffers carried across tiles, the short last band of the tile order when the number of tile
rows is not a multiple of the band height) and, for K = 12288, 48 k-tiles per output tile.

Reference: the CPU oracle's scaled_mm_* (both operands expanded to fp32 exactly, fp32 matmul, bias)
on a sample of rows -- the first 128, the last 128 and 256 random ones, all N columns.  Rows of a
GEMM are independent, so a row sample checks the same arithmetic as the full product; the sampled
rows' codes and (re-tiled) block scales are what the oracle sees.  Tolerance, as in the reference's
GEMM tests (tests/test_qdq.py:452-509 compare with a high-precision linear):
max |y - ref| <= 1e-2 * max(|ref|, rms(ref)) for bf16 outputs.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

CONFIG_SHAPES = [(m, n, k) for m in (4608, 9216, 18432)
                 for (n, k) in ((9216, 3072), (3072, 3072), (12288, 3072), (3072, 12288))]
# tile rows not a multiple of the band height, M and N not multiples of 256 / 192, long K
RAGGED_SHAPES = [(2344, 1160, 12288), (1300, 3000, 6176)]


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
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (0.02 * torch.randn(N, K, device="cuda", generator=g)).bfloat16()
    bias = 0.02 * torch.randn(N, device="cuda", generator=g)
    return x, w, bias


def _row_sample(M, seed):
    g = torch.Generator().manual_seed(seed)
    idx = torch.cat([torch.arange(min(128, M)), torch.arange(max(M - 128, 0), M), torch.randint(0, M, (256,), generator=g)])
    return torch.unique(idx)


def _sampled_scales(orc, scales, rows, cols, idx):
    """Block scales of the sampled rows, re-tiled for a matrix that holds just those rows."""
    plain = orc.from_blocked(scales.cpu().view(torch.uint8), rows, cols)
    return orc.to_blocked(plain[idx].contiguous())


@pytest.mark.parametrize("M,N,K", CONFIG_SHAPES + RAGGED_SHAPES)
def test_scaled_mm_nvfp4_config_shape(ck, orc, M, N, K):
    x, w, bias = _operands(M, N, K, 10)
    gx = (x.float().abs().max() / (6 * 448)).float()
    gw = (w.float().abs().max() / (6 * 448)).float()
    qx, sx = ck.quantize_nvfp4(x, gx)
    qw, sw = ck.quantize_nvfp4(w, gw)
    y = ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, bias=bias, out_dtype=torch.bfloat16)
    assert ck.gemm_device_status() == 0
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    idx = _row_sample(M, M + N + K)
    sxs = _sampled_scales(orc, sx, M, K // 16, idx)
    ref = orc.scaled_mm_nvfp4(qx[idx.cuda()].cpu(), qw.cpu(), gx.cpu(), gw.cpu(), sxs.view(torch.float8_e4m3fn),
                              sw.cpu(), bias=bias.cpu(), out_dtype=torch.float32)
    err = _rel_err(y[idx.cuda()], ref)
    assert err <= 1e-2, f"max rel err {err}"
    # every row was written (no tile skipped): rows outside the sample have the magnitude of the sampled ones
    assert torch.isfinite(y.float()).all()
    rms_all, rms_s = y.float().pow(2).mean().sqrt().item(), ref.pow(2).mean().sqrt().item()
    assert abs(rms_all - rms_s) <= 0.05 * rms_s


@pytest.mark.parametrize("M,N,K", CONFIG_SHAPES + RAGGED_SHAPES)
def test_scaled_mm_mxfp8_config_shape(ck, orc, M, N, K):
    x, w, bias = _operands(M, N, K, 11)
    qx, sx = ck.quantize_mxfp8(x)
    qw, sw = ck.quantize_mxfp8(w)
    y = ck.scaled_mm_mxfp8(qx, qw, sx, sw, bias=bias, out_dtype=torch.bfloat16)
    assert ck.gemm_device_status() == 0
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    idx = _row_sample(M, M + N + K + 1)
    sxs = _sampled_scales(orc, sx, M, K // 32, idx)
    ref = orc.scaled_mm_mxfp8(qx[idx.cuda()].cpu(), qw.cpu(), sxs.view(torch.float8_e8m0fnu), sw.cpu(),
                              bias=bias.cpu(), out_dtype=torch.float32)
    err = _rel_err(y[idx.cuda()], ref)
    assert err <= 1e-2, f"max rel err {err}"
    assert torch.isfinite(y.float()).all()
    rms_all, rms_s = y.float().pow(2).mean().sqrt().item(), ref.pow(2).mean().sqrt().item()
    assert abs(rms_all - rms_s) <= 0.05 * rms_s


def test_full_product_against_fp64_of_exact_dequantizers(ck):
    """One large shape compared in full.  The reference here is the GPU dequantizers (bit-exact against the
    oracle in the quantizer tests) followed by an fp64 matmul, so that all 18432 x 3072 outputs are checked."""
    M, N, K = 18432, 3072, 12288
    x, w, bias = _operands(M, N, K, 12)
    gx = (x.float().abs().max() / (6 * 448)).float()
    gw = (w.float().abs().max() / (6 * 448)).float()
    qx, sx = ck.quantize_nvfp4(x, gx)
    qw, sw = ck.quantize_nvfp4(w, gw)
    y = ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, bias=bias, out_dtype=torch.float32)
    assert ck.gemm_device_status() == 0
    b = ck.dequantize_nvfp4(qw, gw, sw, torch.float32).double()
    worst = 0.0
    for r0 in range(0, M, 2048):
        a = ck.dequantize_nvfp4(qx[r0:r0 + 2048].contiguous(), gx, _tile_rows(sx, r0, 2048, K // 16), torch.float32)
        ref = (a.double() @ b.t()).float() + bias
        worst = max(worst, _rel_err(y[r0:r0 + 2048], ref))
    assert worst <= 1e-4, f"max rel err {worst}"   # fp32 output: accumulation order only


def _tile_rows(scales, r0, n, cols):
    """Rows r0 .. r0+n-1 of a tiled scale buffer (r0 and n multiples of 128): whole 128-row tiles are contiguous."""
    cpad = (cols + 3) // 4 * 4
    return scales.view(torch.uint8).reshape(-1)[r0 * cpad:(r0 + n) * cpad].view(scales.dtype).reshape(n, cpad)
