"""GPU parity of RoPE and AdaLN (and the fused AdaLN -> quantize kernels), through the C ABI."""
import pytest
import torch

from conftest import cases_of

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ck():
    from comfy_kitchen.backends import cuda

    return cuda


@pytest.fixture(scope="module")
def orc():
    from oracle import ck_oracle

    return ck_oracle


def _same_bits(a, b):
    return torch.equal(a.contiguous().view(torch.uint8).cpu(), b.contiguous().view(torch.uint8).cpu())


def _mismatch_ratio(a, b, rtol=1e-3, atol=1e-3):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).abs() > atol + rtol * b.abs()).float().mean().item()


def flux_freqs(batch, n_txt=512, side=64, theta=10000.0, axes=(16, 56, 56)):
    """fp32 [B,1,N,64,2,2] rotation table from 3-axis position ids: text tokens (0,0,0), image
    tokens (0,row,col) on a side x side grid; axis dims 16/56/56 -> 8/28/28 pairs."""
    ids = torch.zeros(n_txt + side * side, 3)
    rr, cc = torch.meshgrid(torch.arange(side), torch.arange(side), indexing="ij")
    ids[n_txt:, 1], ids[n_txt:, 2] = rr.reshape(-1).float(), cc.reshape(-1).float()
    parts = []
    for a, d in enumerate(axes):
        omega = 1.0 / theta ** (torch.arange(0, d, 2).double() / d)
        ang = ids[:, a].double().unsqueeze(1) * omega.unsqueeze(0)
        parts.append(torch.stack([ang.cos(), -ang.sin(), ang.sin(), ang.cos()], -1).reshape(-1, d // 2, 2, 2))
    f = torch.cat(parts, 1).float()
    return f.reshape(1, 1, *f.shape).expand(batch, 1, -1, -1, -1, -1).contiguous()


# ------------------------------------------------------------------------- RoPE


def test_rope_golden(ck, golden):
    for c in cases_of(golden, "rope"):
        fdt, xdt = c["freqs"].dtype, c["xq"].dtype
        ratio = 1e-5 if (fdt == torch.float32 and xdt == torch.float16) else (0.25 if fdt == torch.bfloat16 else 0.05)
        oq, ok = ck.apply_rope(c["xq"].cuda(), c["xk"].cuda(), c["freqs"].cuda())
        assert _mismatch_ratio(oq, c["oq"]) <= ratio and _mismatch_ratio(ok, c["ok"]) <= ratio
        if "sq" in c:
            sq, sk = ck.apply_rope_split_half(c["xq"].cuda(), c["xk"].cuda(), c["freqs"].cuda())
            assert _mismatch_ratio(sq, c["sq"]) <= ratio and _mismatch_ratio(sk, c["sk"]) <= ratio


@pytest.mark.parametrize("xshape,fshape", [
    ((1, 24, 4352, 128), (1, 1, 4352, 64, 2, 2)),      # BHND, table broadcast over heads
    ((2, 32, 500, 64), (2, 1, 500, 32, 2, 2)),
    ((1, 512, 30, 128), (1, 512, 1, 64, 2, 2)),        # BNHD
    ((2, 3, 17, 20), (2, 1, 17, 10, 2, 2)),            # D not a multiple of 8 -> generic path
    ((1, 2, 8, 16), (1, 1, 12, 8, 2, 2)),              # table longer than the sequence
])
@pytest.mark.parametrize("xdt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("fdt", [torch.float32, torch.bfloat16, torch.float16])
def test_rope_bit_exact_vs_oracle(ck, orc, xshape, fshape, xdt, fdt):
    g = torch.Generator().manual_seed(11)
    xq = torch.randn(xshape, generator=g).to(xdt)
    xk = torch.randn(xshape, generator=g).to(xdt)
    fr = torch.randn(fshape, generator=g).to(fdt)
    oq, ok = ck.apply_rope(xq.cuda(), xk.cuda(), fr.cuda())
    rq, rk = orc.apply_rope(xq, xk, fr)
    # same operation order as the oracle and no fused multiply-add: identical bits
    assert _same_bits(oq, rq) and _same_bits(ok, rk)
    assert _same_bits(ck.apply_rope1(xk.cuda(), fr.cuda()), rk)
    if fshape[2] in (1, xshape[2]):
        sq, sk = ck.apply_rope_split_half(xq.cuda(), xk.cuda(), fr.cuda())
        tq, tk = orc.apply_rope_split_half(xq, xk, fr)
        assert _same_bits(sq, tq) and _same_bits(sk, tk)


def test_rope_flux_table_preserves_norm(ck, orc):
    # full config size: q,k [1,24,4608,128] with a real rotation table.  Rotations preserve the norm
    # of every pair; a 512-token slice is checked against the oracle bit for bit.
    fr = flux_freqs(1).cuda()
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn(1, 24, 4608, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(1, 24, 4608, 128, device="cuda", generator=g).bfloat16()
    oq, ok = ck.apply_rope(q, k, fr)
    n_in = q.float().reshape(-1, 2).norm(dim=1)
    n_out = oq.float().reshape(-1, 2).norm(dim=1)
    assert torch.allclose(n_in, n_out, rtol=2e-2, atol=2e-2)
    sl = slice(400, 912)
    rq, rk = orc.apply_rope(q[:, :, sl].cpu().contiguous(), k[:, :, sl].cpu().contiguous(), fr[:, :, sl].cpu().contiguous())
    assert _same_bits(oq[:, :, sl].contiguous(), rq) and _same_bits(ok[:, :, sl].contiguous(), rk)


# ------------------------------------------------------------------------- AdaLN


def test_adaln_golden(ck, golden):
    for c in cases_of(golden, "adaln"):
        dt = c["x"].dtype
        tol = 1e-2 if dt != torch.float32 else 1e-4
        y = ck.adaln(c["x"].cuda(), c["scale"].cuda(), c["shift"].cuda(), c["eps"])
        torch.testing.assert_close(y.float().cpu(), c["y"].float(), rtol=tol, atol=tol)
        torch.testing.assert_close(y.float().cpu(), c["y_fp32"].to(dt).float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("xshape,mshape", [((2, 256, 768), (2, 1, 768)), ((1, 4608, 3072), (1, 1, 3072)),
                                           ((3, 5, 100), (3, 5, 100)), ((2, 7, 5000), (2, 1, 5000)),
                                           ((1, 300, 12288), (1, 1, 12288)), ((2, 130, 6144), (2, 1, 6144)),
                                           ((2, 16, 64), (2, 1, 64))])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_adaln_vs_oracle(ck, orc, xshape, mshape, dt):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(xshape, generator=g).to(dt)
    sc = (0.1 * torch.randn(mshape, generator=g)).to(dt)
    sh = (0.1 * torch.randn(mshape, generator=g)).to(dt)
    y = ck.adaln(x.cuda(), sc.cuda(), sh.cuda(), 1e-6)
    ref = orc.adaln(x, sc, sh, 1e-6, single_rounding=True)
    tol = 1e-2 if dt != torch.float32 else 1e-4
    torch.testing.assert_close(y.float().cpu(), ref.float(), rtol=tol, atol=tol)
    if dt != torch.float32:
        # one unit in the last place at most, on a tiny fraction of elements (summation order only)
        assert (y.cpu().view(torch.int16) != ref.view(torch.int16)).float().mean().item() < 0.02


@pytest.mark.parametrize("D", [3072, 4096, 1008])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_adaln_rows_with_a_large_mean(ck, orc, D, dt):
    """16-bit rows get their statistics from unshifted sums (tensor cores); a row whose mean is many standard
    deviations away from zero must come out as accurately as one centred on zero (the kernel then sums again,
    shifted).  Offsets on both sides of that switch, and constant rows."""
    g = torch.Generator().manual_seed(12)
    offsets = torch.tensor([0.0, 3.0, -8.0, 12.0, 20.0, -50.0, 100.0, 7.5])
    N = 8 * 40
    spread = torch.tensor([1.0, 0.5, 2.0, 0.25, 1.0])
    x = torch.randn(N, D, generator=g) * spread[torch.arange(N) % 5, None] + offsets[torch.arange(N) % 8, None]
    x[5] = 3.25      # constant rows
    x[6] = -100.0
    x = x.to(dt).reshape(1, N, D)
    sc = (0.1 * torch.randn(1, 1, D, generator=g)).to(dt)
    sh = (0.1 * torch.randn(1, 1, D, generator=g)).to(dt)
    y = ck.adaln(x.cuda(), sc.cuda(), sh.cuda(), 1e-6)
    ref = orc.adaln(x, sc, sh, 1e-6, single_rounding=True)
    torch.testing.assert_close(y.float().cpu(), ref.float(), rtol=1e-2, atol=1e-2)
    assert (y.cpu().view(torch.int16) != ref.view(torch.int16)).float().mean().item() < 0.02
    # the fused kernel sees the same statistics
    yy = y.reshape(N, D)
    gs = (yy.float().abs().max() / (6 * 448)).float()
    q, sf = ck.adaln_quantize_nvfp4(x.cuda(), sc.cuda(), sh.cuda(), gs, 1e-6)
    q2, sf2 = ck.quantize_nvfp4(yy, gs)
    assert torch.equal(q, q2) and torch.equal(sf.view(torch.uint8), sf2.view(torch.uint8))


@pytest.mark.parametrize("B,T,D", [(5, 130, 1024), (3, 1000, 3072), (7, 64, 512)])
def test_norm_with_several_modulation_groups(ck, orc, B, T, D):
    """Each modulation group (batch entry) gets its own share of the CTAs; group sizes that are no multiple of the
    128-row scale tiles, so the last CTA also owns the scale buffer's padding rows.  Plain output against the oracle,
    fused outputs against norm kernel -> quantizer (padding bytes of the scale buffer included)."""
    g = torch.Generator().manual_seed(21)
    x = torch.randn(B, T, D, generator=g).bfloat16()
    sc = (0.2 * torch.randn(B, 1, D, generator=g)).bfloat16()
    sh = (0.2 * torch.randn(B, 1, D, generator=g)).bfloat16()
    y = ck.adaln(x.cuda(), sc.cuda(), sh.cuda(), 1e-6)
    ref = orc.adaln(x, sc, sh, 1e-6, single_rounding=True)
    torch.testing.assert_close(y.float().cpu(), ref.float(), rtol=1e-2, atol=1e-2)
    assert (y.cpu().view(torch.int16) != ref.view(torch.int16)).float().mean().item() < 0.02
    yy = y.reshape(B * T, D)
    gs = (yy.float().abs().max() / (6 * 448)).float()
    q, sf = ck.adaln_quantize_nvfp4(x.cuda(), sc.cuda(), sh.cuda(), gs, 1e-6)
    q2, sf2 = ck.quantize_nvfp4(yy, gs)
    assert torch.equal(q, q2) and torch.equal(sf.view(torch.uint8), sf2.view(torch.uint8))
    q8, sf8 = ck.adaln_quantize_mxfp8(x.cuda(), sc.cuda(), sh.cuda(), 1e-6)
    q8b, sf8b = ck.quantize_mxfp8(yy)
    assert torch.equal(q8.view(torch.uint8), q8b.view(torch.uint8))
    assert torch.equal(sf8.view(torch.uint8), sf8b.view(torch.uint8))


def test_rmsnorm_vs_torch(ck):
    g = torch.Generator().manual_seed(6)
    x = torch.randn(64, 24, 128, generator=g).bfloat16().cuda()
    w = (1 + 0.1 * torch.randn(128, generator=g)).bfloat16().cuda()
    y = ck.rmsnorm(x, w, 1e-6)
    ref = torch.nn.functional.rms_norm(x.float(), (128,), w.float(), 1e-6).bfloat16()
    torch.testing.assert_close(y.float(), ref.float(), rtol=1e-2, atol=1e-2)


# 3072 and 4096: fully unrolled builds; 6144: one row buffer per warp; 12288: no modulation cache (it would
# leave room for four warps only); 8192: between the two
@pytest.mark.parametrize("N,D,B", [(4608, 3072, 1), (9216, 3072, 2), (200, 1024, 2), (130, 64, 1), (77, 4096, 1),
                                   (520, 6144, 2), (300, 8192, 1), (300, 12288, 1)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_fused_adaln_quantize_is_adaln_then_quantize(ck, orc, N, D, B, dt):
    g = torch.Generator().manual_seed(8)
    T = N // B if N % B == 0 else N
    B = N // T
    x = torch.randn(B, T, D, generator=g).to(dt).cuda()
    sc = (0.1 * torch.randn(B, 1, D, generator=g)).to(dt).cuda()
    sh = (0.1 * torch.randn(B, 1, D, generator=g)).to(dt).cuda()
    y = ck.adaln(x, sc, sh, 1e-6).reshape(N, D)
    gs = (y.float().abs().max() / (6 * 448)).float()
    q, sf = ck.adaln_quantize_nvfp4(x, sc, sh, gs, 1e-6)
    q2, sf2 = ck.quantize_nvfp4(y, gs)
    assert torch.equal(sf.view(torch.uint8), sf2.view(torch.uint8))
    assert torch.equal(q, q2)
    # and "adaln kernel then quantize" equals the CPU oracle's quantizer on the same activation
    q3, sf3 = orc.quantize_nvfp4(y.cpu(), gs.cpu())
    assert torch.equal(q.cpu(), q3) and torch.equal(sf.view(torch.uint8).cpu(), sf3.view(torch.uint8))
    if D % 32 == 0:
        q8, sf8 = ck.adaln_quantize_mxfp8(x, sc, sh, 1e-6)
        q8b, sf8b = ck.quantize_mxfp8(y)
        assert torch.equal(q8.view(torch.uint8), q8b.view(torch.uint8))
        assert torch.equal(sf8.view(torch.uint8), sf8b.view(torch.uint8))


def test_fused_vs_all_eager_composition_mismatch_rate(ck, orc, golden):
    # against "eager adaln, eager quantize" only a small fraction of codes may differ (LayerNorm
    # summation order moves a few activations across an FP4 rounding boundary)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(1, 256, 3072, generator=g).bfloat16()
    sc = (0.1 * torch.randn(1, 1, 3072, generator=g)).bfloat16()
    sh = (0.1 * torch.randn(1, 1, 3072, generator=g)).bfloat16()
    y_eager = orc.adaln(x, sc, sh, 1e-6).reshape(256, 3072)
    gs = (y_eager.float().abs().max() / (6 * 448)).float()
    q_ref, _ = orc.quantize_nvfp4(y_eager, gs)
    q, _ = ck.adaln_quantize_nvfp4(x.cuda(), sc.cuda(), sh.cuda(), gs.cuda(), 1e-6)
    lo = (q.cpu() & 0xF) != (q_ref & 0xF)
    hi = (q.cpu() >> 4) != (q_ref >> 4)
    assert (lo.float().mean() + hi.float().mean()).item() / 2 < 0.02


@pytest.mark.parametrize("group", [2, 4])
@pytest.mark.parametrize("N,D", [(300, 2048), (257, 4352), (130, 12288)])
def test_warp_groups_per_row(ck, orc, group, N, D):
    """Rows shared by 2 or 4 warps (forced here on narrow rows too; the launcher uses them for rows that do not
    fit 16 single warps): the fused outputs still equal adaln -> quantize byte for byte, AdaLN itself stays
    within one bf16 step of the exactly rounded value, RMSNorm takes the same path, padding rows and columns of the scale buffer
    are written, and no bounded wait runs out."""
    g = torch.Generator().manual_seed(12)
    x = torch.randn(1, N, D, generator=g).bfloat16().cuda()
    sc = (0.1 * torch.randn(1, 1, D, generator=g)).bfloat16().cuda()
    sh = (0.1 * torch.randn(1, 1, D, generator=g)).bfloat16().cuda()
    w = (1 + 0.1 * torch.randn(D, generator=g)).bfloat16().cuda()
    ck.set_option("norm_group", group)
    try:
        y = ck.adaln(x, sc, sh, 1e-6).reshape(N, D)
        gs = (y.float().abs().max() / (6 * 448)).float()
        q, sf = ck.adaln_quantize_nvfp4(x, sc, sh, gs, 1e-6)
        q2, sf2 = ck.quantize_nvfp4(y, gs)
        assert torch.equal(q, q2) and torch.equal(sf.view(torch.uint8), sf2.view(torch.uint8))
        q8, sf8 = ck.adaln_quantize_mxfp8(x, sc, sh, 1e-6)
        q8b, sf8b = ck.quantize_mxfp8(y)
        assert torch.equal(q8.view(torch.uint8), q8b.view(torch.uint8))
        assert torch.equal(sf8.view(torch.uint8), sf8b.view(torch.uint8))
        yr = ck.rmsnorm(x.reshape(N, D), w, 1e-6)
        qr, sr = ck.rmsnorm_quantize_nvfp4(x.reshape(N, D), w, gs, 1e-6)
        qr2, sr2 = ck.quantize_nvfp4(yr, gs)
        assert torch.equal(qr, qr2) and torch.equal(sr.view(torch.uint8), sr2.view(torch.uint8))
    finally:
        ck.set_option("norm_group", 0)
    # against the fp64 value rounded once to bf16: at most one bf16 step away, and rarely (the kernel's fp32
    # statistics move a few values across a rounding boundary, with one warp per row just as with four)
    xd = x.cpu().double()
    mean, var = xd.mean(-1, keepdim=True), xd.var(-1, unbiased=False, keepdim=True)
    exact = ((xd - mean) / torch.sqrt(var + 1e-6) * (1 + sc.cpu().double()) + sh.cpu().double()).reshape(N, D)
    want = exact.float().bfloat16()
    got = y.cpu()
    assert (got != want).float().mean().item() < 1e-3
    # (the absolute floor covers values that are themselves the small difference of terms of size one, where fp32
    # evaluation is only accurate to about 1e-7 absolute)
    assert ((got.float() - want.float()).abs() <= 2.0 ** -7 * want.float().abs() + 1e-6).all()
    assert ck.norm_device_status() == 0


def test_rmsnorm_quantize(ck):
    g = torch.Generator().manual_seed(10)
    x = torch.randn(300, 1024, generator=g).bfloat16().cuda()
    w = (1 + 0.1 * torch.randn(1024, generator=g)).bfloat16().cuda()
    y = ck.rmsnorm(x, w, 1e-6)
    gs = (y.float().abs().max() / (6 * 448)).float()
    q, sf = ck.rmsnorm_quantize_nvfp4(x, w, gs, 1e-6)
    q2, sf2 = ck.quantize_nvfp4(y, gs)
    assert torch.equal(q, q2) and torch.equal(sf.view(torch.uint8), sf2.view(torch.uint8))


def test_norm_status_word_is_clear(ck):
    """The norm kernels' bounded waits have not run out in anything this file launched."""
    x = torch.randn(2, 300, 3072, device="cuda").bfloat16()
    sc = (0.1 * torch.randn(2, 1, 3072, device="cuda")).bfloat16()
    ck.adaln(x, sc, sc, 1e-6)
    assert ck.norm_device_status() == 0


@pytest.mark.parametrize("group", [0, 2])
def test_norm_bounded_wait_runs_out_and_recovers(ck, group):
    """The time-out path of the norm kernel's row waits, exercised without any fault: with the library's
    poll limit set to "no poll" every consumer gives its first row up at once, records the status word and
    leaves (after waiting, with the normal limit, for the copies it had in flight).  The call returns, the
    status call reports CK_ERR_DEVICE_TIMEOUT once and clears, and the next normal call is correct."""
    g = torch.Generator().manual_seed(21)
    x = torch.randn(1, 200, 3072, generator=g).bfloat16().cuda()
    sc = (0.1 * torch.randn(1, 1, 3072, generator=g)).bfloat16().cuda()
    sh = (0.1 * torch.randn(1, 1, 3072, generator=g)).bfloat16().cuda()
    want = ck.adaln(x, sc, sh, 1e-6)
    assert ck.norm_device_status() == 0
    ck.set_option("norm_poll_limit", -1)
    ck.set_option("norm_group", group)
    try:
        ck.adaln(x, sc, sh, 1e-6)
        status = ck.norm_device_status()      # synchronises: the kernel has returned
    finally:
        ck.set_option("norm_poll_limit", 0)
        ck.set_option("norm_group", 0)
    assert status == -6                        # CK_ERR_DEVICE_TIMEOUT
    from comfy_kitchen import _native
    assert b"bounded wait" in _native.load().ck_last_error()
    assert ck.norm_device_status() == 0       # cleared by the read
    again = ck.adaln(x, sc, sh, 1e-6)
    assert torch.equal(again, want)
    assert ck.norm_device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_qk_norm_rope_matches_composition(ck, dtype):
    """Fused per-head RMSNorm + RoPE + relayout against rms_norm (fp32) -> oracle rope -> permute; two calls fill a
    joint sequence (text then image tokens); the qkv of the second call is a column slice of a wider matrix."""
    from tests import dit_oracle_ops as ops

    g = torch.Generator().manual_seed(3)
    heads, t_txt, t_img = 3, 37, 210
    total = t_txt + t_img
    ang = torch.rand(total, 64, generator=g) * 6.28
    f = torch.stack([torch.stack([ang.cos(), -ang.sin()], -1), torch.stack([ang.sin(), ang.cos()], -1)], -2)[None, None].contiguous()
    qkv_txt = (2 * torch.randn(t_txt, 3 * heads * 128, generator=g)).to(dtype)
    wide = (2 * torch.randn(t_img, 3 * heads * 128 + 256, generator=g)).to(dtype)
    qw = (1 + 0.1 * torch.randn(128, generator=g)).to(dtype)
    kw = (1 + 0.1 * torch.randn(128, generator=g)).to(dtype)
    want = ops.qk_norm_rope(qkv_txt, qw, kw, f, heads, None, None, None, 0, 1e-6)
    want = ops.qk_norm_rope(wide[:, :3 * heads * 128], qw, kw, f, heads, *want, t_txt, 1e-6)
    got = ck.qk_norm_rope(qkv_txt.cuda(), qw.cuda(), kw.cuda(), f.cuda(), heads, None, None, None, 0, 1e-6)
    wide_d = wide.cuda()
    got = ck.qk_norm_rope(wide_d[:, :3 * heads * 128], qw.cuda(), kw.cuda(), f.cuda(), heads, *got, t_txt, 1e-6)
    assert got[0].shape == (1, heads, total, 128)
    assert torch.equal(got[2].cpu(), want[2])                       # v is a copy
    for a, b in zip(got[:2], want[:2]):
        # the norm's rounding to the 16-bit dtype can differ by one ulp between summation orders and is then rotated
        torch.testing.assert_close(a.float().cpu(), b.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("heads", [24, 7])
def test_qk_norm_rope_heads_per_warp_setting_changes_no_byte(ck, heads):
    """One head per warp (the default), compile-time counts that divide the heads, a count that does not (the
    run-time walk) and all heads in one warp: the same bytes, the arithmetic per (token, head) is the same."""
    g = torch.Generator().manual_seed(9)
    tokens = 333
    ang = torch.rand(tokens, 64, generator=g) * 6.28
    f = torch.stack([torch.stack([ang.cos(), -ang.sin()], -1), torch.stack([ang.sin(), ang.cos()], -1)], -2)[None, None].contiguous().cuda()
    qkv = (2 * torch.randn(tokens, 3 * heads * 128, generator=g)).bfloat16().cuda()
    qw = (1 + 0.1 * torch.randn(128, generator=g)).bfloat16().cuda()
    kw = (1 + 0.1 * torch.randn(128, generator=g)).bfloat16().cuda()
    try:
        base = ck.qk_norm_rope(qkv, qw, kw, f, heads)
        for hpw in (2, 3, 4, 5, 6, heads):
            ck.set_option("qk_heads_per_warp", hpw)
            got = ck.qk_norm_rope(qkv, qw, kw, f, heads)
            for a, b in zip(got, base):
                assert torch.equal(a, b), f"heads per warp {hpw}"
    finally:
        ck.set_option("qk_heads_per_warp", 0)
