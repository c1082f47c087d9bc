"""GPU parity of the quantizers / dequantizers, through the C ABI, against the CPU oracle
and the reference-generated fixtures.  Integer outputs must be bit-identical."""
import pytest
import torch

from conftest import cases_of

pytestmark = pytest.mark.gpu

DT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


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


def _outliers(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    mask = torch.rand(shape, generator=g) < 0.001
    return torch.where(mask, 50.0 * torch.randn(shape, generator=g), x).to(dtype)


# ----------------------------------------------------------------- golden fixtures


def test_nvfp4_golden(ck, golden):
    for c in cases_of(golden, "quantize_nvfp4"):
        x = c["x"].cuda()
        q, sf = ck.quantize_nvfp4(x, c["scale"].cuda(), pad_16x=c["pad"], hi_first=c["hi_first"])
        assert torch.equal(sf.view(torch.uint8).cpu(), c["sf"]), f"scales {tuple(x.shape)} {x.dtype}"
        assert torch.equal(q.cpu(), c["q"]), f"codes {tuple(x.shape)} {x.dtype}"
        for name, dt in DT.items():
            if "dq_" + name in c:
                out = ck.dequantize_nvfp4(c["q"].cuda(), c["scale"].cuda(), c["sf"].cuda().view(torch.float8_e4m3fn),
                                          dt, hi_first=c["hi_first"])
                assert _same_bits(out, c["dq_" + name]), f"dequant {name} {tuple(x.shape)}"


def test_mxfp8_golden(ck, golden):
    for c in cases_of(golden, "quantize_mxfp8"):
        x = c["x"].cuda()
        q, sf = ck.quantize_mxfp8(x, pad_32x=c["pad"])
        assert torch.equal(sf.view(torch.uint8).cpu(), c["sf"]), f"scales {tuple(x.shape)} {x.dtype}"
        assert torch.equal(q.view(torch.uint8).cpu(), c["q"]), f"data {tuple(x.shape)} {x.dtype}"
        for name, dt in DT.items():
            if "dq_" + name in c:
                out = ck.dequantize_mxfp8(c["q"].cuda().view(torch.float8_e4m3fn),
                                          c["sf"].cuda().view(torch.float8_e8m0fnu), dt)
                assert _same_bits(out, c["dq_" + name]), f"dequant {name} {tuple(x.shape)}"


def test_fp8_golden(ck, golden):
    for c in cases_of(golden, "quantize_fp8"):
        ot = torch.float8_e4m3fn if c["out"] == "e4m3" else torch.float8_e5m2
        q = ck.quantize_per_tensor_fp8(c["x"].cuda(), c["scale"].cuda(), ot)
        assert torch.equal(q.view(torch.uint8).cpu(), c["q"]), f"{c['x'].dtype} {c['out']} {float(c['scale'])}"
        for name, dt in DT.items():
            if "dq_" + name in c:
                out = ck.dequantize_per_tensor_fp8(c["q"].cuda().view(ot), c["scale"].cuda(), dt)
                assert _same_bits(out, c["dq_" + name])


# ----------------------------------------------------------------- known answers


def test_known_answers(ck):
    x = (torch.arange(16).float() / 2).reshape(1, 16).bfloat16().cuda()
    g = torch.tensor(7.5 / (6 * 448), device="cuda")
    q, sf = ck.quantize_nvfp4(x, g)
    assert q.flatten().tolist() == [1, 34, 52, 69, 86, 102, 103, 119]
    assert int(sf.view(torch.uint8)[0, 0]) == 126
    assert int(sf.view(torch.uint8).sum()) == 126  # every padding byte of the 128x4 buffer is zero
    x = torch.zeros(1, 16).bfloat16()
    x[0, 0], x[0, 1] = 6.0, 3.0
    g = torch.tensor(1.0 / 448, device="cuda")
    assert int(ck.quantize_nvfp4(x.cuda(), g, hi_first=True)[0][0, 0]) == 0x75
    assert int(ck.quantize_nvfp4(x.cuda(), g, hi_first=False)[0][0, 0]) == 0x57
    # E2M1 ties and signed zero: one value per block so the block scale is exactly 1 when amax = 6
    v = [0, 0.1, 0.25, 0.2500001, 0.5, 0.75, 1, 1.25, 1.5, 1.75, 2, 2.5, 3, 3.5, 4, 5, 5.0000005, 6,
         -0.25, -0.75, -5, -6, -0.0]
    want = [0, 0, 0, 1, 1, 2, 2, 2, 3, 4, 4, 4, 5, 6, 6, 6, 7, 7, 8, 10, 14, 15, 8]
    x = torch.zeros(len(v), 16)
    x[:, 0] = torch.tensor(v)
    x[:, 1] = 6.0
    q, sf = ck.quantize_nvfp4(x.cuda(), torch.tensor(1.0 / 64, device="cuda"))  # block scale 64, total exactly 1
    assert int(sf.view(torch.uint8)[0, 0]) == 0x68
    assert (q[:, 0] >> 4).tolist() == want
    for val, e, qv in [(448.0, 127, 448.0), (449.0, 127, 448.0), (1.75, 119, 448.0), (1e-30, 19, 320.0),
                       (3e38, 247, 224.0)]:
        x = torch.zeros(1, 32).bfloat16()
        x[0, 0] = val
        q, sf = ck.quantize_mxfp8(x.cuda())
        assert int(sf.view(torch.uint8)[0, 0]) == e and float(q[0, 0].float()) == qv, val
    x = torch.tensor([1.0039062, 3.140625, 447, 500]).bfloat16().cuda()
    assert ck.quantize_per_tensor_fp8(x, torch.tensor(0.3, device="cuda")).view(torch.uint8).tolist() == [69, 82, 126, 126]


# ----------------------------------------------------------------- oracle parity on seeded inputs


@pytest.mark.parametrize("shape,pad", [((1024, 3072), False), ((129, 128), False), ((33, 65), True),
                                       ((4608, 256), False), ((200, 1040), False), ((2048, 4096), False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_nvfp4_vs_oracle(ck, orc, shape, pad, dtype):
    if dtype != torch.bfloat16 and shape[0] * shape[1] > 2_000_000:
        pytest.skip("large shapes only in bf16")
    x = _outliers(shape, 1, dtype)
    g = (x.float().abs().max() / (6.0 * 448.0)).float()
    q_ref, sf_ref = orc.quantize_nvfp4(x, g, pad_16x=pad)
    q, sf = ck.quantize_nvfp4(x.cuda(), g.cuda(), pad_16x=pad)
    assert torch.equal(sf.view(torch.uint8).cpu(), sf_ref.view(torch.uint8))
    assert torch.equal(q.cpu(), q_ref)
    for odt in (torch.bfloat16, torch.float32, torch.float16):
        d = ck.dequantize_nvfp4(q, g.cuda(), sf, odt)
        assert _same_bits(d, orc.dequantize_nvfp4(q_ref, g, sf_ref, odt))


@pytest.mark.parametrize("shape,pad", [((1024, 3072), False), ((65, 96), True), ((257, 288), False),
                                       ((4608, 128), False), ((2048, 4096), False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_mxfp8_vs_oracle(ck, orc, shape, pad, dtype):
    if dtype != torch.bfloat16 and shape[0] * shape[1] > 2_000_000:
        pytest.skip("large shapes only in bf16")
    x = _outliers(shape, 2, dtype)
    q_ref, sf_ref = orc.quantize_mxfp8(x, pad_32x=pad)
    q, sf = ck.quantize_mxfp8(x.cuda(), pad_32x=pad)
    assert torch.equal(sf.view(torch.uint8).cpu(), sf_ref.view(torch.uint8))
    assert torch.equal(q.view(torch.uint8).cpu(), q_ref.view(torch.uint8))
    for odt in (torch.bfloat16, torch.float32, torch.float16):
        d = ck.dequantize_mxfp8(q, sf, odt)
        assert _same_bits(d, orc.dequantize_mxfp8(q_ref, sf_ref, odt))


def test_mxfp8_tiny_blocks(ck, orc):
    # blocks whose scale byte is 0 or 1 (|amax| around 2^-118): the reference's 0-scale corner
    x = torch.zeros(2, 64).bfloat16()
    x[0, 0], x[0, 1], x[0, 32], x[0, 33] = 2.0 ** -120, -(2.0 ** -125), 2.0 ** -117, 2.0 ** -126
    x[1, 5] = 2.0 ** -119
    q_ref, sf_ref = orc.quantize_mxfp8(x)
    q, sf = ck.quantize_mxfp8(x.cuda())
    assert torch.equal(sf.view(torch.uint8).cpu(), sf_ref.view(torch.uint8))
    assert torch.equal(q.view(torch.uint8).cpu(), q_ref.view(torch.uint8))


@pytest.mark.parametrize("numel_shape", [(1024, 3072), (7, 13), (4097, 33), (2048, 4096)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("ot", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_fp8_vs_oracle(ck, orc, numel_shape, dtype, ot):
    x = _outliers(numel_shape, 3, dtype)
    lp_max = 448.0 if ot == torch.float8_e4m3fn else 57344.0
    s = (x.float().abs().max() / lp_max).float()
    q_ref = orc.quantize_per_tensor_fp8(x, s, ot)
    q = ck.quantize_per_tensor_fp8(x.cuda(), s.cuda(), ot)
    assert torch.equal(q.view(torch.uint8).cpu(), q_ref.view(torch.uint8))
    for odt in (torch.bfloat16, torch.float32, torch.float16):
        assert _same_bits(ck.dequantize_per_tensor_fp8(q, s.cuda(), odt), orc.dequantize_per_tensor_fp8(q_ref, s, odt))


# ----------------------------------------------------------------- size-independent properties at full size


def test_full_size_properties(ck, orc):
    M, K = 65536, 3072
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(M, K, device="cuda", generator=g, dtype=torch.float32)
    x = torch.where(torch.rand(M, K, device="cuda", generator=g) < 0.001, 50.0 * x, x).bfloat16()
    gs = (x.float().abs().max() / (6.0 * 448.0)).float()
    q, sf = ck.quantize_nvfp4(x, gs)
    # rows are independent: any row slice quantizes to the same bytes, and the oracle agrees on a sample
    rows = torch.cat([torch.arange(0, 256), torch.randint(0, M, (1024,), generator=torch.Generator().manual_seed(0))])
    rows = rows.unique()[: 1152 // 128 * 128]
    xs = x[rows.cuda()].contiguous()
    q_s, sf_s = ck.quantize_nvfp4(xs, gs)
    assert torch.equal(q_s, q[rows.cuda()])
    q_ref, sf_ref = orc.quantize_nvfp4(xs.cpu(), gs.cpu())
    assert torch.equal(q_s.cpu(), q_ref) and torch.equal(sf_s.view(torch.uint8).cpu(), sf_ref.view(torch.uint8))
    # idempotence: quantizing the dequantized tensor with the same scale reproduces codes and scales
    d = ck.dequantize_nvfp4(q, gs, sf, torch.float32)
    q2, sf2 = ck.quantize_nvfp4(d, gs)
    assert torch.equal(sf2.view(torch.uint8), sf.view(torch.uint8)) and torch.equal(q2, q)
    # MXFP8: the round trip stays within half an E4M3 step of the block's scale
    q8, sf8 = ck.quantize_mxfp8(x)
    d8 = ck.dequantize_mxfp8(q8, sf8, torch.float32)
    from comfy_kitchen.float_utils import e8m0_to_f32, from_blocked
    step = e8m0_to_f32(from_blocked(sf8.view(torch.uint8), M, K // 32)).repeat_interleave(32, dim=1)
    err = (d8 - x.float()).abs()
    bound = torch.maximum(x.float().abs() * 2.0 ** -4, step * 2.0 ** -10)
    assert bool((err <= bound).all())
    del step, err, bound, d8
    # FP8: dequantize(quantize(x)) requantizes to the same codes.  The fp32 dequantized value is code * scale
    # rounded once, and multiplying it by fp32(1 / scale) lands within 2^-22 of the code, far inside the
    # E4M3 rounding interval, so the bytes must come back unchanged.
    s = (x.float().abs().max() / 448.0).float()
    q1 = ck.quantize_per_tensor_fp8(x, s)
    d1 = ck.dequantize_per_tensor_fp8(q1, s, torch.float32)
    q1b = ck.quantize_per_tensor_fp8(d1, s)
    assert torch.equal(q1b.view(torch.uint8), q1.view(torch.uint8))


SWEEP_SHAPES = [(m, k) for m in (1024, 4608, 18432, 65536) for k in (3072, 12288)]


@pytest.mark.parametrize("M,K", SWEEP_SHAPES)
def test_sweep_shapes_vs_oracle_row_samples(ck, orc, M, K):
    """Every shape of the quantizer sweep, all three formats: the device result on the whole tensor must equal the
    CPU oracle's on a row sample (rows 0..255, the last 128 and 640 random ones).  Rows are independent for all
    three quantizers -- only the per-tensor scale is global and it is passed in -- and block scales of sampled
    rows are compared after un-tiling."""
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(M, K, device="cuda", generator=g, dtype=torch.float32)
    x = torch.where(torch.rand(M, K, device="cuda", generator=g) < 0.001, 50.0 * torch.randn(M, K, device="cuda", generator=g), x)
    x = x.bfloat16()
    rows = torch.cat([torch.arange(0, 256), torch.arange(M - 128, M),
                      torch.randint(0, M, (640,), generator=torch.Generator().manual_seed(M + K))]).unique()
    rc = rows.cuda()
    xs = x[rc].cpu()
    amax = x.float().abs().max()
    # NVFP4
    gs = (amax / (6.0 * 448.0)).float()
    q, sf = ck.quantize_nvfp4(x, gs)
    q_ref, sf_ref = orc.quantize_nvfp4(xs, gs.cpu())
    assert torch.equal(q[rc].cpu(), q_ref)
    sf_plain = orc.from_blocked(sf.view(torch.uint8).cpu(), M, K // 16)
    assert torch.equal(sf_plain[rows], orc.from_blocked(sf_ref.view(torch.uint8), len(rows), K // 16))
    d = ck.dequantize_nvfp4(q, gs, sf, torch.bfloat16)
    assert _same_bits(d[rc], orc.dequantize_nvfp4(q_ref, gs.cpu(), sf_ref, torch.bfloat16))
    del q, sf, d
    # MXFP8
    q8, sf8 = ck.quantize_mxfp8(x)
    q8_ref, sf8_ref = orc.quantize_mxfp8(xs)
    assert torch.equal(q8[rc].view(torch.uint8).cpu(), q8_ref.view(torch.uint8))
    sf8_plain = orc.from_blocked(sf8.view(torch.uint8).cpu(), M, K // 32)
    assert torch.equal(sf8_plain[rows], orc.from_blocked(sf8_ref.view(torch.uint8), len(rows), K // 32))
    d8 = ck.dequantize_mxfp8(q8, sf8, torch.bfloat16)
    assert _same_bits(d8[rc], orc.dequantize_mxfp8(q8_ref, sf8_ref, torch.bfloat16))
    del q8, sf8, d8
    # FP8 per tensor
    s = (amax / 448.0).float()
    qf = ck.quantize_per_tensor_fp8(x, s)
    qf_ref = orc.quantize_per_tensor_fp8(xs, s.cpu())
    assert torch.equal(qf[rc].view(torch.uint8).cpu(), qf_ref.view(torch.uint8))
    df = ck.dequantize_per_tensor_fp8(qf, s, torch.bfloat16)
    assert _same_bits(df[rc], orc.dequantize_per_tensor_fp8(qf_ref, s.cpu(), torch.bfloat16))


def test_nvfp4_reciprocal_division_is_exact(ck):
    """The quantizer's shared-reciprocal divisions must give the same bytes as plain IEEE
    divisions: compared on the device over many tensors, per-tensor scales and dtypes."""
    gen = torch.Generator(device="cuda").manual_seed(123)
    total = 0
    for i in range(40):
        dt = (torch.bfloat16, torch.float16, torch.float32)[i % 3]
        M, K = 8192, 2048
        x = torch.randn(M, K, device="cuda", generator=gen)
        if i % 4 == 1:
            x = x * torch.exp2(torch.randint(-12, 12, (M, 1), device="cuda", generator=gen).float())
        if i % 4 == 2:
            x = torch.where(torch.rand(M, K, device="cuda", generator=gen) < 0.01, 40.0 * x, x)
        if i % 4 == 3:
            x = (x * 4).round() / 4  # many exact ties, and both signs of zero
            x = torch.where(x == 0, torch.where(torch.rand(M, K, device="cuda", generator=gen) < 0.5, -0.0, 0.0), x)
        x = x.to(dt)
        amax = x.float().abs().max()
        # a spread of per-tensor scales: the natural one, ones that clamp block scales at 448, tiny, huge
        g = amax / (6.0 * 448.0) * float(torch.tensor([1.0, 0.037, 1.7, 1e-3, 64.0][i % 5]))
        if i == 7:
            g = torch.tensor(2.0 ** -100, device="cuda")   # outside the fast range: IEEE path inside the kernel
        g = g.float().reshape(1)
        ck.set_option("nvfp4_exact_div", 0)
        q_fast, sf_fast = ck.quantize_nvfp4(x, g)
        ck.set_option("nvfp4_exact_div", 1)
        try:
            q_ref, sf_ref = ck.quantize_nvfp4(x, g)
        finally:
            ck.set_option("nvfp4_exact_div", 0)
        assert torch.equal(sf_fast.view(torch.uint8), sf_ref.view(torch.uint8)), f"scales differ in tensor {i}"
        assert torch.equal(q_fast, q_ref), f"codes differ in tensor {i}"
        total += x.numel()
    assert total > 6e8


def test_argument_errors(ck):
    x = torch.randn(16, 24, device="cuda").bfloat16()
    with pytest.raises((AssertionError, RuntimeError)):
        ck.quantize_nvfp4(x, torch.tensor(1.0, device="cuda"))  # 24 is not a multiple of 16
    with pytest.raises((AssertionError, RuntimeError)):
        ck.quantize_mxfp8(x)
    with pytest.raises(ValueError):
        ck.quantize_per_tensor_fp8(x, torch.tensor(1.0, device="cuda"), torch.bfloat16)
    from comfy_kitchen import _native
    import ctypes
    with pytest.raises(RuntimeError, match="multiple of 16"):
        _native.call("launch_quantize_nvfp4_kernel", ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x.data_ptr()),
                     ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x.data_ptr()), 16, 24, 16, 24, 0.0, 2, True,
                     ctypes.c_void_p(0))


def test_quantize_nvfp4_gather_matches_concatenation():
    """Gathered source (attention layout + column slice) without activation: bytes equal cat -> quantize_nvfp4;
    with GELU on the second segment: equal to the oracle on torch's gelu except where the two tanh
    implementations round a bf16 value differently (a handful of blocks)."""
    from comfy_kitchen.backends import cuda as ck
    from tests import dit_oracle_ops as ops

    g = torch.Generator().manual_seed(5)
    heads, rows, d = 3, 300, 128
    o_full = torch.randn(heads, rows + 50, d, generator=g).bfloat16()       # a token range of a longer sequence
    wide = (1.5 * torch.randn(rows, 3 * heads * d + 512, generator=g)).bfloat16()
    seg0, seg1 = o_full[:, 50:], wide[:, 3 * heads * d:]
    gs = torch.tensor(4.0 / (6 * 448))
    o_d, wide_d = o_full.cuda(), wide.cuda()
    seg0_d, seg1_d = o_d[:, 50:], wide_d[:, 3 * heads * d:]
    # no activation: exact
    q, sf = ck.quantize_nvfp4_gather([(seg0_d, None), (seg1_d, None)], gs.cuda())
    q_ref, sf_ref = ops.quantize_nvfp4_gather([(seg0, None), (seg1, None)], gs)
    assert q.shape == (rows, (heads * d + 512) // 2)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(sf.view(torch.uint8).cpu(), sf_ref.view(torch.uint8))
    # one segment only
    q1, sf1 = ck.quantize_nvfp4_gather([(seg0_d, None)], gs.cuda())
    q1_ref, sf1_ref = ops.quantize_nvfp4_gather([(seg0, None)], gs)
    assert torch.equal(q1.cpu(), q1_ref) and torch.equal(sf1.view(torch.uint8).cpu(), sf1_ref.view(torch.uint8))
    # GELU on the second segment
    q2, sf2 = ck.quantize_nvfp4_gather([(seg0_d, None), (seg1_d, "gelu_tanh")], gs.cuda())
    q2_ref, sf2_ref = ops.quantize_nvfp4_gather([(seg0, None), (seg1, "gelu_tanh")], gs)
    n0 = heads * d // 2
    assert torch.equal(q2.cpu()[:, :n0], q2_ref[:, :n0])                     # the plain segment stays exact
    bad_codes = (q2.cpu() != q2_ref).float().mean().item()
    bad_scales = (sf2.view(torch.uint8).cpu() != sf2_ref.view(torch.uint8)).float().mean().item()
    assert bad_codes < 2e-3 and bad_scales < 2e-3, (bad_codes, bad_scales)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_quantize_nvfp4_gather_table_path_equals_arithmetic_path(dt):
    """Large activated inputs go through a per-CTA table of round(gelu(x)) over all 65536 input values; forced
    here on a small input (option gelu_table_min = 0) and compared with the arithmetic kernel (option -1): the
    bytes are the same, for every input value (the second segment holds all 65536 bit patterns, NaNs included)
    and for random data, with and without a plain first segment, at a ragged row count."""
    from comfy_kitchen.backends import cuda as ck

    g = torch.Generator().manual_seed(6)
    rows = 300
    every = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(dt).reshape(64, 1024)   # each value once
    rnd = (2.0 * torch.randn(rows - 64, 1024, generator=g)).to(dt)
    act = torch.cat([every, rnd]).cuda()
    plain = torch.randn(rows, 384, generator=g).to(dt).cuda()
    gs = torch.tensor(4.0 / (6 * 448)).cuda()
    outs = {}
    try:
        for mode in (-1, 0):
            ck.set_option("gelu_table_min", mode)
            outs[mode] = (ck.quantize_nvfp4_gather([(plain, None), (act, "gelu_tanh")], gs),
                          ck.quantize_nvfp4_gather([(act, "gelu_tanh")], gs))
    finally:
        ck.set_option("gelu_table_min", 8 << 20)
    for (qa, sa), (qb, sb) in zip(outs[-1], outs[0]):
        assert torch.equal(qa, qb)
        assert torch.equal(sa.view(torch.uint8), sb.view(torch.uint8))


@pytest.mark.parametrize("ot", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_stochastic_rounding_exhaustive(ck, orc, ot):
    """All 65536 fp16 inputs x all 256 random bytes against the oracle (which the reference fixtures pin), and
    bf16 / fp32 / ragged inputs through the public API."""
    import comfy_kitchen as api

    h = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.float16)
    x = h.repeat(256)
    r = torch.arange(256, dtype=torch.uint8).repeat_interleave(65536)
    want = orc.stochastic_rounding_fp8(x, r, ot).view(torch.uint8)
    got = ck.stochastic_rounding_fp8(x.cuda(), r.cuda(), ot).view(torch.uint8).cpu()
    bad = (got != want).nonzero().flatten()
    assert bad.numel() == 0, (bad[:8].tolist(), got[bad[:8]].tolist(), want[bad[:8]].tolist())
    g = torch.Generator().manual_seed(9)
    for dtype, n in ((torch.bfloat16, 4099), (torch.float32, 12345), (torch.float16, 7)):
        v = (torch.randn(n, generator=g) * torch.exp2(torch.randint(-18, 17, (n,), generator=g).float())).to(dtype)
        rb = torch.randint(0, 256, (n,), generator=g, dtype=torch.uint8)
        want = orc.stochastic_rounding_fp8(v, rb, ot).view(torch.uint8)
        got = api.stochastic_rounding_fp8(v.cuda(), rb.cuda(), ot)
        assert got.dtype == ot and torch.equal(got.view(torch.uint8).cpu(), want)
