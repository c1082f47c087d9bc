"""Pin the CPU oracle against fixtures produced by the reference's eager backend.

The fixtures (tests/golden/eager_golden.pt, made by tests/golden/make_golden.py)
hold the reference's outputs bit for bit.  Integer and byte results must be
identical; RoPE and AdaLN are floating point and carry the tolerances of the
reference's own tests (tests/test_rope.py:73-96, tests/test_adaln.py:66-72).
"""
import torch

from conftest import cases_of
from oracle import ck_oracle as orc

DT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def _same_bits(a, b):
    return torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))


def test_nvfp4_quantize_bit_exact(golden):
    cases = cases_of(golden, "quantize_nvfp4")
    assert len(cases) > 40
    for c in cases:
        q, sf = orc.quantize_nvfp4(c["x"], c["scale"], pad_16x=c["pad"], hi_first=c["hi_first"])
        assert q.shape == c["q"].shape and sf.shape == c["sf"].shape
        assert torch.equal(sf.view(torch.uint8), c["sf"]), f"scales differ {tuple(c['x'].shape)} {c['x'].dtype}"
        assert torch.equal(q, c["q"]), f"codes differ {tuple(c['x'].shape)} {c['x'].dtype}"


def test_nvfp4_dequantize_bit_exact(golden):
    for c in cases_of(golden, "quantize_nvfp4"):
        for name, dt in DT.items():
            if "dq_" + name not in c:
                continue
            out = orc.dequantize_nvfp4(c["q"], c["scale"], c["sf"].view(torch.float8_e4m3fn), dt, hi_first=c["hi_first"])
            assert _same_bits(out, c["dq_" + name]), f"dequant {name} differs {tuple(c['x'].shape)}"


def test_mxfp8_quantize_bit_exact(golden):
    cases = cases_of(golden, "quantize_mxfp8")
    assert len(cases) > 30
    for c in cases:
        q, sf = orc.quantize_mxfp8(c["x"], pad_32x=c["pad"])
        assert torch.equal(sf.view(torch.uint8), c["sf"]), f"scales differ {tuple(c['x'].shape)} {c['x'].dtype}"
        assert torch.equal(q.view(torch.uint8), c["q"]), f"data differ {tuple(c['x'].shape)} {c['x'].dtype}"


def test_mxfp8_dequantize_bit_exact(golden):
    for c in cases_of(golden, "quantize_mxfp8"):
        for name, dt in DT.items():
            if "dq_" + name not in c:
                continue
            out = orc.dequantize_mxfp8(c["q"].view(torch.float8_e4m3fn), c["sf"].view(torch.float8_e8m0fnu), dt)
            assert _same_bits(out, c["dq_" + name])


def test_fp8_quantize_dequantize_bit_exact(golden):
    cases = cases_of(golden, "quantize_fp8")
    assert len(cases) > 30
    for c in cases:
        ot = torch.float8_e4m3fn if c["out"] == "e4m3" else torch.float8_e5m2
        q = orc.quantize_per_tensor_fp8(c["x"], c["scale"], ot)
        assert torch.equal(q.view(torch.uint8), c["q"]), f"{c['x'].dtype} {c['out']} scale {float(c['scale'])}"
        for name, dt in DT.items():
            if "dq_" + name not in c:
                continue
            out = orc.dequantize_per_tensor_fp8(c["q"].view(ot), c["scale"], dt)
            assert _same_bits(out, c["dq_" + name])


def test_scale_layout(golden):
    (c,) = cases_of(golden, "to_blocked")
    blocked = orc.to_blocked(c["m"])
    assert torch.equal(blocked, c["blocked"])
    assert torch.equal(orc.from_blocked(blocked, *c["m"].shape), c["m"])
    # spot values of the offset rule inside one 128x4 tile
    m = torch.zeros(128, 4, dtype=torch.uint8)
    for (r, col), off in {(1, 0): 16, (32, 0): 4, (33, 2): 22, (127, 3): 511}.items():
        m.zero_()
        m[r, col] = 1
        assert int(orc.to_blocked(m).flatten().argmax()) == off


def test_e2m1_rounding(golden):
    (c,) = cases_of(golden, "e2m1")
    assert torch.equal(orc.e2m1_codes(c["v"]), c["codes"])
    v = torch.tensor([0, 0.1, 0.25, 0.2500001, 0.5, 0.75, 1, 1.25, 1.5, 1.75, 2, 2.5, 3, 3.5, 4, 5, 5.0000005, 6,
                      -0.25, -0.75, -5, -6, -0.0])
    want = [0, 0, 0, 1, 1, 2, 2, 2, 3, 4, 4, 4, 5, 6, 6, 6, 7, 7, 8, 10, 14, 15, 8]
    assert orc.e2m1_codes(v).tolist() == want


def test_known_answers():
    # NVFP4: one row 0, .5, ... 7.5 with a per-tensor scale that makes the block scale 448
    x = (torch.arange(16).float() / 2).reshape(1, 16).bfloat16()
    g = torch.tensor(7.5 / (6 * 448))
    q, sf = orc.quantize_nvfp4(x, g)
    assert q.flatten().tolist() == [1, 34, 52, 69, 86, 102, 103, 119]
    assert int(sf.view(torch.uint8)[0, 0]) == 126
    q0, sf0 = orc.quantize_nvfp4(torch.zeros(16, 32).bfloat16(), g)
    assert int(q0.sum()) == 0 and int(sf0.view(torch.uint8).sum()) == 0
    # nibble order
    x = torch.zeros(1, 16).bfloat16()
    x[0, 0], x[0, 1] = 6.0, 3.0
    g = torch.tensor(6.0 / (6 * 448))
    assert int(orc.quantize_nvfp4(x, g, hi_first=True)[0][0, 0]) == 0x75
    assert int(orc.quantize_nvfp4(x, g, hi_first=False)[0][0, 0]) == 0x57
    # MXFP8: first element of one 32-block set
    for val, e, qv in [(448.0, 127, 448.0), (449.0, 127, 448.0), (1.75, 119, 448.0), (1e-30, 19, 320.0),
                       (3e38, 247, 224.0)]:
        x = torch.zeros(1, 32).bfloat16()
        x[0, 0] = val
        q, sf = orc.quantize_mxfp8(x)
        assert int(sf.view(torch.uint8)[0, 0]) == e, val
        assert float(q[0, 0].float()) == qv, val
    q, sf = orc.quantize_mxfp8(torch.zeros(1, 32).bfloat16())
    assert int(sf.view(torch.uint8)[0, 0]) == 0 and int(q.view(torch.uint8).sum()) == 0
    # FP8 per tensor, bf16 arithmetic
    x = torch.tensor([1.0039062, 3.140625, 447, 500]).bfloat16()
    assert orc.quantize_per_tensor_fp8(x, torch.tensor(0.3)).view(torch.uint8).tolist() == [69, 82, 126, 126]


def _mismatch_ratio(a, b, rtol, atol):
    a, b = a.float(), b.float()
    bad = (a - b).abs() > atol + rtol * b.abs()
    return bad.float().mean().item()


def test_rope_matches_reference(golden):
    cases = cases_of(golden, "rope")
    assert len(cases) >= 20
    for c in cases:
        fdt, xdt = c["freqs"].dtype, c["xq"].dtype
        # tolerances of the reference's RoPE tests: exact-ish for fp32 tables, a
        # tolerated fraction of 1e-3 misses for 16-bit tables
        ratio = 1e-5 if (fdt == torch.float32 and xdt == torch.float16) else (0.25 if fdt == torch.bfloat16 else 0.05)
        oq, ok = orc.apply_rope(c["xq"], c["xk"], c["freqs"])
        assert _mismatch_ratio(oq, c["oq"], 1e-3, 1e-3) <= ratio
        assert _mismatch_ratio(ok, c["ok"], 1e-3, 1e-3) <= ratio
        assert _same_bits(orc.apply_rope1(c["xk"], c["freqs"]), ok)
        if "sq" in c:
            sq, sk = orc.apply_rope_split_half(c["xq"], c["xk"], c["freqs"])
            assert _mismatch_ratio(sq, c["sq"], 1e-3, 1e-3) <= ratio
            assert _mismatch_ratio(sk, c["sk"], 1e-3, 1e-3) <= ratio


def test_rope_fp32_tables_bit_exact(golden):
    # With fp32 tables the only freedom is whether a*b+c is fused; the reference's
    # CPU path rounds the product, and so does the oracle.
    n = bad = 0
    for c in cases_of(golden, "rope"):
        if c["freqs"].dtype != torch.float32:
            continue
        oq, _ = orc.apply_rope(c["xq"], c["xk"], c["freqs"])
        n += oq.numel()
        bad += (oq.view(torch.int16) != c["oq"].view(torch.int16)).sum().item()
    assert n > 0 and bad / n < 1e-3


def test_adaln_matches_reference(golden):
    for c in cases_of(golden, "adaln"):
        dt = c["x"].dtype
        tol = 1e-2 if dt != torch.float32 else 1e-4
        y = orc.adaln(c["x"], c["scale"], c["shift"], c["eps"])
        torch.testing.assert_close(y.float(), c["y"].float(), rtol=tol, atol=tol)
        y1 = orc.adaln(c["x"], c["scale"], c["shift"], c["eps"], single_rounding=True)
        torch.testing.assert_close(y1.float(), c["y_fp32"].to(dt).float(), rtol=tol, atol=tol)


def test_stochastic_rounding_golden():
    """Every fp16 input against six random-byte choices, both formats, plus bf16 / fp32 inputs: byte-exact."""
    import os

    import torch
    from oracle import ck_oracle as orc

    d = torch.load(os.path.join(os.path.dirname(__file__), "golden", "stochastic_rounding_golden.pt"))
    h = d["fp16_bits"].view(torch.float16)
    for (fmt, src, rname), want in d["cases"].items():
        ot = torch.float8_e4m3fn if fmt == "e4m3" else torch.float8_e5m2
        if src == "fp16":
            got = orc.stochastic_rounding_fp8(h, d["rng"][rname], ot)
        else:
            got = orc.stochastic_rounding_fp8(d["extra"][src], d["extra_rng"], ot)
        bad = (got.view(torch.uint8) != want).nonzero().flatten()
        assert bad.numel() == 0, (fmt, src, rname, bad[:8].tolist())
