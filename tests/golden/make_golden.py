"""Generate the golden fixtures in this folder from the reference's eager backend.

Run where the reference checkout is available (it is a pure-Python import; only
its ``eager`` backend registers on a machine without a GPU):

    python tests/golden/make_golden.py --reference /path/to/comfy-kitchen

Every fixture stores the exact input bits and the reference's output bits, so the
tests that read them need neither the reference nor a particular RNG.  The
fixtures pin ``oracle/`` (CPU) and, through it, the CUDA kernels.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _inputs(shape, dtype, seed, kind):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    if kind == "outliers":
        mask = torch.rand(shape, generator=g) < 0.01
        x = torch.where(mask, 50.0 * torch.randn(shape, generator=g), x)
    elif kind == "zeros":
        x[:, : shape[1] // 2] = 0.0
        x[::3] = 0.0
    elif kind == "tiny":
        x = x * 1e-4
    elif kind == "wide":
        x = x * torch.exp2(torch.randint(-20, 12, shape, generator=g).float())
    return x.to(dtype)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference repository")
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    import comfy_kitchen  # noqa: F401  (registers the eager backend)
    from comfy_kitchen.backends.eager import quantization as rq
    from comfy_kitchen.backends.eager import rope as rr
    ra = sys.modules["comfy_kitchen.backends.eager.adaln"]  # the package re-exports a function of the same name

    torch.set_num_threads(1)
    dts = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}
    cases = []

    # ---------------- NVFP4 quantize / dequantize
    seed = 100
    for shape, pad in [((16, 16), False), ((32, 64), False), ((129, 128), False), ((33, 65), True),
                       ((257, 272), False), ((130, 144), True)]:
        for dn, dt in dts.items():
            for kind in ("normal", "outliers", "zeros", "tiny"):
                if shape[0] > 100 and (dn != "bf16" or kind not in ("normal", "outliers")):
                    continue
                seed += 1
                x = _inputs(shape, dt, seed, kind)
                amax = x.float().abs().max()
                for gname, gs in (("amax", amax / (6.0 * 448.0)), ("small", amax / (6.0 * 448.0) / 37.0)):
                    if gname == "small" and kind != "outliers":
                        continue
                    gs = gs.float().clamp_min(1e-30)
                    for hi in (True, False):
                        if not hi and (kind != "normal" or dn != "bf16"):
                            continue
                        q, sf = rq.quantize_nvfp4(x, gs, pad_16x=pad, hi_first=hi)
                        case = {"op": "quantize_nvfp4", "x": x, "scale": gs, "pad": pad, "hi_first": hi,
                                "q": q, "sf": sf.view(torch.uint8)}
                        for on, ot in dts.items():
                            if on == "bf16" or x.numel() <= 1100:
                                case["dq_" + on] = rq.dequantize_nvfp4(q, gs, sf, ot, hi_first=hi)
                        cases.append(case)

    # ---------------- MXFP8 quantize / dequantize
    for shape, pad in [((32, 32), False), ((64, 128), False), ((65, 96), True), ((128, 256), False),
                       ((257, 288), False)]:
        for dn, dt in dts.items():
            for kind in ("normal", "outliers", "zeros", "tiny", "wide"):
                if shape[0] > 100 and (dn != "bf16" or kind in ("zeros", "tiny")):
                    continue
                seed += 1
                x = _inputs(shape, dt, seed, kind)
                if dn == "f16":
                    x = torch.nan_to_num(x, posinf=60000.0, neginf=-60000.0)
                q, sf = rq.quantize_mxfp8(x, pad_32x=pad)
                case = {"op": "quantize_mxfp8", "x": x, "pad": pad, "q": q.view(torch.uint8),
                        "sf": sf.view(torch.uint8)}
                for on, ot in dts.items():
                    if on == "bf16" or x.numel() <= 1100:
                        case["dq_" + on] = rq.dequantize_mxfp8(q, sf, ot)
                cases.append(case)

    # ---------------- FP8 per-tensor
    for shape in [(7, 13), (24, 80)]:
        for dn, dt in dts.items():
            for kind in ("normal", "outliers"):
                for on, ot in (("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)):
                    seed += 1
                    x = _inputs(shape, dt, seed, kind)
                    lp_max = 448.0 if on == "e4m3" else 57344.0
                    for sname, sc in (("amax", x.float().abs().max() / lp_max), ("one", torch.tensor(1.0)),
                                      ("third", torch.tensor(0.3))):
                        sc = sc.float()
                        q = rq.quantize_per_tensor_fp8(x, sc, ot)
                        case = {"op": "quantize_fp8", "x": x, "scale": sc, "out": on, "q": q.view(torch.uint8)}
                        for o2n, o2t in dts.items():
                            if o2n == "bf16" or x.numel() <= 1100:
                                case["dq_" + o2n] = rq.dequantize_per_tensor_fp8(q, sc, o2t)
                        cases.append(case)

    # ---------------- RoPE
    g = torch.Generator().manual_seed(7)
    for xshape, fshape in [((2, 3, 17, 64), (2, 1, 17, 32, 2, 2)), ((1, 2, 9, 128), (1, 1, 9, 64, 2, 2)),
                           ((2, 7, 3, 32), (1, 7, 1, 16, 2, 2)), ((1, 2, 8, 16), (1, 1, 12, 8, 2, 2))]:
        for xn in ("bf16", "f16"):
            for fn in ("f32", "bf16", "f16"):
                xq = torch.randn(xshape, generator=g).to(dts[xn])
                xk = torch.randn(xshape, generator=g).to(dts[xn])
                fr = torch.randn(fshape, generator=g).to(dts[fn])
                oq, ok = rr.apply_rope(xq, xk, fr)
                case = {"op": "rope", "xq": xq, "xk": xk, "freqs": fr, "oq": oq, "ok": ok}
                if fshape[2] in (1, xshape[2]):  # only the interleaved form slices a longer table
                    case["sq"], case["sk"] = rr.apply_rope_split_half(xq, xk, fr)
                cases.append(case)

    # ---------------- AdaLN
    for xshape, mshape in [((2, 16, 64), (2, 1, 64)), ((2, 6, 768), (2, 1, 768)), ((1, 3, 3072), (1, 1, 3072)),
                           ((3, 5, 96), (3, 5, 96))]:
        for dn, dt in dts.items():
            x = torch.randn(xshape, generator=g).to(dt)
            sc = (0.1 * torch.randn(mshape, generator=g)).to(dt)
            sh = (0.1 * torch.randn(mshape, generator=g)).to(dt)
            y = ra.adaln(x, sc, sh, 1e-6)
            y32 = ra.adaln(x.float(), sc.float(), sh.float(), 1e-6)
            cases.append({"op": "adaln", "x": x, "scale": sc, "shift": sh, "eps": 1e-6, "y": y, "y_fp32": y32})

    # ---------------- scale layout and scalar conversions
    m = torch.arange(257 * 19, dtype=torch.int64).remainder(251).to(torch.uint8).reshape(257, 19)
    from comfy_kitchen import float_utils as fu
    cases.append({"op": "to_blocked", "m": m, "blocked": fu.to_blocked(m, flatten=False)})
    v = torch.cat([torch.linspace(-7, 7, 2801), torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.0,
                                                               0.2500001, 5.0000005])])
    cases.append({"op": "e2m1", "v": v, "codes": fu._f32_to_floatx_unpacked(v.clamp(-6, 6).float(), 2, 1)})

    out = os.path.join(HERE, "eager_golden.pt")
    torch.save({"reference_version": "0.2.18", "torch": str(torch.__version__), "cases": cases}, out)
    print(f"wrote {len(cases)} cases, {os.path.getsize(out) / 1e6:.2f} MB -> {out}")


if __name__ == "__main__":
    main()
