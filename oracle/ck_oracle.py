"""Python face of the CPU oracle (oracle/ck_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and
by the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  The shipped
package never imports this module.

Every function takes and returns CPU ``torch`` tensors and mirrors the keyword
signature of the reference function it restates, so a parity test reads like
the reference's own tests.  The arithmetic lives in the C file; this module only
allocates outputs and passes raw pointers.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libck_oracle.so")

DTYPE_TO_CODE = {
    torch.float32: 0,
    torch.float16: 1,
    torch.bfloat16: 2,
    torch.float8_e4m3fn: 5,
    torch.float8_e5m2: 6,
}


def build(force: bool = False) -> str:
    """Compile the C oracle with the Makefile beside it and return the library path."""
    src = os.path.join(_HERE, "ck_oracle.c")
    stale = not os.path.exists(_LIB_PATH) or (
        os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(_LIB_PATH)
    )
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _p(t: torch.Tensor | None):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _i64(*v):
    return (ctypes.c_int64 * len(v))(*v)


def _check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"oracle {what} failed with status {rc}")


def roundup(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def set_threads(n: int = 0) -> int:
    """Set (n > 0) and return the OpenMP thread count the oracle uses."""
    return int(lib().ck_oracle_set_threads(ctypes.c_int(n)))


def _scalar_f32(s) -> torch.Tensor:
    if not isinstance(s, torch.Tensor):
        s = torch.tensor(float(s))
    return s.detach().to(device="cpu", dtype=torch.float32).reshape(1).contiguous()


# --------------------------------------------------------------------- FP8


def quantize_per_tensor_fp8(x, scale, output_type=torch.float8_e4m3fn):
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=torch.uint8)
    s = _scalar_f32(scale)
    _check(
        lib().ck_oracle_quantize_fp8(
            _p(x), _p(s), _p(out), ctypes.c_int64(x.numel()), DTYPE_TO_CODE[x.dtype], DTYPE_TO_CODE[output_type]
        ),
        "quantize_fp8",
    )
    return out.view(output_type)


def dequantize_per_tensor_fp8(x, scale, output_type=torch.bfloat16):
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=output_type)
    s = _scalar_f32(scale)
    _check(
        lib().ck_oracle_dequantize_fp8(
            _p(x), _p(s), _p(out), ctypes.c_int64(x.numel()), DTYPE_TO_CODE[x.dtype], DTYPE_TO_CODE[output_type]
        ),
        "dequantize_fp8",
    )
    return out


# ------------------------------------------------------------------- NVFP4


def quantize_nvfp4(x, per_tensor_scale, epsilon: float = 0.0, pad_16x: bool = False, hi_first: bool = True):
    assert x.dim() == 2
    x = x.contiguous()
    orig_rows, orig_cols = x.shape
    rows, cols = (roundup(orig_rows, 16), roundup(orig_cols, 16)) if pad_16x else (orig_rows, orig_cols)
    assert cols % 16 == 0, "K dimension must be divisible by 16"
    q = torch.empty((rows, cols // 2), dtype=torch.uint8)
    sf = torch.empty((roundup(rows, 128), roundup(cols // 16, 4)), dtype=torch.uint8)
    g = _scalar_f32(per_tensor_scale)
    _check(
        lib().ck_oracle_quantize_nvfp4(
            _p(x), _p(g), _p(q), _p(sf),
            ctypes.c_int64(rows), ctypes.c_int64(cols), ctypes.c_int64(orig_rows), ctypes.c_int64(orig_cols),
            DTYPE_TO_CODE[x.dtype], int(bool(hi_first)),
        ),
        "quantize_nvfp4",
    )
    return q, sf.view(torch.float8_e4m3fn)


def dequantize_nvfp4(qx, per_tensor_scale, block_scales, output_type=torch.bfloat16, hi_first: bool = True):
    qx = qx.contiguous()
    rows, cols = qx.shape[0], qx.shape[1] * 2
    out = torch.empty((rows, cols), dtype=output_type)
    g = _scalar_f32(per_tensor_scale)
    sf = block_scales.contiguous().view(torch.uint8)
    _check(
        lib().ck_oracle_dequantize_nvfp4(
            _p(qx), _p(g), _p(sf), _p(out), ctypes.c_int64(rows), ctypes.c_int64(cols),
            DTYPE_TO_CODE[output_type], int(bool(hi_first)),
        ),
        "dequantize_nvfp4",
    )
    return out


# ------------------------------------------------------------------- MXFP8


def quantize_mxfp8(x, pad_32x: bool = False):
    assert x.dim() == 2
    x = x.contiguous()
    orig_rows, orig_cols = x.shape
    rows, cols = (roundup(orig_rows, 32), roundup(orig_cols, 32)) if pad_32x else (orig_rows, orig_cols)
    assert cols % 32 == 0, "K dimension must be divisible by 32"
    q = torch.empty((rows, cols), dtype=torch.uint8)
    sf = torch.empty((roundup(rows, 128), roundup(cols // 32, 4)), dtype=torch.uint8)
    _check(
        lib().ck_oracle_quantize_mxfp8(
            _p(x), _p(q), _p(sf),
            ctypes.c_int64(rows), ctypes.c_int64(cols), ctypes.c_int64(orig_rows), ctypes.c_int64(orig_cols),
            DTYPE_TO_CODE[x.dtype],
        ),
        "quantize_mxfp8",
    )
    return q.view(torch.float8_e4m3fn), sf.view(torch.float8_e8m0fnu)


def dequantize_mxfp8(qx, block_scales, output_type=torch.bfloat16):
    qx = qx.contiguous()
    rows, cols = qx.shape
    out = torch.empty((rows, cols), dtype=output_type)
    sf = block_scales.contiguous().view(torch.uint8)
    _check(
        lib().ck_oracle_dequantize_mxfp8(
            _p(qx), _p(sf), _p(out), ctypes.c_int64(rows), ctypes.c_int64(cols), DTYPE_TO_CODE[output_type]
        ),
        "dequantize_mxfp8",
    )
    return out


# -------------------------------------------------------------------- GEMM


def expand_nvfp4(q, block_scales, hi_first: bool = True) -> torch.Tensor:
    """codes x block scales as fp32, without the per-tensor scale (exact)."""
    q = q.contiguous()
    rows, cols = q.shape[0], q.shape[1] * 2
    out = torch.empty((rows, cols), dtype=torch.float32)
    sf = block_scales.contiguous().view(torch.uint8)
    _check(
        lib().ck_oracle_expand_nvfp4(_p(q), _p(sf), _p(out), ctypes.c_int64(rows), ctypes.c_int64(cols), int(bool(hi_first))),
        "expand_nvfp4",
    )
    return out


def expand_mxfp8(q, block_scales) -> torch.Tensor:
    q = q.contiguous()
    rows, cols = q.shape
    out = torch.empty((rows, cols), dtype=torch.float32)
    sf = block_scales.contiguous().view(torch.uint8)
    _check(
        lib().ck_oracle_expand_mxfp8(_p(q), _p(sf), _p(out), ctypes.c_int64(rows), ctypes.c_int64(cols)),
        "expand_mxfp8",
    )
    return out


def scaled_mm_nvfp4(a, b, tensor_scale_a, tensor_scale_b, block_scale_a, block_scale_b,
                    bias=None, out_dtype=torch.bfloat16, alpha=None) -> torch.Tensor:
    """y = alpha * (a4*sa) @ (b4*sb)^T + bias, fp32 accumulate, one cast at the end.

    The eager reference (backends/eager/quantization.py:224-248) forwards to
    torch's scaled_mm, which has no CPU kernel; the reference's own GEMM tests
    (tests/test_qdq.py:452-509) compare with dequantize -> F.linear, which is
    what this function evaluates in fp32.
    """
    if alpha is None:
        alpha = _scalar_f32(tensor_scale_a) * _scalar_f32(tensor_scale_b)
    alpha = _scalar_f32(alpha)
    y = expand_nvfp4(a, block_scale_a) @ expand_nvfp4(b, block_scale_b).t()
    y = y * alpha
    if bias is not None:
        y = y + bias.detach().float().cpu()
    return y.to(out_dtype)


def scaled_mm_mxfp8(a, b, block_scale_a, block_scale_b, bias=None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """y = (a8*2^ea) @ (b8*2^eb)^T + bias (backends/eager/quantization.py:369-404)."""
    y = expand_mxfp8(a.view(torch.uint8), block_scale_a) @ expand_mxfp8(b.view(torch.uint8), block_scale_b).t()
    if bias is not None:
        y = y + bias.detach().float().cpu()
    return y.to(out_dtype)


# -------------------------------------------------------------------- RoPE


def _rope(x, freqs_cis, split_half: bool):
    assert x.dim() == 4 and freqs_cis.dim() == 6
    out = torch.empty(x.shape, dtype=x.dtype)
    _check(
        lib().ck_oracle_rope(
            _p(x), _p(freqs_cis), _p(out),
            _i64(*x.shape), _i64(*freqs_cis.shape[:3]), _i64(*x.stride()), _i64(*freqs_cis.stride()),
            DTYPE_TO_CODE[x.dtype], DTYPE_TO_CODE[freqs_cis.dtype], int(split_half),
        ),
        "rope",
    )
    return out


def apply_rope1(x, freqs_cis):
    return _rope(x, freqs_cis, False)


def apply_rope(xq, xk, freqs_cis):
    return _rope(xq, freqs_cis, False), _rope(xk, freqs_cis, False)


def apply_rope_split_half1(x, freqs_cis):
    return _rope(x, freqs_cis, True)


def apply_rope_split_half(xq, xk, freqs_cis):
    return _rope(xq, freqs_cis, True), _rope(xk, freqs_cis, True)


def stochastic_rounding_fp8(x, rng, output_type=torch.float8_e4m3fn):
    """backends/eager/quantization.py:77-114: x.half() rounded to FP8 with one random byte per element."""
    assert output_type in (torch.float8_e4m3fn, torch.float8_e5m2)
    x = x.contiguous()
    rng = rng.contiguous()
    assert rng.dtype == torch.uint8 and rng.numel() == x.numel()
    out = torch.empty(x.shape, dtype=torch.uint8)
    _check(lib().ck_oracle_stochastic_rounding_fp8(_p(x), _p(rng), _p(out), ctypes.c_int64(x.numel()), DTYPE_TO_CODE[x.dtype],
                                                   int(output_type == torch.float8_e4m3fn)), "stochastic_rounding_fp8")
    return out.view(output_type)


# ------------------------------------------------------------------- AdaLN


def _modulation_rows(t: torch.Tensor, x: torch.Tensor, n: int, d: int):
    """(rows, group): row r of x reads modulation row r // group.

    Covers the broadcast shapes the hot path uses ([B,1,D] against [B,T,D], or the
    same shape as x); anything else is materialised (group 1).
    """
    if t.shape[-1] == d and t.numel() % d == 0:
        rows = t.numel() // d
        lead = tuple(t.shape[:-1])
        lead = (1,) * (x.dim() - 1 - len(lead)) + lead
        kept = [i for i, (a, b) in enumerate(zip(lead, x.shape[:-1])) if a == b and b != 1]
        bc = [i for i, (a, b) in enumerate(zip(lead, x.shape[:-1])) if a == 1 and b != 1]
        ok = all(a in (1, b) for a, b in zip(lead, x.shape[:-1]))
        if ok and rows > 0 and n % rows == 0 and (not kept or not bc or max(kept) < min(bc)):
            return t.reshape(rows, d).contiguous(), n // rows
    return t.expand_as(x).reshape(n, d).contiguous(), 1


def adaln(x, scale, shift, eps: float = 1e-6, single_rounding: bool = False, rms: bool = False):
    """Eager-ordered AdaLN (rounding after each op) or, with ``single_rounding``,
    the fp32 formulation with one final cast (what the CUDA kernels compute)."""
    d = x.shape[-1]
    n = x.numel() // d
    xf = x.reshape(n, d).contiguous()
    sc, sg = _modulation_rows(scale.to(x.dtype), x, n, d)
    sh, hg = _modulation_rows(shift.to(x.dtype), x, n, d)
    out = torch.empty_like(xf)
    code = DTYPE_TO_CODE[x.dtype]
    if single_rounding or rms:
        rc = lib().ck_oracle_adaln_f32(_p(xf), _p(sc), _p(sh), _p(out), ctypes.c_int64(n), ctypes.c_int64(d),
                                       ctypes.c_int64(sg), ctypes.c_int64(hg), ctypes.c_float(eps), code, int(rms))
    else:
        rc = lib().ck_oracle_adaln(_p(xf), _p(sc), _p(sh), _p(out), ctypes.c_int64(n), ctypes.c_int64(d),
                                   ctypes.c_int64(sg), ctypes.c_int64(hg), ctypes.c_float(eps), code)
    _check(rc, "adaln")
    return out.reshape(x.shape)


# ------------------------------------------------------------ scale layout


def to_blocked(m: torch.Tensor) -> torch.Tensor:
    rows, cols = m.shape
    src = m.contiguous().view(torch.uint8)
    dst = torch.empty((roundup(rows, 128), roundup(cols, 4)), dtype=torch.uint8)
    _check(lib().ck_oracle_to_blocked(_p(src), _p(dst), ctypes.c_int64(rows), ctypes.c_int64(cols)), "to_blocked")
    return dst


def from_blocked(blocked: torch.Tensor, num_rows: int, num_cols: int) -> torch.Tensor:
    src = blocked.contiguous().view(torch.uint8)
    dst = torch.empty((num_rows, num_cols), dtype=torch.uint8)
    _check(lib().ck_oracle_from_blocked(_p(src), _p(dst), ctypes.c_int64(num_rows), ctypes.c_int64(num_cols)), "from_blocked")
    return dst


def e2m1_codes(v: torch.Tensor) -> torch.Tensor:
    v = v.float().contiguous()
    out = torch.empty(v.shape, dtype=torch.uint8)
    _check(lib().ck_oracle_e2m1_codes(_p(v), _p(out), ctypes.c_int64(v.numel())), "e2m1")
    return out
