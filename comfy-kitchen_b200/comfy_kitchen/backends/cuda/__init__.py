"""The single compute backend: hand-written sm_100a kernels behind a C ABI.

Function names, keyword names, return types and error behaviour mirror the
reference's CUDA backend module (comfy_kitchen/backends/cuda/__init__.py:369-529,
1338-1498, 1681-1817) so the registry and the layout classes can call it
unchanged.  Differences, all additive: fp32 inputs to the block quantizers, fp32
bias in ``scaled_mm_*``, ``dequantize_mxfp8`` / ``scaled_mm_mxfp8`` on the device,
no zero-fill pass over the scale buffers (the kernels write the padding), and the
fused ``adaln_quantize_*`` / ``rmsnorm`` entry points.

Every output is allocated here with torch (caching allocator, CUDA-graph safe);
the native side only launches on the current stream.  Nothing synchronises.
"""
from __future__ import annotations

import ctypes

import torch

from comfy_kitchen import _native
from comfy_kitchen.backends._modulation import adaln_prep_modulation
from comfy_kitchen.float_utils import roundup

DTYPE_CODE_TO_DTYPE = {
    0: torch.float32,
    1: torch.float16,
    2: torch.bfloat16,
    5: torch.float8_e4m3fn,
    6: torch.float8_e5m2,
}
DTYPE_TO_CODE = {v: k for k, v in DTYPE_CODE_TO_DTYPE.items()}

_native.load()  # fail at import when the library is absent: there is no other path


def _ptr(t: torch.Tensor | None):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _code(dtype: torch.dtype, what: str) -> int:
    try:
        return DTYPE_TO_CODE[dtype]
    except KeyError:
        raise TypeError(f"{what}: unsupported dtype {dtype}") from None


def _plain(t):
    return t.data if isinstance(t, torch.nn.Parameter) else t


# ------------------------------------------------------------------ FP8 per tensor


def quantize_per_tensor_fp8(
    x: torch.Tensor, scale: torch.Tensor, output_type: torch.dtype = torch.float8_e4m3fn
) -> torch.Tensor:
    if output_type not in (torch.float8_e4m3fn, torch.float8_e5m2):
        raise ValueError(
            f"Unsupported output_type: {output_type}. Expected torch.float8_e4m3fn or torch.float8_e5m2"
        )
    x = _plain(x)
    if not x.is_contiguous():
        x = x.contiguous()
    scale = _scalar_on(scale, x.device)
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    _native.call(
        "launch_quantize_fp8_kernel", _ptr(x), _ptr(out), _ptr(scale), x.numel(),
        _code(x.dtype, "quantize_per_tensor_fp8"), DTYPE_TO_CODE[output_type], _stream(x.device),
    )
    return out.view(output_type)


def dequantize_per_tensor_fp8(
    x: torch.Tensor, scale: torch.Tensor, output_type: torch.dtype = torch.bfloat16
) -> torch.Tensor:
    assert scale.numel() == 1, "Scale must be a scalar tensor"
    x = _plain(x)
    if not x.is_contiguous():
        x = x.contiguous()
    scale = _scalar_on(scale, x.device)
    out = torch.empty(x.shape, dtype=output_type, device=x.device)
    _native.call(
        "launch_dequantize_fp8_kernel", _ptr(x), _ptr(out), _ptr(scale), x.numel(),
        _code(x.dtype, "dequantize_per_tensor_fp8"), _code(output_type, "dequantize_per_tensor_fp8"),
        _stream(x.device),
    )
    return out


def stochastic_rounding_fp8(
    x: torch.Tensor, rng: torch.Tensor, output_type: torch.dtype = torch.float8_e4m3fn
) -> torch.Tensor:
    """x.half() rounded to FP8 up or down according to one random byte per element (same bytes as the
    reference's eager function)."""
    if output_type not in (torch.float8_e4m3fn, torch.float8_e5m2):
        raise ValueError(f"Unsupported output_type: {output_type}. Expected torch.float8_e4m3fn or torch.float8_e5m2")
    x = _plain(x)
    assert rng.dtype == torch.uint8 and rng.shape == x.shape, "rng must be uint8 with x's shape"
    xc = x if x.is_contiguous() else x.contiguous()
    rc = rng if rng.is_contiguous() else rng.contiguous()
    out = torch.empty(x.shape, device=x.device, dtype=torch.uint8)
    _native.call("launch_stochastic_rounding_fp8_kernel", _ptr(xc), _ptr(rc), _ptr(out), xc.numel(),
                 _code(x.dtype, "stochastic_rounding_fp8"), DTYPE_TO_CODE[output_type], _stream(x.device))
    return out.view(output_type)


def _scalar_on(s, device) -> torch.Tensor:
    """fp32 one-element device tensor without a host round trip when it already is one."""
    s = _plain(s)
    if not isinstance(s, torch.Tensor):
        s = torch.tensor(float(s), dtype=torch.float32, device=device)
    if s.dtype != torch.float32 or s.device != device:
        s = s.to(device=device, dtype=torch.float32)
    return s.reshape(1) if s.dim() == 0 else s.contiguous()


def _bias_for(bias: torch.Tensor, n: int) -> torch.Tensor:
    """Bias vector for an output of n columns; a weight padded to the block multiple gets zero bias
    on its padding columns (they are cropped by the layout handlers afterwards)."""
    bias = bias.contiguous()
    if bias.numel() == n:
        return bias
    if bias.dim() != 1 or bias.numel() > n:
        raise RuntimeError(f"bias has {bias.numel()} elements, output has {n} columns")
    return torch.nn.functional.pad(bias, (0, n - bias.numel()))


# ------------------------------------------------------------------ NVFP4


def quantize_nvfp4(
    x: torch.Tensor,
    per_tensor_scale: torch.Tensor,
    epsilon: float = 0.0,
    pad_16x: bool = False,
    hi_first: bool = True,
) -> tuple[torch.Tensor, torch.Tensor]:
    x = _plain(x)
    assert x.dim() == 2, "Input must be 2D"
    assert x.is_contiguous(), "Input tensor must be contiguous"
    orig_rows, orig_cols = x.shape
    if pad_16x:
        num_rows, num_cols = roundup(orig_rows, 16), roundup(orig_cols, 16)
    else:
        num_rows, num_cols = orig_rows, orig_cols
        assert num_cols % 16 == 0, f"num_cols must be divisible by 16, got {num_cols}"
    qx = torch.empty((num_rows, num_cols // 2), device=x.device, dtype=torch.uint8)
    # the kernel writes every byte of the tiled scale buffer, padding included
    sx = torch.empty((roundup(num_rows, 128), roundup(num_cols // 16, 4)), device=x.device, dtype=torch.uint8)
    g = _scalar_on(per_tensor_scale, x.device)
    _native.call(
        "launch_quantize_nvfp4_kernel", _ptr(x), _ptr(g), _ptr(qx), _ptr(sx), num_rows, num_cols, orig_rows,
        orig_cols, float(epsilon), _code(x.dtype, "quantize_nvfp4"), bool(hi_first), _stream(x.device),
    )
    return qx, sx.view(torch.float8_e4m3fn)


def _segment(t: torch.Tensor, what: str):
    """(tensor, cols, group, group_stride, row_stride, rows) of one gather-quantizer segment."""
    if t.dim() == 2:      # [rows, cols], unit column stride, any row pitch
        assert t.stride(1) == 1, f"{what}: 2-D segments need unit column stride"
        return t, t.shape[1], t.shape[1], 0, t.stride(0), t.shape[0]
    if t.dim() == 3:      # [groups, rows, d] read as [rows, groups * d]  (attention's [heads, tokens, head_dim])
        assert t.stride(2) == 1, f"{what}: 3-D segments need unit stride in the last dim"
        return t, t.shape[0] * t.shape[2], t.shape[2], t.stride(0), t.stride(1), t.shape[1]
    raise ValueError(f"{what}: segments are 2-D [rows, cols] or 3-D [groups, rows, d]")


def quantize_nvfp4_gather(
    segments, per_tensor_scale: torch.Tensor, hi_first: bool = True
) -> tuple[torch.Tensor, torch.Tensor]:
    """quantize_nvfp4 of the column concatenation of one or two segments, without materialising it.

    segments: [(tensor, activation), ...] with activation None or "gelu_tanh"; a tensor is 2-D [rows, cols] with
    unit column stride (any row pitch: a column slice is fine) or 3-D [groups, rows, d], read as [rows, groups*d].
    Widths and strides must be multiples of 16 elements.  With no activation the result equals
    quantize_nvfp4(torch.cat(...)) byte for byte.
    """
    assert 1 <= len(segments) <= 2, "one or two segments"
    segs = []
    for t, act in segments:
        assert act in (None, "gelu_tanh"), f"unknown activation {act!r}"
        segs.append((*_segment(t, "quantize_nvfp4_gather"), 0 if act is None else 1))
    rows = segs[0][5]
    assert all(sg[5] == rows for sg in segs), "segments must have the same number of rows"
    dtype, device = segs[0][0].dtype, segs[0][0].device
    assert all(sg[0].dtype == dtype for sg in segs)
    cols = sum(sg[1] for sg in segs)
    qx = torch.empty((rows, cols // 2), device=device, dtype=torch.uint8)
    sx = torch.empty((roundup(rows, 128), roundup(cols // 16, 4)), device=device, dtype=torch.uint8)
    g = _scalar_on(per_tensor_scale, device)
    flat = []
    for i in range(2):
        if i < len(segs):
            t, c, grp, gs, rs, _, act = segs[i]
            flat += [_ptr(t), c, grp, gs, rs, act]
        else:
            flat += [None, 0, 16, 0, 16, 0]
    _native.call("launch_quantize_nvfp4_gather_kernel", *flat, _ptr(g), _ptr(qx), _ptr(sx), rows,
                 _code(dtype, "quantize_nvfp4_gather"), bool(hi_first), _stream(device))
    return qx, sx.view(torch.float8_e4m3fn)


def dequantize_nvfp4(
    qx: torch.Tensor,
    per_tensor_scale: torch.Tensor,
    block_scales: torch.Tensor,
    output_type: torch.dtype = torch.bfloat16,
    hi_first: bool = True,
) -> torch.Tensor:
    qx = _plain(qx)
    assert qx.is_contiguous(), "Input tensor must be contiguous"
    num_rows, packed = qx.shape
    num_cols = packed * 2
    out = torch.empty((num_rows, num_cols), device=qx.device, dtype=output_type)
    g = _scalar_on(per_tensor_scale, qx.device)
    sf = _plain(block_scales).contiguous().view(torch.uint8)
    _native.call(
        "launch_dequantize_nvfp4_kernel", _ptr(qx), _ptr(g), _ptr(sf), _ptr(out), num_rows, num_cols,
        _code(output_type, "dequantize_nvfp4"), bool(hi_first), _stream(qx.device),
    )
    return out


def scaled_mm_nvfp4(
    a: torch.Tensor,
    b: torch.Tensor,
    tensor_scale_a: torch.Tensor,
    tensor_scale_b: torch.Tensor,
    block_scale_a: torch.Tensor,
    block_scale_b: torch.Tensor,
    bias: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    alpha: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    gate: torch.Tensor | None = None,
    scatter=None,
) -> torch.Tensor:
    """``out`` (not in the reference's signature): a contiguous [M, N] tensor of ``out_dtype`` to write into,
    e.g. a row range of a larger buffer.  ``residual`` [M, N] and ``gate`` [N] (both of ``out_dtype``, bf16 or
    fp16; also additions): the kernel's epilogue returns ``residual + gate * y`` instead of ``y`` (bytes equal to
    the GEMM followed by ``torch.addcmul``); ``out`` may be ``residual`` itself.  ``scatter`` = (dests, bounds, world,
    row_offset) with ctypes arrays of peer-mapped destination pointers and row bounds (a tensor-parallel group's
    reduce-scatter fused into the epilogue, see ``launch_scaled_mm_nvfp4_scatter_kernel``): nothing is returned."""
    a, b = _plain(a), _plain(b)
    block_scale_a, block_scale_b = _plain(block_scale_a), _plain(block_scale_b)
    if alpha is None:
        alpha = _plain(tensor_scale_a) * _plain(tensor_scale_b)  # device op, no sync
    alpha = _scalar_on(alpha, a.device)
    assert alpha.numel() == 1, "alpha must be a scalar"
    m, k_a = a.shape
    n, k_b = b.shape
    assert k_a == k_b, "Matrix dimensions do not match"
    k = 2 * k_a
    assert n % 8 == 0, "B tensor must have 8 alignment in N dimension"
    assert block_scale_a.dtype == block_scale_b.dtype, "A and B scale dtype must match"
    if block_scale_a.dtype == torch.float8_e8m0fnu:
        raise ValueError("MXFP4 is not supported")
    if block_scale_a.dtype != torch.float8_e4m3fn:
        raise ValueError(f"Unsupported scale dtype: {block_scale_a.dtype}")
    sk = roundup(k // 16, 4)
    assert tuple(block_scale_a.shape) == (roundup(m, 128), sk), "Invalid A scale shape"
    assert tuple(block_scale_b.shape) == (roundup(n, 128), sk), "Invalid B scale shape"
    if out_dtype is None:
        out_dtype = torch.bfloat16
    bias_code = 0
    if bias is not None and bias.numel() > 0:
        bias = _bias_for(_plain(bias), n)
        assert bias.dtype in (torch.float16, torch.bfloat16, torch.float32), "bias must be fp16, bf16 or fp32"
        bias_code = DTYPE_TO_CODE[bias.dtype]
    else:
        bias = None
    if scatter is not None:
        dests, bounds, world, row_offset = scatter
        assert out is None and residual is None and out_dtype in (torch.bfloat16, torch.float16)
        _native.call(
            "launch_scaled_mm_nvfp4_scatter_kernel", _ptr(a.contiguous()), _ptr(block_scale_a.contiguous().view(torch.uint8)),
            _ptr(b.contiguous()), _ptr(block_scale_b.contiguous().view(torch.uint8)), dests, bounds, int(world), int(row_offset),
            _ptr(bias), bias_code, m, n, k, _ptr(alpha), _code(out_dtype, "scaled_mm_nvfp4"), _stream(a.device),
        )
        return None
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=a.device)
    else:
        assert out.shape == (m, n) and out.dtype == out_dtype and out.is_contiguous() and out.device == a.device
    if residual is not None:
        assert gate is not None, "residual needs a gate"
        gate = gate.reshape(-1)
        assert out_dtype in (torch.bfloat16, torch.float16), "the fused residual update needs a 16-bit output"
        assert residual.shape == (m, n) and residual.dtype == out_dtype and residual.is_contiguous()
        assert gate.numel() == n and gate.dtype == out_dtype and gate.is_contiguous()
        _native.call(
            "launch_scaled_mm_nvfp4_residual_kernel", _ptr(a.contiguous()), _ptr(block_scale_a.contiguous().view(torch.uint8)),
            _ptr(b.contiguous()), _ptr(block_scale_b.contiguous().view(torch.uint8)), _ptr(out), _ptr(bias), bias_code,
            _ptr(residual), _ptr(gate), m, n, k, _ptr(alpha), _code(out_dtype, "scaled_mm_nvfp4"), _stream(a.device),
        )
        return out
    _native.call(
        "launch_scaled_mm_nvfp4_kernel", _ptr(a.contiguous()), _ptr(block_scale_a.contiguous().view(torch.uint8)),
        _ptr(b.contiguous()), _ptr(block_scale_b.contiguous().view(torch.uint8)), _ptr(out), _ptr(bias), bias_code,
        m, n, k, _ptr(alpha), _code(out_dtype, "scaled_mm_nvfp4"), _stream(a.device),
    )
    return out


launch_residual_supported = True   # scaled_mm_nvfp4 accepts residual= / gate= (see its docstring)


# ------------------------------------------------------------------ MXFP8


def quantize_mxfp8(x: torch.Tensor, pad_32x: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    x = _plain(x)
    assert x.dim() == 2, "Input must be 2D"
    assert x.is_contiguous(), "Input tensor must be contiguous"
    orig_rows, orig_cols = x.shape
    if pad_32x:
        num_rows, num_cols = roundup(orig_rows, 32), roundup(orig_cols, 32)
    else:
        num_rows, num_cols = orig_rows, orig_cols
        assert num_cols % 32 == 0, f"num_cols must be divisible by 32, got {num_cols}"
    qx = torch.empty((num_rows, num_cols), device=x.device, dtype=torch.uint8)
    sx = torch.empty((roundup(num_rows, 128), roundup(num_cols // 32, 4)), device=x.device, dtype=torch.uint8)
    _native.call(
        "launch_quantize_mxfp8_kernel", _ptr(x), _ptr(qx), _ptr(sx), num_rows, num_cols, orig_rows, orig_cols,
        _code(x.dtype, "quantize_mxfp8"), _stream(x.device),
    )
    return qx.view(torch.float8_e4m3fn), sx.view(torch.float8_e8m0fnu)


def dequantize_mxfp8(
    qx: torch.Tensor, block_scales: torch.Tensor, output_type: torch.dtype = torch.bfloat16
) -> torch.Tensor:
    qx = _plain(qx)
    assert qx.is_contiguous(), "Input tensor must be contiguous"
    rows, cols = qx.shape
    out = torch.empty((rows, cols), device=qx.device, dtype=output_type)
    sf = _plain(block_scales).contiguous().view(torch.uint8)
    _native.call(
        "launch_dequantize_mxfp8_kernel", _ptr(qx), _ptr(sf), _ptr(out), rows, cols,
        _code(output_type, "dequantize_mxfp8"), _stream(qx.device),
    )
    return out


def scaled_mm_mxfp8(
    a: torch.Tensor,
    b: torch.Tensor,
    block_scale_a: torch.Tensor,
    block_scale_b: torch.Tensor,
    bias: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
) -> torch.Tensor:
    a, b = _plain(a), _plain(b)
    block_scale_a, block_scale_b = _plain(block_scale_a), _plain(block_scale_b)
    m, k = a.shape
    n, k_b = b.shape
    assert k == k_b, "Matrix dimensions do not match"
    assert n % 8 == 0, "B tensor must have 8 alignment in N dimension"
    sk = roundup(k // 32, 4)
    assert tuple(block_scale_a.shape) == (roundup(m, 128), sk), "Invalid A scale shape"
    assert tuple(block_scale_b.shape) == (roundup(n, 128), sk), "Invalid B scale shape"
    if out_dtype is None:
        out_dtype = torch.bfloat16
    bias_code = 0
    if bias is not None and bias.numel() > 0:
        bias = _bias_for(_plain(bias), n)
        bias_code = _code(bias.dtype, "scaled_mm_mxfp8")
    else:
        bias = None
    out = torch.empty(m, n, dtype=out_dtype, device=a.device)
    _native.call(
        "launch_scaled_mm_mxfp8_kernel", _ptr(a.contiguous()), _ptr(block_scale_a.contiguous().view(torch.uint8)),
        _ptr(b.contiguous()), _ptr(block_scale_b.contiguous().view(torch.uint8)), _ptr(out), _ptr(bias), bias_code,
        m, n, k, _code(out_dtype, "scaled_mm_mxfp8"), _stream(a.device),
    )
    return out


# ------------------------------------------------------------------ RoPE


def _rope(xq, xk, freqs_cis, split_half: bool):
    if xq.dim() != 4 or freqs_cis.dim() != 6:
        raise ValueError("apply_rope expects x [B, H, N, D] (or [B, N, H, D]) and freqs_cis [b, h, n, D/2, 2, 2]")
    xq = xq if xq.is_contiguous() else xq.contiguous()
    if xk is not None:
        xk = xk if xk.is_contiguous() else xk.contiguous()
    if not freqs_cis.is_contiguous():
        freqs_cis = freqs_cis.contiguous()
    oq = torch.empty_like(xq)
    ok = torch.empty_like(xk) if xk is not None else None
    sx, sf = xq.stride(), freqs_cis.stride()
    _native.call(
        "launch_apply_rope_kernel", _ptr(xq), _ptr(xk), _ptr(freqs_cis), _ptr(oq), _ptr(ok),
        *xq.shape, *freqs_cis.shape[:3], *sx, *sf,
        _code(xq.dtype, "apply_rope"), _code(freqs_cis.dtype, "apply_rope"), bool(split_half), _stream(xq.device),
    )
    return oq, ok


def apply_rope1(x: torch.Tensor, freqs_cis: torch.Tensor) -> torch.Tensor:
    return _rope(x, None, freqs_cis, False)[0]


def apply_rope(xq: torch.Tensor, xk: torch.Tensor, freqs_cis: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    if xq.shape != xk.shape:
        return apply_rope1(xq, freqs_cis), apply_rope1(xk, freqs_cis)
    return _rope(xq, xk, freqs_cis, False)


def apply_rope_split_half1(x: torch.Tensor, freqs_cis: torch.Tensor) -> torch.Tensor:
    return _rope(x, None, freqs_cis, True)[0]


def apply_rope_split_half(
    xq: torch.Tensor, xk: torch.Tensor, freqs_cis: torch.Tensor
) -> tuple[torch.Tensor, torch.Tensor]:
    if xq.shape != xk.shape:
        return apply_rope_split_half1(xq, freqs_cis), apply_rope_split_half1(xk, freqs_cis)
    return _rope(xq, xk, freqs_cis, True)


def qk_norm_rope(
    qkv: torch.Tensor,
    q_weight: torch.Tensor,
    k_weight: torch.Tensor,
    freqs_cis: torch.Tensor,
    heads: int,
    q_out: torch.Tensor | None = None,
    k_out: torch.Tensor | None = None,
    v_out: torch.Tensor | None = None,
    token_offset: int = 0,
    eps: float = 1e-6,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per-head RMSNorm of q and k, RoPE of both and the relayout of q, k, v for attention in one pass.

    qkv: [tokens, >= 3*heads*128], unit column stride (a column slice of a wider matrix is fine), columns
    [q heads | k heads | v heads].  freqs_cis: fp32 [1, 1, total_tokens, 64, 2, 2].  Outputs (allocated when
    not given): [1, heads, total_tokens, 128]; rows token_offset .. token_offset + tokens - 1 are written, so
    two calls can fill the text and the image part of one joint sequence.
    """
    assert qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= 3 * heads * 128, "qkv must be [tokens, 3*heads*128]"
    assert freqs_cis.dtype == torch.float32 and freqs_cis.is_contiguous() and freqs_cis.shape[-3:] == (64, 2, 2)
    assert freqs_cis.dim() == 6 and freqs_cis.shape[0] == freqs_cis.shape[1] == 1, "freqs_cis must be [1, 1, N, 64, 2, 2]"
    tokens, total = qkv.shape[0], freqs_cis.shape[2]
    outs = []
    for o in (q_out, k_out, v_out):
        if o is None:
            o = torch.empty((1, heads, total, 128), device=qkv.device, dtype=qkv.dtype)
        assert o.shape == (1, heads, total, 128) and o.is_contiguous() and o.dtype == qkv.dtype
        outs.append(o)
    qw = q_weight.to(qkv.dtype).contiguous()
    kw = k_weight.to(qkv.dtype).contiguous()
    _native.call(
        "launch_qk_norm_rope_kernel", _ptr(qkv), qkv.stride(0), _ptr(qw), _ptr(kw), _ptr(freqs_cis), _ptr(outs[0]),
        _ptr(outs[1]), _ptr(outs[2]), tokens, heads, int(token_offset), total, float(eps), _code(qkv.dtype, "qk_norm_rope"),
        _stream(qkv.device),
    )
    return outs[0], outs[1], outs[2]


# ------------------------------------------------------------------ AdaLN / RMSNorm


def _norm_inputs(x, scale, shift):
    d = x.shape[-1]
    n = x.numel() // d
    xf = x.reshape(n, d)
    if not xf.is_contiguous():
        xf = xf.contiguous()
    sc, sg = adaln_prep_modulation(scale.to(x.dtype), x, n, d)
    sh, hg = adaln_prep_modulation(shift.to(x.dtype), x, n, d)
    return xf, sc, sg, sh, hg, n, d


def adaln(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf, sc, sg, sh, hg, n, d = _norm_inputs(x, scale, shift)
    out = torch.empty_like(xf)
    _native.call(
        "launch_adaln_kernel", _ptr(xf), _ptr(sc), _ptr(sh), _ptr(out), n, d, sg, hg, float(eps),
        _code(x.dtype, "adaln"), _stream(x.device),
    )
    return out.reshape(x.shape)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor | None = None, eps: float = 1e-6) -> torch.Tensor:
    d = x.shape[-1]
    n = x.numel() // d
    xf = x.reshape(n, d)
    if not xf.is_contiguous():
        xf = xf.contiguous()
    w = None if weight is None else weight.to(x.dtype).contiguous()
    out = torch.empty_like(xf)
    _native.call(
        "launch_rmsnorm_kernel", _ptr(xf), _ptr(w), _ptr(out), n, d, float(eps), _code(x.dtype, "rmsnorm"),
        _stream(x.device),
    )
    return out.reshape(x.shape)


def adaln_quantize_nvfp4(
    x: torch.Tensor,
    scale: torch.Tensor,
    shift: torch.Tensor,
    per_tensor_scale: torch.Tensor,
    eps: float = 1e-6,
    hi_first: bool = True,
) -> tuple[torch.Tensor, torch.Tensor]:
    """quantize_nvfp4(adaln(x, scale, shift, eps), per_tensor_scale) in one pass over x."""
    xf, sc, sg, sh, hg, n, d = _norm_inputs(x, scale, shift)
    assert d % 16 == 0, f"last dim must be divisible by 16, got {d}"
    qx = torch.empty((n, d // 2), device=x.device, dtype=torch.uint8)
    sx = torch.empty((roundup(n, 128), roundup(d // 16, 4)), device=x.device, dtype=torch.uint8)
    g = _scalar_on(per_tensor_scale, x.device)
    _native.call(
        "launch_adaln_quantize_nvfp4_kernel", _ptr(xf), _ptr(sc), _ptr(sh), _ptr(g), _ptr(qx), _ptr(sx), n, d, sg, hg,
        float(eps), _code(x.dtype, "adaln_quantize_nvfp4"), bool(hi_first), 0, _stream(x.device),
    )
    return qx, sx.view(torch.float8_e4m3fn)


def adaln_quantize_nvfp4_rows(
    x: torch.Tensor,
    scale: torch.Tensor,
    shift: torch.Tensor,
    per_tensor_scale: torch.Tensor,
    qx: torch.Tensor,
    sx: torch.Tensor,
    row_begin: int,
    row_end: int,
    eps: float = 1e-6,
    hi_first: bool = True,
) -> None:
    """adaln_quantize_nvfp4 for rows [row_begin, row_end) of x only, written into the caller's whole-tensor buffers
    ``qx`` [N, D/2] uint8 and ``sx`` [roundup(N, 128), roundup(D/16, 4)] (the bytes of other rows are left alone).
    For sequence-parallel callers: each rank quantizes its rows of a shared activation."""
    xf, sc, sg, sh, hg, n, d = _norm_inputs(x, scale, shift)
    assert d % 16 == 0, f"last dim must be divisible by 16, got {d}"
    assert qx.shape == (n, d // 2) and qx.dtype == torch.uint8 and qx.is_contiguous()
    assert tuple(sx.shape) == (roundup(n, 128), roundup(d // 16, 4)) and sx.element_size() == 1 and sx.is_contiguous()
    g = _scalar_on(per_tensor_scale, x.device)
    _native.call(
        "launch_adaln_quantize_nvfp4_rows_kernel", _ptr(xf), _ptr(sc), _ptr(sh), _ptr(g), _ptr(qx), _ptr(sx), n, d, sg, hg,
        float(eps), _code(x.dtype, "adaln_quantize_nvfp4"), bool(hi_first), 0, int(row_begin), int(row_end), _stream(x.device),
    )


def adaln_quantize_mxfp8(
    x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float = 1e-6
) -> tuple[torch.Tensor, torch.Tensor]:
    """quantize_mxfp8(adaln(x, scale, shift, eps)) in one pass over x."""
    xf, sc, sg, sh, hg, n, d = _norm_inputs(x, scale, shift)
    assert d % 32 == 0, f"last dim must be divisible by 32, got {d}"
    qx = torch.empty((n, d), device=x.device, dtype=torch.uint8)
    sx = torch.empty((roundup(n, 128), roundup(d // 32, 4)), device=x.device, dtype=torch.uint8)
    _native.call(
        "launch_adaln_quantize_mxfp8_kernel", _ptr(xf), _ptr(sc), _ptr(sh), _ptr(qx), _ptr(sx), n, d, sg, hg,
        float(eps), _code(x.dtype, "adaln_quantize_mxfp8"), 0, _stream(x.device),
    )
    return qx.view(torch.float8_e4m3fn), sx.view(torch.float8_e8m0fnu)


def rmsnorm_quantize_nvfp4(
    x: torch.Tensor, weight: torch.Tensor | None, per_tensor_scale: torch.Tensor, eps: float = 1e-6,
    hi_first: bool = True,
) -> tuple[torch.Tensor, torch.Tensor]:
    """quantize_nvfp4(rmsnorm(x, weight, eps), per_tensor_scale) in one pass over x."""
    d = x.shape[-1]
    n = x.numel() // d
    assert d % 16 == 0
    xf = x.reshape(n, d)
    if not xf.is_contiguous():
        xf = xf.contiguous()
    w = None if weight is None else weight.to(x.dtype).contiguous()
    qx = torch.empty((n, d // 2), device=x.device, dtype=torch.uint8)
    sx = torch.empty((roundup(n, 128), roundup(d // 16, 4)), device=x.device, dtype=torch.uint8)
    g = _scalar_on(per_tensor_scale, x.device)
    _native.call(
        "launch_adaln_quantize_nvfp4_kernel", _ptr(xf), _ptr(w), _ptr(None), _ptr(g), _ptr(qx), _ptr(sx), n, d, n, n,
        float(eps), _code(x.dtype, "rmsnorm_quantize_nvfp4"), bool(hi_first), 1, _stream(x.device),
    )
    return qx, sx.view(torch.float8_e4m3fn)


def build_constraints() -> dict:
    """What this backend accepts, per function (checked by the registry before dispatch)."""
    from comfy_kitchen.constraints import DivisibleBy, ExactDims, FunctionConstraints, ParamConstraint

    dev = frozenset({"cuda"})
    floats = frozenset({torch.float32, torch.float16, torch.bfloat16})
    fp8 = frozenset({torch.float8_e4m3fn, torch.float8_e5m2})
    sm100 = (10, 0)

    def fc(**params):
        return FunctionConstraints(params=params, default_devices=dev, min_compute_capability=sm100)

    two_d = (ExactDims(2),)
    rope = fc(x=ParamConstraint(dtypes=floats, shape_rules=(ExactDims(4),)),
              freqs_cis=ParamConstraint(dtypes=floats, shape_rules=(ExactDims(6),)))
    rope2 = fc(xq=ParamConstraint(dtypes=floats, shape_rules=(ExactDims(4),)),
               xk=ParamConstraint(dtypes=floats, shape_rules=(ExactDims(4),)),
               freqs_cis=ParamConstraint(dtypes=floats, shape_rules=(ExactDims(6),)))
    norm = dict(x=ParamConstraint(dtypes=floats), scale=ParamConstraint(dtypes=floats), shift=ParamConstraint(dtypes=floats))
    return {
        "quantize_per_tensor_fp8": fc(x=ParamConstraint(dtypes=floats), scale=ParamConstraint(dtypes=frozenset({torch.float32})),
                                      output_type=ParamConstraint(dtypes=fp8)),
        "dequantize_per_tensor_fp8": fc(x=ParamConstraint(dtypes=fp8), output_type=ParamConstraint(dtypes=floats)),
        "quantize_nvfp4": fc(x=ParamConstraint(dtypes=floats, shape_rules=two_d),
                             per_tensor_scale=ParamConstraint(dtypes=frozenset({torch.float32}))),
        "dequantize_nvfp4": fc(qx=ParamConstraint(dtypes=frozenset({torch.uint8}), shape_rules=two_d + (DivisibleBy(1, 8),)),
                               per_tensor_scale=ParamConstraint(dtypes=frozenset({torch.float32})),
                               block_scales=ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn})),
                               output_type=ParamConstraint(dtypes=floats)),
        "scaled_mm_nvfp4": fc(a=ParamConstraint(dtypes=frozenset({torch.uint8}), shape_rules=two_d + (DivisibleBy(1, 16),)),
                              b=ParamConstraint(dtypes=frozenset({torch.uint8}), shape_rules=two_d + (DivisibleBy(1, 16), DivisibleBy(0, 8))),
                              block_scale_a=ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn})),
                              block_scale_b=ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn})),
                              bias=ParamConstraint(dtypes=floats), out_dtype=ParamConstraint(dtypes=floats)),
        "quantize_mxfp8": fc(x=ParamConstraint(dtypes=floats, shape_rules=two_d)),
        "dequantize_mxfp8": fc(qx=ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn}), shape_rules=two_d + (DivisibleBy(1, 32),)),
                               block_scales=ParamConstraint(dtypes=frozenset({torch.float8_e8m0fnu})),
                               output_type=ParamConstraint(dtypes=floats)),
        "scaled_mm_mxfp8": fc(a=ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn}), shape_rules=two_d + (DivisibleBy(1, 32),)),
                              b=ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn}), shape_rules=two_d + (DivisibleBy(1, 32), DivisibleBy(0, 8))),
                              block_scale_a=ParamConstraint(dtypes=frozenset({torch.float8_e8m0fnu})),
                              block_scale_b=ParamConstraint(dtypes=frozenset({torch.float8_e8m0fnu})),
                              bias=ParamConstraint(dtypes=floats), out_dtype=ParamConstraint(dtypes=floats)),
        "apply_rope": rope2, "apply_rope1": rope, "apply_rope_split_half": rope2, "apply_rope_split_half1": rope,
        "adaln": fc(**norm),
        "rmsnorm": fc(x=ParamConstraint(dtypes=floats), weight=ParamConstraint(dtypes=floats)),
        "adaln_quantize_nvfp4": fc(**norm, per_tensor_scale=ParamConstraint(dtypes=frozenset({torch.float32}))),
        "adaln_quantize_mxfp8": fc(**norm),
        "stochastic_rounding_fp8": fc(x=ParamConstraint(dtypes=floats), rng=ParamConstraint(dtypes=frozenset({torch.uint8}))),
        "qk_norm_rope": fc(qkv=ParamConstraint(dtypes=frozenset({torch.bfloat16, torch.float16})),
                           freqs_cis=ParamConstraint(dtypes=frozenset({torch.float32}))),
        "quantize_nvfp4_gather": fc(per_tensor_scale=ParamConstraint(dtypes=frozenset({torch.float32}))),
    }


def set_option(name: str, value: int) -> None:
    """Process-wide library option (see ``ck_set_option`` in the C header)."""
    _native.call("ck_set_option", name.encode(), int(value))


def gemm_device_status() -> int:
    """Synchronise and return the GEMM kernels' device status word (0 = fine)."""
    return int(_native.load().ck_gemm_device_status())


def norm_device_status() -> int:
    """Synchronise and return (then clear) the norm kernels' device-side status word; 0 = healthy."""
    return int(_native.load().ck_norm_device_status())
