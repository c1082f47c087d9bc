"""``torch.library`` custom ops: the traceable entry points of the public API.

Op names and schemas are the reference's (comfy_kitchen/backends/eager/quantization.py:413-716,
rope.py:40-99, adaln.py:22-36): dtypes cross the op boundary as integer codes, every op asks the
registry for an implementation with the call's keyword arguments, and every op has a fake kernel
that fixes the output shapes for ``torch.compile``.
"""
from __future__ import annotations

import torch

from .float_utils import roundup
from .registry import registry

DTYPE_CODE_TO_DTYPE = {
    0: torch.float32,
    1: torch.float16,
    2: torch.bfloat16,
    5: torch.float8_e4m3fn,
    6: torch.float8_e5m2,
}
DTYPE_TO_CODE = {v: k for k, v in DTYPE_CODE_TO_DTYPE.items()}


def _dispatch(name: str, **kwargs):
    return registry.get_implementation(name, kwargs=kwargs)(**kwargs)


# ------------------------------------------------------------------ FP8 per tensor


@torch.library.custom_op("comfy_kitchen::quantize_fp8", mutates_args=())
def _op_quantize_fp8(x: torch.Tensor, scale: torch.Tensor, output_dtype_code: int) -> torch.Tensor:
    return _dispatch("quantize_per_tensor_fp8", x=x, scale=scale, output_type=DTYPE_CODE_TO_DTYPE[output_dtype_code])


@_op_quantize_fp8.register_fake
def _(x, scale, output_dtype_code):
    return torch.empty_like(x, dtype=DTYPE_CODE_TO_DTYPE[output_dtype_code])


@torch.library.custom_op("comfy_kitchen::dequantize_fp8", mutates_args=())
def _op_dequantize_fp8(x: torch.Tensor, scale: torch.Tensor, output_dtype_code: int) -> torch.Tensor:
    return _dispatch("dequantize_per_tensor_fp8", x=x, scale=scale, output_type=DTYPE_CODE_TO_DTYPE[output_dtype_code])


@_op_dequantize_fp8.register_fake
def _(x, scale, output_dtype_code):
    return torch.empty_like(x, dtype=DTYPE_CODE_TO_DTYPE[output_dtype_code])


# ------------------------------------------------------------------ NVFP4


@torch.library.custom_op("comfy_kitchen::quantize_nvfp4", mutates_args=())
def _op_quantize_nvfp4(x: torch.Tensor, per_tensor_scale: torch.Tensor, epsilon: float, pad_16x: bool,
                       hi_first: bool) -> tuple[torch.Tensor, torch.Tensor]:
    return _dispatch("quantize_nvfp4", x=x, per_tensor_scale=per_tensor_scale, epsilon=epsilon, pad_16x=pad_16x,
                     hi_first=hi_first)


@_op_quantize_nvfp4.register_fake
def _(x, per_tensor_scale, epsilon, pad_16x, hi_first):
    rows, cols = x.shape
    if pad_16x:
        rows, cols = roundup(rows, 16), roundup(cols, 16)
    q = torch.empty((rows, cols // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty((roundup(rows, 128), roundup(cols // 16, 4)), dtype=torch.float8_e4m3fn, device=x.device)
    return q, sf


@torch.library.custom_op("comfy_kitchen::dequantize_nvfp4", mutates_args=())
def _op_dequantize_nvfp4(qx: torch.Tensor, per_tensor_scale: torch.Tensor, block_scales: torch.Tensor,
                         output_dtype_code: int, hi_first: bool) -> torch.Tensor:
    return _dispatch("dequantize_nvfp4", qx=qx, per_tensor_scale=per_tensor_scale, block_scales=block_scales,
                     output_type=DTYPE_CODE_TO_DTYPE[output_dtype_code], hi_first=hi_first)


@_op_dequantize_nvfp4.register_fake
def _(qx, per_tensor_scale, block_scales, output_dtype_code, hi_first):
    rows, packed = qx.shape
    return torch.empty((rows, packed * 2), dtype=DTYPE_CODE_TO_DTYPE[output_dtype_code], device=qx.device)


@torch.library.custom_op("comfy_kitchen::scaled_mm_nvfp4", mutates_args=())
def _op_scaled_mm_nvfp4(a: torch.Tensor, b: torch.Tensor, tensor_scale_a: torch.Tensor, tensor_scale_b: torch.Tensor,
                        block_scale_a: torch.Tensor, block_scale_b: torch.Tensor, bias: torch.Tensor | None,
                        output_dtype_code: int, alpha: torch.Tensor | None) -> torch.Tensor:
    return _dispatch("scaled_mm_nvfp4", a=a, b=b, tensor_scale_a=tensor_scale_a, tensor_scale_b=tensor_scale_b,
                     block_scale_a=block_scale_a, block_scale_b=block_scale_b, bias=bias,
                     out_dtype=DTYPE_CODE_TO_DTYPE[output_dtype_code], alpha=alpha)


@_op_scaled_mm_nvfp4.register_fake
def _(a, b, tensor_scale_a, tensor_scale_b, block_scale_a, block_scale_b, bias, output_dtype_code, alpha):
    return torch.empty((a.shape[0], b.shape[0]), dtype=DTYPE_CODE_TO_DTYPE[output_dtype_code], device=a.device)


# ------------------------------------------------------------------ MXFP8


@torch.library.custom_op("comfy_kitchen::quantize_mxfp8", mutates_args=())
def _op_quantize_mxfp8(x: torch.Tensor, pad_32x: bool) -> tuple[torch.Tensor, torch.Tensor]:
    return _dispatch("quantize_mxfp8", x=x, pad_32x=pad_32x)


@_op_quantize_mxfp8.register_fake
def _(x, pad_32x):
    rows, cols = x.shape
    if pad_32x:
        rows, cols = roundup(rows, 32), roundup(cols, 32)
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=x.device)
    sf = torch.empty((roundup(rows, 128), roundup(cols // 32, 4)), dtype=torch.float8_e8m0fnu, device=x.device)
    return q, sf


@torch.library.custom_op("comfy_kitchen::dequantize_mxfp8", mutates_args=())
def _op_dequantize_mxfp8(qx: torch.Tensor, block_scales: torch.Tensor, output_dtype_code: int) -> torch.Tensor:
    return _dispatch("dequantize_mxfp8", qx=qx, block_scales=block_scales,
                     output_type=DTYPE_CODE_TO_DTYPE[output_dtype_code])


@_op_dequantize_mxfp8.register_fake
def _(qx, block_scales, output_dtype_code):
    return torch.empty_like(qx, dtype=DTYPE_CODE_TO_DTYPE[output_dtype_code])


@torch.library.custom_op("comfy_kitchen::scaled_mm_mxfp8", mutates_args=())
def _op_scaled_mm_mxfp8(a: torch.Tensor, b: torch.Tensor, block_scale_a: torch.Tensor, block_scale_b: torch.Tensor,
                        bias: torch.Tensor | None, output_dtype_code: int) -> torch.Tensor:
    return _dispatch("scaled_mm_mxfp8", a=a, b=b, block_scale_a=block_scale_a, block_scale_b=block_scale_b, bias=bias,
                     out_dtype=DTYPE_CODE_TO_DTYPE[output_dtype_code])


@_op_scaled_mm_mxfp8.register_fake
def _(a, b, block_scale_a, block_scale_b, bias, output_dtype_code):
    return torch.empty((a.shape[0], b.shape[0]), dtype=DTYPE_CODE_TO_DTYPE[output_dtype_code], device=a.device)


# ------------------------------------------------------------------ RoPE, AdaLN


def _define_rope(op_name: str, func_name: str, pair: bool):
    if pair:
        @torch.library.custom_op(f"comfy_kitchen::{op_name}", mutates_args=())
        def op(xq: torch.Tensor, xk: torch.Tensor, freqs_cis: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
            return _dispatch(func_name, xq=xq, xk=xk, freqs_cis=freqs_cis)

        @op.register_fake
        def _(xq, xk, freqs_cis):
            return torch.empty_like(xq), torch.empty_like(xk)
    else:
        @torch.library.custom_op(f"comfy_kitchen::{op_name}", mutates_args=())
        def op(x: torch.Tensor, freqs_cis: torch.Tensor) -> torch.Tensor:
            return _dispatch(func_name, x=x, freqs_cis=freqs_cis)

        @op.register_fake
        def _(x, freqs_cis):
            return torch.empty_like(x)
    return op


_op_apply_rope = _define_rope("apply_rope", "apply_rope", True)
_op_apply_rope1 = _define_rope("apply_rope1", "apply_rope1", False)
_op_apply_rope_split_half = _define_rope("apply_rope_split_half", "apply_rope_split_half", True)
_op_apply_rope_split_half1 = _define_rope("apply_rope_split_half1", "apply_rope_split_half1", False)


@torch.library.custom_op("comfy_kitchen::adaln", mutates_args=())
def _op_adaln(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float) -> torch.Tensor:
    return _dispatch("adaln", x=x, scale=scale, shift=shift, eps=eps)


@_op_adaln.register_fake
def _(x, scale, shift, eps):
    return torch.empty_like(x)


# ---- additions of this build (no counterpart in the reference): the fused front ends


@torch.library.custom_op("comfy_kitchen::adaln_quantize_nvfp4", mutates_args=())
def _op_adaln_quantize_nvfp4(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, per_tensor_scale: torch.Tensor,
                             eps: float, hi_first: bool) -> tuple[torch.Tensor, torch.Tensor]:
    return _dispatch("adaln_quantize_nvfp4", x=x, scale=scale, shift=shift, per_tensor_scale=per_tensor_scale, eps=eps,
                     hi_first=hi_first)


@_op_adaln_quantize_nvfp4.register_fake
def _(x, scale, shift, per_tensor_scale, eps, hi_first):
    d = x.shape[-1]
    n = x.numel() // d
    return (torch.empty((n, d // 2), dtype=torch.uint8, device=x.device),
            torch.empty((roundup(n, 128), roundup(d // 16, 4)), dtype=torch.float8_e4m3fn, device=x.device))


@torch.library.custom_op("comfy_kitchen::adaln_quantize_mxfp8", mutates_args=())
def _op_adaln_quantize_mxfp8(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor,
                             eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    return _dispatch("adaln_quantize_mxfp8", x=x, scale=scale, shift=shift, eps=eps)


@_op_adaln_quantize_mxfp8.register_fake
def _(x, scale, shift, eps):
    d = x.shape[-1]
    n = x.numel() // d
    return (torch.empty((n, d), dtype=torch.float8_e4m3fn, device=x.device),
            torch.empty((roundup(n, 128), roundup(d // 32, 4)), dtype=torch.float8_e8m0fnu, device=x.device))


@torch.library.custom_op("comfy_kitchen::qk_norm_rope", mutates_args=())
def _op_qk_norm_rope(qkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, freqs_cis: torch.Tensor,
                     heads: int, eps: float) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _dispatch("qk_norm_rope", qkv=qkv, q_weight=q_weight, k_weight=k_weight, freqs_cis=freqs_cis, heads=heads,
                     eps=eps)


@_op_qk_norm_rope.register_fake
def _(qkv, q_weight, k_weight, freqs_cis, heads, eps):
    shape = (1, heads, freqs_cis.shape[2], 128)
    return tuple(torch.empty(shape, dtype=qkv.dtype, device=qkv.device) for _ in range(3))


@torch.library.custom_op("comfy_kitchen::stochastic_rounding_fp8", mutates_args=())
def _op_stochastic_rounding_fp8(x: torch.Tensor, rng: torch.Tensor, output_type: torch.dtype) -> torch.Tensor:
    return _dispatch("stochastic_rounding_fp8", x=x, rng=rng, output_type=output_type)


@_op_stochastic_rounding_fp8.register_fake
def _(x, rng, output_type):
    return torch.empty(x.shape, dtype=output_type, device=x.device)
