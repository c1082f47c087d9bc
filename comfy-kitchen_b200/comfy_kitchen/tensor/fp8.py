"""Per-tensor-scaled FP8 layout (TensorCoreFP8Layout): behaviour of the reference's
comfy_kitchen/tensor/fp8.py:23-216.  Quantize / dequantize run on this package's kernels; the
per-tensor FP8 matmul is a plain library GEMM through torch."""
from __future__ import annotations

import logging
from dataclasses import dataclass

import torch

import comfy_kitchen as ck
from comfy_kitchen.scaled_mm_v2 import scaled_mm_v2

from .base import BaseLayoutParams, QuantizedLayout, QuantizedTensor, dequantize_args, register_layout_op

logger = logging.getLogger(__name__)
_NAME = "TensorCoreFP8Layout"


class TensorCoreFP8Layout(QuantizedLayout):
    """E4M3 (or E5M2) data, one fp32 scale for the whole tensor; storage is 1:1 with the logical shape."""

    MIN_SM_VERSION = (8, 9)

    @dataclass(frozen=True)
    class Params(BaseLayoutParams):
        def _validate_tensor_fields(self):
            if isinstance(self.scale, torch.Tensor):
                object.__setattr__(self, "scale", self.scale.to(dtype=torch.float32, non_blocking=True))

    @classmethod
    def quantize(cls, tensor, scale=None, dtype=torch.float8_e4m3fn, **kwargs):
        if scale is None or (isinstance(scale, str) and scale == "recalculate"):
            scale = torch.amax(tensor.abs()) / torch.finfo(dtype).max
        if not isinstance(scale, torch.Tensor):
            scale = torch.tensor(scale)
        scale = scale.to(device=tensor.device, dtype=torch.float32)
        qdata = ck.quantize_per_tensor_fp8(tensor, scale, dtype)
        return qdata, cls.Params(scale=scale, orig_dtype=tensor.dtype, orig_shape=tuple(tensor.shape))

    @classmethod
    def dequantize(cls, qdata, params):
        return ck.dequantize_per_tensor_fp8(qdata, params.scale, params.orig_dtype)

    @classmethod
    def get_plain_tensors(cls, qtensor):
        return qtensor._qdata, qtensor._params.scale

    @classmethod
    def state_dict_tensors(cls, qdata, params):
        return {"": qdata, "_scale": params.scale}


def _both_quantized(*tensors) -> bool:
    return all(isinstance(t, QuantizedTensor) for t in tensors)


def _matmul(a_q, b_q, scale_a, scale_b, bias, out_dtype):
    return scaled_mm_v2(a_q.contiguous(), b_q, scale_a=scale_a, scale_b=scale_b, bias=bias, out_dtype=out_dtype)


@register_layout_op(torch.ops.aten.linear.default, TensorCoreFP8Layout)
def _fp8_linear(qt, args, kwargs):
    x, w = args[0], args[1]
    bias = args[2] if len(args) > 2 else None
    if not _both_quantized(x, w):
        return torch.nn.functional.linear(*dequantize_args((x, w, bias)))
    xq, sx = TensorCoreFP8Layout.get_plain_tensors(x)
    wq, sw = TensorCoreFP8Layout.get_plain_tensors(w)
    out_dtype = kwargs.get("out_dtype", x._params.orig_dtype)
    try:
        out = _matmul(xq, wq.t(), sx, sw, bias, out_dtype)
    except (RuntimeError, TypeError) as e:
        logger.warning(f"FP8 _scaled_mm failed: {e}, falling back to dequantization")
        return torch.nn.functional.linear(*dequantize_args((x, w, bias)))
    if out.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):  # an FP8 result stays quantized
        params = TensorCoreFP8Layout.Params(scale=sx * sw, orig_dtype=x._params.orig_dtype, orig_shape=tuple(out.shape))
        return QuantizedTensor(out, _NAME, params)
    return out


@register_layout_op(torch.ops.aten.mm.default, TensorCoreFP8Layout)
def _fp8_mm(qt, args, kwargs):
    a, b = args[0], args[1]
    if not _both_quantized(a, b):
        return torch.mm(*dequantize_args(args))
    try:
        return _matmul(a._qdata, b._qdata, a._params.scale, b._params.scale, None,
                       kwargs.get("out_dtype", a._params.orig_dtype))
    except (RuntimeError, TypeError):
        return torch.mm(*dequantize_args(args))


@register_layout_op(torch.ops.aten.addmm.default, TensorCoreFP8Layout)
def _fp8_addmm(qt, args, kwargs):
    bias, a, b = args[0], args[1], args[2]
    if not _both_quantized(a, b):
        return torch.addmm(*dequantize_args(args))
    try:
        return _matmul(a._qdata, b._qdata, a._params.scale, b._params.scale, bias,
                       kwargs.get("out_dtype", a._params.orig_dtype))
    except (RuntimeError, TypeError):
        return torch.addmm(*dequantize_args(args))


def _shape_op(aten_op):
    """view / reshape / t act on the FP8 bytes directly (one byte per element, no block structure)."""

    def handler(qt, args, kwargs):
        src = args[0]
        if not isinstance(src, QuantizedTensor):
            return aten_op(*args, **kwargs)
        qdata = aten_op(src._qdata, *args[1:], **kwargs)
        params = TensorCoreFP8Layout.Params(scale=src._params.scale, orig_dtype=src._params.orig_dtype,
                                            orig_shape=tuple(qdata.shape))
        return QuantizedTensor(qdata, _NAME, params)

    return handler


for _op in (torch.ops.aten.view.default, torch.ops.aten.reshape.default, torch.ops.aten.t.default):
    register_layout_op(_op, TensorCoreFP8Layout)(_shape_op(_op))
