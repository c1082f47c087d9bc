"""Shared handlers of the two block-scaled layouts (NVFP4, MXFP8).

Both store a 2-D tensor row-major with per-block scales along K, pad to their block multiple, treat
``.t()`` as a flag flip (the bytes stay where they are) and reach the tensor cores only in the
"activation @ weight^T" orientation, i.e. ``linear(x, w)`` or ``mm(x, w.t())`` / ``addmm(b, x, w.t())``.
Anything else dequantizes.  Behaviour: reference tensor/nvfp4.py:126-260 and tensor/mxfp8.py:132-230.
"""
from __future__ import annotations

import logging

import torch

from .base import QuantizedTensor, dequantize_args, register_layout_op

logger = logging.getLogger(__name__)


def _crop(result: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Drop the padding rows / columns of a GEMM on padded operands."""
    if result.shape[0] != rows or result.shape[1] != cols:
        return result[:rows, :cols]
    return result


def _flag(t) -> bool:
    return bool(getattr(t._params, "transposed", False))


def install_blockscaled_ops(layout, name: str, gemm, make_params):
    """Register t / mm / addmm / linear for ``layout``.

    gemm(x_qt, w_qt, bias, out_dtype) -> padded [M, N] product of x and w^T (both stored K-major);
    make_params(src_params, orig_shape, transposed) -> params of the transposed view.
    """

    @register_layout_op(torch.ops.aten.t.default, layout)
    def _t(qt, args, kwargs):
        src = args[0]
        if not isinstance(src, QuantizedTensor):
            return torch.ops.aten.t.default(*args, **kwargs)
        r, c = src._params.orig_shape
        return QuantizedTensor(src._qdata, name, make_params(src._params, (c, r), not _flag(src)))

    def _fast_ok(x, w, need_w_transposed: bool) -> bool:
        if not (isinstance(x, QuantizedTensor) and isinstance(w, QuantizedTensor)):
            return False
        if x._qdata.dim() != 2:
            return False
        return (not _flag(x)) and (_flag(w) == need_w_transposed)

    def _run(x, w, bias, out_dtype, rows, cols, fallback, what):
        try:
            return _crop(gemm(x, w, bias, out_dtype), rows, cols)
        except (RuntimeError, TypeError) as e:
            logger.warning(f"{name} {what} failed: {e}, falling back to dequantization")
            return fallback()

    @register_layout_op(torch.ops.aten.mm.default, layout)
    def _mm(qt, args, kwargs):
        a, b = args[0], args[1]
        slow = lambda: torch.mm(*dequantize_args(args))  # noqa: E731
        if not _fast_ok(a, b, need_w_transposed=True):
            return slow()
        return _run(a, b, None, kwargs.get("out_dtype", a._params.orig_dtype),
                    a._params.orig_shape[0], b._params.orig_shape[1], slow, "mm")

    @register_layout_op(torch.ops.aten.addmm.default, layout)
    def _addmm(qt, args, kwargs):
        bias, a, b = args[0], args[1], args[2]
        slow = lambda: torch.addmm(*dequantize_args((bias, a, b)))  # noqa: E731
        if not _fast_ok(a, b, need_w_transposed=True):
            return slow()
        return _run(a, b, bias, a._params.orig_dtype, a._params.orig_shape[0], b._params.orig_shape[1], slow, "addmm")

    @register_layout_op(torch.ops.aten.linear.default, layout)
    def _linear(qt, args, kwargs):
        x, w = args[0], args[1]
        bias = args[2] if len(args) > 2 else None
        slow = lambda: torch.nn.functional.linear(*dequantize_args((x, w, bias)))  # noqa: E731
        if not _fast_ok(x, w, need_w_transposed=False):
            return slow()
        return _run(x, w, bias, kwargs.get("out_dtype", x._params.orig_dtype),
                    x._params.orig_shape[0], w._params.orig_shape[0], slow, "linear")

    return _t, _mm, _addmm, _linear
