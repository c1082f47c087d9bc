"""MXFP8 layout (TensorCoreMXFP8Layout): E4M3 data, one E8M0 (power-of-two) scale per 32 elements.
Behaviour of the reference's comfy_kitchen/tensor/mxfp8.py:23-230."""
from __future__ import annotations

from dataclasses import dataclass

import comfy_kitchen as ck
from comfy_kitchen.float_utils import roundup

from ._blockscaled import install_blockscaled_ops
from .base import BaseLayoutParams, QuantizedLayout

_NAME = "TensorCoreMXFP8Layout"


class TensorCoreMXFP8Layout(QuantizedLayout):
    """2-D only; rows and columns are padded to 32; ``scale`` holds the tiled E8M0 block scales."""

    MIN_SM_VERSION = (10, 0)

    @dataclass(frozen=True)
    class Params(BaseLayoutParams):
        transposed: bool = False

        def _tensor_fields(self) -> list[str]:
            return ["scale"]

    @classmethod
    def quantize(cls, tensor, **kwargs):
        if tensor.dim() != 2:
            raise ValueError(f"MXFP8 requires 2D tensor, got {tensor.dim()}D")
        shape = tuple(tensor.shape)
        qdata, block_scale = ck.quantize_mxfp8(tensor, pad_32x=cls.get_padded_shape(shape) != shape)
        return qdata, cls.Params(scale=block_scale, orig_dtype=tensor.dtype, orig_shape=shape)

    @classmethod
    def dequantize(cls, qdata, params):
        return ck.dequantize_mxfp8(qdata, params.scale, params.orig_dtype)

    @classmethod
    def get_plain_tensors(cls, qtensor):
        return qtensor._qdata, qtensor._params.scale

    @classmethod
    def state_dict_tensors(cls, qdata, params):
        return {"": qdata, "_scale": params.scale}

    @classmethod
    def get_padded_shape(cls, orig_shape):
        if len(orig_shape) != 2:
            raise ValueError(f"MXFP8 requires 2D shape, got {len(orig_shape)}D")
        return (roundup(orig_shape[0], 32), roundup(orig_shape[1], 32))

    @classmethod
    def get_storage_shape(cls, orig_shape):
        return cls.get_padded_shape(orig_shape)

    @classmethod
    def get_logical_shape_from_storage(cls, storage_shape):
        return storage_shape


def _gemm(x, w, bias, out_dtype):
    xq, sx = TensorCoreMXFP8Layout.get_plain_tensors(x)
    wq, sw = TensorCoreMXFP8Layout.get_plain_tensors(w)
    return ck.scaled_mm_mxfp8(xq, wq, block_scale_a=sx, block_scale_b=sw, bias=bias, out_dtype=out_dtype)


def _transposed_params(p, shape, flag):
    return TensorCoreMXFP8Layout.Params(scale=p.scale, orig_dtype=p.orig_dtype, orig_shape=shape, transposed=flag)


_handle_mxfp8_transpose, _handle_mxfp8_mm, _handle_mxfp8_addmm, _handle_mxfp8_linear = install_blockscaled_ops(
    TensorCoreMXFP8Layout, _NAME, _gemm, _transposed_params)
