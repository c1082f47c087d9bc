"""NVFP4 layout (TensorCoreNVFP4Layout): E2M1 codes, E4M3 scale per 16 elements, fp32 tensor scale.
Behaviour of the reference's comfy_kitchen/tensor/nvfp4.py:23-260."""
from __future__ import annotations

from dataclasses import dataclass

import torch

import comfy_kitchen as ck
from comfy_kitchen.float_utils import F4_E2M1_MAX, F8_E4M3_MAX, roundup

from ._blockscaled import install_blockscaled_ops
from .base import BaseLayoutParams, QuantizedLayout

_NAME = "TensorCoreNVFP4Layout"


class TensorCoreNVFP4Layout(QuantizedLayout):
    """2-D only; rows and columns are padded to 16; two codes per stored byte."""

    MIN_SM_VERSION = (10, 0)

    @dataclass(frozen=True)
    class Params(BaseLayoutParams):
        block_scale: torch.Tensor  # tiled E4M3 block scales
        transposed: bool = False

        def _tensor_fields(self) -> list[str]:
            return ["scale", "block_scale"]

        def _validate_tensor_fields(self):
            if isinstance(self.scale, torch.Tensor):
                object.__setattr__(self, "scale", self.scale.to(dtype=torch.float32, non_blocking=True))

    @classmethod
    def quantize(cls, tensor, scale=None, **kwargs):
        if tensor.dim() != 2:
            raise ValueError(f"NVFP4 requires 2D tensor, got {tensor.dim()}D")
        shape = tuple(tensor.shape)
        if scale is None or (isinstance(scale, str) and scale == "recalculate"):
            scale = torch.amax(tensor.abs()) / (F8_E4M3_MAX * F4_E2M1_MAX)
        if not isinstance(scale, torch.Tensor):
            scale = torch.tensor(scale)
        scale = scale.to(device=tensor.device, dtype=torch.float32)
        qdata, block_scale = ck.quantize_nvfp4(tensor, scale, pad_16x=cls.get_padded_shape(shape) != shape)
        return qdata, cls.Params(scale=scale, orig_dtype=tensor.dtype, orig_shape=shape, block_scale=block_scale)

    @classmethod
    def dequantize(cls, qdata, params):
        return ck.dequantize_nvfp4(qdata, params.scale, params.block_scale, params.orig_dtype)

    @classmethod
    def get_plain_tensors(cls, qtensor):
        return qtensor._qdata, qtensor._params.scale, qtensor._params.block_scale

    @classmethod
    def state_dict_tensors(cls, qdata, params):
        return {"": qdata, "_scale": params.block_scale, "_scale_2": params.scale}

    @classmethod
    def get_padded_shape(cls, orig_shape):
        if len(orig_shape) != 2:
            raise ValueError(f"NVFP4 requires 2D shape, got {len(orig_shape)}D")
        return (roundup(orig_shape[0], 16), roundup(orig_shape[1], 16))

    @classmethod
    def get_storage_shape(cls, orig_shape):
        rows, cols = cls.get_padded_shape(orig_shape)
        return (rows, cols // 2)

    @classmethod
    def get_logical_shape_from_storage(cls, storage_shape):
        return (storage_shape[0], storage_shape[1] * 2)


def _gemm(x, w, bias, out_dtype):
    xq, sx, bx = TensorCoreNVFP4Layout.get_plain_tensors(x)
    wq, sw, bw = TensorCoreNVFP4Layout.get_plain_tensors(w)
    return ck.scaled_mm_nvfp4(xq, wq, tensor_scale_a=sx, tensor_scale_b=sw, block_scale_a=bx, block_scale_b=bw,
                              bias=bias, out_dtype=out_dtype)


def _transposed_params(p, shape, flag):
    return TensorCoreNVFP4Layout.Params(scale=p.scale, orig_dtype=p.orig_dtype, orig_shape=shape,
                                        block_scale=p.block_scale, transposed=flag)


_handle_nvfp4_transpose, _handle_nvfp4_mm, _handle_nvfp4_addmm, _handle_nvfp4_linear = install_blockscaled_ops(
    TensorCoreNVFP4Layout, _NAME, _gemm, _transposed_params)
