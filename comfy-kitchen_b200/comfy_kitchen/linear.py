"""Linear layers on block-quantized weights, loading the reference's checkpoint key contract.

Counterparts of the reference's samples: ``NVFP4Linear`` (samples/nvfp4_linear.py:10-80: keys ``weight``
packed codes, ``weight_scale`` tiled E4M3 block scales stored as uint8, ``weight_scale_2`` fp32 per-tensor
scale, optional ``input_scale`` for static activation quantization, ``bias``) and ``MXFP8Linear`` /
``patch_model_with_mxfp8`` (samples/mxfp8_model_patcher.py:15-76 and following).  Both route
``torch.nn.functional.linear`` through ``QuantizedTensor`` and therefore through this package's kernels.

Addition: tensor parallelism.  With ``parallel="column"`` or ``"row"`` and (rank, world), a module keeps only
its shard of the checkpoint's weight, cut out of the packed codes and the tiled scale buffer without
re-quantizing (comfy_kitchen/sharding.py); ``in_features`` / ``out_features`` stay those of the full layer.
A row-parallel module returns this rank's partial sum (bias on rank 0 only); the caller sums over the ranks.
"""
from __future__ import annotations

import logging

import torch
import torch.nn as nn

from comfy_kitchen.sharding import shard_linear_state
from comfy_kitchen.tensor import QuantizedTensor, TensorCoreNVFP4Layout

logger = logging.getLogger(__name__)


class NVFP4Linear(nn.Module):
    """Linear layer whose weight lives only as NVFP4 codes + block scales (no full-precision copy)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 parallel: str | None = None, rank: int = 0, world: int = 1) -> None:
        super().__init__()
        assert parallel in (None, "column", "row")
        self.device = "cpu" if device is None else device
        self.compute_dtype = torch.bfloat16 if dtype is None else dtype
        self.in_features, self.out_features = in_features, out_features
        self.parallel, self.rank, self.world = (parallel if world > 1 else None), rank, world
        self.weight = None   # set while loading a state dict
        self.input_scale = None
        local_out = out_features // world if self.parallel == "column" else out_features
        keeps_bias = bias and not (self.parallel == "row" and rank != 0)
        if keeps_bias:
            self.bias = nn.Parameter(torch.empty(local_out, dtype=self.compute_dtype, device=self.device))
        else:
            self.register_parameter("bias", None)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        keys = [prefix + "weight", prefix + "weight_scale_2", prefix + "weight_scale"]
        absent = [k for k in keys if k not in state_dict]
        if absent:
            missing_keys.extend(absent)
            return
        if self.parallel is None:
            weight = state_dict.pop(prefix + "weight").to(device=self.device)
            scale = state_dict.pop(prefix + "weight_scale_2").to(device=self.device)
            block = state_dict.pop(prefix + "weight_scale").to(device=self.device).view(dtype=torch.float8_e4m3fn)
            params = TensorCoreNVFP4Layout.Params(scale=scale, orig_dtype=self.compute_dtype,
                                                  orig_shape=(self.out_features, self.in_features), block_scale=block)
            qt = QuantizedTensor(weight, "TensorCoreNVFP4Layout", params)
        else:
            local = {k[len(prefix):]: state_dict[k] for k in keys + [prefix + "bias"] if k in state_dict}
            shard = shard_linear_state({prefix + k: v for k, v in local.items()}, prefix, self.parallel, self.rank,
                                       self.world, "TensorCoreNVFP4Layout", self.compute_dtype)
            qt = shard["weight"].to(device=self.device)
            for k in keys:
                state_dict.pop(k)
            if prefix + "bias" in state_dict:
                b = state_dict.pop(prefix + "bias")
                if self.bias is not None:
                    state_dict[prefix + "bias"] = shard["bias"].to(self.compute_dtype)
                del b
        self.weight = nn.Parameter(qt, requires_grad=False)
        input_scale = state_dict.pop(prefix + "input_scale", None)
        if input_scale is None:
            missing_keys.append(prefix + "input_scale")   # dynamic activation quantization
            self.input_scale = None
        else:
            self.input_scale = nn.Parameter(input_scale.to(device=self.device), requires_grad=False)
            keys.append(prefix + "input_scale")
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)
        for k in keys:
            if k in missing_keys:
                missing_keys.remove(k)

    def state_dict(self, *args, **kwargs) -> dict:
        sd = super().state_dict(*args, **kwargs)
        prefix = kwargs.get("prefix", args[1] if len(args) > 1 else "")
        sd.pop(prefix + "weight", None)   # the QuantizedTensor itself
        sd.update(self.weight.state_dict(prefix + "weight"))
        return sd

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not isinstance(x, QuantizedTensor):
            x = QuantizedTensor.from_float(x, "TensorCoreNVFP4Layout", scale=self.input_scale)
        return torch.nn.functional.linear(x, self.weight, self.bias)


class MXFP8Linear(nn.Module):
    """Linear layer with an MXFP8 weight (32-element E4M3 blocks, E8M0 scales)."""

    def __init__(self, in_features: int, out_features: int, bias: nn.Parameter | None = None,
                 weight_qt: QuantizedTensor | None = None, compute_dtype: torch.dtype = torch.bfloat16) -> None:
        super().__init__()
        self.in_features, self.out_features, self.compute_dtype = in_features, out_features, compute_dtype
        self.weight = nn.Parameter(weight_qt, requires_grad=False) if weight_qt is not None else None
        self.bias = bias

    @classmethod
    def from_linear(cls, linear: nn.Linear, device: str = "cuda") -> "MXFP8Linear":
        weight = linear.weight.data
        if weight.device.type != "cuda":
            weight = weight.to(device)   # the quantizer is a device kernel
        bias = linear.bias
        if bias is not None and bias.device.type != "cuda":
            bias = nn.Parameter(bias.data.to(device))
        return cls(linear.in_features, linear.out_features, bias, QuantizedTensor.from_float(weight, "TensorCoreMXFP8Layout"),
                   weight.dtype)

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        if not isinstance(x, QuantizedTensor):
            if x.ndim == 3:
                x = x.reshape(-1, shape[2])
            if x.ndim != 2:
                return torch.nn.functional.linear(x.reshape(shape), self.weight.dequantize(), self.bias)
            x = QuantizedTensor.from_float(x, "TensorCoreMXFP8Layout")
        out = torch.nn.functional.linear(x, self.weight, self.bias)
        return out.reshape(shape[0], shape[1], self.out_features) if len(shape) == 3 else out


def patch_model_with_mxfp8(model: nn.Module, min_features: int = 64, skip_names: list[str] | None = None,
                           verbose: bool = False) -> tuple[nn.Module, int]:
    """Replace every suitable nn.Linear of ``model`` by an MXFP8Linear (features at least ``min_features`` and a
    multiple of 32, name not matching ``skip_names``).  Returns (model, number of layers replaced)."""
    skip_names = skip_names or []
    todo = []
    for name, module in model.named_modules():
        if not isinstance(module, nn.Linear):
            continue
        if any(pat in name for pat in skip_names):
            continue
        if min(module.in_features, module.out_features) < min_features or module.in_features % 32:
            continue
        todo.append(name)
    count = 0
    for name in todo:
        parent = model
        *path, leaf = name.split(".")
        for p in path:
            parent = getattr(parent, p)
        try:
            setattr(parent, leaf, MXFP8Linear.from_linear(getattr(parent, leaf)))
            count += 1
        except Exception as e:  # noqa: BLE001 - leave the layer as it was
            logger.warning("MXFP8 patch of %s failed: %s", name, e)
    if verbose:
        logger.info("MXFP8: %d of %d candidate linear layers replaced", count, len(todo))
    return model, count
