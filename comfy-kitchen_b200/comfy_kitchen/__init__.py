"""comfy_kitchen, B200 build: the quantized-linear hot path on hand-written sm_100a kernels.

Public names and signatures follow the reference package (comfy_kitchen/__init__.py:28-72 for the
functions of this path).  Every function goes through a ``torch.library`` custom op and the backend
registry; the registry holds one compute backend, ``cuda``.  There is no CPU or Triton path: a call
the ``cuda`` backend cannot take raises ``NoCapableBackendError``.
"""
from __future__ import annotations

import torch

from . import _ops  # noqa: F401  (defines torch.ops.comfy_kitchen.*)
from ._ops import DTYPE_CODE_TO_DTYPE, DTYPE_TO_CODE  # noqa: F401
from .exceptions import BackendError, BackendNotFoundError, BackendNotImplementedError, NoCapableBackendError
from .float_utils import from_blocked, swap_nibbles, to_blocked
from .registry import registry

__version__ = "0.2.18+b200"

__all__ = [
    "adaln", "rmsnorm", "adaln_quantize_nvfp4", "adaln_quantize_mxfp8", "qk_norm_rope", "quantize_nvfp4_gather",
    "quantize_per_tensor_fp8", "dequantize_per_tensor_fp8", "stochastic_rounding_fp8", "quantize_nvfp4", "dequantize_nvfp4",
    "quantize_mxfp8", "dequantize_mxfp8", "scaled_mm_nvfp4", "scaled_mm_mxfp8",
    "apply_rope", "apply_rope1", "apply_rope_split_half", "apply_rope_split_half1",
    "swap_nibbles", "to_blocked", "from_blocked",
    "list_backends", "set_backend_priority", "enable_backend", "disable_backend", "use_backend",
    "BackendError", "BackendNotFoundError", "BackendNotImplementedError", "NoCapableBackendError",
]

class _Ops:
    """Calls into the custom ops of ``torch.ops.comfy_kitchen``.

    A custom op costs ~30 us of host time per call in torch's dispatcher (measured: 55 us for the public
    ``quantize_nvfp4`` against 18 us for the backend function it ends in, of which the registry's lookup and
    constraint validation are 5 us) -- more than most of this path's kernels run.  The dispatcher is only needed
    when something intercepts the call: ``torch.compile`` tracing, fake / functional tensor modes, tensor
    subclasses.  For plain tensors outside any of those the op's Python body is called directly: same registry
    lookup, same validation, same backend function (the reference pays the dispatcher on every call,
    comfy_kitchen/backends/eager/quantization.py:413-432)."""

    def __init__(self):
        self._ns = torch.ops.comfy_kitchen
        self._direct = {}
        for attr in dir(_ops):
            fn = getattr(_ops, attr)
            if attr.startswith("_op_") and hasattr(fn, "_init_fn") and hasattr(fn, "_qualname"):
                self._direct[fn._qualname.split("::")[1]] = fn._init_fn

    @staticmethod
    def _plain(args) -> bool:
        if torch.compiler.is_compiling() or torch._C._len_torch_dispatch_stack() > 0:
            return False
        if torch._C._len_torch_function_stack() > 0:
            return False
        for a in args:
            if isinstance(a, torch.Tensor) and type(a) is not torch.Tensor and type(a) is not torch.nn.Parameter:
                return False
        return True

    def __getattr__(self, name: str):
        direct, op = self._direct.get(name), getattr(self._ns, name)
        if direct is None:
            return op

        def call(*args):
            return direct(*args) if self._plain(args) else op(*args)

        setattr(self, name, call)   # (resolved once per op)
        return call


_ops_ns = _Ops()


# ------------------------------------------------------------------ normalisation


def adaln(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """layer_norm(x, no affine, eps) * (1 + scale) + shift, scale/shift broadcastable to x."""
    return _ops_ns.adaln(x, scale, shift, eps)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor | None = None, eps: float = 1e-6) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight over the last dimension."""
    return registry.get_implementation("rmsnorm", kwargs={"x": x, "weight": weight})(x, weight, eps)


def adaln_quantize_nvfp4(x, scale, shift, per_tensor_scale, eps: float = 1e-6, hi_first: bool = True):
    """``quantize_nvfp4(adaln(x, scale, shift, eps).reshape(-1, D), per_tensor_scale)`` in one pass over x."""
    return _ops_ns.adaln_quantize_nvfp4(x, scale, shift, per_tensor_scale, eps, hi_first)


def adaln_quantize_mxfp8(x, scale, shift, eps: float = 1e-6):
    """``quantize_mxfp8(adaln(x, scale, shift, eps).reshape(-1, D))`` in one pass over x."""
    return _ops_ns.adaln_quantize_mxfp8(x, scale, shift, eps)


def qk_norm_rope(qkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, freqs_cis: torch.Tensor, heads: int,
                 eps: float = 1e-6):
    """Per-head RMSNorm of q and k, RoPE of both, and q, k, v in attention's [1, heads, tokens, 128] layout, from
    the output of a fused QKV projection ([tokens, 3 * heads * 128]) in one pass.  The backend function of the same
    name also takes output buffers and a token offset (two segments of one joint sequence)."""
    return _ops_ns.qk_norm_rope(qkv, q_weight, k_weight, freqs_cis, heads, eps)


def quantize_nvfp4_gather(segments, per_tensor_scale: torch.Tensor, hi_first: bool = True):
    """quantize_nvfp4 of the column concatenation of one or two (tensor, activation) segments read in place;
    see the backend function for the accepted layouts."""
    first = segments[0][0]
    impl = registry.get_implementation("quantize_nvfp4_gather", kwargs={"x": first, "per_tensor_scale": per_tensor_scale})
    return impl(segments, per_tensor_scale, hi_first)


# ------------------------------------------------------------------ quantize / dequantize


def stochastic_rounding_fp8(x: torch.Tensor, rng: torch.Tensor,
                            output_type: torch.dtype = torch.float8_e4m3fn) -> torch.Tensor:
    """Stochastically round ``x`` (via fp16) to FP8; ``rng`` is a uint8 tensor of x's shape."""
    return _ops_ns.stochastic_rounding_fp8(x, rng, output_type)


def quantize_per_tensor_fp8(x: torch.Tensor, scale: torch.Tensor,
                            output_type: torch.dtype = torch.float8_e4m3fn) -> torch.Tensor:
    return _ops_ns.quantize_fp8(x, scale, DTYPE_TO_CODE[output_type])


def dequantize_per_tensor_fp8(x: torch.Tensor, scale: torch.Tensor,
                              output_type: torch.dtype = torch.bfloat16) -> torch.Tensor:
    return _ops_ns.dequantize_fp8(x, scale, DTYPE_TO_CODE[output_type])


def quantize_nvfp4(x: torch.Tensor, per_tensor_scale: torch.Tensor, epsilon: float = 0.0, pad_16x: bool = False,
                   hi_first: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """-> (uint8 codes [M, K/2], float8_e4m3fn block scales in the tiled 128x4 layout)."""
    return _ops_ns.quantize_nvfp4(x, per_tensor_scale, epsilon, pad_16x, hi_first)


def dequantize_nvfp4(qx: torch.Tensor, per_tensor_scale: torch.Tensor, block_scales: torch.Tensor,
                     output_type: torch.dtype = torch.bfloat16, hi_first: bool = True) -> torch.Tensor:
    return _ops_ns.dequantize_nvfp4(qx, per_tensor_scale, block_scales, DTYPE_TO_CODE[output_type], hi_first)


def quantize_mxfp8(x: torch.Tensor, pad_32x: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """-> (float8_e4m3fn data [M, K], float8_e8m0fnu block scales in the tiled 128x4 layout)."""
    return _ops_ns.quantize_mxfp8(x, pad_32x)


def dequantize_mxfp8(qx: torch.Tensor, block_scales: torch.Tensor,
                     output_type: torch.dtype = torch.bfloat16) -> torch.Tensor:
    return _ops_ns.dequantize_mxfp8(qx, block_scales, DTYPE_TO_CODE[output_type])


# ------------------------------------------------------------------ block-scaled GEMMs


def scaled_mm_nvfp4(a, b, tensor_scale_a, tensor_scale_b, block_scale_a, block_scale_b, bias=None, out_dtype=None,
                    alpha=None) -> torch.Tensor:
    """y = (a @ b.T) * (tensor_scale_a * tensor_scale_b) + bias with a [M, K/2], b [N, K/2] NVFP4."""
    return _ops_ns.scaled_mm_nvfp4(a, b, tensor_scale_a, tensor_scale_b, block_scale_a, block_scale_b, bias,
                                   DTYPE_TO_CODE[out_dtype or torch.bfloat16], alpha)


def scaled_mm_mxfp8(a, b, block_scale_a, block_scale_b, bias=None, out_dtype=None) -> torch.Tensor:
    """y = a @ b.T + bias with a [M, K], b [N, K] MXFP8."""
    return _ops_ns.scaled_mm_mxfp8(a, b, block_scale_a, block_scale_b, bias, DTYPE_TO_CODE[out_dtype or torch.bfloat16])


# ------------------------------------------------------------------ RoPE


def apply_rope(xq: torch.Tensor, xk: torch.Tensor, freqs_cis: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    return _ops_ns.apply_rope(xq, xk, freqs_cis)


def apply_rope1(x: torch.Tensor, freqs_cis: torch.Tensor) -> torch.Tensor:
    return _ops_ns.apply_rope1(x, freqs_cis)


def apply_rope_split_half(xq: torch.Tensor, xk: torch.Tensor, freqs_cis: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    return _ops_ns.apply_rope_split_half(xq, xk, freqs_cis)


def apply_rope_split_half1(x: torch.Tensor, freqs_cis: torch.Tensor) -> torch.Tensor:
    return _ops_ns.apply_rope_split_half1(x, freqs_cis)


# ------------------------------------------------------------------ backend configuration


def set_backend_priority(priority: list[str]) -> None:
    registry.set_priority(priority)


def disable_backend(name: str) -> None:
    registry.disable(name)


def enable_backend(name: str) -> None:
    registry.enable(name)


def list_backends() -> dict:
    return registry.list_backends()


def use_backend(name: str):
    return registry.use_backend(name)


# ------------------------------------------------------------------ backend registration

from .backends import register_backends as _register_backends  # noqa: E402

_register_backends()
