"""Per-tensor-scaled FP8 matmul through torch (a library GEMM; the block-scaled formats have
their own kernels in this package).  Same call shape as the reference's
comfy_kitchen/scaled_mm_v2.py:26-83."""
from __future__ import annotations

import torch

_HAS_V2 = hasattr(torch.nn.functional, "scaled_mm")

if _HAS_V2:
    from torch.nn.functional import ScalingType, SwizzleType  # noqa: F401
else:  # pragma: no cover - older torch

    class ScalingType:  # type: ignore[no-redef]
        TensorWise = "TensorWise"
        BlockWise1x16 = "BlockWise1x16"
        BlockWise1x32 = "BlockWise1x32"

    class SwizzleType:  # type: ignore[no-redef]
        NO_SWIZZLE = "NO_SWIZZLE"
        SWIZZLE_32_4_4 = "SWIZZLE_32_4_4"


def has_scaled_mm_v2() -> bool:
    return _HAS_V2


def scaled_mm_v2(input, weight, scale_a, scale_b, bias=None, out_dtype=None,
                 scale_recipe_a=ScalingType.TensorWise, scale_recipe_b=ScalingType.TensorWise,
                 swizzle_a=SwizzleType.NO_SWIZZLE, swizzle_b=SwizzleType.NO_SWIZZLE) -> torch.Tensor:
    if _HAS_V2:
        return torch.nn.functional.scaled_mm(
            input, weight, scale_a=scale_a, scale_recipe_a=scale_recipe_a, scale_b=scale_b,
            scale_recipe_b=scale_recipe_b, swizzle_a=swizzle_a, swizzle_b=swizzle_b, bias=bias,
            output_dtype=out_dtype, use_fast_accum=False,
        )
    out = torch._scaled_mm(input, weight, scale_a=scale_a, scale_b=scale_b, out_dtype=out_dtype, bias=bias)
    return out[0] if isinstance(out, tuple) else out
