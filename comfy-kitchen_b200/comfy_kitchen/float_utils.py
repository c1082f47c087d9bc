"""Bit-level helpers of the quantized formats (host side, torch).

Constants and the 128x4 tiled scale layout match
comfy_kitchen/float_utils.py:20-29 and :292-352 of the reference.  These run on
whatever device their argument lives on and are used for layout bookkeeping
(shapes, un-tiling a scale buffer for inspection); the quantization arithmetic
itself lives in the CUDA kernels.
"""
from __future__ import annotations

import torch

F4_E2M1_MAX = 6.0
F4_E2M1_EPS = 0.5
F8_E4M3_MAX = 448.0
F8_E4M3_EPS = 0.125
F8_E5M2_MAX = 57344.0
F8_E5M2_EPS = 0.0625
E8M0_BIAS = 127


def roundup(x: int, multiple: int) -> int:
    return -(-x // multiple) * multiple


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def _tile_index(rows: int, cols: int, device) -> torch.Tensor:
    """Flat byte offset of scale (r, c) in the tiled buffer, for all r < rows, c < cols."""
    cpad = roundup(cols, 4)
    r = torch.arange(rows, device=device).unsqueeze(1)
    c = torch.arange(cols, device=device).unsqueeze(0)
    return ((r // 128) * (cpad // 4) + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4


def to_blocked(input_matrix: torch.Tensor, flatten: bool = True) -> torch.Tensor:
    """Row-major [H, W] scales -> tiled buffer [roundup(H,128), roundup(W,4)] (zero padded)."""
    rows, cols = input_matrix.shape
    rpad, cpad = roundup(rows, 128), roundup(cols, 4)
    out = torch.zeros(rpad * cpad, dtype=input_matrix.dtype, device=input_matrix.device)
    out[_tile_index(rows, cols, input_matrix.device).reshape(-1)] = input_matrix.reshape(-1)
    return out if flatten else out.view(rpad, cpad)


def from_blocked(blocked_matrix: torch.Tensor, num_rows: int, num_cols: int) -> torch.Tensor:
    """Inverse of :func:`to_blocked`, cropped to [num_rows, num_cols]."""
    idx = _tile_index(num_rows, num_cols, blocked_matrix.device)
    return blocked_matrix.reshape(-1)[idx.reshape(-1)].view(num_rows, num_cols)


def swap_nibbles(packed: torch.Tensor) -> torch.Tensor:
    """0xAB -> 0xBA in every byte: converts between the two FP4 nibble orders."""
    return ((packed << 4) | (packed >> 4)).to(torch.uint8)


def e8m0_to_f32(x: torch.Tensor) -> torch.Tensor:
    """E8M0 byte -> 2^(e-127); byte 0 decodes to 0.0 (float_utils.py:376-382 of the reference)."""
    e = x.to(torch.int32)
    return torch.where(e == 0, torch.zeros_like(e), e << 23).view(torch.float32)
