"""Tensor-parallel slicing of block-quantized weights without re-quantizing them.

A checkpoint in the reference's key contract (samples/nvfp4_linear.py:39-80: ``weight`` packed codes,
``weight_scale`` tiled block scales, ``weight_scale_2`` per-tensor scale, optional ``input_scale``) holds
each weight [N, K] quantized as a whole.  Megatron tensor parallelism needs a row range (column-parallel
linear: split N) or a column range (row-parallel linear: split K) of it on each rank.  Because the block
scales are stored in 128 x 4 tiles (comfy_kitchen/float_utils.py:292-326), a range that starts and ends
on tile boundaries — 128 rows, or 4 scale columns = 64 NVFP4 / 128 MXFP8 elements — is a plain slice of
the codes and a plain slice of the tiled scale buffer: the shard's bytes equal what quantizing the sliced
float weight with the same per-tensor scale would give.
"""
from __future__ import annotations

import torch

from comfy_kitchen.float_utils import roundup
from comfy_kitchen.tensor import QuantizedTensor

_FORMATS = {
    # layout name -> (elements per block, codes per stored byte)
    "TensorCoreNVFP4Layout": (16, 2),
    "TensorCoreMXFP8Layout": (32, 1),
}


def slice_tiled_scales(block_scale: torch.Tensor, rows: tuple[int, int], scale_cols: tuple[int, int]) -> torch.Tensor:
    """Rows [r0, r1) and scale columns [c0, c1) of a tiled scale buffer [R, C] (R % 128 == 0, C % 4 == 0),
    r0 % 128 == 0 and c0 % 4 == 0; the result is again a tiled buffer, padded like a fresh one."""
    r0, r1 = rows
    c0, c1 = scale_cols
    big_r, big_c = block_scale.shape
    assert big_r % 128 == 0 and big_c % 4 == 0, "not a tiled scale buffer"
    assert r0 % 128 == 0 and c0 % 4 == 0, "ranges must start on a scale-tile boundary (128 rows, 4 scale columns)"
    assert 0 <= r0 < r1 <= big_r and 0 <= c0 < c1 <= big_c
    # tile (i, j) of the buffer is 512 contiguous bytes at ((i * C/4) + j) * 512
    tiles = block_scale.contiguous().view(torch.uint8).reshape(big_r // 128, big_c // 4, 512)
    t_r1, t_c1 = roundup(r1, 128) // 128, roundup(c1, 4) // 4
    part = tiles[r0 // 128:t_r1, c0 // 4:t_c1].clone()
    # rows / columns of the last tiles that lie beyond the range must read as padding (zero)
    if r1 % 128 or c1 % 4:
        cell = part.reshape(part.shape[0], part.shape[1], 32, 4, 4)   # [.., r % 32, (r % 128) // 32, c % 4]
        if r1 % 128:
            keep = (r1 - r0) - (part.shape[0] - 1) * 128                # valid rows in the last row tile
            r = torch.arange(32).view(32, 1) + 32 * torch.arange(4).view(1, 4)
            cell[-1][:, (r >= keep).to(cell.device)] = 0
        if c1 % 4:
            cell[:, -1, :, :, (c1 - c0) - (part.shape[1] - 1) * 4:] = 0
    out = part.reshape(part.shape[0] * 128, part.shape[1] * 4)
    return out.view(block_scale.dtype)


def shard_quantized(qt: QuantizedTensor, dim: int, rank: int, world: int) -> QuantizedTensor:
    """Rank's equal share of a 2-D NVFP4 / MXFP8 QuantizedTensor along ``dim`` (0 = rows, 1 = columns)."""
    name = qt._layout_cls
    if name not in _FORMATS:
        raise ValueError(f"shard_quantized: unsupported layout {name}")
    block, per_byte = _FORMATS[name]
    params = qt._params
    if getattr(params, "transposed", False):
        raise ValueError("shard_quantized: shard the stored (untransposed) weight")
    n, k = params.orig_shape
    size = (n, k)[dim]
    if size % world:
        raise ValueError(f"dimension {dim} of size {size} does not split over {world} ranks")
    lo, hi = rank * (size // world), (rank + 1) * (size // world)
    unit = 128 if dim == 0 else 4 * block
    if lo % unit or (hi % unit and hi != size):
        raise ValueError(f"shard boundaries {lo}:{hi} must be multiples of {unit} along dim {dim}")
    scale_field = "block_scale" if hasattr(params, "block_scale") else "scale"   # MXFP8 keeps them in `scale`
    qdata, scales = qt._qdata, getattr(params, scale_field)
    if dim == 0:
        q = qdata[lo:hi].contiguous()
        s = slice_tiled_scales(scales, (lo, hi), (0, scales.shape[1]))
        shape = (hi - lo, k)
    else:
        q = qdata[:, lo // per_byte:hi // per_byte].contiguous()
        s = slice_tiled_scales(scales, (0, scales.shape[0]), (lo // block, hi // block))
        shape = (n, hi - lo)
    fields = {f: getattr(params, f) for f in params.__dataclass_fields__}
    fields.update({scale_field: s, "orig_shape": shape})
    return QuantizedTensor(q, name, type(params)(**fields))


def shard_linear_state(state: dict, prefix: str, parallel: str, rank: int, world: int, layout: str = "TensorCoreNVFP4Layout",
                       orig_dtype: torch.dtype = torch.bfloat16) -> dict:
    """One linear of a checkpoint in the reference's key contract -> this rank's tensors.

    parallel = "column" splits the output features (weight rows, bias), "row" splits the input features
    (weight columns; the bias stays on rank 0 only because the partial results are summed).
    Returns {"weight": QuantizedTensor, "bias": tensor | None, "input_scale": tensor | None}.
    """
    assert parallel in ("column", "row")
    from comfy_kitchen.tensor import get_layout_class

    w = state[prefix + "weight"]
    block, per_byte = _FORMATS[layout]
    n, k = w.shape[0], w.shape[1] * per_byte
    klass = get_layout_class(layout)
    fields = dict(orig_dtype=orig_dtype, orig_shape=(n, k))
    if layout == "TensorCoreNVFP4Layout":
        fields["block_scale"] = state[prefix + "weight_scale"].view(torch.float8_e4m3fn)
        fields["scale"] = state[prefix + "weight_scale_2"]
    else:
        fields["scale"] = state[prefix + "weight_scale"].view(torch.float8_e8m0fnu)
    full = QuantizedTensor(w, layout, klass.Params(**fields))
    shard = shard_quantized(full, 0 if parallel == "column" else 1, rank, world)
    bias = state.get(prefix + "bias")
    if bias is not None:
        if parallel == "column":
            per = n // world
            bias = bias[rank * per:(rank + 1) * per].contiguous()
        elif rank != 0:
            bias = None
    return {"weight": shard, "bias": bias, "input_scale": state.get(prefix + "input_scale")}


def take_ranges(qt: QuantizedTensor, dim: int, ranges) -> QuantizedTensor:
    """Concatenation, along ``dim``, of several [lo, hi) ranges of a 2-D NVFP4 / MXFP8 QuantizedTensor
    (0 = rows, 1 = columns).  Every range starts and ends on a scale-tile boundary (128 rows; 64 NVFP4 or 128
    MXFP8 columns), so the result is assembled from whole tiles of codes and scales: a rank's heads of a fused
    q | k | v weight, or its attention and MLP columns of a fused second linear, without re-quantizing."""
    name = qt._layout_cls
    if name not in _FORMATS:
        raise ValueError(f"take_ranges: unsupported layout {name}")
    block, per_byte = _FORMATS[name]
    params = qt._params
    if getattr(params, "transposed", False):
        raise ValueError("take_ranges: slice the stored (untransposed) weight")
    n, k = params.orig_shape
    unit = 128 if dim == 0 else 4 * block
    size = (n, k)[dim]
    scale_field = "block_scale" if hasattr(params, "block_scale") else "scale"
    qdata, scales = qt._qdata, getattr(params, scale_field)
    qs, ss, total = [], [], 0
    for lo, hi in ranges:
        if not (0 <= lo < hi <= size) or lo % unit or hi % unit:
            raise ValueError(f"range {lo}:{hi} along dim {dim} must lie in 0:{size} on multiples of {unit}")
        if dim == 0:
            qs.append(qdata[lo:hi])
            ss.append(slice_tiled_scales(scales, (lo, hi), (0, scales.shape[1])))
        else:
            qs.append(qdata[:, lo // per_byte:hi // per_byte])
            ss.append(slice_tiled_scales(scales, (0, scales.shape[0]), (lo // block, hi // block)))
        total += hi - lo
    q = torch.cat(qs, dim=dim).contiguous()
    if dim == 0:
        s = torch.cat([t.view(torch.uint8) for t in ss], dim=0)      # whole 128-row tiles stack along the rows
        shape = (total, k)
    else:
        # tiles of one row block are contiguous along the scale columns: interleave per row block
        parts = [t.view(torch.uint8).reshape(t.shape[0] // 128, t.shape[1] // 4, 512) for t in ss]
        tiles = torch.cat(parts, dim=1)
        s = tiles.reshape(tiles.shape[0] * 128, tiles.shape[1] * 4)
        shape = (n, total)
    fields = {f: getattr(params, f) for f in params.__dataclass_fields__}
    fields.update({scale_field: s.contiguous().view(scales.dtype), "orig_shape": shape})
    return QuantizedTensor(q, name, type(params)(**fields))
