"""Broadcast bookkeeping for AdaLN scale / shift tensors.

The kernels read a modulation tensor as ``rows`` vectors of length D plus one
integer ``group``: output row r uses vector ``r // group``.  That covers the
shapes AdaLN uses in practice ([B, 1, D] against [B, T, D]; per-row modulation)
without expanding the tensor.  Same contract as the reference helper
(comfy_kitchen/backends/_modulation.py:12-57).
"""
from __future__ import annotations

import torch


def _contiguous_groups(mod_lead: tuple[int, ...], x_lead: tuple[int, ...]) -> bool:
    """True when every kept dim lies outside (to the left of) every broadcast dim,
    i.e. equal vectors occupy contiguous runs of output rows."""
    broadcast_seen = False
    for m, n in zip(mod_lead, x_lead):
        if m == n:
            if n != 1 and broadcast_seen:
                return False
        elif m == 1:
            broadcast_seen = broadcast_seen or n != 1
        else:
            return False  # not broadcastable at all
    return True


def adaln_prep_modulation(t: torch.Tensor, x: torch.Tensor, n: int, d: int):
    """Return ``(flat, group)`` with ``flat`` of shape (n // group, d), contiguous."""
    if t.dim() >= 1 and t.shape[-1] == d and t.dim() <= x.dim():
        lead = (1,) * (x.dim() - t.dim()) + tuple(t.shape[:-1])
        rows = t.numel() // d
        if rows > 0 and n % rows == 0 and _contiguous_groups(lead, tuple(x.shape[:-1])):
            return t.reshape(rows, d).contiguous(), n // rows
    # anything else: materialise one vector per row
    return t.expand_as(x).reshape(n, d).contiguous(), 1
