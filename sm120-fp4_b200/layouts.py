"""128x4 block-scale layout on the GPU: the interface of sm120fp4/layouts.py (padded_sf_shape, to_128x4, from_128x4)."""
from __future__ import annotations

import torch

from . import _lib

SF_BLOCK_ROWS, SF_BLOCK_COLS = 128, 4


def padded_sf_shape(rows: int, sf_cols: int) -> tuple[int, int]:
    """Rows padded to a multiple of 128 and scale columns to a multiple of 4 (sm120fp4/layouts.py:32-36)."""
    return -(-rows // SF_BLOCK_ROWS) * SF_BLOCK_ROWS, -(-sf_cols // SF_BLOCK_COLS) * SF_BLOCK_COLS


def _u8(t: torch.Tensor) -> torch.Tensor:
    if t.element_size() != 1:
        raise TypeError("block scales are one byte per element (uint8 or float8_e4m3fn)")
    return t.view(torch.uint8)


def to_128x4(sf_linear: torch.Tensor) -> torch.Tensor:
    """Row-major [rows, sf_cols] (or batched [B, rows, sf_cols]) -> 128x4 swizzled [padded_rows, padded_cols] (batched:
    [B, padded_rows, padded_cols]); padding entries are zero (sm120fp4/layouts.py:56-68)."""
    if sf_linear.dim() not in (2, 3):
        raise ValueError(f"expected a 2-D [rows, sf_cols] tensor, got {tuple(sf_linear.shape)}")
    if not sf_linear.is_cuda:
        raise RuntimeError("to_128x4 runs on the GPU; there is no CPU path in this package")
    src = _u8(sf_linear).contiguous()
    batch = 1 if src.dim() == 2 else src.shape[0]
    rows, cols = src.shape[-2], src.shape[-1]
    pr, pc = padded_sf_shape(rows, cols)
    out = torch.empty((batch, pr, pc) if src.dim() == 3 else (pr, pc), dtype=torch.uint8, device=src.device)
    _lib.check(_lib.lib().b200moe_to_128x4(_lib.ptr(src), _lib.ptr(out), batch, rows, cols, _lib.stream_ptr()), "to_128x4")
    return out.view(sf_linear.dtype)


def from_128x4(sf_swizzled: torch.Tensor, rows: int, sf_cols: int) -> torch.Tensor:
    """Inverse of to_128x4 -> row-major [rows, sf_cols] (sm120fp4/layouts.py:71-78); batched if the input is 3-D."""
    pr, pc = padded_sf_shape(rows, sf_cols)
    batch = sf_swizzled.shape[0] if sf_swizzled.dim() == 3 else 1
    if sf_swizzled.numel() != batch * pr * pc:
        raise ValueError(f"swizzled buffer has {sf_swizzled.numel()} elements; expected {pr}*{pc}={pr * pc} for rows={rows}, sf_cols={sf_cols}")
    if not sf_swizzled.is_cuda:
        raise RuntimeError("from_128x4 runs on the GPU; there is no CPU path in this package")
    src = _u8(sf_swizzled).contiguous()
    out = torch.empty((batch, rows, sf_cols) if sf_swizzled.dim() == 3 else (rows, sf_cols), dtype=torch.uint8, device=src.device)
    _lib.check(_lib.lib().b200moe_from_128x4(_lib.ptr(src), _lib.ptr(out), batch, rows, sf_cols, _lib.stream_ptr()), "from_128x4")
    return out.view(sf_swizzled.dtype)
