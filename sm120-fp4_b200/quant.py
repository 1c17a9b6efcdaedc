"""NVFP4 quantizer on the GPU with the interface of sm120fp4/reference.py (global_scale_for, quantize_nvfp4); results are
bit-identical to the reference's CPU code. `quantize_nvfp4_128x4` is the fused form that writes the block scales
directly in the 128x4 swizzle (optionally gathering source rows), as the W4A4 path consumes them."""
from __future__ import annotations

import torch

from . import _lib
from .layouts import padded_sf_shape

BLOCK = 16


def _dtype_code(x: torch.Tensor) -> int:
    if x.dtype == torch.bfloat16:
        return 0
    if x.dtype == torch.float32:
        return 1
    raise TypeError(f"the quantizer takes bf16 or fp32, not {x.dtype}")


def global_scale_for(x: torch.Tensor) -> torch.Tensor:
    """448 * 6 / amax(|x|) as fp32 [1] (sm120fp4/reference.py:68-71), computed on the device."""
    x = x.contiguous()
    scratch = torch.empty(1, dtype=torch.int32, device=x.device)
    gs = torch.empty(1, dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().b200moe_global_scale(_lib.ptr(x), _dtype_code(x), x.numel(), _lib.ptr(scratch), _lib.ptr(gs),
                                               _lib.stream_ptr()), "global_scale_for")
    return gs


def _check_2d(x: torch.Tensor) -> None:
    if x.dim() != 2 or x.shape[1] % BLOCK:
        raise ValueError(f"expected [M, K] with K a multiple of {BLOCK}, got {tuple(x.shape)}")
    if not x.is_cuda:
        raise RuntimeError("quantize_nvfp4 runs on the GPU; there is no CPU path in this package")


def quantize_nvfp4(x: torch.Tensor, global_scale: torch.Tensor | None = None):
    """x [M, K] bf16/fp32 -> (packed u8 [M, K/2], sf u8 [M, K/16] E4M3 bits row-major, global_scale f32 [1])
    (sm120fp4/reference.py:74-90)."""
    _check_2d(x)
    if x.dtype not in (torch.bfloat16, torch.float32):
        x = x.float()
    x = x.contiguous()
    gs = global_scale_for(x) if global_scale is None else global_scale.to(device=x.device, dtype=torch.float32).reshape(1).contiguous()
    m, k = x.shape
    packed = torch.empty(m, k // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(m, k // BLOCK, dtype=torch.uint8, device=x.device)
    _lib.check(_lib.lib().b200moe_quantize_nvfp4(_lib.ptr(x), _dtype_code(x), 0, m, k, _lib.ptr(gs), 0, _lib.ptr(packed), _lib.ptr(sf), 0,
                                                 _lib.stream_ptr()), "quantize_nvfp4")
    return packed, sf, gs


def quantize_nvfp4_128x4(x: torch.Tensor, global_scale: torch.Tensor, src_row: torch.Tensor | None = None,
                         out_rows: int | None = None):
    """Fused quantizer: packed u8 [R, K/2] and block scales written directly in the 128x4 swizzle ([pad128(R), pad4(K/16)]).
    With `src_row` (int32 [R]) destination row r reads x[src_row[r]] (negative: a zero row), which lays tokens out in
    per-expert segments without a separate gather."""
    _check_2d(x)
    x = x.contiguous()
    k = x.shape[1]
    rows = x.shape[0] if src_row is None else (int(src_row.numel()) if out_rows is None else out_rows)
    pr, pc = padded_sf_shape(rows, k // BLOCK)
    gs = global_scale.to(device=x.device, dtype=torch.float32).reshape(1).contiguous()
    packed = torch.empty(rows, k // 2, dtype=torch.uint8, device=x.device)
    zero = (pr != rows) or (pc != k // BLOCK)
    sf = (torch.zeros if zero else torch.empty)(pr, pc, dtype=torch.uint8, device=x.device)
    if src_row is not None:
        src_row = src_row.to(device=x.device, dtype=torch.int32).contiguous()
    _lib.check(_lib.lib().b200moe_quantize_nvfp4(_lib.ptr(x), _dtype_code(x), _lib.ptr(src_row), rows, k, _lib.ptr(gs), 0, _lib.ptr(packed),
                                                 _lib.ptr(sf), 1, _lib.stream_ptr()), "quantize_nvfp4_128x4")
    return packed, sf, gs


def quantize_nvfp4_experts(w: torch.Tensor, swizzle: bool = False):
    """Stacked expert matrices w [E, R, K] -> (packed u8 [E, R, K/2], sf u8 [E, R, K/16] row-major or [E, pad128(R),
    pad4(K/16)] in the 128x4 swizzle, global_scale f32 [E]): each expert quantised with its own global scale
    2688 / amax, exactly as E separate calls of the reference's quantize_nvfp4 would, in three launches."""
    if w.dim() != 3 or w.shape[2] % BLOCK:
        raise ValueError(f"expected [E, R, K] with K a multiple of {BLOCK}, got {tuple(w.shape)}")
    if not w.is_cuda:
        raise RuntimeError("quantize_nvfp4_experts runs on the GPU; there is no CPU path in this package")
    w = w.contiguous()
    e, r, k = w.shape
    h = _lib.lib()
    scratch = torch.empty(e, dtype=torch.int32, device=w.device)
    gs = torch.empty(e, dtype=torch.float32, device=w.device)
    _lib.check(h.b200moe_global_scale_grouped(_lib.ptr(w), _dtype_code(w), e, r * k, _lib.ptr(scratch), _lib.ptr(gs), _lib.stream_ptr()),
               "quantize_nvfp4_experts")
    packed = torch.empty(e, r, k // 2, dtype=torch.uint8, device=w.device)
    if swizzle and r % 128 == 0 and (k // BLOCK) % 4 == 0:
        sf = torch.empty(e, r, k // BLOCK, dtype=torch.uint8, device=w.device)   # pad-free: expert e starts at row e*R
        _lib.check(h.b200moe_quantize_nvfp4(_lib.ptr(w), _dtype_code(w), 0, e * r, k, _lib.ptr(gs), r, _lib.ptr(packed), _lib.ptr(sf), 1,
                                            _lib.stream_ptr()), "quantize_nvfp4_experts")
        return packed, sf, gs
    sf = torch.empty(e, r, k // BLOCK, dtype=torch.uint8, device=w.device)
    _lib.check(h.b200moe_quantize_nvfp4(_lib.ptr(w), _dtype_code(w), 0, e * r, k, _lib.ptr(gs), r, _lib.ptr(packed), _lib.ptr(sf), 0,
                                        _lib.stream_ptr()), "quantize_nvfp4_experts")
    if swizzle:
        from .layouts import to_128x4
        sf = to_128x4(sf)
    return packed, sf, gs
