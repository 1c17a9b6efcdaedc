"""Token-to-expert routing tables on the GPU: `route(ids, num_experts, experts, offsets, pairs)` has the signature of the
reference's pybind function (sm120fp4/kernels/moe_w4a16.py:85-91) and fills the caller's buffers in its padded form."""
from __future__ import annotations

import torch

from . import _lib


_WS: dict = {}   # (device index, stream) -> scratch tensor, grown on demand: steady-state calls allocate nothing


def _workspace(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    key = (device.index, stream)
    ws = _WS.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
        _WS[key] = ws
    return ws


def route(ids: torch.Tensor, num_experts: int, experts: torch.Tensor, offsets: torch.Tensor, pairs: torch.Tensor) -> None:
    """Fills the caller's tables on the current stream. The scratch memory of the counting sort is kept per (device, stream)
    and only grows, so a call of a size seen before allocates nothing (it can be captured into a CUDA graph) and calls on
    different streams do not share scratch."""
    if ids.dtype != torch.int32 or experts.dtype != torch.int32 or offsets.dtype != torch.int32 or pairs.dtype != torch.int32:
        raise TypeError("route takes int32 tensors")
    p, umax = ids.numel(), experts.numel()
    if offsets.numel() != umax + 1 or pairs.numel() != p:
        raise RuntimeError("shape")   # the reference's TORCH_CHECK message
    ids = ids.contiguous()
    h = _lib.lib()
    nbytes = h.b200moe_route_workspace_bytes(p, num_experts)
    if nbytes < 0:
        _lib.check(int(nbytes), "route")
    st = _lib.stream_ptr()
    ws = _workspace(ids.device, st, int(nbytes))
    _lib.check(h.b200moe_route(_lib.ptr(ids), p, num_experts, umax, _lib.ptr(experts), _lib.ptr(offsets), _lib.ptr(pairs), _lib.ptr(ws),
                               ws.numel(), st), "route")


def route_tables(ids: torch.Tensor, num_experts: int):
    """Allocate and fill (experts [min(E, P)], offsets [min(E, P) + 1], pairs [P]) for `ids`."""
    ids = ids.to(torch.int32).contiguous()
    p = ids.numel()
    umax = min(num_experts, p)
    experts = torch.empty(umax, dtype=torch.int32, device=ids.device)
    offsets = torch.empty(umax + 1, dtype=torch.int32, device=ids.device)
    pairs = torch.empty(p, dtype=torch.int32, device=ids.device)
    route(ids, num_experts, experts, offsets, pairs)
    return experts, offsets, pairs
