"""Kernel-level entry points under the reference's names and argument order, each group with a `build()` that returns the
object holding them, as the reference's per-kernel modules do (`load_inline(...)` in `build()`):

  moe.build().route(ids, num_experts, experts, offsets, pairs)                      sm120fp4/kernels/moe_w4a16.py:38,85-91
  fc1.build().fc1_w4a16(q1, s1, x, experts, offsets, pairs, alpha, act, inter, top_k)  sm120fp4/kernels/fc1_w4a16.py:37-38,251-262
  fc1m.build().fc1_mma(...same arguments...)                                         sm120fp4/kernels/fc1_mma.py:49-50,266-282
  fc2.build().fc2_w4a16(q2, s2, act, experts, offsets, pairs, weights, alpha, out, top_k)  sm120fp4/kernels/fc2_w4a16.py:37-38,276-279
  fc2p.build().fc2_pf(q2, s2, act, experts, offsets, pairs, weights, alpha, out, scratch, counters, top_k, groups)
                                                                                     sm120fp4/kernels/fc2_mma_pf.py:44-46,403-421
  *_set_pdl(on)                                                                      the reference's module-wide PDL switches

Nothing is compiled here: the library is prebuilt, `build()` only binds it (and raises if it is missing). The halves run on
the library's stand-alone FC1 / FC2 kernels (`b200moe_decode_fc1`, `b200moe_decode_fc2`), which work from a layer handle:
the weight tensors passed in must be those of a live `Weights` (they are looked up by address) - a layer's tensor maps and
swizzled scales are built once at construction, not per call. `act` is bf16 [tokens * top_k, I] with row = pair index.
"""
from __future__ import annotations

import weakref
from types import SimpleNamespace

import torch

from . import _lib
from .router import route

_OWNERS: dict[int, "weakref.ref"] = {}
_PDL = {"fc1": True, "fc1_mma": True, "fc2": True, "fc2_pf": True}


def register(weights) -> None:
    """Called by Weights.__init__: lets the kernel-level entry points find the layer a weight tensor belongs to."""
    ref = weakref.ref(weights)
    _OWNERS[weights.q1.data_ptr()] = ref
    _OWNERS[weights.q2.data_ptr()] = ref


def _owner(t: torch.Tensor, what: str):
    ref = _OWNERS.get(t.data_ptr())
    w = ref() if ref is not None else None
    if w is None or w.q1 is None:
        raise RuntimeError(f"{what}: the codes tensor is not the q1 / q2 of a live Weights (the kernels work from a layer handle)")
    return w


def _ids_from_tables(experts: torch.Tensor, offsets: torch.Tensor, pairs: torch.Tensor, p: int) -> torch.Tensor:
    """topk_ids (flat int32 [P], -1 for pairs that appear in no segment) from the router's tables."""
    ids = torch.full((p,), -1, dtype=torch.int32, device=pairs.device)
    routed = int(offsets[experts.numel()]) if experts.numel() < offsets.numel() else p
    pos = torch.arange(p, device=pairs.device)
    seg = torch.searchsorted(offsets[1:].to(torch.int64), pos, right=True).clamp_(max=max(experts.numel() - 1, 0))
    live = pos < routed
    ids[pairs[live].long()] = experts[seg[live]].to(torch.int32)
    return ids


def _check(x, what, dtype):
    if x.dtype != dtype:
        raise RuntimeError(f"{what}: dtype")        # the reference's TORCH_CHECK failures surface as RuntimeError


def fc1_w4a16(q1, s1, x, experts, offsets, pairs, alpha, act, inter, top_k) -> None:
    w = _owner(q1, "fc1_w4a16")
    m = x.shape[0]
    if m > 16:
        raise RuntimeError("decode kernel: at most 16 tokens")
    _check(x, "fc1_w4a16 x", torch.bfloat16)
    _check(act, "fc1_w4a16 act", torch.bfloat16)
    if int(inter) != w.I or int(top_k) != w.k or x.shape[1] != w.H or act.shape[0] < m * w.k:
        raise RuntimeError("shape")
    ids = _ids_from_tables(experts, offsets, pairs, m * w.k).view(m, w.k)
    wts = torch.ones(m, w.k, dtype=torch.float32, device=x.device)
    w.fc1(x.contiguous(), ids, wts, act)


def fc2_w4a16(q2, s2, act, experts, offsets, pairs, weights, alpha, out, top_k) -> None:
    w = _owner(q2, "fc2_w4a16")
    m = out.shape[0]
    if m > 16:
        raise RuntimeError("decode kernel: at most 16 tokens")
    _check(act, "fc2_w4a16 act", torch.bfloat16)
    _check(out, "fc2_w4a16 out", torch.bfloat16)
    if int(top_k) != w.k or out.shape[1] != w.H or act.shape[1] != w.I or weights.numel() < m * w.k:
        raise RuntimeError("shape")
    ids = _ids_from_tables(experts, offsets, pairs, m * w.k).view(m, w.k)
    w.fc2(act, ids, weights.reshape(-1)[: m * w.k].to(torch.float32).view(m, w.k).contiguous(), out)


def fc2_pf(q2, s2, act, experts, offsets, pairs, weights, alpha, out, scratch, counters, top_k, groups) -> None:
    """The reference's prefetching FC2 takes its own scratch and counters; the layer's workspace holds both here, so the two
    arguments are accepted and left untouched."""
    if not 1 <= int(groups) <= 4:
        raise RuntimeError("scratch")
    fc2_w4a16(q2, s2, act, experts, offsets, pairs, weights, alpha, out, top_k)


def _setter(name):
    def set_pdl(on: bool) -> None:
        _PDL[name] = bool(on)     # recorded only: a stand-alone half is a single launch with nothing to chain to
    return set_pdl


def _bind() -> None:
    _lib.lib()                    # raises if the library has not been built: there is no other code path


def _group(**fns):
    ns = SimpleNamespace(**fns)

    def build(verbose: bool = False):
        _bind()
        return ns
    return SimpleNamespace(build=build, **fns)


moe = _group(route=route)
fc1 = _group(fc1_w4a16=fc1_w4a16, fc1_set_pdl=_setter("fc1"))
fc1m = _group(fc1_mma=fc1_w4a16, fc1_mma_set_pdl=_setter("fc1_mma"))
fc2 = _group(fc2_w4a16=fc2_w4a16, fc2_set_pdl=_setter("fc2"))
fc2p = _group(fc2_pf=fc2_pf, fc2_pf_set_pdl=_setter("fc2_pf"))
