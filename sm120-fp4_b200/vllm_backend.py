"""The engine-free operator: `Weights` and `Weights.forward`, with the constructor and call signature of
sm120fp4/vllm_backend.py:95-172, on the B200 kernels of this package.

Differences from the reference, all widening: any hidden size that is a multiple of 128 and intermediate size that is a
multiple of 64 (the reference takes 2048 x {768, 1024} only, vllm_backend.py:44-45,102-103); block scales may be handed
over already in the 128x4 swizzle (`scale_layout="128x4"`) or row-major as the checkpoint stores them (converted once on
the device); a decode batch (up to 16 tokens) is ONE kernel launch instead of router + FC1 + FC2.
"""
from __future__ import annotations

import ctypes as C
import os
import sys
from types import SimpleNamespace

import torch

from . import _lib, moe_layer
from .layouts import padded_sf_shape, to_128x4

ENV = "SM120FP4_MOE"
PREFILL_ENV = "SM120FP4_PREFILL"
METHOD_NAME = "modelopt_fp4"
MAXM = 16  # tokens per decode launch


def enabled() -> bool:
    return os.environ.get(ENV, "") == "1"


def prefill_mode() -> str:
    """"w4a4" (default: batches above MAXM tokens run the W4A4 tensor-core path when activation scales were given) or
    "slices" (SM120FP4_PREFILL=slices: slices of MAXM tokens through the decode kernel). The reference's value "cutlass"
    (sm120fp4/vllm_backend.py:55-61) is accepted as a synonym of the default."""
    return "slices" if os.environ.get(PREFILL_ENV, "") == "slices" else "w4a4"


def prefill_explicit() -> bool:
    return os.environ.get(PREFILL_ENV, "") in ("cutlass", "w4a4")


_KERNELS = None


def kernels() -> SimpleNamespace:
    """The kernel groups under the names the reference's loader returns (sm120fp4/vllm_backend.py:64-80): `layer` (the
    selection rule), `route`, `fc1_cc`, `fc2_cc`, `fc1_tc`, `fc2_pf`. Binding only: the library is prebuilt."""
    global _KERNELS
    if _KERNELS is None:
        from . import kernels as K, moe_layer
        _KERNELS = SimpleNamespace(layer=moe_layer, route=K.moe.build(), fc1_cc=K.fc1.build(), fc2_cc=K.fc2.build(),
                                   fc1_tc=K.fc1m.build(), fc2_pf=K.fc2p.build())
    return _KERNELS


def set_pdl(k: SimpleNamespace, on: bool) -> None:
    """The reference's module-wide switch (sm120fp4/vllm_backend.py:83-87); here `forward(..., pdl=...)` carries it per call."""
    k.fc1_cc.fc1_set_pdl(on)
    k.fc2_cc.fc2_set_pdl(on)
    k.fc1_tc.fc1_mma_set_pdl(on)
    k.fc2_pf.fc2_pf_set_pdl(on)


def rotate_halves(t: torch.Tensor, inter: int) -> torch.Tensor:
    """[gate; up] -> [up; gate] along dim 1 (sm120fp4/vllm_backend.py:90-92)."""
    return torch.cat([t[:, inter:], t[:, :inter]], dim=1).contiguous()


class Weights:
    """The layer's weights and work buffers as the kernels read them (sm120fp4/vllm_backend.py:95-121)."""

    def __init__(self, q1: torch.Tensor, s1: torch.Tensor, alpha1: torch.Tensor, q2: torch.Tensor, s2: torch.Tensor,
                 alpha2: torch.Tensor, top_k: int, scale_layout: str = "linear"):
        if q1.dim() != 3:
            raise ValueError("checkpoint layout expected: q1 [E,2I,H/2] s1 [E,2I,H/16] q2 [E,H,I/2] s2 [E,H,I/16]")
        e_n, two_i, h2 = q1.shape
        self.E, self.I, self.H, self.k = e_n, two_i // 2, h2 * 2, top_k
        if self.H % 128 or self.I % 64 or two_i % 2:
            raise ValueError(f"the kernels take a hidden size that is a multiple of 128 and an intermediate size that is a multiple of 64, not {self.H}/{self.I}")
        if e_n > 256 or not 1 <= top_k <= 16:
            raise ValueError(f"the kernels take at most 256 experts and top_k in 1..16, not {e_n}/{top_k}")
        if q1.dtype != torch.uint8 or q2.dtype != torch.uint8 or s1.dtype != torch.uint8 or s2.dtype != torch.uint8:
            raise TypeError("codes and block scales must be uint8 views")
        if scale_layout not in ("linear", "128x4"):
            raise ValueError("scale_layout is 'linear' (checkpoint order) or '128x4' (swizzled per expert)")
        p1, p2 = padded_sf_shape(two_i, self.H // 16), padded_sf_shape(self.H, self.I // 16)
        want1 = (e_n, two_i, self.H // 16) if scale_layout == "linear" else (e_n, *p1)
        want2 = (e_n, self.H, self.I // 16) if scale_layout == "linear" else (e_n, *p2)
        if tuple(q2.shape) != (e_n, self.H, self.I // 2) or s1.numel() != want1[0] * want1[1] * want1[2] \
                or s2.numel() != want2[0] * want2[1] * want2[2]:
            raise ValueError("checkpoint layout expected: q1 [E,2I,H/2] s1 [E,2I,H/16] q2 [E,H,I/2] s2 [E,H,I/16]")
        if alpha1.dtype != torch.float32 or alpha2.dtype != torch.float32 or alpha1.numel() != e_n or alpha2.numel() != e_n:
            raise TypeError("one float32 global scale per expert and projection")
        if not q1.is_cuda:
            raise RuntimeError("Weights lives on a CUDA device; there is no CPU path in this package")
        self.q1, self.alpha1 = q1.contiguous(), alpha1.contiguous()
        self.q2, self.alpha2 = q2.contiguous(), alpha2.contiguous()
        if scale_layout == "linear":
            self.s1_linear, self.s2_linear = s1.contiguous().view(want1), s2.contiguous().view(want2)
            self.s1 = to_128x4(self.s1_linear)          # [E, pad128(2I), pad4(H/16)]
            self.s2 = to_128x4(self.s2_linear)
        else:
            self.s1_linear = self.s2_linear = None
            self.s1, self.s2 = s1.contiguous().view(want1), s2.contiguous().view(want2)
        h = _lib.lib()
        handle = C.c_void_p()
        _lib.check(h.b200moe_layer_create(C.byref(handle), self.E, self.H, self.I, self.k, _lib.ptr(self.q1), _lib.ptr(self.s1),
                                          _lib.ptr(self.alpha1), _lib.ptr(self.q2), _lib.ptr(self.s2), _lib.ptr(self.alpha2)),
                   "Weights")
        self._h = handle
        dev = self.device = q1.device
        self.ws_bytes = int(h.b200moe_layer_workspace_bytes(self._h))
        self.workspace = torch.zeros(self.ws_bytes, dtype=torch.uint8, device=dev)
        # kernel-native copies for the tcgen05 decode kernel (FC1 scale tiles per 64-column block, alpha2 normaliser)
        self.prepack = torch.empty(int(h.b200moe_layer_prepack_bytes(self._h)), dtype=torch.uint8, device=dev)
        _lib.check(h.b200moe_layer_prepack(self._h, _lib.ptr(self.prepack), self.prepack.numel(), _lib.stream_ptr()), "prepack")
        if os.environ.get("B200MOE_DECODE", "") in ("mma", "tcgen05"):   # force one decode kernel (default: chosen by batch size)
            self.set_decode_impl(os.environ["B200MOE_DECODE"])
        umax, pmax = min(e_n, MAXM * top_k), MAXM * top_k
        self.experts = torch.empty(umax, dtype=torch.int32, device=dev)
        self.offsets = torch.empty(umax + 1, dtype=torch.int32, device=dev)
        self.pairs = torch.empty(pmax, dtype=torch.int32, device=dev)
        self.act = torch.empty(pmax, self.I, dtype=torch.bfloat16, device=dev)
        self.prefill = None   # set by enable_prefill: the W4A4 path above MAXM tokens
        self.mid = None       # set by enable_mid: one W4A16 call for 17..max_tokens tokens
        self._host_checked: set = set()   # (addresses, tokens) of host tensor sets forward_host has validated
        from . import kernels as _k
        _k.register(self)
        self._fwd_host = h.b200moe_decode_forward_host
        self._fwd = h.b200moe_decode_forward
        self._fwd_ex = h.b200moe_decode_forward_ex
        self._ws_ptr = self.workspace.data_ptr()

    def release_checkpoint_layout(self) -> None:
        """Drop the checkpoint-layout codes and scales (about half of the layer's device memory): every tcgen05 path reads
        the tile records of the prepack only. Afterwards `set_decode_impl("mma")`, `fc1` and `fc2` raise."""
        _lib.check(_lib.lib().b200moe_layer_release_checkpoint(self._h), "release_checkpoint_layout")
        self.q1 = self.q2 = self.s1 = self.s2 = self.s1_linear = self.s2_linear = None

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                _lib.lib().b200moe_layer_destroy(self._h)
                self._h = None
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass

    def enable_prefill(self, a1_scale: torch.Tensor | float | None = None, a2_scale: torch.Tensor | float | None = None,
                       max_tokens: int = 8192, workspace: torch.Tensor | None = None) -> None:
        """Above MAXM tokens, run the layer's own W4A4 tensor-core path (NVFP4 activations) instead of slices of MAXM.
        a1_scale / a2_scale: the checkpoint's activation input scales of FC1 and FC2 (the largest over the experts is used,
        as in the reference's enable_cutlass_prefill, sm120fp4/vllm_backend.py:123-145); None means 1.0, the global scale
        of the reference's own W4A4 arithmetic. `workspace`: a zeroed uint8 tensor to share between the layers of a stack
        (it only holds transient data of one call); allocated here when None."""
        def one(a):
            if a is None:
                return 1.0
            v = float(torch.as_tensor(a).float().max())
            if not (v > 0 and v == v and v != float("inf")):
                raise ValueError("the input scales must be finite and positive")
            return v
        h = _lib.lib()
        nbytes = int(h.b200moe_prefill_workspace_bytes(self._h, int(max_tokens)))
        if nbytes < 0:
            _lib.check(nbytes, "enable_prefill")
        if workspace is None:
            workspace = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        elif workspace.numel() < nbytes or workspace.dtype != torch.uint8:
            raise ValueError(f"the shared prefill workspace needs {nbytes} bytes of uint8")
        self.prefill = SimpleNamespace(max_tokens=int(max_tokens), gs_x=1.0 / one(a1_scale), gs_a=1.0 / one(a2_scale),
                                       workspace=workspace, forward=self._prefill_forward)

    enable_cutlass_prefill = enable_prefill   # the reference's name for the same switch

    def enable_mid(self, max_tokens: int = 256, workspace: torch.Tensor | None = None, min_tokens: int = 2 * MAXM + 1) -> None:
        """Batches of 33..max_tokens tokens run as ONE W4A16 call (the decode arithmetic, a grouped GEMM over per-expert
        gathered rows) instead of slices of 16 that each stream the touched experts again. `workspace`: a zeroed uint8
        tensor to share between the layers of a stack (transient data of one call); allocated here when None. `min_tokens`:
        first batch size that takes this path (an expert-parallel shard with few local experts gains from 17 on)."""
        h = _lib.lib()
        nbytes = int(h.b200moe_mid_workspace_bytes(self._h, int(max_tokens)))
        if nbytes < 0:
            _lib.check(nbytes, "enable_mid")
        if workspace is None:
            workspace = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        elif workspace.numel() < nbytes or workspace.dtype != torch.uint8:
            raise ValueError(f"the shared mid-batch workspace needs {nbytes} bytes of uint8")
        self.mid = SimpleNamespace(max_tokens=int(max_tokens), min_tokens=max(int(min_tokens), MAXM + 1), workspace=workspace)

    def mid_workspace_bytes(self, max_tokens: int) -> int:
        """Bytes of the mid-batch workspace for `max_tokens`; raises for shapes the one-call path does not take."""
        n = int(_lib.lib().b200moe_mid_workspace_bytes(self._h, int(max_tokens)))
        if n < 0:
            _lib.check(n, "mid workspace")
        return n

    def prefill_workspace_bytes(self, max_tokens: int) -> int:
        n = int(_lib.lib().b200moe_prefill_workspace_bytes(self._h, int(max_tokens)))
        if n < 0:
            _lib.check(n, "prefill workspace")
        return n

    def mid_status(self) -> None:
        _lib.check(_lib.lib().b200moe_mid_status(self._h, _lib.ptr(self.mid.workspace), self.mid.max_tokens, _lib.stream_ptr()), "mid status")

    def _prefill_forward(self, x, ids, wts, out):
        pf = self.prefill
        for s in range(0, x.shape[0], pf.max_tokens):
            e = min(x.shape[0], s + pf.max_tokens)
            _lib.check(_lib.lib().b200moe_prefill_forward(self._h, _lib.ptr(x[s:e]), _lib.ptr(ids[s:e]), _lib.ptr(wts[s:e]), e - s,
                                                          _lib.ptr(out[s:e]), _lib.ptr(pf.workspace), pf.workspace.numel(), pf.max_tokens,
                                                          pf.gs_x, pf.gs_a, _lib.stream_ptr()), "prefill forward")
        return out

    def prefill_status(self) -> None:
        _lib.check(_lib.lib().b200moe_prefill_status(self._h, _lib.ptr(self.prefill.workspace), self.prefill.max_tokens, _lib.stream_ptr()),
                   "prefill status")

    # ------------------------------------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, out: torch.Tensor | None = None,
                pdl: bool | None = None) -> torch.Tensor:
        """The MoE forward for a batch of any size (sm120fp4/vllm_backend.py:147-172). `pdl` (the reference's per-call
        switch for programmatic dependent launch): None or True - the two launches of a decode call are programmatic, so the
        call overlaps the tail of its predecessor in the stream and reads topk_ids / topk_weights at kernel entry (they must
        be complete when the kernel before this call starts; a violation is reported by `status()`); False - ordinary
        stream-ordered launches, no such requirement."""
        if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != self.H:
            raise TypeError(f"x must be bf16 [tokens, {self.H}]")
        m = x.shape[0]
        if tuple(topk_ids.shape) != (m, self.k) or tuple(topk_weights.shape) != (m, self.k):
            raise ValueError("topk_ids and topk_weights must be [tokens, top_k]")
        if not x.is_contiguous():
            x = x.contiguous()
        ids = topk_ids if topk_ids.dtype == torch.int32 and topk_ids.is_contiguous() else topk_ids.to(torch.int32).contiguous()
        wts = topk_weights if topk_weights.dtype == torch.float32 and topk_weights.is_contiguous() else topk_weights.to(torch.float32).contiguous()
        if out is None:
            out = torch.empty_like(x)
        if m <= MAXM:   # the decode call: one foreign-function call, no slicing
            if m:
                st = torch.cuda.current_stream(x.device).cuda_stream
                if pdl is False:
                    rc = self._fwd_ex(self._h, x.data_ptr(), ids.data_ptr(), wts.data_ptr(), m, out.data_ptr(), self._ws_ptr, self.ws_bytes, 1, st)
                else:
                    rc = self._fwd(self._h, x.data_ptr(), ids.data_ptr(), wts.data_ptr(), m, out.data_ptr(), self._ws_ptr, self.ws_bytes, st)
                if rc:
                    _lib.check(rc, "forward")
            return out
        path = moe_layer.regime(m, self.H, self.I, prefill=self.prefill is not None and prefill_mode() != "slices",
                                mid_max_tokens=self.mid.max_tokens if self.mid is not None else 0,
                                mid_min_tokens=self.mid.min_tokens if self.mid is not None else 0)
        if path == "prefill_w4a4":   # W4A4, as the reference's batches above 16 tokens in that mode
            return self.prefill.forward(x, ids, wts, out)
        if path == "mid_w4a16":      # W4A16 in one call
            _lib.check(_lib.lib().b200moe_mid_forward(self._h, x.data_ptr(), ids.data_ptr(), wts.data_ptr(), m, out.data_ptr(),
                                                      self.mid.workspace.data_ptr(), self.mid.workspace.numel(), self.mid.max_tokens,
                                                      torch.cuda.current_stream(x.device).cuda_stream), "mid forward")
            return out
        for s in range(0, m, MAXM):  # "decode_slices"
            e = min(m, s + MAXM)
            self._slice(x[s:e], ids[s:e], wts[s:e], out[s:e], 1 if pdl is False else 0)
        return out

    def forward_host(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """The forward for tensors in host memory: x bf16 [tokens, H], ids int32 and weights f32 [tokens, top_k], out bf16
        [tokens, H], all on the CPU. One library call per 16 tokens enqueues everything on the current stream of the layer's
        device (the inputs are staged by three small copies, a page-locked `out` is written by the kernel directly); nothing
        synchronises - read `out` after synchronising the stream. A set of tensors is validated once and then recognised by
        its addresses, so that a serving loop that reuses its buffers pays for one foreign-function call only."""
        m = x.shape[0]
        key = (x.data_ptr(), topk_ids.data_ptr(), topk_weights.data_ptr(), out.data_ptr(), m)
        if key not in self._host_checked:
            if x.is_cuda or topk_ids.is_cuda or topk_weights.is_cuda or out.is_cuda:
                raise TypeError("forward_host takes host tensors; use forward for device tensors")
            if x.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or topk_ids.dtype != torch.int32 or topk_weights.dtype != torch.float32:
                raise TypeError("x/out bf16, topk_ids int32, topk_weights float32")
            if tuple(x.shape) != (m, self.H) or tuple(out.shape) != (m, self.H) or tuple(topk_ids.shape) != (m, self.k) \
                    or tuple(topk_weights.shape) != (m, self.k):
                raise ValueError("x/out [tokens, H], topk_ids/topk_weights [tokens, top_k]")
            if not (x.is_contiguous() and out.is_contiguous() and topk_ids.is_contiguous() and topk_weights.is_contiguous()):
                raise ValueError("contiguous host tensors expected")
            if len(self._host_checked) > 4096:
                self._host_checked.clear()
            self._host_checked.add(key)
        st = torch.cuda.current_stream(self.device).cuda_stream
        fn = self._fwd_host
        px, pi, pw, po = key[0], key[1], key[2], key[3]
        for s in range(0, m, MAXM):
            n = min(m, s + MAXM) - s
            rc = fn(self._h, px + s * self.H * 2, pi + s * self.k * 4, pw + s * self.k * 4, n, po + s * self.H * 2, self._ws_ptr, self.ws_bytes, st)
            if rc:
                _lib.check(rc, "forward_host")
        return out

    def _slice(self, x, ids, wts, out, flags: int = 0) -> None:
        _lib.check(_lib.lib().b200moe_decode_forward_ex(self._h, _lib.ptr(x), _lib.ptr(ids), _lib.ptr(wts), x.shape[0], _lib.ptr(out),
                                                        _lib.ptr(self.workspace), self.ws_bytes, flags, _lib.stream_ptr()), "forward")

    def fc1(self, x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, act: torch.Tensor) -> None:
        """FC1 + SiLU*mul alone: act bf16 [tokens*top_k, I], row = pair index."""
        _lib.check(_lib.lib().b200moe_decode_fc1(self._h, _lib.ptr(x), _lib.ptr(ids), _lib.ptr(wts), x.shape[0], _lib.ptr(act),
                                                 _lib.ptr(self.workspace), self.ws_bytes, _lib.stream_ptr()), "fc1")

    def fc2(self, act: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, out: torch.Tensor) -> None:
        """FC2 + weighted combine alone, from act bf16 [tokens*top_k, I]."""
        _lib.check(_lib.lib().b200moe_decode_fc2(self._h, _lib.ptr(act), _lib.ptr(ids), _lib.ptr(wts), ids.shape[0], _lib.ptr(out),
                                                 _lib.ptr(self.workspace), self.ws_bytes, _lib.stream_ptr()), "fc2")

    def route_tables(self, m: int):
        """The routing tables the last decode launch of `m` tokens wrote, in the router's padded form."""
        umax, p = min(self.E, m * self.k), m * self.k
        ex, off, pairs = self.experts[:umax], self.offsets[:umax + 1], self.pairs[:p]
        _lib.check(_lib.lib().b200moe_layer_route_tables(self._h, _lib.ptr(self.workspace), m, _lib.ptr(ex), _lib.ptr(off), _lib.ptr(pairs),
                                                         _lib.stream_ptr()), "route_tables")
        return ex, off, pairs

    def set_decode_impl(self, impl: str) -> None:
        """'auto' / 'tcgen05' (FP4 tensor-core kernel) or 'mma' (mma.sync kernel with in-register dequantisation)."""
        code = {"auto": 0, "mma": 1, "tcgen05": 2}[impl]
        _lib.check(_lib.lib().b200moe_layer_set_decode_impl(self._h, code), "set_decode_impl")

    def set_act_scale(self, g1: float) -> None:
        _lib.check(_lib.lib().b200moe_layer_set_act_scale(self._h, float(g1)), "set_act_scale")

    def status(self) -> None:
        """Synchronise and raise if a bounded device-side wait ran out or an expert id was out of range."""
        _lib.check(_lib.lib().b200moe_layer_status(self._h, _lib.ptr(self.workspace), _lib.stream_ptr()), "status")

    def reset_workspace(self) -> None:
        _lib.check(_lib.lib().b200moe_layer_workspace_init(self._h, _lib.ptr(self.workspace), self.ws_bytes, _lib.stream_ptr()), "reset")

    def expert_bytes(self) -> int:
        """Packed FP4 + scale bytes of one expert (sm120fp4/kernels/bench_moe_baseline.py:190-191)."""
        return 3 * self.I * self.H // 2 + 3 * self.I * self.H // 16


def map_expert_ids(topk_ids: torch.Tensor, topk_weights: torch.Tensor, expert_map: torch.Tensor):
    """Global expert ids -> the ids of this rank's shard under an engine's expert map (int tensor [global experts]: local id,
    or -1 for an expert another rank owns). Slots of other ranks' experts become id -1 with weight 0, which every kernel of
    this package skips; the row such a call returns is the partial sum over this rank's experts."""
    emap = expert_map.to(device=topk_ids.device)
    local = emap[topk_ids.long()].to(torch.int32)
    own = local >= 0
    return torch.where(own, local, torch.full_like(local, -1)), torch.where(own, topk_weights.to(torch.float32), torch.zeros((), device=topk_ids.device))


_SHARED_WS: dict = {}


def shared_workspace(kind: str, device, nbytes: int) -> torch.Tensor:
    """One zeroed workspace per (kind, device) for all layers of a model: the prefill and mid-batch workspaces only hold
    transient data of one layer call, and the layers of a model run one after the other on one stream."""
    key = (kind, str(device))
    t = _SHARED_WS.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.zeros(int(nbytes), dtype=torch.uint8, device=device)
        _SHARED_WS[key] = t
    return t


def weights_from_vllm_layout(w13: torch.Tensor, w13_scale: torch.Tensor, w13_scale_2: torch.Tensor, w2: torch.Tensor,
                             w2_scale: torch.Tensor, w2_scale_2: torch.Tensor, top_k: int) -> Weights:
    """Build Weights from the tensors vLLM's loader fills: w13 [E, 2I, H/2] as [gate; up], e4m3 block scales [E, 2I, H/16],
    w13_scale_2 [E, 2] (gate, up), w2 [E, H, I/2], w2 scales [E, H, I/16], w2_scale_2 [E] (sm120fp4/vllm_backend.py:193-206)."""
    e_n, two_i = w13.shape[0], w13.shape[1]
    inter = two_i // 2
    g = w13_scale_2.reshape(e_n, -1).to(torch.float32)
    if g.shape[1] == 2 and not torch.equal(g[:, 0], g[:, 1]):
        n = int((g[:, 0] != g[:, 1]).sum())
        raise ValueError(f"gate and up global scales differ on {n} of {e_n} experts; FC1 applies one alpha per expert")
    alpha1 = g[:, 0].contiguous()
    return Weights(rotate_halves(w13, inter).view(torch.uint8), rotate_halves(w13_scale, inter).view(torch.uint8), alpha1,
                   w2.view(torch.uint8), w2_scale.view(torch.uint8), w2_scale_2.to(torch.float32).reshape(-1), top_k)


# ----------------------------------------------------------------------------------------------------------------------
def _vllm():
    from vllm.model_executor.layers.quantization import register_quantization_config
    return SimpleNamespace(register=register_quantization_config)


def classes() -> SimpleNamespace:
    from . import vllm_classes as vc
    return SimpleNamespace(Config=vc.SM120Fp4Config, Method=vc.SM120Fp4MoEMethod)


def _log(msg: str) -> None:
    try:
        from vllm.logger import init_logger
        init_logger("vllm.sm120fp4").info("sm120fp4_b200: %s", msg)
    except Exception:  # noqa: BLE001 - logging must never fail the engine
        print("sm120fp4_b200:", msg, file=sys.stderr)


def register() -> bool:
    """The `vllm.general_plugins` entry point (sm120fp4/vllm_backend.py:232-245): re-registers `modelopt_fp4` with
    SM120Fp4Config when SM120FP4_MOE=1; a no-op otherwise."""
    if not enabled():
        return False
    v = _vllm()
    v.register(METHOD_NAME)(classes().Config)
    _log(f"{METHOD_NAME} now resolves to SM120Fp4Config ({ENV}=1); routed-experts layers the kernels fit run on them")
    return True
