"""Kernel-selection rule of the layer, with the interface of sm120fp4/kernels/moe_layer.py:60-93 (`choice`, `use_pdl`).

The reference picks, per batch size and shape, between CUDA-core and mma.sync kernels for FC1 and FC2 and decides whether
its three launches are chained programmatically. Here the same three functions state the rule THIS library runs - they are
what `Weights.forward` consults, not a description beside it:

  tokens 1..16     one fused launch (routing + FC1 + SiLU*mul + FC2 + combine). The tcgen05 kernel ("tcgen05_fused": FP4
                   weights straight into kind::mxf4nvf4 MMAs) whenever the hidden size is at most 3072 (its x scale tiles
                   stay resident in TMEM: 12 K boxes of 256) and there is a worker per 128-row output block; otherwise the
                   mma.sync kernel ("mma_sync_fused"). Both BASELINE shapes (2048 x 768 and 2816 x 704) take the tcgen05 kernel
                   at every batch size: on B200 there is no CUDA-core / tensor-core crossover inside the decode regime.
  tokens 17 and up "prefill_w4a4" when activation scales were given (`Weights.enable_prefill`): the reference's rule for
                   every batch above 16 tokens (sm120fp4/vllm_backend.py:161-168). Otherwise "mid_w4a16" (one W4A16 grouped
                   GEMM call) from `min_tokens` (33 by default: up to two slices the decode kernel is ahead) up to the
                   `max_tokens` the path was enabled for, if hidden and intermediate sizes are at most 3072; otherwise
                   "decode_slices" (slices of 16 through the decode kernel, the reference's fallback,
                   sm120fp4/vllm_backend.py:169-172).
"""
from __future__ import annotations

DECODE_MAX = 16       # tokens of one fused decode launch
TCGEN05_MAX_HIDDEN = 3072
MID_MAX_DIM = 3072
MID_MIN_TOKENS = 33


def decode_kernel(hidden: int = 2048, inter: int = 768, sm_count: int = 148, prepacked: bool = True) -> str:
    """The kernel `b200moe_decode_forward` launches for this shape."""
    if hidden % 128 or inter % 64:
        raise ValueError(f"the kernels take a hidden size that is a multiple of 128 and an intermediate size that is a multiple of 64, not {hidden}/{inter}")
    if prepacked and hidden <= TCGEN05_MAX_HIDDEN and hidden // 128 <= sm_count <= 256:
        return "tcgen05_fused"
    return "mma_sync_fused"


def choice(m: int, hidden: int = 2048, inter: int = 768) -> tuple[str, str]:
    """(FC1 kernel, FC2 kernel) for a decode batch of m tokens, as the reference's `choice`. One fused kernel runs both
    halves, so both entries name it."""
    if not 1 <= m <= DECODE_MAX:
        raise ValueError(f"the layer's decode kernel takes 1 to {DECODE_MAX} tokens, not {m}")
    k = decode_kernel(hidden, inter)
    return k, k


def regime(m: int, hidden: int = 2048, inter: int = 768, prefill: bool = False, mid_max_tokens: int = 0,
           mid_min_tokens: int = MID_MIN_TOKENS) -> str:
    """Which path a batch of m tokens takes: "decode", "prefill_w4a4", "mid_w4a16" or "decode_slices". `prefill`: the W4A4
    path is enabled; `mid_max_tokens`: the size the one-call W4A16 path was enabled for (0: not enabled)."""
    if m < 1:
        raise ValueError(f"the layer takes at least one token, not {m}")
    if m <= DECODE_MAX:
        return "decode"
    if prefill:
        return "prefill_w4a4"
    if mid_max_tokens and max(mid_min_tokens, DECODE_MAX + 1) <= m <= mid_max_tokens and hidden <= MID_MAX_DIM and inter <= MID_MAX_DIM:
        return "mid_w4a16"
    return "decode_slices"


def use_pdl(m: int) -> bool:
    """Whether the launches of a decode call are chained programmatically when the caller does not say (`pdl=None`). The
    reference measured a gain below 16 tokens and a loss at 16 (sm120fp4/kernels/moe_layer.py:89-93); here the chained form
    is ahead at every decode batch size (about 2 us per call), so the default is on throughout."""
    return 1 <= m <= DECODE_MAX


def __getattr__(name):   # moe, fc1, fc2, fc1m, fc2p: the kernel modules under the names the reference's moe_layer gives them
    if name in ("moe", "fc1", "fc2", "fc1m", "fc2p"):
        from . import kernels
        return getattr(kernels, name)
    raise AttributeError(name)
