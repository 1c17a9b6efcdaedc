"""Kernel-selection rule of the layer, with the interface of sm120fp4/kernels/moe_layer.py:60-93 (`choice`, `use_pdl`).

The reference picks between CUDA-core and mma.sync kernels per batch size and shape; on B200 the decode regime is one
persistent kernel for every batch size up to 16 tokens, so the rule names the regime instead of a kernel pair."""
from __future__ import annotations

DECODE_MAX = 16       # tokens: one fused W4A16 launch
PREFILL_MIN = 17      # tokens: W4A4 tensor-core path when activation scales are available, else decode slices


def regime(m: int) -> str:
    if m < 1:
        raise ValueError(f"the layer takes at least one token, not {m}")
    return "decode_w4a16" if m <= DECODE_MAX else "prefill_w4a4"


def choice(m: int, hidden: int = 2048, inter: int = 768) -> tuple[str, str]:
    """(FC1 kernel, FC2 kernel) for a batch of m tokens. Both entries name the same fused kernel in the decode regime."""
    if not 1 <= m <= DECODE_MAX:
        raise ValueError(f"the layer's decode kernel takes 1 to {DECODE_MAX} tokens, not {m}")
    return "fused_tma_stream", "fused_tma_stream"


def use_pdl(m: int) -> bool:
    """The reference toggles programmatic dependent launch between its three kernels (moe_layer.py:89-93). One launch has
    no dependent launch inside it; kept for signature compatibility."""
    return False
