"""Seeded synthetic inputs with the shapes and distributions of the benchmark configurations.

The reference measured on a public checkpoint that is not available offline; these recipes stand in for it. Every
draw uses a CPU `torch.Generator`, so two machines with the same torch build produce identical tensors (the method of
the reference's tests/test_mm_fp4.py:16-18).
"""
from __future__ import annotations

import torch

QWEN = dict(experts=128, hidden=2048, inter=768, top_k=8)     # Qwen3-30B-A3B-shaped layer
GEMMA = dict(experts=128, hidden=2816, inter=704, top_k=8)    # Gemma-4-26B-A4B-shaped layer
TINY = dict(experts=8, hidden=256, inter=128, top_k=2)        # CPU-sized layer for parity tests


def layer_weights_bf16(experts: int, hidden: int, inter: int, seed: int = 0, std: float = 0.02):
    """w13 bf16 [E, 2I, H] with rows [up ; gate] and w2 bf16 [E, H, I], drawn N(0, std) then rounded to bf16."""
    g = torch.Generator().manual_seed(seed)
    w13 = (torch.randn(experts, 2 * inter, hidden, generator=g) * std).to(torch.bfloat16)
    w2 = (torch.randn(experts, hidden, inter, generator=g) * std).to(torch.bfloat16)
    return w13, w2


def decode_inputs(m: int, experts: int, hidden: int, top_k: int, seed: int, routing: str = "random"):
    """(x bf16 [m, H], topk_ids int32 [m, k], topk_weights fp32 [m, k]).

    random: logits N(0,1) -> softmax -> top-k -> renormalised (sm120fp4/kernels/moe_layer.py:195-200).
    fixed8: every token on experts arange(k) * (E // k), weights 1/k (sm120fp4/kernels/moe_layer.py:201-205)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, hidden, generator=g).to(torch.bfloat16)
    if routing == "random":
        wts, ids = torch.topk(torch.softmax(torch.randn(m, experts, generator=g), dim=-1), top_k, dim=-1)
        wts = (wts / wts.sum(-1, keepdim=True)).float()
        return x, ids.to(torch.int32).contiguous(), wts.contiguous()
    if routing == "fixed8":
        ids = (torch.arange(top_k, dtype=torch.int32) * (experts // top_k)).repeat(m, 1).contiguous()
        return x, ids, torch.full((m, top_k), 1.0 / top_k)
    raise ValueError(f"routing {routing!r}")
