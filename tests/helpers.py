"""Test helpers: build one synthetic layer both as the GPU operator and as the CPU oracle's weights."""
from __future__ import annotations

import numpy as np
import torch

from oracle import nvfp4_oracle as O


def make_layer(experts, hidden, inter, top_k, seed=0, std=0.02, device="cuda", scale_layout="linear"):
    """(Weights on the GPU, ExpertWeights for the oracle). Weights are drawn on the CPU (seeded), quantised on the GPU by
    the library's quantizer (bit-exact with the reference, tested separately) and copied back for the oracle."""
    import sm120fp4_b200 as pkg
    from sm120fp4_b200 import synth
    from sm120fp4_b200.vllm_backend import Weights

    w13, w2 = synth.layer_weights_bf16(experts, hidden, inter, seed=seed, std=std)
    q1, s1, g1 = pkg.quantize_nvfp4_experts(w13.to(device))
    q2, s2, g2 = pkg.quantize_nvfp4_experts(w2.to(device))
    a1, a2 = 1.0 / g1, 1.0 / g2
    if scale_layout == "128x4":
        w = Weights(q1, pkg.to_128x4(s1), a1, q2, pkg.to_128x4(s2), a2, top_k, scale_layout="128x4")
    else:
        w = Weights(q1, s1, a1, q2, s2, a2, top_k)
    ow = O.ExpertWeights(q1.cpu().numpy(), s1.cpu().numpy(), a1.cpu().numpy(), q2.cpu().numpy(), s2.cpu().numpy(), a2.cpu().numpy())
    return w, ow


def check_layer_output(got: torch.Tensor, want: np.ndarray, what=""):
    """The parity bar of the layer: bf16 max-abs error <= 2e-2 x output RMS; also reports the normwise error."""
    g = got.float().cpu().numpy()
    assert np.isfinite(g).all(), f"{what}: non-finite output"
    rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
    err = float(np.abs(g - want).max())
    rel = float(np.linalg.norm(g - want) / max(np.linalg.norm(want), 1e-30))
    assert err <= 2e-2 * rms, f"{what}: max-abs error {err:.3e} > 2e-2 * rms ({rms:.3e}); normwise {rel:.3e}"
    assert rel < 1e-2, f"{what}: normwise error {rel:.3e}"
    return err / rms, rel


def check_w4a4_output(got: torch.Tensor, want: np.ndarray, what=""):
    """W4A4 bar. The SiLU*mul activations are re-quantised to FP4 between the two GEMMs; an activation that sits on a
    rounding boundary can take the neighbouring code when the fp32 sum feeding it was accumulated in another order, which
    moves single outputs by more than fp32 round-off. So: normwise error < 1 %, at most 0.1 % of the elements beyond the
    layer bar of 2e-2 x output RMS, and none beyond 8e-2 x RMS."""
    g = got.float().cpu().numpy()
    assert np.isfinite(g).all(), f"{what}: non-finite output"
    rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
    err = np.abs(g - want)
    rel = float(np.linalg.norm(g - want) / max(np.linalg.norm(want), 1e-30))
    frac = float((err > 2e-2 * rms).mean())
    assert rel < 1e-2, f"{what}: normwise error {rel:.3e}"
    assert frac <= 1e-3, f"{what}: {frac:.2e} of the elements beyond 2e-2 * rms"
    assert err.max() <= 8e-2 * rms, f"{what}: max-abs error {err.max():.3e} > 8e-2 * rms ({rms:.3e})"
    return float(err.max()) / rms, rel
