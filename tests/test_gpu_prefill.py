"""GPU parity of the W4A4 prefill path (tcgen05 grouped GEMM) against the oracle's W4A4 arithmetic
(sm120fp4/kernels/bench_moe_baseline.py:53-74 with act_quant=True) and against the reference's golden outputs."""
import numpy as np
import pytest
import torch

from helpers import check_w4a4_output as check_layer_output
from oracle import nvfp4_oracle as O
from test_gpu_decode import inputs, layer

pytestmark = pytest.mark.gpu


def run_prefill(w, x, ids, wts, max_tokens=512):
    if w.prefill is None or w.prefill.max_tokens < max_tokens:
        w.enable_prefill(max_tokens=max_tokens)
    out = w.forward(x.cuda(), ids.cuda(), wts.cuda())
    w.prefill_status()
    return out


@pytest.mark.parametrize("name,m", [("tiny", 17), ("tiny", 40), ("tiny", 130), ("tiny", 300), ("mid", 64), ("mid", 257), ("odd", 100)])
def test_prefill_matches_w4a4_oracle(name, m):
    cfg, w, ow = layer(name)
    x, ids, wts = inputs(cfg, m, 500 + m)
    out = run_prefill(w, x, ids, wts)
    want = O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy(), act_quant=True)
    err, rel = check_layer_output(out, want, f"prefill {name} m={m}")
    print(f"prefill {name} m={m}: max-abs/rms {err:.2e} normwise {rel:.2e}")


def test_prefill_matches_golden_reference_output(golden):
    cfg, w, _ = layer("tiny")
    x, ids, wts = inputs(cfg, 40, 15)
    check_layer_output(run_prefill(w, x, ids, wts), golden.load("layer_tiny")["tiny_m40_random_w4a4"], "golden tiny m=40 w4a4")


def test_prefill_is_deterministic_and_row_independent():
    cfg, w, _ = layer("mid")
    x, ids, wts = inputs(cfg, 200, 77)
    a = run_prefill(w, x, ids, wts).clone()
    for _ in range(3):
        assert torch.equal(run_prefill(w, x, ids, wts), a)
    # a token's output does not depend on which other tokens share its tiles: permuting the batch permutes the output
    perm = torch.randperm(200, generator=torch.Generator().manual_seed(3))
    b = run_prefill(w, x[perm], ids[perm], wts[perm])
    assert torch.equal(b, a[perm.cuda()])
    # routing skew: all tokens on one expert (two full tiles of one expert), and an expert with exactly 128 rows
    ids2 = ids.clone()
    ids2[:, 0] = 5
    ids2[:, 1:] = torch.tensor([1, 2, 3])[None, :]
    out = run_prefill(w, x, ids2, wts)
    assert torch.isfinite(out.float()).all()


def test_qwen_shape_prefill_m256_and_chunk_consistency():
    cfg, w, ow = layer("qwen")
    x, ids, wts = inputs(cfg, 1024, 4242)
    full = run_prefill(w, x, ids, wts, max_tokens=1024).clone()
    # the first 256 tokens against the oracle (W4A4 arithmetic, fp32)
    want = O.moe_reference(x[:64].float().numpy(), ow, ids[:64].numpy(), wts[:64].numpy(), act_quant=True)
    check_layer_output(full[:64], want, "qwen prefill (64 of 1024 tokens vs oracle)")
    # size-independent property: a batch of 1024 equals its four chunks of 256, bit for bit
    parts = torch.cat([run_prefill(w, x[s:s + 256], ids[s:s + 256], wts[s:s + 256], max_tokens=1024) for s in range(0, 1024, 256)])
    assert torch.equal(full, parts)
