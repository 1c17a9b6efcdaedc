"""GPU parity of the W4A4 prefill path (tcgen05 grouped GEMM) against the oracle's W4A4 arithmetic
(sm120fp4/kernels/bench_moe_baseline.py:53-74 with act_quant=True), stage by stage from the workspace a call leaves behind:
router tables and the activation quantiser bit-exact (sm120fp4/reference.py:74-90 + sm120fp4/layouts.py:56-68), the
re-quantised SiLU*mul activations a member of what the reference quantiser can produce (the tie/defect split of
sm120fp4/oracle.py:199-252), and the outputs within 2e-2 x RMS of the oracle evaluated on the kernel's own codes."""
import numpy as np
import pytest
import torch

from helpers import check_prefill_call, check_w4a4_output
from oracle import nvfp4_oracle as O
from test_gpu_decode import inputs, layer

pytestmark = pytest.mark.gpu


def run_prefill(w, x, ids, wts, max_tokens=512):
    if w.prefill is None or w.prefill.max_tokens != max_tokens:
        w.enable_prefill(max_tokens=max_tokens)
    out = w.forward(x.cuda(), ids.cuda(), wts.cuda())
    w.prefill_status()
    return out


def sample(ids, n_tokens, seed=0):
    """Tokens for the per-pair checks: some of the largest expert (its last, ragged tile included: the pairs of an expert are
    in ascending pair order, so its last tokens sit in its last tile), some of the smallest expert, the rest spread."""
    idn = ids.numpy()
    cnt = np.bincount(idn.reshape(-1), minlength=int(idn.max()) + 1)
    big, small = int(np.argmax(cnt)), int(np.argmin(np.where(cnt > 0, cnt, 1 << 30)))
    tb, ts = np.nonzero((idn == big).any(axis=1))[0], np.nonzero((idn == small).any(axis=1))[0]
    rng = np.random.default_rng(seed)
    pick = set(tb[-3:].tolist()) | set(tb[:1].tolist()) | set(ts[-2:].tolist())
    while len(pick) < min(n_tokens, idn.shape[0]):
        pick.add(int(rng.integers(idn.shape[0])))
    return np.array(sorted(pick))


@pytest.mark.parametrize("name,m", [("tiny", 17), ("tiny", 40), ("tiny", 130), ("tiny", 300), ("mid", 64), ("mid", 257), ("odd", 100)])
def test_prefill_stage_by_stage_small_layers(name, m):
    cfg, w, ow = layer(name)
    x, ids, wts = inputs(cfg, m, 500 + m)
    out = run_prefill(w, x, ids, wts)
    r = check_prefill_call(w, ow, x, ids, wts, out, 512, what=f"prefill {name} m={m}")
    want = O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy(), act_quant=True)
    err, rel = check_w4a4_output(out, want, f"prefill {name} m={m}")
    print(f"prefill {name} m={m}: own codes {r['max_abs_over_rms_own_codes']:.2e} x rms, {r['max_err_over_bound']:.2f} x bound; "
          f"{r['flips']} code / {r['scale_flips']} scale flips in {r['pairs']} rows (closest {r['max_flip']:.2f} half-widths); "
          f"plain oracle {err:.2e} x rms, normwise {rel:.2e}")


@pytest.mark.parametrize("m", [256, 1024, 4096, 8192])
def test_prefill_qwen_shape_stage_by_stage(m):
    """The Qwen3-30B-A3B-shaped layer at the prefill sizes of the benchmark: tables and the x quantiser on ALL rows, the
    per-pair checks on a sample of tokens that includes the last (ragged) tile of the largest expert."""
    cfg, w, ow = layer("qwen")
    x, ids, wts = inputs(cfg, m, 4242 + m)
    out = run_prefill(w, x, ids, wts, max_tokens=8192)
    r = check_prefill_call(w, ow, x, ids, wts, out, 8192, sample_tokens=sample(ids, 8, m), what=f"qwen prefill m={m}")
    print(f"qwen prefill m={m}: own codes {r['max_abs_over_rms_own_codes']:.2e} x rms, {r['max_err_over_bound']:.2f} x bound; "
          f"{r['flips']} code / {r['scale_flips']} scale flips in {r['pairs']} rows; plain oracle {r['max_abs_over_rms_plain_oracle']:.2e} x rms, "
          f"normwise {r['normwise_plain_oracle']:.2e}")


def test_prefill_gemma_shape_stage_by_stage():
    cfg, w, ow = layer("gemma")
    x, ids, wts = inputs(cfg, 256, 99)
    out = run_prefill(w, x, ids, wts, max_tokens=256)
    r = check_prefill_call(w, ow, x, ids, wts, out, 256, sample_tokens=sample(ids, 8, 1), what="gemma prefill m=256")
    print(f"gemma prefill m=256: own codes {r['max_abs_over_rms_own_codes']:.2e} x rms, {r['max_err_over_bound']:.2f} x bound; "
          f"{r['flips']} code flips in {r['pairs']} rows; plain oracle {r['max_abs_over_rms_plain_oracle']:.2e} x rms")


def test_prefill_matches_golden_reference_output(golden):
    cfg, w, _ = layer("tiny")
    x, ids, wts = inputs(cfg, 40, 15)
    check_w4a4_output(run_prefill(w, x, ids, wts), golden.load("layer_tiny")["tiny_m40_random_w4a4"], "golden tiny m=40 w4a4")


def test_prefill_empty_slots_and_input_scales():
    """Masked slots (negative ids: the form an expert-parallel shard receives) and activation input scales other than 1."""
    cfg, w, ow = layer("mid")
    x, ids, wts = inputs(cfg, 150, 31)
    ids = ids.clone()
    ids[::3, 1] = -1
    ids[5] = -1
    wts = wts.clone()
    wts[ids < 0] = 0
    w.enable_prefill(a1_scale=0.5, a2_scale=0.25, max_tokens=512)
    out = w.forward(x.cuda(), ids.cuda(), wts.cuda())
    w.prefill_status()
    assert not out[5].float().abs().max().item(), "a token whose slots are all empty gets a zero row"
    r = check_prefill_call(w, ow, x, ids, wts, out, 512, what="masked slots, gs_x = 2, gs_a = 4")
    print(f"masked: own codes {r['max_abs_over_rms_own_codes']:.2e} x rms, {r['flips']} flips in {r['pairs']} rows")
    w.prefill = None


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


def test_qwen_shape_chunk_consistency():
    """Size-independent property at full size: a batch of 1024 equals its four chunks of 256, bit for bit."""
    cfg, w, ow = layer("qwen")
    x, ids, wts = inputs(cfg, 1024, 4242)
    full = run_prefill(w, x, ids, wts, max_tokens=8192).clone()
    parts = torch.cat([run_prefill(w, x[s:s + 256], ids[s:s + 256], wts[s:s + 256], max_tokens=8192) for s in range(0, 1024, 256)])
    assert torch.equal(full, parts)
