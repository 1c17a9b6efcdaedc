"""GPU parity of the W4A16 mid-batch path (17 tokens up to a few hundred in one call) against the oracle's W4A16 arithmetic
(sm120fp4/kernels/bench_moe_baseline.py:53-74) and against the 16-token slices it replaces."""
import pytest
import torch

from helpers import check_layer_output
from oracle import nvfp4_oracle as O
from test_gpu_decode import inputs, layer

pytestmark = pytest.mark.gpu


def run_mid(w, x, ids, wts, max_tokens=256):
    if w.mid is None or w.mid.max_tokens < max_tokens:
        w.enable_mid(max_tokens=max_tokens)
    out = w.forward(x.cuda(), ids.cuda(), wts.cuda())
    w.mid_status()
    return out


@pytest.mark.parametrize("name,m", [("tiny", 33), ("tiny", 40), ("tiny", 130), ("mid", 33), ("mid", 64), ("mid", 255), ("odd", 100), ("gemma", 48)])
def test_mid_batches_match_the_w4a16_oracle(name, m):
    cfg, w, ow = layer(name)
    x, ids, wts = inputs(cfg, m, 700 + m)
    out = run_mid(w, x, ids, wts)
    err, rel = check_layer_output(out, O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy()), f"mid {name} m={m}")
    print(f"mid {name} m={m}: max-abs/rms {err:.2e} normwise {rel:.2e}")


def test_mid_is_deterministic_row_independent_and_close_to_the_slices():
    cfg, w, ow = layer("mid")
    x, ids, wts = inputs(cfg, 96, 31)
    slices = w.forward(x.cuda(), ids.cuda(), wts.cuda()).clone()        # without the mid path: slices of 16
    a = run_mid(w, x, ids, wts).clone()
    for _ in range(3):
        assert torch.equal(run_mid(w, x, ids, wts), a)
    perm = torch.randperm(96, generator=torch.Generator().manual_seed(5))
    b = run_mid(w, x[perm], ids[perm], wts[perm])
    assert torch.equal(b, a[perm.cuda()])                                # a token's output does not depend on its neighbours
    rms = float(a.float().pow(2).mean().sqrt())
    assert float((a.float() - slices.float()).abs().max()) <= 2e-2 * rms  # same arithmetic up to summation order and bf16 rounding
    # masked slots (expert-parallel shards) and a fully masked row
    masked = ids.clone()
    masked[:, 1] = -1
    masked[0, :] = -1
    wz = wts.clone()
    wz[masked < 0] = 0
    out = run_mid(w, x, masked, wz)
    check_layer_output(out, O.moe_reference(x.float().numpy(), ow, ids.numpy(), wz.numpy()), "mid masked")
    assert float(out[0].float().abs().max()) == 0.0


def test_qwen_shape_mid_batches():
    cfg, w, ow = layer("qwen")
    for m in (40, 128):
        x, ids, wts = inputs(cfg, m, 8100 + m)
        out = run_mid(w, x, ids, wts)
        check_layer_output(out, O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy()), f"mid qwen m={m}")
