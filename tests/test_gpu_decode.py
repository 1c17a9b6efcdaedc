"""GPU parity of the fused decode layer (M <= 16, W4A16) against the CPU oracle and the golden layer outputs."""
import numpy as np
import pytest
import torch

from helpers import check_layer_output, make_layer
from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu

SHAPES = {
    "tiny": dict(experts=8, hidden=256, inter=128, top_k=2),
    "mid": dict(experts=16, hidden=512, inter=192, top_k=4),
    "odd": dict(experts=12, hidden=384, inter=320, top_k=3),
}
_cache = {}


def layer(name, scale_layout="linear"):
    key = (name, scale_layout)
    if key not in _cache:
        from sm120fp4_b200 import synth
        cfg = {"qwen": synth.QWEN, "gemma": synth.GEMMA}.get(name) or SHAPES[name]
        seed = {"tiny": 3, "qwen": 0}.get(name, 21)
        _cache[key] = (cfg, *make_layer(cfg["experts"], cfg["hidden"], cfg["inter"], cfg["top_k"], seed=seed, scale_layout=scale_layout))
    _cache[key][1].prefill = None        # the layers are shared between tests: each test starts without the W4A4 path
    _cache[key][1].mid = None            # ... and without the one-call W4A16 path for mid-sized batches
    _cache[key][1].set_decode_impl("auto")
    return _cache[key]


def inputs(cfg, m, seed, routing="random"):
    from sm120fp4_b200 import synth
    return synth.decode_inputs(m, cfg["experts"], cfg["hidden"], cfg["top_k"], seed, routing)


def run(w, x, ids, wts):
    out = w.forward(x.cuda(), ids.cuda(), wts.cuda())
    w.status()
    return out


@pytest.mark.parametrize("name", ["tiny", "mid", "odd"])
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 13, 16])
def test_small_layers_match_oracle(name, m):
    cfg, w, ow = layer(name)
    x, ids, wts = inputs(cfg, m, 100 + m)
    out = run(w, x, ids, wts)
    want = O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy())
    check_layer_output(out, want, f"{name} m={m}")
    ex, off, pairs = w.route_tables(m)
    wex, woff, wpairs = O.route_padded(ids.numpy(), cfg["experts"])
    assert np.array_equal(ex.cpu().numpy(), wex) and np.array_equal(off.cpu().numpy(), woff) and np.array_equal(pairs.cpu().numpy(), wpairs)


@pytest.mark.parametrize("name,m", [("tiny", 3), ("mid", 7), ("odd", 16), ("qwen", 16), ("gemma", 5)])
def test_both_decode_kernels_meet_the_bar(name, m):
    """The tcgen05 kernel (FP4 tensor cores, activations as a four-term NVFP4 expansion) and the mma.sync kernel
    (in-register dequantisation) are two implementations of the same contract."""
    cfg, w, ow = layer(name)
    x, ids, wts = inputs(cfg, m, 300 + m)
    want = O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy())
    errs = {}
    try:
        for impl in ("mma", "tcgen05"):
            w.set_decode_impl(impl)
            out = run(w, x, ids, wts)
            errs[impl] = check_layer_output(out, want, f"{name} m={m} {impl}")
            first = out.clone()
            for _ in range(3):
                assert torch.equal(run(w, x, ids, wts), first), f"{impl}: not bit-identical from call to call"
    finally:
        w.set_decode_impl("auto")
    print(f"{name} m={m}: (max-abs/rms, normwise) {errs}")


def test_tiny_layer_matches_golden_reference_outputs(golden):
    cfg, w, ow = layer("tiny")
    g = golden.load("layer_tiny")
    for m, routing, seed in [(1, "random", 11), (6, "random", 12), (16, "random", 13), (5, "fixed8", 14)]:
        x, ids, wts = inputs(cfg, m, seed, routing)
        check_layer_output(run(w, x, ids, wts), g[f"tiny_m{m}_{routing}_w4a16"], f"golden tiny m={m} {routing}")


def test_swizzled_scale_input_and_determinism():
    cfg, w, _ = layer("mid")
    _, w2, _ = layer("mid", "128x4")
    x, ids, wts = inputs(cfg, 7, 5)
    a = run(w, x, ids, wts).clone()
    b = run(w2, x, ids, wts)
    assert torch.equal(a, b), "scales handed over row-major and pre-swizzled must give identical bits"
    for _ in range(20):   # the reference's 50-call bit-identity check, shortened
        assert torch.equal(run(w, x, ids, wts), a)


def test_fixed_routing_duplicates_and_skew():
    cfg, w, ow = layer("mid")
    for m in (4, 16):
        x, ids, wts = inputs(cfg, m, 9, "fixed8")
        check_layer_output(run(w, x, ids, wts), O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy()), f"fixed m={m}")
    # a token that names the same expert twice: two pairs, both weights count
    x, ids, wts = inputs(cfg, 6, 10)
    ids[2, 1] = ids[2, 0]
    ids[5, :] = ids[5, 0]
    check_layer_output(run(w, x, ids, wts), O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy()), "duplicate experts")
    # every token on one expert
    ids[:] = 3
    check_layer_output(run(w, x, ids, wts), O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy()), "one expert")


def test_fc1_and_fc2_entry_points():
    cfg, w, ow = layer("mid")
    m = 11
    x, ids, wts = inputs(cfg, m, 31)
    xd, idd, wd = x.cuda(), ids.cuda(), wts.cuda()
    act = torch.full((m * cfg["top_k"], cfg["inter"]), float("nan"), dtype=torch.bfloat16, device="cuda")
    w.fc1(xd, idd, wd, act)
    w.status()
    want = np.zeros((m * cfg["top_k"], cfg["inter"]), dtype=np.float32)
    for t in range(m):
        for j in range(cfg["top_k"]):
            w1d, _ = ow.dequant(int(ids[t, j]))
            hmid = x[t].float().numpy() @ w1d.T
            want[t * cfg["top_k"] + j] = O.silu(hmid[cfg["inter"]:]) * hmid[:cfg["inter"]]
    got = act.float().cpu().numpy()
    assert np.isfinite(got).all()
    # act is stored in bf16: allow its rounding (2^-8 relative) on top of the layer's bar
    assert (np.abs(got - want) <= 2e-2 * np.sqrt((want ** 2).mean()) * 0.25 + np.abs(want) * 2.0 ** -8 + 1e-6).all()
    out2 = torch.empty(m, cfg["hidden"], dtype=torch.bfloat16, device="cuda")
    w.fc2(act, idd, wd, out2)
    w.status()
    check_layer_output(out2, O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy(), bf16_mid=False), "fc1 -> fc2 entry points")


def test_operator_errors_and_slicing():
    cfg, w, ow = layer("tiny")
    x, ids, wts = inputs(cfg, 40, 15)
    out = run(w, x, ids, wts)                      # 40 tokens: 16 + 16 + 8 through the decode kernel
    parts = torch.cat([run(w, x[s:s + 16], ids[s:s + 16], wts[s:s + 16]) for s in (0, 16, 32)])
    assert torch.equal(out, parts)
    with pytest.raises(TypeError):
        w.forward(x.float().cuda(), ids.cuda(), wts.cuda())
    with pytest.raises(ValueError):
        w.forward(x.cuda(), ids[:, :1].cuda(), wts.cuda())
    assert w.forward(x[:0].cuda(), ids[:0].cuda(), wts[:0].cuda()).shape == (0, cfg["hidden"])
    # int64 ids and bf16 weights are converted, as the reference does
    out2 = w.forward(x[:4].cuda(), ids[:4].long().cuda(), wts[:4].to(torch.bfloat16).cuda())
    assert out2.shape == (4, cfg["hidden"])


def test_qwen_shape_config0_golden(golden):
    """Configuration 0: Qwen3-30B-A3B-shaped layer, M = 4, seed 0, against the output of the reference's own CPU path."""
    import hashlib
    cfg, w, ow = layer("qwen")
    meta = golden.meta["cfg0"]
    h = lambda t: hashlib.sha256(np.ascontiguousarray(t.cpu().numpy()).tobytes()).hexdigest()  # noqa: E731
    assert h(w.q1) == meta["q1_sha256"] and h(w.q2) == meta["q2_sha256"], "GPU-quantised weights differ from the reference's bytes"
    assert h(w.s1_linear) == meta["s1_sha256"] and h(w.s1) == meta["s1_128x4_sha256"]
    assert h(w.s2_linear) == meta["s2_sha256"] and h(w.s2) == meta["s2_128x4_sha256"]
    assert h(w.alpha1) == meta["alpha1_sha256"] and h(w.alpha2) == meta["alpha2_sha256"]
    g = golden.load("layer_cfg0")
    x, ids, wts = inputs(cfg, 4, 100)
    assert np.array_equal(ids.numpy(), g["ids"])
    err, rel = check_layer_output(run(w, x, ids, wts), g["out_m4"], "configuration 0")
    print(f"config 0: max-abs/rms {err:.2e}, normwise {rel:.2e}")


@pytest.mark.parametrize("m,routing", [(1, "random"), (16, "random"), (16, "fixed8"), (8, "fixed8"), (2, "random")])
def test_qwen_shape_sweep(m, routing):
    cfg, w, ow = layer("qwen")
    x, ids, wts = inputs(cfg, m, 1000 + m if routing == "random" else 7, routing)
    out = run(w, x, ids, wts)
    check_layer_output(out, O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy()), f"qwen m={m} {routing}")
    first = out.clone()
    for _ in range(5):
        assert torch.equal(run(w, x, ids, wts), first)


@pytest.mark.parametrize("m,routing", [(4, "random"), (16, "random"), (16, "fixed8")])
def test_gemma_shape(m, routing):
    cfg, w, ow = layer("gemma")
    x, ids, wts = inputs(cfg, m, 2000 + m, routing)
    check_layer_output(run(w, x, ids, wts), O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy()), f"gemma m={m} {routing}")


@pytest.mark.parametrize("name,m", [("mid", 48), ("tiny", 40), ("qwen", 40)])
def test_back_to_back_launches_on_one_workspace(name, m):
    """Batches above 16 tokens run as consecutive launches on the same workspace, and each launch lets the next one be
    scheduled before it has finished (programmatic dependent launch). Some workers of a launch finish before its last
    FC1 gate opens; the next launch must still find the gate words final. Every slice is checked against the oracle and
    the whole sequence must repeat bit for bit."""
    cfg, w, ow = layer(name)
    x, ids, wts = inputs(cfg, m, 4000 + m)
    first = run(w, x, ids, wts).clone()
    check_layer_output(first, O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy()), f"{name} m={m} in slices")
    xd, idd, wd = x.cuda(), ids.cuda(), wts.cuda()
    for _ in range(20):
        assert torch.equal(w.forward(xd, idd, wd), first)
    w.status()


@pytest.mark.parametrize("m", [1, 16, 37])
def test_host_buffer_entry_point_equals_the_device_call(m):
    """b200moe_decode_forward_host: pinned host tensors in, pinned host tensor out, same bits as the device-tensor call."""
    cfg, w, ow = layer("mid")
    x, ids, wts = inputs(cfg, m, 6000 + m)
    want = run(w, x, ids, wts).cpu()
    hx, hid, hw = x.pin_memory(), ids.pin_memory(), wts.pin_memory()
    hout = torch.empty_like(x).pin_memory()
    for _ in range(2):
        hout.zero_()
        w.forward_host(hx, hid, hw, hout)
        torch.cuda.synchronize()
        assert torch.equal(hout, want)
    # pageable host memory takes the staged-copy route of the same entry point
    pout = torch.zeros_like(x)
    w.forward_host(x.clone(), ids.clone(), wts.clone(), pout)
    torch.cuda.synchronize()
    assert torch.equal(pout, want)
    w.status()
    with pytest.raises(TypeError):
        w.forward_host(hx.cuda(), hid, hw, hout)


def test_routing_inputs_written_by_the_kernel_just_before_the_call():
    """topk_ids / topk_weights are read at kernel entry, before the stream dependency of the programmatic launch has resolved.
    Here they are written by a copy kernel enqueued immediately before every call, alternating between two routings without
    any synchronisation in between: every output must be the one of its own routing, and no call may report stale inputs."""
    cfg, w, ow = layer("mid")
    sets = []
    for seed in (41, 42):
        x, ids, wts = inputs(cfg, 9, seed)
        want = run(w, x, ids, wts).clone()
        check_layer_output(want, O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy()), f"seed {seed}")
        sets.append((x.cuda(), ids.cuda(), wts.cuda(), want))
    ids_live, wts_live = torch.empty_like(sets[0][1]), torch.empty_like(sets[0][2])
    outs = []
    for i in range(24):
        xd, idd, wd, _ = sets[i & 1]
        ids_live.copy_(idd)
        wts_live.copy_(wd)
        outs.append(w.forward(xd, ids_live, wts_live))
    w.status()                      # raises on B200MOE_ERR_ORDER
    for i, o in enumerate(outs):
        assert torch.equal(o, sets[i & 1][3]), f"call {i} used stale routing inputs"


def test_ordered_launch_flag_gives_the_same_bits():
    """pdl=False: both kernels of the call are ordinary stream-ordered launches (the reference's per-call PDL switch)."""
    cfg, w, ow = layer("mid")
    for m in (3, 16, 40):
        x, ids, wts = inputs(cfg, m, 7000 + m)
        a = run(w, x, ids, wts).clone()
        b = w.forward(x.cuda(), ids.cuda(), wts.cuda(), pdl=False)
        w.status()
        assert torch.equal(a, b)


def test_activation_range_is_reported_not_clipped_silently():
    """The FC1 -> FC2 activations are expanded with a fixed first-term scale: block maxima above 2688 / scale are clipped, and
    the status call says so; with a scale that covers the range the same input meets the bar again."""
    import sm120fp4_b200._lib as L
    cfg, w, ow = layer("tiny")
    x, ids, wts = inputs(cfg, 6, 77)
    x = (x.float() * 250.0).to(torch.bfloat16)
    try:
        w.forward(x.cuda(), ids.cuda(), wts.cuda())
        with pytest.raises(L.B200MoEError) as ei:
            w.status()
        assert ei.value.code == L.ERR_RANGE
        w.status()                                   # the flag is cleared by the read
        w.set_act_scale(8.0 / 4096.0)
        out = run(w, x, ids, wts)
        check_layer_output(out, O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy()), "large activations, wider scale")
    finally:
        w.set_act_scale(8.0)


def test_fifty_calls_are_bit_identical():
    """The reference's determinism check (sm120fp4/kernels/moe_layer.py:177-181): 50 calls, one result."""
    for name, m, routing in (("qwen", 16, "random"), ("qwen", 1, "fixed8"), ("mid", 7, "random")):
        cfg, w, _ = layer(name)
        x, ids, wts = inputs(cfg, m, 123, routing)
        xd, idd, wd = x.cuda(), ids.cuda(), wts.cuda()
        first = w.forward(xd, idd, wd).clone()
        for _ in range(50):
            assert torch.equal(w.forward(xd, idd, wd), first), f"{name} m={m}"
        w.status()


def test_released_checkpoint_layout_keeps_the_tensor_core_paths():
    import sm120fp4_b200._lib as L
    from helpers import make_layer
    cfg = SHAPES["mid"]
    w, ow = make_layer(cfg["experts"], cfg["hidden"], cfg["inter"], cfg["top_k"], seed=21)
    x, ids, wts = inputs(cfg, 12, 5)
    a = run(w, x, ids, wts).clone()
    w.release_checkpoint_layout()
    assert w.q1 is None
    assert torch.equal(run(w, x, ids, wts), a)
    with pytest.raises(L.B200MoEError):
        w.set_decode_impl("mma")
    with pytest.raises(L.B200MoEError):
        w.fc1(x.cuda(), ids.cuda(), wts.cuda(), torch.empty(12 * cfg["top_k"], cfg["inter"], dtype=torch.bfloat16, device="cuda"))
    x2, ids2, wts2 = inputs(cfg, 100, 6)
    w.enable_prefill(max_tokens=128)
    out = w.forward(x2.cuda(), ids2.cuda(), wts2.cuda())
    w.prefill_status()
    from helpers import check_w4a4_output
    check_w4a4_output(out, O.moe_reference(x2.float().numpy(), ow, ids2.numpy(), wts2.numpy(), act_quant=True), "prefill after release")


@pytest.mark.parametrize("name,m,routing", [("tiny", 3, "random"), ("mid", 8, "random"), ("mid", 16, "fixed8"), ("odd", 5, "random"),
                                            ("qwen", 1, "random"), ("qwen", 16, "random"), ("qwen", 4, "fixed8"), ("gemma", 8, "random")])
def test_decode_conformance_gate_without_a_tolerance(name, m, routing):
    """The interval gate (the reference's distinctive quality bar: sm120fp4/oracle.py:96-183, sm120fp4/moe_oracle.py:82-150)
    with this kernel's rounding points, on the operands the call left in its workspace."""
    from helpers import check_decode_call
    cfg, w, ow = layer(name)
    w.set_decode_impl("tcgen05")
    try:
        x, ids, wts = inputs(cfg, m, 8100 + m, routing)
        out = run(w, x, ids, wts)
        r = check_decode_call(w, ow, x, ids, wts, out, f"{name} m={m} {routing}")
        print(f"{name} m={m} {routing}: x residual {r['x_residual_over_bound']:.2f} of its bound, activations {r['activation_excess_over_slack']:.2f} "
              f"of the slack beyond the interval, output {r['out_err_over_bound']:.2f} of its bound ({r['out_max_abs_over_rms_own_operands']:.2e} x rms)")
    finally:
        w.set_decode_impl("auto")
