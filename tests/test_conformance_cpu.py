"""The exact / interval oracle harness (oracle/conformance.py) against vectors produced by the reference's own oracle
(sm120fp4/oracle.py) and against the known answers of its selftest (sm120fp4/oracle.py:255-351,
sm120fp4/moe_oracle_w4a4.py:289-345): what a conformant kernel looks like, and which faults fall outside the bound."""
import numpy as np
import pytest

from oracle import conformance as C
from oracle import nvfp4_oracle as O


@pytest.fixture(scope="module")
def g(golden):
    return golden.load("conformance")


@pytest.mark.parametrize("i", [0, 1, 2])
def test_exact_gemm_and_bound_equal_the_reference_oracle(g, i):
    exact, bound = C.exact_gemm_nvfp4(g[f"g{i}_ap"], g[f"g{i}_asf"], g[f"g{i}_ags"], g[f"g{i}_bp"], g[f"g{i}_bsf"], g[f"g{i}_bgs"])
    assert np.array_equal(exact, g[f"g{i}_exact"])
    np.testing.assert_allclose(bound, g[f"g{i}_bound"], rtol=1e-12, atol=0)
    e16, b16 = C.exact_gemm_bf16_nvfp4(g[f"g{i}_a_bf16"], g[f"g{i}_bp"], g[f"g{i}_bsf"], g[f"g{i}_bgs"])
    assert np.array_equal(e16, g[f"g{i}_exact16"])
    np.testing.assert_allclose(b16, g[f"g{i}_bound16"], rtol=1e-12, atol=0)


@pytest.mark.parametrize("i", [0, 1, 2])
def test_fp32_reference_inside_faults_outside(g, i):
    ap, asf, ags, bp, bsf, bgs = (g[f"g{i}_{n}"] for n in ("ap", "asf", "ags", "bp", "bsf", "bgs"))
    exact, bound = C.exact_gemm_nvfp4(ap, asf, ags, bp, bsf, bgs)
    k = ap.shape[1] * 2
    # a correct fp32-accumulating implementation, rounded to bf16, is inside the bound
    ref = (O.dequantize_nvfp4(ap, asf, ags) @ O.dequantize_nvfp4(bp, bsf, bgs).T).astype(np.float32)
    v = C.conformance(C.round_bf16(ref), exact, bound)
    assert v["conformant"], v
    # the exact value agrees with an independent term-by-term sum
    sa, sb = C.scaled_operand(ap, asf), C.scaled_operand(bp, bsf)
    s0 = sum(float(sa[0, kk]) * float(sb[0, kk]) for kk in range(k))
    e0 = s0 / (4.0 * float(ags[0]) * float(bgs[0]))
    assert abs(e0 - exact[0, 0]) <= 4 * C.U64 * abs(e0) + 1e-300
    # one wrong operand code: visible at K <= 1024, below the fp32 floor at K = 4096 (sm120fp4/oracle.py:37-46)
    bad = ap.copy()
    bad[0, 0] ^= 0x07
    wrong, _ = C.exact_gemm_nvfp4(bad, asf, ags, bp, bsf, bgs)
    v3 = C.conformance(C.round_bf16(wrong), exact, bound)
    if k <= 1024:
        assert v3["outside_bound"] >= 1 and not v3["conformant"]
    # a lost 16-wide block partial is caught at every K
    lost = exact.copy()
    lost[1] -= (sa[1, :16][None, :] * sb[:, :16]).sum(axis=1) / (4.0 * float(ags[0]) * float(bgs[0]))
    assert C.conformance(C.round_bf16(lost), exact, bound)["outside_bound"] >= 1
    # the quantizer check accepts the reference quantizer's output and rejects a changed code
    q = C.quantizer_conformance(g[f"g{i}_a"], ap, asf, ags)
    assert [q["codes_differ"], q["scales_differ"], int(q["conformant"])] == list(g[f"g{i}_qconf"])
    q2 = C.quantizer_conformance(g[f"g{i}_a"], bad, asf, ags)
    assert not q2["conformant"] and q2["codes_differ_not_at_tie"] >= 1


def test_scale_tie_is_a_tie_and_a_moved_scale_is_a_defect(g):
    """x = 2.265625, gs = 307.2: the fp32 scale 116 sits midway between the E4M3 values 112 and 120 (sm120fp4/oracle.py:302-314)."""
    x, gs = np.full((1, 16), 2.265625, dtype=np.float32), np.array([307.2], dtype=np.float32)
    p, sf, _ = O.quantize_nvfp4(x, gs)
    assert np.array_equal(sf, g["tie_ref_sf"]) and np.array_equal(p, g["tie_ref_packed"])
    up = sf.copy()
    up[0, 0] = O.e4m3_encode(np.array([120.0], dtype=np.float32))[0]
    qt = C.quantizer_conformance(x, g["tie_up_packed"], up, gs)
    assert [qt["scales_differ_at_tie"], qt["scales_differ_not_at_tie"], int(qt["conformant"])] == list(g["tie_up_verdict"]) == [1, 0, 1]
    off = sf.copy()
    off[0, 0] = O.e4m3_encode(np.array([128.0], dtype=np.float32))[0]
    qo = C.quantizer_conformance(x, p, off, gs)
    assert [qo["scales_differ_at_tie"], qo["scales_differ_not_at_tie"], int(qo["conformant"])] == list(g["tie_off_verdict"]) == [0, 1, 0]


def test_grouped_oracle_equals_the_dense_one_and_catches_a_misrouted_expert(g):
    ap, asf, ags, bp, bsf, bgs, indptr = (g[f"grp_{n}"] for n in ("ap", "asf", "ags", "bp", "bsf", "bgs", "indptr"))
    ge, gb = C.exact_grouped_gemm_nvfp4(ap, asf, ags, bp, bsf, bgs, indptr)
    assert np.array_equal(ge, g["grp_exact"])
    np.testing.assert_allclose(gb, g["grp_bound"], rtol=1e-12)
    d2, _ = C.exact_gemm_nvfp4(ap[4:10], asf[4:10], ags, bp[2], bsf[2], bgs[2:3])
    swapped, _ = C.exact_gemm_nvfp4(ap[0:4], asf[0:4], ags, bp[1], bsf[1], bgs[1:2])
    assert not C.conformance(C.round_bf16(np.concatenate([swapped, d2])), ge, gb)["conformant"]


def _tiny_layer(seed=20261011, e_count=4, hdim=256, inter=128, m=6, topk=2):
    rng = np.random.default_rng(seed)
    one = np.ones(1, dtype=np.float32)
    x = O._bf16_round(rng.standard_normal((m, hdim)).astype(np.float32))
    w13 = [O.quantize_nvfp4((rng.standard_normal((2 * inter, hdim)) * 0.05).astype(np.float32), one) for _ in range(e_count)]
    w2 = [O.quantize_nvfp4((rng.standard_normal((hdim, inter)) * 0.05).astype(np.float32), one) for _ in range(e_count)]
    w = O.ExpertWeights(np.stack([q[0] for q in w13]), np.stack([q[1] for q in w13]), np.ones(e_count, np.float32),
                        np.stack([q[0] for q in w2]), np.stack([q[1] for q in w2]), np.ones(e_count, np.float32))
    ids = np.stack([rng.permutation(e_count)[:topk] for _ in range(m)]).astype(np.int32)
    wts = rng.random((m, topk)).astype(np.float32)
    wts = (wts / wts.sum(-1, keepdims=True)).astype(np.float32)
    return x, w, ids, wts


def _emulate_w4a4(x, w, ids, wts, gate_first=False, fault=None):
    """This library's W4A4 rounding points in fp32 numpy: quantised x, fp32 FC1, SiLU*mul in fp32, re-quantisation, fp32 FC2,
    one bf16 row per (token, expert), fp32 sum in slot order, bf16."""
    one = np.ones(1, dtype=np.float32)
    xp, xs, _ = O.quantize_nvfp4(x, one)
    xq = O.dequantize_nvfp4(xp, xs, one)
    out = np.zeros((x.shape[0], w.H), dtype=np.float32)
    for t in range(x.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            w1d, w2d = w.dequant(e)
            h = (xq[t:t + 1].astype(np.float64) @ w1d.astype(np.float64).T).astype(np.float32)
            gate, up = (h[:, :w.I], h[:, w.I:]) if gate_first else (h[:, w.I:], h[:, :w.I])
            a = (O.silu(gate) * up).astype(np.float32)
            ap, asf, _ = O.quantize_nvfp4(a, one)
            c = (O.dequantize_nvfp4(ap, asf, one).astype(np.float64) @ w2d.astype(np.float64).T).astype(np.float32)
            row = O._bf16_round((c * np.float32(wts[t, j])).astype(np.float32))
            if fault is not None:
                row = fault(row, e)
            out[t] += row[0]
    return O._bf16_round(out).astype(np.float64)


def test_w4a4_interval_oracle_accepts_the_faithful_emulation_and_rejects_faults():
    x, w, ids, wts = _tiny_layer()
    o = C.w4a4_layer_oracle(x, w, ids, wts)
    nominal, b = o["nominal"], o["bound"]
    assert np.isfinite(nominal).all() and np.isfinite(b).all() and (b > 0).all()
    y = _emulate_w4a4(x, w, ids, wts)
    assert (np.abs(y - nominal) <= b).all(), float((np.abs(y - nominal) / b).max())
    # the other half of w13 read as the gate: a wrong contract, outside nearly everywhere
    y_other = _emulate_w4a4(x, w, ids, wts, gate_first=True)
    assert (np.abs(y_other - nominal) > b).mean() > 0.9

    def drop_group(row, e):   # a lost 8-column group of expert 1's contribution
        r = row.copy()
        if e == 1:
            r[:, 64:72] = 0.0
        return r
    y3 = _emulate_w4a4(x, w, ids, wts, fault=drop_group)
    affected = (ids == 1).any(axis=1)
    assert (np.abs(y3 - nominal) > b)[affected][:, 64:72].mean() > 0.9

    def off_by(rel):
        return lambda row, e: row * np.float32(1.0 + rel) if e == 2 else row
    affected = (ids == 2).any(axis=1)
    y5 = _emulate_w4a4(x, w, ids, wts, fault=off_by(2.0 ** -3))
    assert (np.abs(y5 - nominal) > b)[affected].mean() > 0.5


def test_requantised_membership_separates_ties_from_defects():
    x, w, ids, wts = _tiny_layer(seed=7)
    one = np.ones(1, dtype=np.float32)
    xp, xs, _ = O.quantize_nvfp4(x, one)
    xq = C.dequant_exact(xp, xs, 1.0)
    e = int(ids[0, 0])
    w1d = C.dequant_exact(w.q1[e], w.s1[e], 1.0)
    lo, hi, nom = C.fc1_activation_interval(xq, w1d, w.I)
    assert (lo <= nom).all() and (nom <= hi).all()
    # the quantisation of an fp32 evaluation of the same activations is a member
    a32 = (O.silu((xq @ w1d[w.I:].T).astype(np.float32)) * (xq @ w1d[:w.I].T).astype(np.float32)).astype(np.float32)
    ap, asf, _ = O.quantize_nvfp4(a32, one)
    v = C.requantised_membership(lo, hi, ap, asf, 1.0, nominal=nom)
    assert v["conformant"], v
    assert v.get("max_flip_distance_over_halfwidth", 0.0) <= 1.0 + 1e-9
    # a code moved by one whole step where no boundary is near is a defect
    bad = ap.copy()
    codes = O.unpack_e2m1(bad)
    r, c = np.unravel_index(np.argmax(np.abs(a32)), a32.shape)
    codes[r, c] = (codes[r, c] & 0x8) | max((codes[r, c] & 0x7) - 2, 0)
    v2 = C.requantised_membership(lo, hi, O.pack_e2m1(codes), asf, 1.0, nominal=nom)
    assert not v2["conformant"] and v2["code_outside"] >= 1
    # a scale byte two steps off is a defect
    sf2 = asf.copy()
    sf2[r, c // 16] += 2
    assert C.requantised_membership(lo, hi, ap, sf2, 1.0)["scale_outside"] >= 1
