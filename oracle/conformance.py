"""Exact and interval oracles for NVFP4 GEMMs, quantizers and the fused MoE layer: TEST INFRASTRUCTURE, not product code.

A numpy restatement of the reference's tolerance-free conformance harness: sm120fp4/oracle.py:96-252 (exact GEMM values,
the bound an fp32-accumulating kernel must respect, `conformance`, `quantizer_conformance` with ties reported apart),
sm120fp4/moe_oracle.py:82-150 and sm120fp4/moe_oracle_w4a4.py:84-236 (a fused layer has no single exact value: the oracle
follows the rounding points of the kernel it judges and carries, at each, the interval of values a correct implementation
can produce). The rounding points modelled here are those of THIS library's kernels:

  W4A4 (prefill)   x -> NVFP4 by the reference's quantiser (exact: x is bf16) -> FC1 in fp32 on the tensor cores -> alpha /
                   gs in fp32 -> SiLU*mul in fp32 with a fast exponential and division, NO bf16 rounding -> NVFP4 again
                   (set-valued where the fp32 value straddles a rounding boundary) -> FC2 in fp32 -> alpha * routing
                   weight -> one bf16 row per (token, expert) -> fp32 sum over the slots in slot order -> bf16.
  W4A16 (decode)   x -> a sum of four NVFP4 terms (residual expansion) -> FC1 per term in fp32, the four columns added
                   with their 1/g_t -> SiLU*mul * routing weight * alpha2 (relative) in fp32 -> four NVFP4 terms with a
                   fixed first scale -> FC2 over all experts in one fp32 accumulation -> partial sums added in a fixed
                   order -> one bf16 rounding.

Products of E2M1 codes and E4M3 scales are exact in float64 (<= 16 significant bits each side, sm120fp4/oracle.py:12-24);
the unit of the fp32 accumulation bound is 2^-23 because tensor cores accumulate with truncation (sm120fp4/oracle.py:61-66).
Parity pin: the exact-GEMM and quantizer-conformance functions are held to the known answers of the reference's own
selftest (sm120fp4/oracle.py:255-351: flipped code, dropped block partial, the 112|120 scale tie, grouped == dense) by
tests/test_conformance_cpu.py.
"""
from __future__ import annotations

import math

import numpy as np

from . import nvfp4_oracle as O

U32 = 2.0 ** -23
U64 = 2.0 ** -53
BLOCK = 16
_MANT = {"bf16": 7, "f16": 10, "f32": 23, "f64": 52}
_TINY = {"bf16": 2.0 ** -126, "f16": 2.0 ** -14, "f32": 2.0 ** -126, "f64": 2.0 ** -1022}


def gamma(k: int) -> float:
    """Higham's gamma_K at the truncation unit: K u / (1 - K u) (sm120fp4/oracle.py:69-76)."""
    ku = k * U32
    if ku >= 1.0:
        raise ValueError(f"K = {k} is too large for a meaningful fp32 accumulation bound")
    return ku / (1.0 - ku)


def ulp(x: np.ndarray, dtype: str) -> np.ndarray:
    """Spacing of `dtype` at |x|; subnormals take the smallest normal spacing (sm120fp4/oracle.py:79-86)."""
    ax = np.maximum(np.abs(np.asarray(x, dtype=np.float64)), _TINY[dtype])
    return np.exp2(np.floor(np.log2(ax)) - _MANT[dtype])


def round_bf16(x: np.ndarray) -> np.ndarray:
    """float64 -> nearest-even bf16 (through fp32, as a kernel's cvt.rn.bf16.f32 of an fp32 value does) -> float64."""
    return O._bf16_round(np.asarray(x, dtype=np.float64).astype(np.float32)).astype(np.float64)


# ------------------------------------------------------------------------------------------------ exact GEMMs
def scaled_operand(packed: np.ndarray, sf_bits: np.ndarray, block: int = BLOCK) -> np.ndarray:
    """2q * sf as float64 [rows, K]: integers times powers of two, exact (sm120fp4/oracle.py:89-94)."""
    codes = O.unpack_e2m1(packed)
    rows, k = codes.shape
    twoq = 2.0 * O.e2m1_decode(codes).astype(np.float64)
    sf = O.e4m3_decode(np.asarray(sf_bits).reshape(rows, k // block)).astype(np.float64)
    return (twoq.reshape(rows, k // block, block) * sf[:, :, None]).reshape(rows, k)


def dequant_exact(packed, sf_bits, gs, block: int = BLOCK) -> np.ndarray:
    """q * sf / gs as float64 (one float64 rounding in the division)."""
    return scaled_operand(packed, sf_bits, block) / (2.0 * float(np.asarray(gs, dtype=np.float64).reshape(())))


def _gemm_bound(s, sabs, inv, k, out_dtype):
    exact = s * inv
    sum_abs = sabs * inv
    bound = gamma(k) * sum_abs + 0.5 * ulp(exact, out_dtype) + 2 * U64 * np.abs(exact) + k * U64 * sum_abs
    return exact, bound


def exact_gemm_nvfp4(a_packed, a_sf, a_gs, b_packed, b_sf, b_gs, out_dtype: str = "bf16", block: int = BLOCK):
    """Exact C[M, N] = dequant(A) @ dequant(B)^T and the per-element bound of an fp32-accumulating kernel writing
    `out_dtype` (sm120fp4/oracle.py:97-122)."""
    sa, sb = scaled_operand(a_packed, a_sf, block), scaled_operand(b_packed, b_sf, block)
    if sa.shape[1] != sb.shape[1]:
        raise ValueError(f"K must match: {sa.shape} vs {sb.shape}")
    inv = 1.0 / (4.0 * float(np.asarray(a_gs, dtype=np.float64).reshape(())) * float(np.asarray(b_gs, dtype=np.float64).reshape(())))
    return _gemm_bound(sa @ sb.T, np.abs(sa) @ np.abs(sb).T, inv, sa.shape[1], out_dtype)


def exact_gemm_bf16_nvfp4(a_bf16, b_packed, b_sf, b_gs, out_dtype: str = "bf16", block: int = BLOCK):
    """W4A16: A holds bf16 values (exact in float64), B is NVFP4 (sm120fp4/oracle.py:125-143)."""
    a = np.asarray(a_bf16, dtype=np.float64)
    sb = scaled_operand(b_packed, b_sf, block)
    if a.shape[1] != sb.shape[1]:
        raise ValueError(f"K must match: {a.shape} vs {sb.shape}")
    inv = 1.0 / (2.0 * float(np.asarray(b_gs, dtype=np.float64).reshape(())))
    return _gemm_bound(a @ sb.T, np.abs(a) @ np.abs(sb).T, inv, a.shape[1], out_dtype)


def exact_grouped_gemm_nvfp4(a_packed, a_sf, a_gs, b_packed, b_sf, b_gs, m_indptr, out_dtype: str = "bf16", block: int = BLOCK):
    """Rows m_indptr[e]:m_indptr[e+1] of A against expert e's B[e] (sm120fp4/oracle.py:146-170)."""
    m_indptr = [int(v) for v in np.asarray(m_indptr).reshape(-1)]
    e_count = b_packed.shape[0]
    if len(m_indptr) != e_count + 1:
        raise ValueError(f"m_indptr has {len(m_indptr)} entries for {e_count} experts")
    n = b_packed.shape[1]
    exact = np.zeros((m_indptr[-1], n))
    bound = np.zeros((m_indptr[-1], n))
    gs_b = np.asarray(b_gs, dtype=np.float64).reshape(-1)
    for e in range(e_count):
        lo, hi = m_indptr[e], m_indptr[e + 1]
        if hi <= lo:
            continue
        g = gs_b[e] if gs_b.size == e_count else gs_b[0]
        exact[lo:hi], bound[lo:hi] = exact_gemm_nvfp4(a_packed[lo:hi], a_sf[lo:hi], a_gs, b_packed[e], b_sf[e], g, out_dtype, block)
    return exact, bound


def conformance(kernel_out, exact, bound) -> dict:
    """Kernel output against the exact value under the bound; every number a report needs, no threshold
    (sm120fp4/oracle.py:173-190)."""
    k = np.asarray(kernel_out, dtype=np.float64)
    err = np.abs(k - exact)
    finite = np.isfinite(k)
    outside = err > bound
    ratio = np.where(bound > 0, err / np.where(bound > 0, bound, 1.0), 0.0)
    return {"elements": int(err.size), "non_finite": int((~finite).sum()), "outside_bound": int(outside.sum()),
            "max_err_over_bound": float(ratio.max()) if ratio.size else 0.0, "max_abs_err": float(err.max()) if err.size else 0.0,
            "all_zero_output": bool((k == 0).all()) if k.size else False, "conformant": bool(finite.all() and not outside.any())}


# ------------------------------------------------------------------------------------------------ quantizer conformance
_E4M3_POS = np.unique(O.E4M3_TABLE[:127][np.isfinite(O.E4M3_TABLE[:127])])      # every non-negative E4M3 value, ascending
_E4M3_POS_NZ = _E4M3_POS[_E4M3_POS > 0]
_E2M1_MIDS = ((O.E2M1_GRID[1:] + O.E2M1_GRID[:-1]) / 2).astype(np.float32)


def _e4m3_neighbours(v: np.ndarray):
    idx = np.searchsorted(_E4M3_POS_NZ, v.reshape(-1))
    lo = _E4M3_POS_NZ[np.clip(idx - 1, 0, None)].reshape(v.shape)
    hi = _E4M3_POS_NZ[np.clip(idx, None, _E4M3_POS_NZ.size - 1)].reshape(v.shape)
    return lo, hi


def quantizer_conformance(x, packed, sf_bits, gs, block: int = BLOCK) -> dict:
    """A library quantizer's codes and scales against the format's definition (the oracle's quantize_nvfp4 with the
    library's own global scale), ties reported apart for scales and for codes (sm120fp4/oracle.py:193-252)."""
    x = np.asarray(x, dtype=np.float32)
    gsf = np.float32(np.asarray(gs, dtype=np.float32).reshape(()))
    ref_packed, ref_sf, _ = O.quantize_nvfp4(x, np.array([gsf], dtype=np.float32), block)
    codes, ref_codes = O.unpack_e2m1(np.asarray(packed)), O.unpack_e2m1(ref_packed)
    rows = x.shape[0]
    sf_lib, sf_ref = np.asarray(sf_bits, dtype=np.uint8).reshape(rows, -1), ref_sf.reshape(rows, -1)
    sf_diff = sf_lib != sf_ref
    xm = x.reshape(rows, -1, block)
    sf_f32 = ((np.abs(xm).max(axis=-1) / O.E2M1_MAX).astype(np.float32) * gsf).astype(np.float32)
    lo, hi = _e4m3_neighbours(sf_f32)
    tie = (sf_f32 == (lo + hi) / 2) & (lo < hi) & (sf_f32 > 0) & (sf_f32 < O.E4M3_MAX)
    lib_val, ref_val = O.e4m3_decode(sf_lib), O.e4m3_decode(sf_ref)
    neighbours = ((lib_val == lo) | (lib_val == hi)) & ((ref_val == lo) | (ref_val == hi))
    sf_diff_tie = sf_diff & tie & neighbours
    sf_diff_other = sf_diff & ~sf_diff_tie
    with np.errstate(divide="ignore", invalid="ignore"):
        scale = np.where(lib_val > 0, (gsf / lib_val).astype(np.float32), np.float32(0))
    y = np.abs((xm * scale[..., None]).astype(np.float32)).reshape(rows, -1)
    ulp_y = np.finfo(np.float32).eps * np.maximum(y, np.finfo(np.float32).tiny)
    at_tie = (np.abs(y[..., None] - _E2M1_MIDS) <= 2 * ulp_y[..., None]).any(axis=-1)
    in_tie_block = np.repeat(sf_diff_tie, block, axis=1)
    diff = codes != ref_codes
    bad_codes = diff & ~at_tie & ~in_tie_block
    return {"elements": int(codes.size), "blocks": int(sf_diff.size), "scales_differ": int(sf_diff.sum()),
            "scales_differ_at_tie": int(sf_diff_tie.sum()), "scales_differ_not_at_tie": int(sf_diff_other.sum()),
            "scales_identical": bool(not sf_diff.any()), "codes_differ": int(diff.sum()),
            "codes_differ_at_tie": int((diff & at_tie & ~in_tie_block).sum()),
            "codes_differ_in_scale_tie_blocks": int((diff & in_tie_block).sum()), "codes_differ_not_at_tie": int(bad_codes.sum()),
            "conformant": int(sf_diff_other.sum()) == 0 and int(bad_codes.sum()) == 0}


# ------------------------------------------------------------------------------------------------ set-valued quantiser
def _block_scale_f32(amax_f32: np.ndarray, gs: np.float32) -> np.ndarray:
    """The reference quantiser's block scale as an E4M3 VALUE (fp32): e4m3(min(amax / 6 * gs, 448))."""
    sf = np.minimum((amax_f32.astype(np.float32) / O.E2M1_MAX).astype(np.float32) * gs, O.E4M3_MAX).astype(np.float32)
    return O.e4m3_decode(O.e4m3_encode(sf))


def _codes_as_values(v_f32: np.ndarray, sf_val: np.ndarray, gs: np.float32) -> np.ndarray:
    """E2M1 codes (as signed values) of v under block scale value sf_val [.., 1]: e2m1(v * (gs / sf)); 0 where sf == 0."""
    with np.errstate(divide="ignore", invalid="ignore"):
        scale = np.where(sf_val > 0, (gs / sf_val).astype(np.float32), np.float32(0)).astype(np.float32)
    return O.e2m1_decode(O.e2m1_encode((v_f32 * scale).astype(np.float32)))


def requantised_membership(lo: np.ndarray, hi: np.ndarray, packed: np.ndarray, sf_bits: np.ndarray, gs: float = 1.0,
                           nominal: np.ndarray | None = None, block: int = BLOCK) -> dict:
    """Is a kernel's NVFP4 re-quantisation (packed codes, scale bytes) of a row a value the reference quantiser can produce
    from SOME input inside [lo, hi] (float64 [rows, K]: the interval of values a correct fp32 computation can hold)?

    The block maximum lies between the maxima of the two ends, and the scale is monotone in it: the kernel's scale byte
    must lie between the scales of the two ends. Under the kernel's own scale every code is monotone in its value: the
    kernel's code must lie between the codes of the two ends (the method of block_quantize_interval,
    sm120fp4/moe_oracle_w4a4.py:84-112, used as a membership test). With `nominal` (the mid-interval value, float64) the
    differences against the quantisation of the nominal value are counted as `flips` - every flip that passes membership
    sits within the interval's half-width of a rounding boundary, which is what distinguishes a tie from a defect."""
    rows, k = lo.shape
    gsf = np.float32(gs)
    blo, bhi = lo.astype(np.float32).reshape(rows, k // block, block), hi.astype(np.float32).reshape(rows, k // block, block)
    mag_hi = np.maximum(np.abs(blo), np.abs(bhi))
    mag_lo = np.where((blo <= 0) & (bhi >= 0), np.float32(0), np.minimum(np.abs(blo), np.abs(bhi)))
    s_a = _block_scale_f32(mag_lo.max(axis=-1), gsf)
    s_b = _block_scale_f32(mag_hi.max(axis=-1), gsf)
    sf_k = O.e4m3_decode(np.asarray(sf_bits, dtype=np.uint8).reshape(rows, k // block))
    scale_ok = (sf_k >= s_a) & (sf_k <= s_b)
    codes_k = O.e2m1_decode(O.unpack_e2m1(np.asarray(packed))).reshape(rows, k // block, block)
    c_lo = _codes_as_values(blo, sf_k[..., None], gsf)
    c_hi = _codes_as_values(bhi, sf_k[..., None], gsf)
    code_ok = (codes_k >= np.minimum(c_lo, c_hi)) & (codes_k <= np.maximum(c_lo, c_hi))
    # the sign of a zero code: the kernel keeps the sign bit of the value; either sign is a correct rounding when the
    # interval contains zero, and a zero-scale block encodes every value as +-0
    out = {"blocks": int(scale_ok.size), "elements": int(code_ok.size), "scale_outside": int((~scale_ok).sum()),
           "code_outside": int((~code_ok & scale_ok[..., None]).sum()), "ambiguous_blocks": int((s_a != s_b).sum())}
    if nominal is not None:
        nom = np.asarray(nominal, dtype=np.float64).astype(np.float32).reshape(rows, k // block, block)
        s_n = _block_scale_f32(np.abs(nom).max(axis=-1), gsf)
        c_n = _codes_as_values(nom, s_n[..., None], gsf)
        out["scale_flips"] = int((s_n != sf_k).sum())
        out["code_flips"] = int(((c_n != codes_k) & (s_n == sf_k)[..., None]).sum())
        # how far a flipped code's pre-rounding value sits from the nearest rounding boundary, in units of the interval's
        # half-width: <= 1 for every flip that passed membership
        flipped = (c_n != codes_k) & (s_n == sf_k)[..., None] & code_ok
        if flipped.any():
            with np.errstate(divide="ignore", invalid="ignore"):
                scale = np.where(sf_k > 0, gsf / sf_k, 0.0)[..., None]
            y = np.abs(nom.astype(np.float64) * scale)
            dist = np.abs(y[..., None] - _E2M1_MIDS.astype(np.float64)).min(axis=-1)
            half = (np.abs(bhi.astype(np.float64) - blo.astype(np.float64)) / 2.0) * scale
            out["max_flip_distance_over_halfwidth"] = float((dist[flipped] / np.maximum(half[flipped], 1e-300)).max())
    out["conformant"] = out["scale_outside"] == 0 and out["code_outside"] == 0
    return out


# ------------------------------------------------------------------------------------------------ layer building blocks
SILU_MIN_X = -1.2784645427610738                       # argmin of x * sigmoid(x) (sm120fp4/moe_oracle.py:47-48)
SILU_MIN = SILU_MIN_X / (1.0 + math.exp(-SILU_MIN_X))
FAST_MATH_REL = 2.0 ** -20                              # ex2.approx, the fast division and the fp32 multiplies, generously


def silu64(x: np.ndarray) -> np.ndarray:
    return x / (1.0 + np.exp(-x))


def hull_silu(lo, hi):
    """Range of silu over [lo, hi] (sm120fp4/moe_oracle.py:56-62)."""
    a, b = silu64(lo), silu64(hi)
    smin, smax = np.minimum(a, b), np.maximum(a, b)
    straddles = (lo <= SILU_MIN_X) & (hi >= SILU_MIN_X)
    return np.where(straddles, SILU_MIN, smin), smax


def hull_prod(alo, ahi, blo, bhi):
    c = np.stack([alo * blo, alo * bhi, ahi * blo, ahi * bhi])
    return c.min(axis=0), c.max(axis=0)


def interval_gemm(alo, ahi, w):
    """A in [alo, ahi] against exact W [N, K]: (mid product, bound = half-width through |W| + the fp32 accumulation bound +
    float64 slack, sum of absolute products) (sm120fp4/moe_oracle_w4a4.py:122-131)."""
    mid, hw = (alo + ahi) / 2.0, (ahi - alo) / 2.0
    k = w.shape[1]
    c = mid @ w.T
    cabs = np.abs(mid) @ np.abs(w).T
    return c, hw @ np.abs(w).T + gamma(k) * cabs + (2.0 + k) * U64 * cabs, cabs


def fc1_activation_interval(xq: np.ndarray, w1d: np.ndarray, inter: int, extra_rel: float = 0.0, xabs: np.ndarray | None = None):
    """The interval [lo, hi] of a = silu(gate) * up for rows xq (float64, exact operand values) against one expert's
    dequantised FC1 weights w1d [2I, H] (rows [up ; gate], alpha folded in), when FC1 is accumulated in fp32 in any order
    and SiLU*mul is evaluated in fp32 with fast math and no intermediate rounding (this library's FC1 epilogues).
    Returns (lo, hi, nominal)."""
    f, fb, cabs = interval_gemm(xq, xq, w1d)
    if xabs is not None:   # the operand is a sum of terms accumulated separately: the bound runs over the terms' magnitudes
        cabs = np.asarray(xabs, dtype=np.float64) @ np.abs(w1d).T
        fb = gamma(w1d.shape[1]) * cabs + (2.0 + w1d.shape[1]) * U64 * cabs + 8 * U32 * cabs
    fb = fb + 4 * U32 * np.abs(f) + extra_rel * np.abs(f)       # the alpha / gs multiplies in fp32
    up, bu, gate, bg = f[:, :inter], fb[:, :inter], f[:, inter:], fb[:, inter:]
    slo, shi = hull_silu(gate - bg, gate + bg)
    gabs = np.abs(gate) + bg
    slack = (FAST_MATH_REL + gabs * 2.0 ** -22) * (np.maximum(np.abs(slo), np.abs(shi)) + gabs)
    plo, phi = hull_prod(slo - slack, shi + slack, up - bu, up + bu)
    w = 2 * U32 * np.maximum(np.abs(plo), np.abs(phi))          # the product's own fp32 rounding
    return plo - w, phi + w, silu64(gate) * up


def w4a4_layer_oracle(x_bf16: np.ndarray, w: O.ExpertWeights, ids: np.ndarray, wts: np.ndarray, gs_in: float = 1.0,
                      gs_mid: float = 1.0) -> dict:
    """Interval oracle of the W4A4 layer with this library's rounding points (module docstring). Returns {"nominal",
    "bound", "abs_contrib", "ambiguous_blocks"}; an output y is conformant when |y - nominal| <= bound everywhere.
    Modelled on fused_moe_w4a4_oracle (sm120fp4/moe_oracle_w4a4.py:134-236) with the exact (not the fast) quantiser and
    this library's combine: one bf16 row per (token, expert), fp32 sum in slot order, one bf16 rounding."""
    x = np.asarray(x_bf16, dtype=np.float32)
    ids, wts = np.asarray(ids), np.asarray(wts, dtype=np.float32)
    m, k = ids.shape
    one = np.array([gs_in], dtype=np.float32)
    xp, xs, _ = O.quantize_nvfp4(x, one)
    xq = dequant_exact(xp, xs, gs_in)
    out = np.zeros((m, w.H))
    bound = np.zeros((m, w.H))
    abs_contrib = np.zeros((m, w.H))
    amb = 0
    for e in sorted(set(int(v) for v in ids.reshape(-1) if v >= 0)):
        tok, slot = np.nonzero(ids == e)
        w1d = dequant_exact(w.q1[e], w.s1[e].reshape(2 * w.I, w.H // BLOCK), 1.0) * float(w.alpha1[e])
        w2d = dequant_exact(w.q2[e], w.s2[e].reshape(w.H, w.I // BLOCK), 1.0) * float(w.alpha2[e])
        lo, hi, _ = fc1_activation_interval(xq[tok], w1d, w.I)
        qlo, qhi, a = block_quantize_interval(lo, hi, gs_mid)
        amb += a
        c, cb, _ = interval_gemm(qlo, qhi, w2d)
        wf = wts[tok, slot].astype(np.float64)[:, None]
        r_lo, r_hi = _round_bf16_interval((c - cb) * wf, (c + cb) * wf, 4 * U32)   # alpha * weight multiply, then the bf16 row
        contrib, cbound = (r_lo + r_hi) / 2.0, (r_hi - r_lo) / 2.0
        np.add.at(out, tok, contrib)
        np.add.at(bound, tok, cbound)
        np.add.at(abs_contrib, tok, np.abs(contrib) + cbound)
    pre = bound + k * U32 * abs_contrib + 2.0 * U64 * abs_contrib
    return {"nominal": out, "bound": pre + 0.5 * ulp(np.abs(out) + pre, "bf16"), "abs_contrib": abs_contrib, "ambiguous_blocks": amb}


def _round_bf16_interval(lo, hi, rel: float = 0.0):
    """The bf16 values a correct rounding of any value in [lo, hi] (widened by `rel` relative and one fp32 ulp) can give
    (sm120fp4/moe_oracle.py:70-78)."""
    mag = np.maximum(np.abs(lo), np.abs(hi))
    wd = ulp(mag, "f32") + rel * mag
    a, b = round_bf16(lo - wd), round_bf16(hi + wd)
    return np.minimum(a, b), np.maximum(a, b)


def block_quantize_interval(lo: np.ndarray, hi: np.ndarray, gs: float = 1.0, block: int = BLOCK):
    """Set-valued quantisation of values in [lo, hi] by the reference quantiser: for every scale candidate between the
    scales of the two ends, the dequantised codes of both ends; the hull is the element's interval. Returns (vlo, vhi,
    ambiguous blocks) (sm120fp4/moe_oracle_w4a4.py:84-112)."""
    rows, k = lo.shape
    gsf = np.float32(gs)
    blo, bhi = lo.astype(np.float32).reshape(rows, k // block, block), hi.astype(np.float32).reshape(rows, k // block, block)
    mag_hi = np.maximum(np.abs(blo), np.abs(bhi))
    mag_lo = np.where((blo <= 0) & (bhi >= 0), np.float32(0), np.minimum(np.abs(blo), np.abs(bhi)))
    s_a = _block_scale_f32(mag_lo.max(axis=-1), gsf)[..., None]
    s_b = _block_scale_f32(mag_hi.max(axis=-1), gsf)[..., None]
    vlo = np.full(blo.shape, np.inf)
    vhi = np.full(blo.shape, -np.inf)
    cands = _E4M3_POS[(_E4M3_POS >= s_a.min()) & (_E4M3_POS <= s_b.max())]
    for g in cands:
        use = (s_a <= g) & (g <= s_b)
        if not use.any():
            continue
        s = np.full(s_a.shape, np.float32(g))
        for v in (blo, bhi):
            c = _codes_as_values(v, s, gsf).astype(np.float64) * float(g) / float(gs)
            vlo = np.where(use, np.minimum(vlo, c), vlo)
            vhi = np.where(use, np.maximum(vhi, c), vhi)
    return vlo.reshape(rows, k), vhi.reshape(rows, k), int((s_a != s_b).sum())


# ------------------------------------------------------------------------------------------------ W4A16 term expansion
EXPANSION_TERMS = 4
# Residual of the expansion of a 16-value block into four NVFP4 terms, relative to the block maximum: every term leaves at
# most one E2M1 step at the top of its range times its (rounded-up) block scale, (1 + 1/16) / 6 of what it was given.
EXPANSION_RESIDUAL = ((1.0 + 1.0 / 16.0) / 6.0) ** EXPANSION_TERMS


def expansion_value(codes: np.ndarray, sf_bits: np.ndarray, g1: np.ndarray, block: int = BLOCK):
    """The value a four-term operand stands for, and the sum of its terms' magnitudes. codes u8 [terms, rows, K/2] packed
    E2M1, sf_bits u8 [terms, rows, K/16], g1 [rows] (or scalar): first-term global scale; term t carries g1 * 6^t."""
    terms = codes.shape[0]
    g = np.asarray(g1, dtype=np.float64).reshape(-1, 1)
    val = 0.0
    mag = 0.0
    for t in range(terms):
        v = scaled_operand(codes[t], sf_bits[t], block) / (2.0 * g * 6.0 ** t)
        val = val + v
        mag = mag + np.abs(v)
    return val, mag
