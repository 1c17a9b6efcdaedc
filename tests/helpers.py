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
    """W4A4 output against the plain fp32 oracle: reported, and held to the normwise bar only. The SiLU*mul activations are
    re-quantised to FP4 between the two GEMMs, so an activation whose fp32 value sits on a rounding boundary may take the
    neighbouring code; whether every such difference IS a boundary case, and the 2e-2 x RMS bar on the outputs given the
    kernel's own codes, is what check_prefill_call establishes."""
    g = got.float().cpu().numpy()
    assert np.isfinite(g).all(), f"{what}: non-finite output"
    rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
    err = np.abs(g - want)
    rel = float(np.linalg.norm(g - want) / max(np.linalg.norm(want), 1e-30))
    assert rel < 1e-2, f"{what}: normwise error {rel:.3e}"
    return float(err.max()) / rms, rel


# ---------------------------------------------------------------------------------------------------- prefill read-back
REC = 18432


def prefill_map(w, max_tokens: int) -> dict:
    import ctypes as C
    import sm120fp4_b200._lib as L
    buf = (C.c_longlong * 14)()
    L.check(L.lib().b200moe_prefill_workspace_map(w._h, int(max_tokens), buf), "prefill map")
    names = ("experts", "offsets", "pairs", "ntiles", "tile_expert", "tile_first", "tile_end", "row_pair", "dst_row", "xrec", "arec", "y",
             "max_tiles", "total")
    return dict(zip(names, [int(v) for v in buf]))


def _i32(ws: torch.Tensor, off: int, n: int) -> np.ndarray:
    return ws[off:off + 4 * n].view(torch.int32).cpu().numpy()


_r = np.arange(128)[:, None]
_CODE_IDX = (_r * 128 + (((np.arange(128)[None, :] >> 4) ^ (_r & 7)) << 4) + (np.arange(128)[None, :] & 15))          # [row, byte of the 128-byte row]
_b = np.arange(16)[None, :]
_SF_IDX = 16384 + (_b >> 2) * 512 + (_r & 31) * 16 + (_r >> 5) * 4 + (_b & 3)                                           # [row, 16-value block]


def read_records(ws: torch.Tensor, off: int, ntiles: int, kb: int):
    """Tile records [ntiles][kb][18432] -> (packed codes u8 [ntiles*128, kb*128], scale bytes u8 [ntiles*128, kb*16], raw)."""
    raw = ws[off:off + ntiles * kb * REC].cpu().numpy().reshape(ntiles, kb, REC)
    codes = raw[:, :, _CODE_IDX]            # [t, kb, row, 128]
    sf = raw[:, :, _SF_IDX]                 # [t, kb, row, 16]
    return (codes.transpose(0, 2, 1, 3).reshape(ntiles * 128, kb * 128), sf.transpose(0, 2, 1, 3).reshape(ntiles * 128, kb * 16), raw)


def check_prefill_call(w, ow, x, ids, wts, out, max_tokens, sample_tokens=None, what=""):
    """Stage-by-stage parity of one W4A4 prefill call that has just run on `w` (Weights with enable_prefill) against the
    oracle, from the workspace the call left behind:
      1. router tables bit-exact;
      2. the x records (codes and 128x4 scale tiles) byte-equal to oracle.quantize_nvfp4 + to_128x4 of the gathered rows;
      3. the re-quantised SiLU*mul activations: every scale byte and code a value the reference quantiser can produce from
         an input inside the fp32-accumulation interval of the exact activation (differences from the nominal quantisation
         are counted as flips and each must sit within that interval of a rounding boundary);
      4. the oracle's FC2 + combine computed from the KERNEL'S OWN activation codes against the kernel's output: bf16 max-abs
         error <= 2e-2 x output RMS with zero exceptions, and inside the exact accumulation bound.
    Returns a dict of the measured maxima."""
    from oracle import conformance as C
    m, k = ids.shape
    h, inter, e_n = ow.H, ow.I, ow.E
    kb1, kb2 = (h + 255) // 256, (inter + 255) // 256
    mp = prefill_map(w, max_tokens)
    ws = w.prefill.workspace
    idn, wn, xf = ids.numpy(), wts.numpy(), x.float().numpy()
    p = m * k
    umax = min(e_n, p)
    # ---- 1. router
    flat = idn.reshape(-1)
    live = np.nonzero(flat >= 0)[0]                        # empty slots (negative ids) appear in no table
    ex_l, off_l, order = O.route(flat[live])
    wex = np.full(umax, -1, dtype=np.int32)
    woff = np.full(umax + 1, live.size, dtype=np.int32)
    wex[: ex_l.size], woff[: off_l.size] = ex_l, off_l
    assert np.array_equal(_i32(ws, mp["experts"], umax), wex), f"{what}: experts"
    assert np.array_equal(_i32(ws, mp["offsets"], umax + 1), woff), f"{what}: offsets"
    assert np.array_equal(_i32(ws, mp["pairs"], p)[: live.size], live[order]), f"{what}: pairs"
    nt = int(_i32(ws, mp["ntiles"], 1)[0])
    counts = np.diff(woff[: (wex >= 0).sum() + 1])
    import os
    setting = os.environ.get("B200MOE_PREFILL_PAIR", "")
    if setting == "1" and kb1 <= 9:   # CTA pairs (opt-in): an even number of tiles per expert
        assert nt == int((2 * ((counts + 255) // 256)).sum()), f"{what}: tile count (pairs)"
    else:
        assert nt == int(((counts + 127) // 128).sum()), f"{what}: tile count"
    row_pair = _i32(ws, mp["row_pair"], nt * 128)
    tile_expert = _i32(ws, mp["tile_expert"], nt)
    valid = row_pair >= 0
    routed = np.nonzero(idn.reshape(-1) >= 0)[0]          # empty slots (negative ids) own no row
    assert np.array_equal(np.sort(row_pair[valid]), routed), f"{what}: every routed pair owns exactly one row"
    assert np.array_equal(idn.reshape(-1)[row_pair[valid]], np.repeat(tile_expert, 128)[valid]), f"{what}: rows sit in their expert's tiles"
    dst_row = _i32(ws, mp["dst_row"], p)
    assert np.array_equal(np.nonzero(valid)[0], np.sort(dst_row[routed])) and np.array_equal(row_pair[dst_row[routed]], routed)
    assert (dst_row[idn.reshape(-1) < 0] == -1).all(), f"{what}: empty slots must map to no row"
    # ---- 2. x records, byte for byte
    one = np.ones(1, dtype=np.float32) * np.float32(w.prefill.gs_x)
    qx, sx, _ = O.quantize_nvfp4(xf, one)
    codes, sfs, raw = read_records(ws, mp["xrec"], nt, kb1)
    tok_of_row = np.where(valid, row_pair // k, 0)
    assert np.array_equal(codes[valid][:, : h // 2], qx[tok_of_row[valid]]), f"{what}: x codes differ from the reference quantiser"
    assert np.array_equal(sfs[valid][:, : h // 16], sx[tok_of_row[valid]]), f"{what}: x block scales differ from the reference quantiser"
    assert not sfs[~valid].any(), f"{what}: padding rows must carry zero scales"
    assert not sfs[:, h // 16:].any(), f"{what}: K padding must carry zero scales"
    for t in sorted({0, nt - 1, int(np.argmin(valid.reshape(nt, 128).sum(axis=1)))}):   # whole scale tiles against to_128x4
        rows = slice(t * 128, t * 128 + 128)
        lin = np.where(valid[rows, None], sx[tok_of_row[rows]], 0).astype(np.uint8)
        lin = np.pad(lin, ((0, 0), (0, kb1 * 16 - lin.shape[1])))
        sw = O.to_128x4(lin).reshape(-1)
        assert np.array_equal(sw, raw[t, :, 16384:].reshape(-1)), f"{what}: scale tiles of row tile {t} differ from to_128x4"
    # ---- 3. / 4. sampled tokens, all of their pairs
    if sample_tokens is None:
        sample_tokens = np.arange(m)
    sample_tokens = np.asarray(sample_tokens)
    acodes, asfs, _ = read_records(ws, mp["arec"], nt, kb2)
    gs_a = float(w.prefill.gs_a)
    xq = C.dequant_exact(qx, sx, float(one[0]))
    got = out.float().cpu().numpy()
    res = dict(flips=0, scale_flips=0, ambiguous=0, blocks=0, max_flip=0.0, pairs=0)
    expect = np.zeros((len(sample_tokens), k, h))
    ebound = np.zeros((len(sample_tokens), k, h))
    pos = {int(t): i for i, t in enumerate(sample_tokens)}
    sel = np.isin(np.arange(m), sample_tokens)
    for e in np.unique(idn[sel]):
        if e < 0:
            continue
        tok, slot = np.nonzero((idn == e) & sel[:, None])
        rows = dst_row[tok * k + slot]
        w1d = C.dequant_exact(ow.q1[e], ow.s1[e].reshape(2 * inter, h // 16), 1.0) * float(ow.alpha1[e])
        lo, hi, nom = C.fc1_activation_interval(xq[tok], w1d, inter)
        v = C.requantised_membership(lo, hi, acodes[rows][:, : inter // 2], asfs[rows][:, : inter // 16], gs_a, nominal=nom)
        assert v["conformant"], f"{what}: expert {e}: re-quantised activations outside what the reference quantiser can produce: {v}"
        res["flips"] += v["code_flips"]; res["scale_flips"] += v["scale_flips"]; res["ambiguous"] += v["ambiguous_blocks"]
        res["blocks"] += v["blocks"]; res["pairs"] += len(rows)
        res["max_flip"] = max(res["max_flip"], v.get("max_flip_distance_over_halfwidth", 0.0))
        a_gpu = C.dequant_exact(acodes[rows][:, : inter // 2], asfs[rows][:, : inter // 16], gs_a)
        w2d = C.dequant_exact(ow.q2[e], ow.s2[e].reshape(h, inter // 16), 1.0) * float(ow.alpha2[e])
        c, cb, _ = C.interval_gemm(a_gpu, a_gpu, w2d)
        wf = wn[tok, slot].astype(np.float64)[:, None]
        r_lo, r_hi = C._round_bf16_interval((c - cb) * wf, (c + cb) * wf, 4 * C.U32)
        for i, (t, sl) in enumerate(zip(tok, slot)):
            expect[pos[int(t)], sl] = (r_lo[i] + r_hi[i]) / 2
            ebound[pos[int(t)], sl] = (r_hi[i] - r_lo[i]) / 2
    nominal = np.zeros((len(sample_tokens), h))
    for sl in range(k):                       # the kernel's combine: fp32 sum in slot order
        nominal = nominal + expect[:, sl]
    bound = ebound.sum(axis=1) + k * C.U32 * np.abs(expect).sum(axis=1)
    bound = bound + 0.5 * C.ulp(np.abs(nominal) + bound, "bf16")
    g = got[sample_tokens]
    plain = O.moe_reference(xf[sample_tokens], ow, idn[sample_tokens], wn[sample_tokens], act_quant=True) if w.prefill.gs_x == 1.0 and gs_a == 1.0 else nominal
    rms = float(np.sqrt((plain.astype(np.float64) ** 2).mean()))
    err = np.abs(g - nominal)
    res["max_abs_over_rms_own_codes"] = float(err.max() / rms)
    res["max_err_over_bound"] = float((err / bound).max())
    res["max_abs_over_rms_plain_oracle"] = float(np.abs(g - plain).max() / rms)
    res["normwise_plain_oracle"] = float(np.linalg.norm(g - plain) / max(np.linalg.norm(plain), 1e-30))
    assert err.max() <= 2e-2 * rms, f"{what}: FC2 + combine from the kernel's own codes: max-abs {err.max():.3e} > 2e-2 x rms {rms:.3e}"
    assert (err <= bound).all(), f"{what}: FC2 + combine outside the exact accumulation bound ({res['max_err_over_bound']:.2f} x)"
    assert res["normwise_plain_oracle"] < 1e-2, f"{what}: normwise error against the plain oracle {res['normwise_plain_oracle']:.3e}"
    return res


# ---------------------------------------------------------------------------------------------------- decode read-back
def decode_map(w) -> dict:
    import ctypes as C
    import sm120fp4_b200._lib as L
    buf = (C.c_longlong * 8)()
    L.check(L.lib().b200moe_layer_workspace_map(w._h, buf), "decode map")
    v = [int(t) for t in buf]
    return dict(xb=v[0], xscale=v[1], aslab=v[2], slab={16: v[3], 32: v[4], 64: v[5]}, act_g1=float(np.array([v[6]], dtype=np.uint32).view(np.float32)[0]),
                umax=v[7])


def _operand_rows(raw: np.ndarray, n: int, kb: int, sf_off: int, nkt: int | None = None):
    """raw u8: kb boxes of [n rows][128 B] (128-byte swizzle) then nkt scale tiles (default 4 per box) from sf_off -> (codes
    [n, kb*128], scales [n, kb*16], zero beyond the last tile)."""
    r = np.arange(n)[:, None]
    by = np.arange(128)[None, :]
    idx = r * 128 + (((by >> 4) ^ (r & 7)) << 4) + (by & 15)
    codes = np.stack([raw[k * n * 128:(k + 1) * n * 128][idx] for k in range(kb)], axis=1).reshape(n, kb * 128)
    nkt = 4 * kb if nkt is None else nkt
    b = np.arange(nkt * 4)[None, :]
    sidx = sf_off + (b >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (b & 3)
    sf = np.zeros((n, kb * 16), dtype=np.uint8)
    sf[:, : nkt * 4] = raw[sidx]
    return codes, sf


def check_decode_call(w, ow, x, ids, wts, out, what=""):
    """The tolerance-free gate of one tcgen05 decode call (M <= 16) that has just run on `w`, from the operands the kernel left
    in its workspace (the method of the reference's interval oracle, sm120fp4/moe_oracle.py:82-150, with this kernel's
    rounding points):
      1. the four-term NVFP4 expansion of x stands for x up to the expansion's residual bound, element by element;
      2. the expanded FC1 -> FC2 activations lie inside the interval of silu(gate) * up * weight that exact FC1 products of
         the kernel's own x operand, accumulated in fp32 in any order, can give - widened by the expansion residual;
      3. the output lies inside the fp32-accumulation bound of the exact FC2 + combine of the kernel's own activation
         operand, plus one bf16 rounding.
    Returns the measured maxima (each as a fraction of its bound)."""
    from oracle import conformance as C
    m, k = ids.shape
    h, inter = ow.H, ow.I
    kb1, kb2 = (h + 255) // 256, (inter + 255) // 256
    n = 16 if m <= 4 else 32 if m <= 8 else 64
    mp = decode_map(w)
    ws = w.workspace
    idn, wn, xf = ids.numpy(), wts.numpy().astype(np.float32), x.float().numpy().astype(np.float64)
    # ---- 1. x operand
    kt1 = (h // 16 + 3) // 4
    raw = ws[mp["xb"]:mp["xb"] + kb1 * n * 128 + kt1 * 512].cpu().numpy()
    codes, sfs = _operand_rows(raw, n, kb1, kb1 * n * 128, kt1)
    colscale = ws[mp["xscale"]:mp["xscale"] + 4 * n].view(torch.float32).cpu().numpy().astype(np.float64)
    tk_codes = codes.reshape(n // 4, 4, -1).transpose(1, 0, 2)[:, :m, : h // 2]          # [term, token, H/2]
    tk_sf = sfs.reshape(n // 4, 4, -1).transpose(1, 0, 2)[:, :m, : h // 16]
    cs = colscale.reshape(n // 4, 4)[:m]                                                  # 1 / g_t per token and term
    xt = 0.0
    xmag = 0.0
    for t in range(4):
        v = C.scaled_operand(tk_codes[t], tk_sf[t]) * 0.5 * cs[:, t:t + 1]
        xt, xmag = xt + v, xmag + np.abs(v)
    bmax = np.repeat(np.abs(xf).reshape(m, -1, 16).max(axis=-1), 16, axis=1)
    res_x = np.abs(xf - xt)
    bound_x = C.EXPANSION_RESIDUAL * bmax + 1e-6 * np.abs(xf).max(axis=1, keepdims=True)
    r = {"x_residual_over_bound": float((res_x / bound_x).max())}
    assert (res_x <= bound_x).all(), f"{what}: the x operand is further from x than four NVFP4 terms leave ({r['x_residual_over_bound']:.2f} x the bound)"
    # ---- 2. activation operand, expert by expert (slab order = ascending touched experts)
    touched = sorted(set(int(e) for e in idn.reshape(-1) if e >= 0))
    a2max = float(np.abs(ow.alpha2).max())
    slab_b = mp["slab"][n]
    g1a = mp["act_g1"]
    act = {}
    worst_a = 0.0
    for u, e in enumerate(touched):
        tok = np.nonzero((idn == e).any(axis=1))[0]
        wsum = np.array([wn[t][idn[t] == e].astype(np.float32).sum(dtype=np.float32) for t in tok], dtype=np.float32)
        wf = (wsum * np.float32(np.float32(ow.alpha2[e]) * np.float32(1.0 / a2max))).astype(np.float64)[:, None]
        w1d = C.dequant_exact(ow.q1[e], ow.s1[e].reshape(2 * inter, h // 16), 1.0) * float(ow.alpha1[e])
        lo, hi, nom = C.fc1_activation_interval(xt[tok], w1d, inter, xabs=xmag[tok])
        lo, hi = np.minimum(lo * wf, hi * wf), np.maximum(lo * wf, hi * wf)
        wid = 4 * C.U32 * np.maximum(np.abs(lo), np.abs(hi))
        lo, hi = lo - wid, hi + wid
        sraw = ws[mp["aslab"] + u * kb2 * slab_b:mp["aslab"] + (u + 1) * kb2 * slab_b].cpu().numpy().reshape(kb2, slab_b)
        ac = np.concatenate([_operand_rows(sraw[kb], n, 1, n * 128)[0] for kb in range(kb2)], axis=1)
        asf = np.concatenate([_operand_rows(sraw[kb], n, 1, n * 128)[1] for kb in range(kb2)], axis=1)
        rows = (tok[:, None] * 4 + np.arange(4)[None, :])                                # operand rows of the routed tokens
        a_t, _ = C.expansion_value(ac[rows.T][:, :, : inter // 2], asf[rows.T][:, :, : inter // 16], g1a)
        bm = np.repeat(np.maximum(np.abs(lo), np.abs(hi)).reshape(len(tok), -1, 16).max(axis=-1), 16, axis=1)
        slack = C.EXPANSION_RESIDUAL * bm + 2.0 ** -9 / (g1a * 216.0)
        ok = (a_t >= lo - slack) & (a_t <= hi + slack)
        dist = np.maximum(lo - a_t, a_t - hi) / slack
        worst_a = max(worst_a, float(dist.max()))
        assert ok.all(), f"{what}: expert {e}: expanded activations outside the interval exact FC1 products allow ({float(dist.max()):.2f} x the slack)"
        for i, t in enumerate(tok):
            act[(int(t), e)] = a_t[i]
    r["activation_excess_over_slack"] = max(worst_a, 0.0)
    # ---- 3. output from the kernel's own activation operand
    exact = np.zeros((m, h))
    sabs = np.zeros((m, h))
    for e in touched:
        w2 = C.dequant_exact(ow.q2[e], ow.s2[e].reshape(h, inter // 16), 1.0) * a2max
        for t in range(m):
            if (t, e) in act:
                exact[t] += act[(t, e)] @ w2.T
                sabs[t] += np.abs(act[(t, e)]) @ np.abs(w2).T
    kk = max(1, len(touched)) * inter
    bound = (C.gamma(kk) + 16 * C.U32) * sabs * 1.25 + 0.5 * C.ulp(np.abs(exact) + C.gamma(kk) * sabs, "bf16")   # 1.25: the terms' magnitudes
    got = out.float().cpu().numpy().astype(np.float64)
    err = np.abs(got - exact)
    r["out_err_over_bound"] = float((err / bound).max())
    rms = float(np.sqrt((exact ** 2).mean()))
    r["out_max_abs_over_rms_own_operands"] = float(err.max() / max(rms, 1e-30))
    assert (err <= bound).all(), f"{what}: output outside the accumulation bound of its own operands ({r['out_err_over_bound']:.2f} x)"
    return r
