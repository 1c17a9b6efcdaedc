"""The CPU oracle against the vectors generated from the reference's own code, and the reference tests' known answers."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_e2m1_probe_and_decode(golden):
    g = golden.load("quantize")
    assert np.array_equal(O.e2m1_encode(g["e2m1_probe_in"]), g["e2m1_probe_codes"])
    assert np.array_equal(O.e2m1_decode(np.arange(16, dtype=np.uint8)), g["e2m1_all_decode"])
    codes = np.arange(16, dtype=np.uint8).reshape(1, 16)
    assert np.array_equal(O.unpack_e2m1(O.pack_e2m1(codes)), codes)
    assert O.pack_e2m1(np.array([[1, 2]], dtype=np.uint8))[0, 0] == 0x21      # even element in the low nibble


def test_e4m3_encode_matches_torch_cast_exhaustively_on_a_dense_grid():
    # every E4M3 value, every midpoint between neighbours and points just off the midpoints
    vals = O.E4M3_TABLE[:0x7F].astype(np.float64)
    mids = (vals[:-1] + vals[1:]) / 2
    pts = np.concatenate([vals, mids, np.nextafter(mids.astype(np.float32), 0), np.nextafter(mids.astype(np.float32), 1e9),
                          np.random.default_rng(0).uniform(0, 448, 200000)]).astype(np.float32)
    pts = np.clip(pts, 0, 448)
    want = torch.from_numpy(pts).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(O.e4m3_encode(pts), want)
    assert np.array_equal(O.e4m3_decode(np.arange(0x7F, dtype=np.uint8)),
                          torch.arange(0x7F, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy())


@pytest.mark.parametrize("name", ["randn3", "act_gs1", "act_auto", "w_small", "edge_gs307", "edge_gs1", "edge_auto"])
def test_quantizer_bytes_equal_reference(golden, name):
    g = golden.load("quantize")
    gs_in = float(g[f"q_{name}_gs_in"][0])
    q, sf, gs = O.quantize_nvfp4(g[f"q_{name}_x"], None if gs_in == 0 else np.array([gs_in], dtype=np.float32))
    assert np.array_equal(q, g[f"q_{name}_packed"])
    assert np.array_equal(sf, g[f"q_{name}_sf"])
    assert np.array_equal(gs.view(np.uint32), g[f"q_{name}_gs"].view(np.uint32))
    deq = O.dequantize_nvfp4(q, sf, gs)
    assert np.allclose(deq, g[f"q_{name}_deq"], rtol=1e-6, atol=0)


def test_quantizer_known_answers_from_the_reference_tests():
    # sign kept on a block that rounds to zero: bytes 0x88, scale byte 0
    x = np.full((1, 16), -1e-9, dtype=np.float32)
    q, sf, _ = O.quantize_nvfp4(x, np.ones(1, dtype=np.float32))
    assert (q == 0x88).all() and sf[0, 0] == 0
    # the scale-tie example: 2.265625 / 6 * 307.2 = 116, midway between 112 and 120 -> even mantissa (112)
    q, sf, _ = O.quantize_nvfp4(np.full((1, 16), 2.265625, dtype=np.float32), np.array([307.2], dtype=np.float32))
    assert O.e4m3_decode(sf)[0, 0] in (112.0, 120.0)
    assert sf[0, 0] == torch.tensor(116.0).to(torch.float8_e4m3fn).view(torch.uint8).item()
    # round-trip error bounded by one grid unit per block (the reference's own quantizer test)
    torch.manual_seed(0)
    x = (torch.randn(64, 256) * 3).numpy()
    q, sf, gs = O.quantize_nvfp4(x)
    y = O.dequantize_nvfp4(q, sf, gs)
    unit = (O.e4m3_decode(sf) / gs.reshape(())).reshape(64, 16, 1)
    err = np.abs(y.reshape(64, 16, 16) - x.reshape(64, 16, 16))
    assert (err <= unit + 1e-5).all() and err.mean() < unit.mean() * 0.35


def test_quantizer_full_size_digest(golden):
    g = torch.Generator().manual_seed(5)
    for shape in ((24, 512), (24, 512), (48, 256)):
        torch.randn(*shape, generator=g)
    big = torch.randn(256, 2048, generator=g).to(torch.bfloat16).float().numpy()
    q, sf, _ = O.quantize_nvfp4(big, np.ones(1, dtype=np.float32))
    m = golden.meta["q_big_gs1"]
    assert sha(q) == m["packed_sha256"] and sha(sf) == m["sf_sha256"] and sha(O.to_128x4(sf)) == m["sf128x4_sha256"]


@pytest.mark.parametrize("rows,cols", [(128, 4), (256, 32), (100, 5), (1, 1), (129, 9), (1024, 256), (1536, 128), (2048, 48),
                                       (1408, 176), (2816, 44)])
def test_layout_equals_reference(golden, rows, cols):
    m = golden.meta[f"layout_{rows}x{cols}"]
    sf = torch.randint(0, 256, (rows, cols), dtype=torch.uint8, generator=torch.Generator().manual_seed(m["seed"])).numpy()
    assert sha(sf) == m["lin_sha256"]
    sw = O.to_128x4(sf)
    assert list(sw.shape) == m["shape"] == list(O.padded_sf_shape(rows, cols))
    assert sha(sw) == m["swz_sha256"]
    assert np.array_equal(O.from_128x4(sw, rows, cols), sf)
    g = golden.load("layouts")
    if f"swz_{rows}x{cols}" in g:
        assert np.array_equal(sw, g[f"swz_{rows}x{cols}"])
        assert np.array_equal(O.linear_to_128x4_index(rows, cols), g[f"idx_{rows}x{cols}"])
    # padding is zero and the index map is a bijection onto the used entries
    idx = O.linear_to_128x4_index(rows, cols)
    assert np.unique(idx).size == rows * cols
    used = np.zeros(sw.size, dtype=bool)
    used[idx.reshape(-1)] = True
    assert (sw.reshape(-1)[~used] == 0).all()


def test_layout_cudnn_worked_example():
    idx = O.linear_to_128x4_index(128, 4)
    for outer in (0, 1, 31, 32, 33, 96, 127):
        for inner in range(4):
            assert idx[outer, inner] == (outer % 32) * 16 + (outer // 32) * 4 + inner
    with pytest.raises(ValueError):
        O.from_128x4(np.zeros(10, dtype=np.uint8), 128, 4)


def test_router_equals_reference(golden):
    g = golden.load("route")
    names = sorted({k.rsplit("_", 1)[0] for k in g.files})
    assert len(names) >= 13
    for n in names:
        ex, off, pairs = O.route(g[f"{n}_ids"])
        assert np.array_equal(ex, g[f"{n}_experts"]) and np.array_equal(off, g[f"{n}_offsets"])
        assert np.array_equal(pairs, g[f"{n}_pairs"])
        e = 256 if n.startswith("e256") else 128
        pex, poff, ppairs = O.route_padded(g[f"{n}_ids"], e)
        u = ex.size
        assert pex.size == min(e, pairs.size) and (pex[u:] == -1).all() and (poff[u:] == pairs.size).all()
        assert np.array_equal(pex[:u], ex) and np.array_equal(poff[:u + 1], off)


def tiny_layer(golden):
    import sm120fp4_b200.synth as synth
    cfg = synth.TINY
    w13, w2 = synth.layer_weights_bf16(cfg["experts"], cfg["hidden"], cfg["inter"], seed=3)
    q1, s1, a1, q2, s2, a2 = [], [], [], [], [], []
    for e in range(cfg["experts"]):
        q, s, gs = O.quantize_nvfp4(w13[e].float().numpy())
        q1.append(q), s1.append(s), a1.append(np.float32(1.0) / gs)
        q, s, gs = O.quantize_nvfp4(w2[e].float().numpy())
        q2.append(q), s2.append(s), a2.append(np.float32(1.0) / gs)
    return cfg, O.ExpertWeights(np.stack(q1), np.stack(s1), np.concatenate(a1), np.stack(q2), np.stack(s2), np.concatenate(a2))


def test_tiny_layer_equals_reference(golden):
    import sm120fp4_b200.synth as synth
    cfg, w = tiny_layer(golden)
    m = golden.meta["tiny_layer"]
    assert sha(w.q1) == m["q1_sha256"] and sha(w.s1) == m["s1_sha256"] and sha(w.q2) == m["q2_sha256"] and sha(w.s2) == m["s2_sha256"]
    g = golden.load("layer_tiny")
    assert np.array_equal(w.alpha1.view(np.uint32), g["tiny_alpha1"].view(np.uint32))
    assert np.array_equal(w.alpha2.view(np.uint32), g["tiny_alpha2"].view(np.uint32))
    for mm, routing, seed in [(1, "random", 11), (6, "random", 12), (16, "random", 13), (5, "fixed8", 14), (40, "random", 15)]:
        x, ids, wts = synth.decode_inputs(mm, cfg["experts"], cfg["hidden"], cfg["top_k"], seed, routing)
        for aq in (False, True):
            want = g[f"tiny_m{mm}_{routing}_{'w4a4' if aq else 'w4a16'}"]
            got = O.moe_reference(x.float().numpy(), w, ids.numpy(), wts.numpy(), act_quant=aq)
            rms = np.sqrt((want ** 2).mean())
            # fp32 GEMMs in a different summation order: round-off only (W4A4: a re-quantised activation may flip a code)
            tol = 1e-5 * rms if not aq else 2e-2 * rms
            assert np.abs(got - want).max() <= tol, (mm, routing, aq, np.abs(got - want).max(), rms)
