"""GPU parity, through the C ABI, of the byte/integer kernels: 128x4 swizzle, NVFP4 quantizer, router. Bit-exact bar."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("rows,cols", [(128, 4), (256, 32), (100, 5), (1, 1), (129, 9), (1024, 256), (1536, 128), (2048, 48),
                                       (1408, 176), (2816, 44)])
def test_swizzle_equals_reference(golden, rows, cols):
    import sm120fp4_b200 as pkg
    m = golden.meta[f"layout_{rows}x{cols}"]
    sf = torch.randint(0, 256, (rows, cols), dtype=torch.uint8, generator=torch.Generator().manual_seed(m["seed"]))
    sw = pkg.to_128x4(sf.cuda())
    assert list(sw.shape) == m["shape"]
    assert sha(sw.cpu().numpy()) == m["swz_sha256"]
    assert torch.equal(pkg.from_128x4(sw, rows, cols).cpu(), sf)


def test_swizzle_batched_and_errors():
    import sm120fp4_b200 as pkg
    sf = torch.randint(0, 256, (5, 200, 22), dtype=torch.uint8)
    sw = pkg.to_128x4(sf.cuda())
    for b in range(5):
        assert np.array_equal(sw[b].cpu().numpy(), O.to_128x4(sf[b].numpy()))
    assert torch.equal(pkg.from_128x4(sw, 200, 22).cpu(), sf)
    with pytest.raises(ValueError):
        pkg.from_128x4(torch.zeros(10, dtype=torch.uint8, device="cuda"), 128, 4)
    with pytest.raises(ValueError):
        pkg.to_128x4(torch.zeros(4, dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("name", ["randn3", "act_gs1", "act_auto", "w_small", "edge_gs307", "edge_gs1", "edge_auto"])
def test_quantizer_bytes_equal_reference(golden, name):
    import sm120fp4_b200 as pkg
    g = golden.load("quantize")
    gs_in = float(g[f"q_{name}_gs_in"][0])
    x = dev(g[f"q_{name}_x"])
    q, sf, gs = pkg.quantize_nvfp4(x, None if gs_in == 0 else torch.tensor([gs_in]))
    assert np.array_equal(gs.cpu().numpy().view(np.uint32), g[f"q_{name}_gs"].view(np.uint32)), "global scale bits"
    bad_sf = int((sf.cpu().numpy() != g[f"q_{name}_sf"]).sum())
    bad_q = int((q.cpu().numpy() != g[f"q_{name}_packed"]).sum())
    assert bad_sf == 0 and bad_q == 0, f"{bad_sf} scale bytes and {bad_q} code bytes differ"
    if name.startswith("act"):    # the same input as bf16: the dtype path must not change a bit
        q2, sf2, _ = pkg.quantize_nvfp4(x.to(torch.bfloat16), gs)
        assert torch.equal(q2, q) and torch.equal(sf2, sf)


def test_quantizer_full_size_digest_and_fused_128x4(golden):
    import sm120fp4_b200 as pkg
    g = torch.Generator().manual_seed(5)
    for shape in ((24, 512), (24, 512), (48, 256)):
        torch.randn(*shape, generator=g)
    big = torch.randn(256, 2048, generator=g).to(torch.bfloat16).cuda()
    one = torch.ones(1)
    q, sf, _ = pkg.quantize_nvfp4(big, one)
    m = golden.meta["q_big_gs1"]
    assert sha(q.cpu().numpy()) == m["packed_sha256"] and sha(sf.cpu().numpy()) == m["sf_sha256"]
    q2, sw, _ = pkg.quantize_nvfp4_128x4(big, one)
    assert torch.equal(q2, q) and sha(sw.cpu().numpy()) == m["sf128x4_sha256"]
    # gather: destination rows read chosen source rows, negative -> zero row; ragged row count (padded to 128 in the scales)
    src = torch.tensor([5, 5, -1, 255, 0, 17, -1] * 29, dtype=torch.int32)
    q3, sw3, _ = pkg.quantize_nvfp4_128x4(big, one, src_row=src.cuda())
    qn, sfn = q.cpu().numpy(), sf.cpu().numpy()
    want_q = np.where(src.numpy()[:, None] >= 0, qn[np.maximum(src.numpy(), 0)], 0)
    want_sf = np.where(src.numpy()[:, None] >= 0, sfn[np.maximum(src.numpy(), 0)], 0)
    assert np.array_equal(q3.cpu().numpy(), want_q)
    assert np.array_equal(sw3.cpu().numpy(), O.to_128x4(want_sf.astype(np.uint8)))


def test_quantizer_oracle_on_random_shapes():
    import sm120fp4_b200 as pkg
    rng = np.random.default_rng(3)
    for m, k, scale in [(1, 16, 1.0), (3, 48, 100.0), (130, 704, 0.01), (17, 2816, 5.0), (64, 768, 1e-3)]:
        x = (rng.standard_normal((m, k)) * scale).astype(np.float32)
        x[rng.random((m, k)) < 0.05] = 0
        for gs in (None, np.array([1.0], dtype=np.float32)):
            wq, wsf, wgs = O.quantize_nvfp4(x, gs)
            q, sf, g = pkg.quantize_nvfp4(dev(x), None if gs is None else torch.from_numpy(gs))
            assert np.array_equal(g.cpu().numpy().view(np.uint32), wgs.view(np.uint32))
            assert np.array_equal(sf.cpu().numpy(), wsf) and np.array_equal(q.cpu().numpy(), wq), (m, k, scale)
    with pytest.raises(ValueError):
        pkg.quantize_nvfp4(torch.zeros(4, 24, device="cuda"))
    with pytest.raises(TypeError):
        pkg.global_scale_for(torch.zeros(4, 32, device="cuda", dtype=torch.float16))


def test_router_equals_reference(golden):
    import sm120fp4_b200 as pkg
    g = golden.load("route")
    for n in sorted({k.rsplit("_", 1)[0] for k in g.files}):
        ids = g[f"{n}_ids"]
        e = 256 if n.startswith("e256") else 128
        ex, off, pairs = pkg.route_tables(dev(ids), e)
        wex, woff, wpairs = O.route_padded(ids, e)
        assert np.array_equal(ex.cpu().numpy(), wex), n
        assert np.array_equal(off.cpu().numpy(), woff), n
        assert np.array_equal(pairs.cpu().numpy(), wpairs), n
        u = g[f"{n}_experts"].size
        assert np.array_equal(ex.cpu().numpy()[:u], g[f"{n}_experts"]) and np.array_equal(pairs.cpu().numpy(), g[f"{n}_pairs"])


@pytest.mark.parametrize("tokens,experts,top_k", [(8192, 128, 8), (4096, 128, 8), (1000, 1024, 3), (1, 4, 1), (777, 7, 7)])
def test_router_large_and_ragged(tokens, experts, top_k):
    import sm120fp4_b200 as pkg
    rng = np.random.default_rng(tokens + experts)
    ids = np.argsort(rng.random((tokens, experts)), axis=1)[:, :top_k].astype(np.int32)
    if experts == 7:
        ids[:, :] = rng.integers(0, 2, ids.shape) * 6          # two experts only, the rest untouched
    ex, off, pairs = pkg.route_tables(dev(ids), experts)
    wex, woff, wpairs = O.route_padded(ids, experts)
    assert np.array_equal(ex.cpu().numpy(), wex) and np.array_equal(off.cpu().numpy(), woff)
    assert np.array_equal(pairs.cpu().numpy(), wpairs)
    # size-independent properties: pairs is a permutation, sorted by (expert, pair index)
    p = pairs.cpu().numpy()
    assert np.array_equal(np.sort(p), np.arange(ids.size))
    key = ids.reshape(-1)[p].astype(np.int64) * ids.size + p
    assert (np.diff(key) > 0).all()


def test_router_empty():
    import sm120fp4_b200 as pkg
    ex, off, pairs = pkg.route_tables(torch.zeros((0, 8), dtype=torch.int32, device="cuda"), 128)
    assert ex.numel() == 0 and off.cpu().tolist() == [0] and pairs.numel() == 0
