"""tcgen05 building blocks (TMEM, descriptors, scale copies, kind::mxf4nvf4) against the oracle's dequantise-then-fp32 GEMM
(the reference GEMM of sm120fp4/reference.py:133-137) on single tiles."""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


def probe(a, b, scale_path=0):
    """a [128, K], b [N, K] fp32 -> (D from the tensor cores, D expected) with NVFP4 operands, global scale 1."""
    import sm120fp4_b200._lib as L
    one = np.ones(1, dtype=np.float32)
    qa, sa, _ = O.quantize_nvfp4(a, one)
    qb, sb, _ = O.quantize_nvfp4(b, one)
    want = O.dequantize_nvfp4(qa, sa, one) @ O.dequantize_nvfp4(qb, sb, one).T
    n, k = b.shape
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()  # noqa: E731
    d = torch.full((128, n), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ta, tsa, tb, tsb = dev(qa), dev(O.to_128x4(sa)), dev(qb), dev(O.to_128x4(sb))
    L.check(L.lib().b200moe_umma_probe(L.ptr(ta), L.ptr(tsa), L.ptr(tb), L.ptr(tsb), n, k, L.ptr(d), scale_path, L.ptr(status), L.stream_ptr()), "probe")
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait ran out in the probe kernel"
    return d.cpu().numpy(), want.astype(np.float32)


@pytest.mark.parametrize("n,k", [(128, 256), (64, 256), (16, 512), (128, 1024), (32, 768)])
def test_block_scaled_fp4_tile_matches_oracle(n, k):
    rng = np.random.default_rng(n * 1000 + k)
    a = rng.standard_normal((128, k)).astype(np.float32) * 3
    b = rng.standard_normal((n, k)).astype(np.float32) * 0.5
    got, want = probe(a, b)
    assert np.isfinite(got).all()
    err = np.abs(got - want).max()
    assert err <= 1e-3 * np.abs(want).max() + 1e-4, f"max err {err} vs max |D| {np.abs(want).max()}"


@pytest.mark.parametrize("n,k", [(64, 256), (16, 1024), (128, 512)])
def test_scales_through_registers_match_the_copy_path(n, k):
    """The decode kernel moves scale tiles shared memory -> registers -> TMEM (tcgen05.st by four warps, one per lane
    quadrant) instead of tcgen05.cp; scale_path = 1 selects that path in the probe, and nothing but 0 and 1 is accepted."""
    rng = np.random.default_rng(n * 77 + k)
    a = rng.standard_normal((128, k)).astype(np.float32) * 2
    b = rng.standard_normal((n, k)).astype(np.float32)
    got_cp, want = probe(a, b)
    got_st, _ = probe(a, b, scale_path=1)
    assert np.array_equal(got_cp, got_st)
    assert np.abs(got_st - want).max() <= 1e-3 * np.abs(want).max() + 1e-4


@pytest.mark.parametrize("k", [256, 512, 1024])
def test_cta_pair_mma_matches_oracle(k):
    """tcgen05 cta_group::2: two CTAs of a cluster as one 256 x 128 x 64 MMA unit (A and accumulator rows split over the two
    CTAs, B rows split over their shared memories, one commit arriving on both)."""
    import sm120fp4_b200._lib as L
    rng = np.random.default_rng(4000 + k)
    a = rng.standard_normal((256, k)).astype(np.float32) * 3
    b = rng.standard_normal((128, k)).astype(np.float32) * 0.5
    one = np.ones(1, dtype=np.float32)
    qa, sa, _ = O.quantize_nvfp4(a, one)
    qb, sb, _ = O.quantize_nvfp4(b, one)
    want = (O.dequantize_nvfp4(qa, sa, one) @ O.dequantize_nvfp4(qb, sb, one).T).astype(np.float32)
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()  # noqa: E731
    d = torch.full((256, 128), float("nan"), device="cuda")
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    ta, tsa, tb, tsb = dev(qa), dev(O.to_128x4(sa)), dev(qb), dev(O.to_128x4(sb))
    L.check(L.lib().b200moe_umma_pair_probe(L.ptr(ta), L.ptr(tsa), L.ptr(tb), L.ptr(tsb), k, L.ptr(d), L.ptr(status), L.stream_ptr()), "pair probe")
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0], "a bounded wait ran out in the pair probe"
    got = d.cpu().numpy()
    assert np.isfinite(got).all()
    err = np.abs(got - want).max()
    assert err <= 1e-3 * np.abs(want).max() + 1e-4, f"max err {err} vs max |D| {np.abs(want).max()}"
