"""The workspace-free router entry point (for hosts that cannot allocate device memory) against the ordinary one.

Collected last on purpose: a run that stops at the first failure has then already exercised everything else."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def tables(fn_name, ids, experts_n, with_workspace):
    import sm120fp4_b200._lib as L
    h = L.lib()
    p = ids.numel()
    umax = min(experts_n, p)
    ex = torch.full((umax,), -7, dtype=torch.int32, device="cuda")
    off = torch.full((umax + 1,), -7, dtype=torch.int32, device="cuda")
    pairs = torch.full((p,), -7, dtype=torch.int32, device="cuda")
    if with_workspace:
        ws = torch.empty(int(h.b200moe_route_workspace_bytes(p, experts_n)), dtype=torch.uint8, device="cuda")
        L.check(h.b200moe_route(L.ptr(ids), p, experts_n, umax, L.ptr(ex), L.ptr(off), L.ptr(pairs), L.ptr(ws), ws.numel(), L.stream_ptr()), fn_name)
    else:
        L.check(h.b200moe_route_static(L.ptr(ids), p, experts_n, umax, L.ptr(ex), L.ptr(off), L.ptr(pairs), L.stream_ptr()), fn_name)
    torch.cuda.synchronize()
    return ex.cpu().numpy(), off.cpu().numpy(), pairs.cpu().numpy()


def test_static_router_matches_the_workspace_router_twice_in_a_row():
    """Two back-to-back calls with different inputs: the second must not see anything the first left in the shared array.
    Integer tables: the comparison is exact."""
    rng = np.random.default_rng(11)
    calls = [(4096, 128, 8), (37, 256, 6)]          # a large batch first, then a small ragged one over more experts
    for tokens, experts_n, top_k in calls:
        ids_np = np.argsort(rng.random((tokens, experts_n)), axis=1)[:, :top_k].astype(np.int32)
        ids = torch.from_numpy(ids_np).cuda()
        want = tables("route", ids, experts_n, True)
        got = tables("route_static", ids, experts_n, False)
        for a, b, name in zip(got, want, ("experts", "offsets", "pairs")):
            assert np.array_equal(a, b), f"{name} differ for {tokens} tokens / {experts_n} experts"


def test_static_router_rejects_sizes_beyond_its_built_in_scratch():
    import sm120fp4_b200._lib as L
    h = L.lib()
    t = torch.zeros(8, dtype=torch.int32, device="cuda")
    assert h.b200moe_route_static(L.ptr(t), 65537, 128, 8, L.ptr(t), L.ptr(t), L.ptr(t), L.stream_ptr()) == L.ERR_LIMIT
    assert h.b200moe_route_static(L.ptr(t), 8, 257, 8, L.ptr(t), L.ptr(t), L.ptr(t), L.stream_ptr()) == L.ERR_LIMIT
