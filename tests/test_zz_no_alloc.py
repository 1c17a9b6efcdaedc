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
    calls = [(4096, 128, 8), (37, 256, 6), (8192, 256, 8)]   # a large batch, a small ragged one over more experts, then the
                                                             # stated limits: 65,536 pairs over 256 experts
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


def test_static_router_reports_an_expert_id_out_of_range():
    """An id >= E is skipped and flagged; the status call (which allocates nothing either) returns the argument error."""
    import sm120fp4_b200._lib as L
    h = L.lib()
    ids = torch.tensor([[0, 3], [9, 1], [2, 2]], dtype=torch.int32, device="cuda")     # 9 is out of range for 8 experts
    ex = torch.empty(6, dtype=torch.int32, device="cuda")
    off = torch.empty(7, dtype=torch.int32, device="cuda")
    pairs = torch.full((6,), -7, dtype=torch.int32, device="cuda")
    L.check(h.b200moe_route_static(L.ptr(ids), 6, 8, 6, L.ptr(ex), L.ptr(off), L.ptr(pairs), L.stream_ptr()), "route_static")
    assert h.b200moe_route_static_status(6, 8, L.stream_ptr()) == L.ERR_ARG
    assert off.cpu().tolist()[:5] == [0, 1, 2, 4, 5] and ex.cpu().tolist() == [0, 1, 2, 3, -1, -1]
    good = torch.tensor([[0, 3], [7, 1], [2, 2]], dtype=torch.int32, device="cuda")
    L.check(h.b200moe_route_static(L.ptr(good), 6, 8, 6, L.ptr(ex), L.ptr(off), L.ptr(pairs), L.stream_ptr()), "route_static")
    assert h.b200moe_route_static_status(6, 8, L.stream_ptr()) == 0
