"""Expert-parallel layer on GPUs: the single-rank path (dispatch / masked slots / combine around the real kernels) always,
and a two-rank NCCL run when the box has two GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT
from helpers import check_layer_output
from oracle import nvfp4_oracle as O
from test_gpu_decode import inputs, layer

pytestmark = pytest.mark.gpu


def test_masked_slots_are_skipped():
    """ids of -1 mark slots another rank owns: the kernels must skip them (decode kernels and the prefill path)."""
    cfg, w, ow = layer("mid")
    for m in (6, 16, 40):
        x, ids, wts = inputs(cfg, m, 900 + m)
        masked = ids.clone()
        masked[:, 1] = -1
        masked[0, :] = -1                       # a row with no local expert at all -> zero output row
        wz = wts.clone()
        wz[masked < 0] = 0
        for impl in ("mma", "tcgen05"):
            w.set_decode_impl(impl)
            out = w.forward(x.cuda(), masked.cuda(), wz.cuda())
            w.status()
            # oracle: the masked slots contribute nothing
            ref_ids = ids.clone()
            want = O.moe_reference(x.float().numpy(), ow, ref_ids.numpy(), wz.numpy())
            check_layer_output(out, want, f"masked m={m} {impl}")
            assert float(out[0].float().abs().max()) == 0.0
        w.set_decode_impl("auto")
    x, ids, wts = inputs(cfg, 150, 77)
    masked = ids.clone()
    masked[::3, 2] = -1
    wz = wts.clone()
    wz[masked < 0] = 0
    w.enable_prefill(max_tokens=256)
    out = w.forward(x.cuda(), masked.cuda(), wz.cuda())
    w.prefill_status()
    from helpers import check_w4a4_output
    check_w4a4_output(out, O.moe_reference(x.float().numpy(), ow, ids.numpy(), wz.numpy(), act_quant=True), "masked prefill")
    w.prefill = None


def test_single_rank_expert_parallel_wrapper_equals_the_layer():
    from sm120fp4_b200.ep import ExpertParallelMoE
    cfg, w, ow = layer("mid")
    x, ids, wts = inputs(cfg, 12, 55)
    base = w.forward(x.cuda(), ids.cuda(), wts.cuda())
    for cap in (None, 16):
        ep = ExpertParallelMoE(w.forward, cfg["experts"], cfg["top_k"], capacity=cap)
        out = ep.forward(x.cuda(), ids.cuda(), wts.cuda())
        assert torch.equal(out, base), f"capacity={cap}"


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import faulthandler
    faulthandler.dump_traceback_later(120, exit=True)   # a rank stuck in a collective shows where, and ends, instead of hanging the test
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import sm120fp4_b200 as pkg
        from sm120fp4_b200 import synth
        from sm120fp4_b200.ep import ExpertParallelMoE, shard_range
        from sm120fp4_b200.vllm_backend import Weights
        cfg = dict(experts=16, hidden=512, inter=192, top_k=4)
        w13, w2 = synth.layer_weights_bf16(cfg["experts"], cfg["hidden"], cfg["inter"], seed=21)
        q1, s1, g1 = pkg.quantize_nvfp4_experts(w13.cuda())
        q2, s2, g2 = pkg.quantize_nvfp4_experts(w2.cuda())
        lo, hi = shard_range(cfg["experts"], rank, world)
        local = Weights(q1[lo:hi].contiguous(), s1[lo:hi].contiguous(), (1 / g1)[lo:hi].contiguous(), q2[lo:hi].contiguous(),
                        s2[lo:hi].contiguous(), (1 / g2)[lo:hi].contiguous(), cfg["top_k"])
        full = O.ExpertWeights(q1.cpu().numpy(), s1.cpu().numpy(), (1 / g1).cpu().numpy(), q2.cpu().numpy(), s2.cpu().numpy(), (1 / g2).cpu().numpy())
        res = []

        def exchange_bound(x, ids, wts):
            """The exchange's rounding points: every owner rank returns ONE bf16 row per token (its experts already summed in
            fp32); the source adds the rows in rank order in fp32 and rounds once. Against the plain oracle (no rounding
            between the experts) each returned row therefore adds at most half a bf16 ulp of its own value, 2^-9 |partial|,
            to the error an un-sharded layer call may have: that sum is the elementwise allowance returned here."""
            extra = np.zeros((x.shape[0], cfg["hidden"]), dtype=np.float32)
            per = cfg["experts"] // world
            for r in range(world):
                wr = np.where((ids.numpy() // per) == r, wts.numpy(), 0.0).astype(np.float32)
                extra += np.abs(O.moe_reference(x.float().numpy(), full, ids.numpy(), wr)) * 2.0 ** -9
            return extra

        for cap, m, transport in ((None, 7 + rank, "nccl"), (16, 16, "nccl"), (None, 40, "nccl"), (16, 9 + rank, "peer"), (16, 3 + 9 * rank, "peer_fence"),
                                   (16, 4 * rank, "peer"), (None, 5 * rank, "nccl")):
            print(f"rank {rank}: capacity={cap} m={m} {transport}", file=sys.stderr, flush=True)
            x, ids, wts = synth.decode_inputs(m, cfg["experts"], cfg["hidden"], cfg["top_k"], 300 + rank + m)
            ep = ExpertParallelMoE(local.forward, cfg["experts"], cfg["top_k"], capacity=cap, transport=transport)
            out = ep.forward(x.cuda(), ids.cuda(), wts.cuda())
            outs = [ep.forward(x.cuda(), ids.cuda(), wts.cuda()) for _ in range(5)]
            local.status()
            ep.status()
            if m == 0:   # an empty batch on one rank: it still takes part in every exchange
                res.append((0.0, 1.0, out.shape == (0, cfg["hidden"]), "empty"))
                continue
            plain = O.moe_reference(x.float().numpy(), full, ids.numpy(), wts.numpy())
            rms = float(np.sqrt((plain ** 2).mean()))
            diff = np.abs(out.float().cpu().numpy() - plain)
            # the un-sharded layer's own bar (2e-2 x RMS) plus the half-ulps of the bf16 rows that crossed the exchange
            over = float((diff - exchange_bound(x, ids, wts)).max())
            used = getattr(getattr(ep, "_buf", None), "peer", False)
            res.append((over, rms, all(torch.equal(out, o) for o in outs), f"cap={cap} m={m} {transport} peer_used={used} "
                        f"max |out - oracle| {float(diff.max()) / rms:.2e} x rms, beyond the exchange's rounding allowance"))
        q.put((rank, res))
    except Exception as ex:  # noqa: BLE001
        import traceback
        q.put((rank, "error", traceback.format_exc()))
    finally:
        # leave without tearing the process group down: the parent has the results, and a teardown that waits for a peer which
        # is already gone would only delay the test
        torch.cuda.synchronize()
        sys.stdout.flush()
        q.close()
        q.join_thread()   # the queue hands its items to a feeder thread: let it finish before the process goes
        os._exit(0)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_expert_parallel_matches_the_full_layer():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=150) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.kill()
    for r in res:
        assert r[1] != "error", r[2]
        for err, rms, same, what in r[1]:
            print(what, f"{err / rms:.2e} x rms")
            assert err <= 2e-2 * rms and same, r


@pytest.mark.parametrize("m,world,k,experts", [(37, 4, 4, 16), (4096, 8, 8, 128), (5, 2, 2, 8), (1500, 16, 8, 128)])
def test_variable_exchange_kernels_match_the_torch_plan(m, world, k, experts):
    """b200moe_ep_plan / _gather / _combine_rows against the torch formulation used on CPU ranks (ep.dispatch_plan,
    ExpertParallelMoE._combine): same rows in the same order, same masked slots, same sums."""
    import sm120fp4_b200._lib as L
    from sm120fp4_b200.ep import dispatch_plan
    lib = L.lib()
    g = torch.Generator().manual_seed(m * 31 + world)
    h, per = 64, experts // world
    ids = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(m)]).to(torch.int32)
    ids[::7, 0] = -1                                                   # some empty slots
    wts = torch.rand(m, k, generator=g)
    x = torch.randn(m, h, generator=g).to(torch.bfloat16)
    idd, wd, xd = ids.cuda(), wts.cuda(), x.cuda()
    # torch plan on the non-empty slots (an empty slot belongs to no rank)
    safe = torch.where(idd >= 0, idd.long(), torch.full_like(idd.long(), experts * 2))
    send_tok_ref, counts_ref, local_ref, own_ref = dispatch_plan(safe, experts, world)
    max_rows = m * min(world, k)
    counts = torch.empty(world, dtype=torch.int32, device="cuda")
    offsets = torch.empty(world + 1, dtype=torch.int32, device="cuda")
    pos = torch.empty(m, world, dtype=torch.int32, device="cuda")
    send_tok = torch.full((max_rows,), -7, dtype=torch.int32, device="cuda")
    L.check(lib.b200moe_ep_plan(L.ptr(idd), m, k, world, per, L.ptr(counts), L.ptr(offsets), L.ptr(pos), L.ptr(send_tok), L.stream_ptr()), "plan")
    total = int(offsets[-1])
    assert torch.equal(counts.long(), counts_ref.long()) and total == int(counts_ref.sum())
    assert torch.equal(send_tok[:total].long(), send_tok_ref)
    sx = torch.zeros(max(total, 1), h, dtype=torch.bfloat16, device="cuda")
    meta = torch.zeros(max(total, 1), 2 * k, dtype=torch.int32, device="cuda")
    L.check(lib.b200moe_ep_gather(L.ptr(xd), L.ptr(idd), L.ptr(wd), L.ptr(send_tok), L.ptr(offsets), h, k, world, per, total, L.ptr(sx), L.ptr(meta),
                                  L.stream_ptr()), "gather")
    assert torch.equal(sx[:total], xd[send_tok_ref])
    assert torch.equal(meta[:total, :k], local_ref)
    want_w = torch.where(own_ref, wd[send_tok_ref], torch.zeros((), device="cuda"))
    assert torch.equal(meta[:total, k:].contiguous().view(torch.float32), want_w)
    # combine: every (token, destination) row exactly once, summed in rank order
    back = torch.randn(max(total, 1), h, generator=torch.Generator(device="cuda").manual_seed(1), device="cuda").to(torch.bfloat16)
    out = torch.empty(m, h, dtype=torch.bfloat16, device="cuda")
    L.check(lib.b200moe_ep_combine_rows(L.ptr(back), L.ptr(pos), m, h, world, L.ptr(out), L.stream_ptr()), "combine")
    ref = torch.zeros(m, h, dtype=torch.float32, device="cuda")
    ends = torch.cumsum(counts_ref, 0).tolist()
    start = 0
    for end in ends:
        if end > start:
            ref.index_add_(0, send_tok_ref[start:end], back[start:end].float())
        start = end
    assert torch.equal(out, ref.to(torch.bfloat16))


def test_peer_store_primitives_on_one_gpu():
    """The kernels of the peer-store exchange with both 'peers' on this GPU: dispatch with counters -> bounded wait -> return
    -> bounded wait -> combine, in stream order (a waiter never runs beside the kernel it waits for here). Then the
    failure path: a counter that nobody bumps makes the wait run out, which sets the status word and returns."""
    import ctypes as C
    import sm120fp4_b200._lib as L
    lib = L.lib()
    world, cap, h, k, experts = 2, 16, 256, 4, 8
    per = experts // world
    g = torch.Generator().manual_seed(5)
    m = 11
    x = torch.randn(m, h, generator=g).to(torch.bfloat16).cuda()
    ids = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(m)]).to(torch.int32).cuda()
    wts = torch.rand(m, k, generator=g).cuda()
    rx = torch.zeros(world, world * cap, h, dtype=torch.bfloat16, device="cuda")       # rx[d]: the receive array of "rank" d
    rid = torch.full((world, world * cap, k), -9, dtype=torch.int32, device="cuda")
    rw = torch.zeros(world, world * cap, k, device="cuda")
    flags = torch.zeros(world, world, dtype=torch.int32, device="cuda")
    calls = torch.zeros(2, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    arr = lambda v: (C.c_void_p * len(v))(*v)  # noqa: E731
    me = 1                                                                               # this "rank" sends as rank 1
    L.check(lib.b200moe_ep_dispatch(L.ptr(x), L.ptr(ids), L.ptr(wts), m, h, k, world, per, cap,
                                    arr([rx[d, me * cap].data_ptr() for d in range(world)]), arr([rid[d, me * cap].data_ptr() for d in range(world)]),
                                    arr([rw[d, me * cap].data_ptr() for d in range(world)]), arr([flags[d, me].data_ptr() for d in range(world)]),
                                    L.stream_ptr()), "dispatch")
    torch.cuda.synchronize()
    assert flags[:, me].tolist() == [cap, cap] and flags[:, 0].tolist() == [0, 0]
    for d in range(world):
        own = (ids // per) == d
        assert torch.equal(rid[d, me * cap:me * cap + m], torch.where(own, ids - d * per, torch.full_like(ids, -1)))
        assert torch.equal(rw[d, me * cap:me * cap + m], torch.where(own, wts, torch.zeros_like(wts)))
        rows = own.any(dim=1)
        assert torch.equal(rx[d, me * cap:me * cap + m][rows], x[rows])
        assert (rid[d, me * cap + m:(me + 1) * cap] == -1).all()                         # rows beyond the batch are empty slots
    # the wait of "rank" 0 on peer 1's counter: already there -> passes at once; peer 0 never sent -> runs out
    one = flags[0, 1:2].contiguous()
    L.check(lib.b200moe_ep_wait(L.ptr(one), 1, cap, L.ptr(calls), L.ptr(status), L.stream_ptr()), "wait")
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(calls[0]) == 1
    L.check(lib.b200moe_ep_wait(L.ptr(flags[0].contiguous()), world, cap, L.ptr(calls[1:]), L.ptr(status), L.stream_ptr()), "wait")
    torch.cuda.synchronize()
    assert int(status.item()) == 1, "the peer whose counter nobody bumped is reported: status = 1 + its rank"
    # return path
    yl = torch.randn(world * cap, h, generator=torch.Generator(device="cuda").manual_seed(2), device="cuda").to(torch.bfloat16)
    back = torch.zeros(world, world, cap, h, dtype=torch.bfloat16, device="cuda")        # back[s]: the array of source s
    bflags = torch.zeros(world, world, dtype=torch.int32, device="cuda")
    L.check(lib.b200moe_ep_return(L.ptr(yl), world, cap, h, me, arr([back[s_].data_ptr() for s_ in range(world)]),
                                  arr([bflags[s_, me].data_ptr() for s_ in range(world)]), L.stream_ptr()), "return")
    torch.cuda.synchronize()
    for s_ in range(world):
        assert torch.equal(back[s_, me], yl[s_ * cap:(s_ + 1) * cap]) and int(bflags[s_, me]) == cap


def test_fused_peer_exchange_kernels_single_rank():
    """dispatch + wait and return + wait + combine as one launch each, with this GPU as its own only peer: the rows a call
    sends to itself come back summed (world 1: the sum is the row), call after call, with the counters never reset."""
    import ctypes as C
    import sm120fp4_b200._lib as L
    lib = L.lib()
    cap, h, k, experts = 8, 256, 4, 8
    g = torch.Generator().manual_seed(9)
    rx = torch.zeros(cap, h, dtype=torch.bfloat16, device="cuda")
    rid = torch.zeros(cap, k, dtype=torch.int32, device="cuda")
    rw = torch.zeros(cap, k, device="cuda")
    back = torch.zeros(1, cap, h, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")
    calls = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    arr = lambda v: (C.c_void_p * len(v))(*v)  # noqa: E731
    for call in range(3):
        m = 5 + call
        x = torch.randn(m, h, generator=g).to(torch.bfloat16).cuda()
        ids = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(m)]).to(torch.int32).cuda()
        wts = torch.rand(m, k, generator=g).cuda()
        out = torch.full((m, h), float("nan"), dtype=torch.bfloat16, device="cuda")
        L.check(lib.b200moe_ep_dispatch_wait(L.ptr(x), L.ptr(ids), L.ptr(wts), m, h, k, 1, experts, cap, arr([rx.data_ptr()]), arr([rid.data_ptr()]),
                                             arr([rw.data_ptr()]), arr([flags[0:].data_ptr()]), L.ptr(flags), L.ptr(calls), L.ptr(status),
                                             L.stream_ptr()), "dispatch_wait")
        yl = (rx.float() * 2).to(torch.bfloat16)                       # stands for the local layer
        L.check(lib.b200moe_ep_return_combine(L.ptr(yl), 1, cap, h, 0, arr([back.data_ptr()]), arr([flags[1:].data_ptr()]), L.ptr(flags[1:]),
                                              L.ptr(calls), L.ptr(status), L.ptr(back), m, L.ptr(out), L.stream_ptr()), "return_combine")
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and int(calls.item()) == call + 1 and flags.tolist() == [cap * (call + 1)] * 2
        assert torch.equal(rid[:m], ids) and torch.equal(rw[:m], wts) and torch.equal(rx[:m], x)
        assert torch.equal(out, (x.float() * 2).to(torch.bfloat16))


def _ll_rank(cap, h, k, world):
    """Buffers of one rank of the flagged-word exchange, as b200moe_ep_dispatch_ll / _return_combine_ll take them."""
    words, hw = h // 2 + 2 * k, h // 2
    z = lambda *shape, dt=torch.int32: torch.zeros(*shape, dtype=dt, device="cuda")  # noqa: E731
    return dict(ll_in=z(world, cap, words, 2), ll_back=z(world * cap * hw + world, 2), rx=z(world * cap, h, dt=torch.bfloat16),
                rid=z(world * cap, k), rw=z(world * cap, k, dt=torch.float32), calls=z(2), status=z(1), words=words, hw=hw)


def _ll_call(lib, L, ranks, r, x, ids, wts, cap, h, k, per, phase, yl=None, out=None):
    import ctypes as C
    arr = lambda v: (C.c_void_p * len(v))(*v)  # noqa: E731
    me, world, m = ranks[r], len(ranks), x.shape[0]
    if phase == "dispatch":
        peers = arr([p["ll_in"].data_ptr() + r * cap * me["words"] * 8 for p in ranks])
        L.check(lib.b200moe_ep_dispatch_ll(L.ptr(x), L.ptr(ids), L.ptr(wts), m, h, k, world, per, cap, peers, L.ptr(me["ll_in"]), L.ptr(me["rx"]),
                                           L.ptr(me["rid"]), L.ptr(me["rw"]), L.ptr(me["calls"]), L.ptr(me["status"]), L.stream_ptr()), "dispatch_ll")
    else:
        peers = arr([p["ll_back"].data_ptr() + r * cap * me["hw"] * 8 for p in ranks])
        L.check(lib.b200moe_ep_return_combine_ll(L.ptr(yl), L.ptr(me["rid"]), world, cap, h, k, r, per, peers, L.ptr(me["ll_back"]), L.ptr(ids), m,
                                                 L.ptr(out), L.ptr(me["calls"]), L.ptr(me["status"]), L.stream_ptr()), "return_combine_ll")
    torch.cuda.synchronize()
    return int(me["status"].item())


def test_flagged_word_exchange_single_rank():
    """The flagged-word form of the peer-store exchange with this GPU as its own only peer: what a call sends to itself
    arrives in the plain arrays and comes back summed, call after call, masked slots and an empty batch included."""
    import sm120fp4_b200._lib as L
    lib = L.lib()
    cap, h, k, experts = 8, 256, 4, 8
    g = torch.Generator().manual_seed(19)
    ranks = [_ll_rank(cap, h, k, 1)]
    for call, m in enumerate((5, 8, 0, 3)):
        x = torch.randn(m, h, generator=g).to(torch.bfloat16).cuda()
        ids = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(max(m, 1))]).to(torch.int32)[:m]
        if m:
            ids[0, 1:] = -1          # a token with one live slot
            ids[m - 1, :] = -1       # a token with none: its row does not travel and its output is zero
        ids = ids.cuda()
        wts = torch.rand(m, k, generator=g).cuda()
        out = torch.full((m, h), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert _ll_call(lib, L, ranks, 0, x, ids, wts, cap, h, k, experts, "dispatch") == 0
        me = ranks[0]
        live = (ids >= 0).any(1)
        assert torch.equal(me["rid"][:m], ids) and torch.equal(me["rw"][:m][ids >= 0], wts[ids >= 0]) and not me["rw"][:m][ids < 0].any()
        assert (me["rid"][m:] == -1).all() and torch.equal(me["rx"][:m][live], x[live])
        yl = (me["rx"].float() * 2).to(torch.bfloat16)                       # stands for the local layer
        assert _ll_call(lib, L, ranks, 0, x, ids, wts, cap, h, k, experts, "return", yl=yl, out=out) == 0
        assert me["calls"].tolist() == [call + 1, call + 1]
        want = torch.where(live[:, None], (x.float() * 2).to(torch.bfloat16), torch.zeros_like(x))
        assert torch.equal(out, want)
    # blocks of more rows than a grid can hold resident are refused before anything is launched
    big = _ll_rank(2048, h, k, 1)
    x, ids, wts = torch.zeros(1, h, dtype=torch.bfloat16, device="cuda"), torch.zeros(1, k, dtype=torch.int32, device="cuda"), torch.zeros(1, k, device="cuda")
    with pytest.raises(L.B200MoEError, match="maximum"):
        _ll_call(lib, L, [big], 0, x, ids, wts, 2048, h, k, experts, "dispatch")


def test_flagged_word_exchange_two_ranks_one_after_the_other():
    """Two ranks' buffers on one GPU, their kernels run one after the other (never at the same time): rank 1 goes first, finds
    nothing from rank 0 and gives up after its bounded wait with the status word naming rank 0 - the context stays usable;
    rank 0 then finds rank 1's words in place and completes, and rank 1 repeats its call to pick up rank 0's rows. Checks the
    cross-rank addressing, the rank-order sum and that a peer that never arrives is an error status, not a hang."""
    import sm120fp4_b200._lib as L
    lib = L.lib()
    cap, h, k, experts, world = 4, 256, 4, 8, 2
    per = experts // world
    g = torch.Generator().manual_seed(23)
    ranks = [_ll_rank(cap, h, k, world) for _ in range(world)]
    batch = []
    for r in range(world):
        m = 3 + r
        x = torch.randn(m, h, generator=g).to(torch.bfloat16).cuda()
        ids = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(m)]).to(torch.int32)
        ids[0] = torch.tensor([0, 1, 2, 3] if r == 0 else [4, 5, 6, 7], dtype=torch.int32)   # a token all of whose experts sit on one rank
        batch.append((x, ids.cuda(), torch.rand(m, k, generator=g).cuda()))
    assert _ll_call(lib, L, ranks, 1, *batch[1], cap, h, k, per, "dispatch") == 1     # 1 + rank 0: its words never came
    ranks[1]["status"].zero_()
    assert _ll_call(lib, L, ranks, 0, *batch[0], cap, h, k, per, "dispatch") == 0
    assert _ll_call(lib, L, ranks, 1, *batch[1], cap, h, k, per, "dispatch") == 0     # the same call again: now rank 0's words are there
    me = ranks[0]
    for src in range(world):
        x, ids, wts = batch[src]
        m = x.shape[0]
        mine = (ids >= 0) & (ids // per == 0)
        blk = slice(src * cap, src * cap + m)
        assert torch.equal(me["rid"][blk], torch.where(mine, ids, torch.full_like(ids, -1)))
        assert torch.equal(me["rw"][blk], torch.where(mine, wts, torch.zeros_like(wts)))
        assert torch.equal(me["rx"][blk][mine.any(1)], x[mine.any(1)])
        assert (me["rid"][src * cap + m:(src + 1) * cap] == -1).all()
    outs = []
    for r in (1, 0):   # rank 1 first again: it returns its partial rows, then waits in vain for rank 0's
        x, ids, wts = batch[r]
        yl = (ranks[r]["rx"].float() * (2 + r)).to(torch.bfloat16)    # rank r's "layer": (2 + r) * x
        out = torch.full_like(x, float("nan"))
        st = _ll_call(lib, L, ranks, r, x, ids, wts, cap, h, k, per, "return", yl=yl, out=out)
        assert st == (1 if r == 1 else 0)
        outs.append(out)
    x, ids, _ = batch[0]
    on0, on1 = ((ids // per) == 0).any(1), ((ids // per) == 1).any(1)
    want = (torch.where(on0[:, None], (x.float() * 2).to(torch.bfloat16).float(), torch.zeros_like(x, dtype=torch.float32))
            + torch.where(on1[:, None], (x.float() * 3).to(torch.bfloat16).float(), torch.zeros_like(x, dtype=torch.float32))).to(torch.bfloat16)
    assert torch.equal(outs[1], want)
    assert ranks[0]["calls"].tolist() == [1, 1]
