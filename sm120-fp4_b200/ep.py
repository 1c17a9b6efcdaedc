"""Expert-parallel MoE layer: experts sharded evenly over the ranks of one process group, tokens data-parallel.

The reference refuses expert parallelism (`fits()` returns False for `use_ep`, sm120fp4/vllm_classes.py:46-47; `apply` raises
on `expert_map`, :95-96); this is the layer it lacks, on NCCL all-to-all over NVLink.

Per layer call, on every rank:
  1. dispatch  - a token row travels ONCE to every rank that owns at least one of its top-k experts (not once per expert),
                 together with its top-k slots re-indexed to the destination's local experts; slots owned by other ranks
                 are masked with id -1 (the kernels skip negative ids) and weight 0.
  2. compute   - the destination runs its ordinary local layer (`Weights.forward`) on the received rows: the routing
                 weights are applied there and the row's local experts are already summed.
  3. combine   - one partial row per (token, destination) comes back; the source adds its partial rows in rank order in
                 fp32 (a fixed order: results are bit-identical call to call) and rounds once to bf16.
Rows are exchanged with `all_to_all_single`; the split sizes travel first as a tiny all-to-all of counts (one host
synchronisation per layer call), or - for decode batches - `capacity` fixes every (source, destination) block at a
constant number of rows so that nothing has to come back to the host and the call is CUDA-graph capturable.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def shard_range(num_experts: int, rank: int, world: int) -> tuple[int, int]:
    """Experts [lo, hi) owned by `rank`: an even split (the number of experts must divide by the world size)."""
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not split evenly over {world} ranks")
    per = num_experts // world
    return rank * per, (rank + 1) * per


def dispatch_plan(topk_ids: torch.Tensor, num_experts: int, world: int):
    """Routing tables of the dispatch, all on the device of `topk_ids`:
    send_tok  int64 [S]     token index of every row sent, grouped by destination rank (ascending), token order within
    counts    int64 [world] rows per destination
    local_ids int32 [S, k]  the row's top-k slots as the destination's local expert ids, -1 where another rank owns the slot
    """
    per = num_experts // world
    dest = torch.div(topk_ids, per, rounding_mode="floor")                     # [m, k]
    ranks = torch.arange(world, device=topk_ids.device)
    hit = (dest[:, None, :] == ranks[None, :, None])                            # [m, world, k]
    mask = hit.any(dim=2)                                                       # [m, world]
    dst_rank, send_tok = mask.t().nonzero(as_tuple=True)                        # rank-major, token ascending
    counts = mask.sum(dim=0)
    local = torch.where(hit[send_tok, dst_rank], (topk_ids[send_tok] - (dst_rank * per)[:, None]),
                        torch.full_like(topk_ids[send_tok], -1))
    return send_tok, counts, local.to(torch.int32), hit[send_tok, dst_rank]


class ExpertParallelMoE:
    """`forward(x, topk_ids, topk_weights)` with GLOBAL expert ids; `local_forward(x, local_ids, weights) -> bf16 rows` is the
    rank's own layer over its shard (e.g. `Weights.forward` built from experts [lo, hi))."""

    def __init__(self, local_forward: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor], num_experts: int, top_k: int,
                 group=None, capacity: int | None = None):
        self.local_forward, self.E, self.k = local_forward, num_experts, top_k
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.lo, self.hi = shard_range(num_experts, self.rank, self.world)
        self.capacity = capacity
        self.last_sent_rows = 0   # rows this rank dispatched in the last call (for traffic accounting)

    # -------------------------------------------------------------------------------------------- variable-size exchange
    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        if self.capacity is not None:
            return self.forward_fixed(x, topk_ids, topk_weights)
        if self.world == 1:   # one rank owns every expert: nothing to dispatch
            self.last_sent_rows = 0
            return self.local_forward(x, topk_ids, topk_weights)
        m, h = x.shape
        if x.is_cuda:
            return self._forward_variable_cuda(x, topk_ids, topk_weights)
        ids = topk_ids.to(torch.int64)
        wts = topk_weights.to(torch.float32)
        send_tok, counts, local_ids, own = dispatch_plan(ids, self.E, self.world)
        send_w = torch.where(own, wts[send_tok], torch.zeros_like(wts[send_tok]))
        if self.world == 1:
            out = self.local_forward(x[send_tok].contiguous(), local_ids, send_w)
            return self._combine(out, send_tok, counts, m, x.dtype)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=self.group)
        s_split, r_split = counts.tolist(), recv_counts.tolist()           # the one host synchronisation of the call
        self.last_sent_rows = int(sum(s_split))
        r_total = int(sum(r_split))
        rx = torch.empty(r_total, h, dtype=x.dtype, device=x.device)
        rid = torch.empty(r_total, self.k, dtype=torch.int32, device=x.device)
        rw = torch.empty(r_total, self.k, dtype=torch.float32, device=x.device)
        dist.all_to_all_single(rx, x[send_tok].contiguous(), r_split, s_split, group=self.group)
        dist.all_to_all_single(rid, local_ids.contiguous(), r_split, s_split, group=self.group)
        dist.all_to_all_single(rw, send_w.contiguous(), r_split, s_split, group=self.group)
        y = self.local_forward(rx, rid, rw) if r_total else rx
        back = torch.empty(int(sum(s_split)), h, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(back, y.contiguous(), s_split, r_split, group=self.group)
        return self._combine(back, send_tok, counts, m, x.dtype)

    def _forward_variable_cuda(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        """The variable-size exchange on a CUDA device: plan, gather and combine are one library kernel each; the only host
        synchronisation is the read of the split sizes (own counts and, after a tiny all-to-all, the peers')."""
        from . import _lib
        lib = _lib.lib()
        m, h = x.shape
        k, world, per, dev = self.k, self.world, self.E // self.world, x.device
        ids = topk_ids.to(torch.int32).contiguous()
        wts = topk_weights.to(torch.float32).contiguous()
        x = x.contiguous()
        max_rows = m * min(world, k)
        plan = torch.empty(2 * world + 1 + m * world + max_rows, dtype=torch.int32, device=dev)
        counts, offsets = plan[:world], plan[world:2 * world + 1]
        pos, send_tok = plan[2 * world + 1:2 * world + 1 + m * world], plan[2 * world + 1 + m * world:]
        st = _lib.stream_ptr()
        _lib.check(lib.b200moe_ep_plan(_lib.ptr(ids), m, k, world, per, _lib.ptr(counts), _lib.ptr(offsets), _lib.ptr(pos), _lib.ptr(send_tok), st),
                   "ep plan")
        both = torch.empty(2, world, dtype=torch.int32, device=dev)
        both[0] = counts
        dist.all_to_all_single(both[1], counts, group=self.group)
        s_split, r_split = both.tolist()                                   # the one host synchronisation of the call
        s_total, r_total = int(sum(s_split)), int(sum(r_split))
        self.last_sent_rows = s_total
        sx = torch.empty(max(s_total, 1), h, dtype=x.dtype, device=dev)
        smeta = torch.empty(max(s_total, 1), 2 * k, dtype=torch.int32, device=dev)
        _lib.check(lib.b200moe_ep_gather(_lib.ptr(x), _lib.ptr(ids), _lib.ptr(wts), _lib.ptr(send_tok), _lib.ptr(offsets), h, k, world, per,
                                         s_total, _lib.ptr(sx), _lib.ptr(smeta), st), "ep gather")
        rx = torch.empty(r_total, h, dtype=x.dtype, device=dev)
        rmeta = torch.empty(r_total, 2 * k, dtype=torch.int32, device=dev)
        dist.all_to_all_single(rx, sx[:s_total], r_split, s_split, group=self.group)
        dist.all_to_all_single(rmeta, smeta[:s_total], r_split, s_split, group=self.group)
        if r_total:
            y = self.local_forward(rx, rmeta[:, :k].contiguous(), rmeta[:, k:].contiguous().view(torch.float32))
        else:
            y = rx
        back = torch.empty(max(s_total, 1), h, dtype=x.dtype, device=dev)
        dist.all_to_all_single(back[:s_total], y.contiguous(), s_split, r_split, group=self.group)
        out = torch.empty(m, h, dtype=x.dtype, device=dev)
        _lib.check(lib.b200moe_ep_combine_rows(_lib.ptr(back), _lib.ptr(pos), m, h, world, _lib.ptr(out), _lib.stream_ptr()), "ep combine")
        return out

    def _combine(self, rows: torch.Tensor, send_tok: torch.Tensor, counts: torch.Tensor, m: int, dtype) -> torch.Tensor:
        """out[t] = sum over destinations (rank order) of the partial row that came back for t; fp32, one rounding."""
        out = torch.zeros(m, rows.shape[1], dtype=torch.float32, device=rows.device)
        ends = torch.cumsum(counts, 0).tolist() if self.world > 1 else [rows.shape[0]]
        start = 0
        for end in ends:                       # within one destination every token appears at most once: index_add is exact
            if end > start:
                out.index_add_(0, send_tok[start:end], rows[start:end].float())
            start = end
        return out.to(dtype)

    # -------------------------------------------------------------------------------------------- fixed-capacity exchange
    def forward_fixed(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        """Every (source, destination) block holds exactly `capacity` rows (>= the tokens of a rank's batch): row t of the
        block is token t, its slots masked to -1 when the destination owns none of its experts. No host synchronisation and
        no allocation after the first call of a shape: the call can be captured into a CUDA graph. On a CUDA device the
        dispatch and the combine are one library kernel each; on the CPU (gloo tests) the same arithmetic runs in torch."""
        m, h = x.shape
        c = self.capacity
        if m > c:
            raise ValueError(f"batch of {m} tokens exceeds the dispatch capacity {c}")
        per = self.E // self.world
        self.last_sent_rows = self.world * c
        if not x.is_cuda:
            return self._forward_fixed_torch(x, topk_ids, topk_weights)
        from . import _lib
        lib = _lib.lib()
        b = self._buffers(h, x.device, x.dtype)
        ids = topk_ids.to(torch.int32).contiguous()
        wts = topk_weights.to(torch.float32).contiguous()
        _lib.check(lib.b200moe_ep_dispatch(_lib.ptr(x.contiguous()), _lib.ptr(ids), _lib.ptr(wts), m, h, self.k, self.world, per, c,
                                           _lib.ptr(b.sx), _lib.ptr(b.smeta), _lib.stream_ptr()), "ep dispatch")
        if self.world == 1:
            rx, rmeta = b.sx, b.smeta
        else:
            dist.all_to_all_single(b.rx.view(-1, h), b.sx.view(-1, h), group=self.group)
            dist.all_to_all_single(b.rmeta.view(-1, 2 * self.k), b.smeta.view(-1, 2 * self.k), group=self.group)
            rx, rmeta = b.rx, b.rmeta
        rid = rmeta[:, :, :self.k].reshape(-1, self.k)
        rw = rmeta[:, :, self.k:].reshape(-1, self.k).view(torch.float32)
        yl = self.local_forward(rx.view(-1, h), rid, rw)
        if self.world == 1:
            y = yl
        else:
            dist.all_to_all_single(b.y.view(-1, h), yl.contiguous().view(-1, h), group=self.group)
            y = b.y
        out = torch.empty(m, h, dtype=x.dtype, device=x.device)
        _lib.check(lib.b200moe_ep_combine(_lib.ptr(y), m, h, self.world, c, _lib.ptr(out), _lib.stream_ptr()), "ep combine")
        return out

    def _buffers(self, h: int, device, dtype):
        key = (h, str(device), dtype)
        if getattr(self, "_buf_key", None) != key:
            from types import SimpleNamespace
            w, c, k = self.world, self.capacity, self.k
            mk = lambda *shape, dt: torch.zeros(*shape, dtype=dt, device=device)  # noqa: E731
            self._buf = SimpleNamespace(sx=mk(w, c, h, dt=dtype), rx=mk(w, c, h, dt=dtype), y=mk(w, c, h, dt=dtype),
                                        smeta=mk(w, c, 2 * k, dt=torch.int32), rmeta=mk(w, c, 2 * k, dt=torch.int32))
            self._buf_key = key
        return self._buf

    def _forward_fixed_torch(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        m, h = x.shape
        c = self.capacity
        per = self.E // self.world
        ids = topk_ids.to(torch.int64)
        wts = topk_weights.to(torch.float32)
        dest = torch.div(ids, per, rounding_mode="floor")
        ranks = torch.arange(self.world, device=x.device)
        own = (dest[None, :, :] == ranks[:, None, None]) & (ids[None] >= 0)                # [world, m, k]
        lid = torch.where(own, ids[None] - (ranks * per)[:, None, None], torch.full_like(ids[None].expand(self.world, -1, -1), -1))
        sw = torch.where(own, wts[None].expand(self.world, -1, -1), torch.zeros((), device=x.device))
        sx = torch.zeros(self.world, c, h, dtype=x.dtype, device=x.device)
        sid = torch.full((self.world, c, self.k), -1, dtype=torch.int32, device=x.device)
        swt = torch.zeros(self.world, c, self.k, dtype=torch.float32, device=x.device)
        sx[:, :m] = x[None]
        sid[:, :m] = lid.to(torch.int32)
        swt[:, :m] = sw
        if self.world == 1:
            y = self.local_forward(sx.view(-1, h), sid.view(-1, self.k), swt.view(-1, self.k)).view(1, c, h)
        else:
            rx, rid, rw = torch.empty_like(sx), torch.empty_like(sid), torch.empty_like(swt)
            dist.all_to_all_single(rx.view(-1, h), sx.view(-1, h), group=self.group)
            dist.all_to_all_single(rid.view(-1, self.k), sid.view(-1, self.k), group=self.group)
            dist.all_to_all_single(rw.view(-1, self.k), swt.view(-1, self.k), group=self.group)
            yl = self.local_forward(rx.view(-1, h), rid.view(-1, self.k), rw.view(-1, self.k))
            y = torch.empty_like(sx)
            dist.all_to_all_single(y.view(-1, h), yl.contiguous().view(-1, h), group=self.group)
        out = torch.zeros(m, h, dtype=torch.float32, device=x.device)
        for r in range(self.world):            # fixed rank order
            out += y[r, :m].float()
        return out.to(x.dtype)


def shard_weights(q1, s1, alpha1, q2, s2, alpha2, rank: int, world: int):
    """The slices of a full layer's tensors that `rank` owns (views; experts along dim 0)."""
    lo, hi = shard_range(q1.shape[0], rank, world)
    return q1[lo:hi], s1[lo:hi], alpha1[lo:hi], q2[lo:hi], s2[lo:hi], alpha2[lo:hi]
