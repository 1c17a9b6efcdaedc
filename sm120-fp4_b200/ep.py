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
constant number of rows so that nothing has to come back to the host and the call is CUDA-graph capturable. The
fixed-capacity exchange has two transports: one packed NCCL all-to-all each way (rows, ids and weights in one buffer), or -
`transport="peer"`, when the ranks can map one another's memory - kernels that store the rows straight into the destination
GPU's memory over NVLink as flagged words (4 bytes of payload + the call number in every 8-byte store, so nothing waits for
an acknowledgement across the link), with a bounded wait on the receiving side (no NCCL call, no multicast; a peer that
never arrives shows up as an error status, not as a hang). `transport="peer_fence"` is the same exchange with plain rows,
a system-scope fence and arrival counters.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


PEER_MAX_BLOCKS = 1024   # rows x ranks the peer-store kernels take (their grids must be resident as a whole on every rank)


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
                 group=None, capacity: int | None = None, transport: str = "nccl"):
        self.local_forward, self.E, self.k = local_forward, num_experts, top_k
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.lo, self.hi = shard_range(num_experts, self.rank, self.world)
        self.capacity = capacity
        if transport not in ("nccl", "peer", "peer_fence"):
            raise ValueError("transport is 'nccl', 'peer' or 'peer_fence'")
        self.transport = transport if (capacity is not None and self.world > 1) else "nccl"
        self.last_sent_rows = 0   # rows this rank dispatched in the last call (for traffic accounting)
        try:
            import inspect
            self._lf_out = "out" in inspect.signature(local_forward).parameters
        except (TypeError, ValueError):
            self._lf_out = False

    # -------------------------------------------------------------------------------------------- variable-size exchange
    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, out: torch.Tensor | None = None,
                rows: int | None = None) -> torch.Tensor:
        if self.capacity is not None:
            return self.forward_fixed(x, topk_ids, topk_weights, out, rows)
        if self.world == 1:   # one rank owns every expert: nothing to dispatch
            self.last_sent_rows = 0
            y = self.local_forward(x, topk_ids, topk_weights)
            return y if out is None else out.copy_(y)
        y = self._forward_variable(x, topk_ids, topk_weights)
        return y if out is None else out.copy_(y)

    def _forward_variable(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
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
        max_rows = m * min(world, k)   # a rank with an empty batch (m == 0) sends nothing but takes part in every collective
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
    def forward_fixed(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, out: torch.Tensor | None = None,
                      rows: int | None = None) -> torch.Tensor:
        """Every (source, destination) block holds exactly `rows` rows (default: `capacity`; at least the tokens of any rank's
        batch, and THE SAME NUMBER ON EVERY RANK - engines that pad decode batches to a common size pass that size, so that a
        destination runs world x rows rows and not world x capacity): row t of the block is token t, its slots masked to -1
        when the destination owns none of its experts. No host synchronisation and no allocation after the first call of a
        shape: the call can be captured into a CUDA graph. On a CUDA device the dispatch, the unpacking and the combine are one
        library kernel each; on the CPU (gloo tests) the same arithmetic runs in torch."""
        m, h = x.shape
        c = self.capacity if rows is None else int(rows)
        if m > c or c > self.capacity:
            raise ValueError(f"batch of {m} tokens / block of {c} rows exceeds the dispatch capacity {self.capacity}")
        if self.transport != "nccl" and c * self.world > PEER_MAX_BLOCKS:
            raise ValueError(f"the peer-store exchange takes decode-sized blocks (rows x ranks <= {PEER_MAX_BLOCKS}, got {c} x {self.world}): "
                             "its kernels wait for the peers' kernels block by block; use transport='nccl' or the variable-size exchange")
        per = self.E // self.world
        self.last_sent_rows = self.world * c
        if not x.is_cuda:
            y = self._forward_fixed_torch(x, topk_ids, topk_weights, c)
            return y if out is None else out.copy_(y)
        from . import _lib
        lib = _lib.lib()
        b = self._buffers(c, h, x.device, x.dtype)
        ids = topk_ids if topk_ids.dtype == torch.int32 and topk_ids.is_contiguous() else topk_ids.to(torch.int32).contiguous()
        wts = topk_weights if topk_weights.dtype == torch.float32 and topk_weights.is_contiguous() else topk_weights.to(torch.float32).contiguous()
        if not x.is_contiguous():
            x = x.contiguous()
        st = torch.cuda.current_stream(x.device).cuda_stream
        w, k = self.world, self.k
        if b.peer == "ll":   # flagged words stored straight into the peers' receive areas; the kernel completes when the peers' rows are here
            _lib.check(lib.b200moe_ep_dispatch_ll(x.data_ptr(), ids.data_ptr(), wts.data_ptr(), m, h, k, w, per, c, b.peers_in, b.ll_in,
                                                  b.rx.data_ptr(), b.rid.data_ptr(), b.rw.data_ptr(), b.calls.data_ptr(), b.status.data_ptr(), st),
                       "ep dispatch")
        elif b.peer:   # rows stored straight into the peers' receive arrays, counters after a system-scope fence
            _lib.check(lib.b200moe_ep_dispatch_wait(x.data_ptr(), ids.data_ptr(), wts.data_ptr(), m, h, k, w, per, c, b.dst_x, b.dst_ids, b.dst_wts,
                                                    b.dst_flag, b.flags_in.data_ptr(), b.calls.data_ptr(), b.status.data_ptr(), st), "ep dispatch")
        else:
            _lib.check(lib.b200moe_ep_dispatch(x.data_ptr(), ids.data_ptr(), wts.data_ptr(), m, h, k, w, per, c, b.dst_x, b.dst_ids, b.dst_wts,
                                               b.dst_flag, st), "ep dispatch")
            if w > 1:
                dist.all_to_all_single(b.rbuf, b.sbuf, group=self.group)
        if not b.peer:   # split the received blocks (world == 1: the send buffer itself) into the arrays the layer call takes
            src = b.rbuf if w > 1 else b.sbuf
            _lib.check(lib.b200moe_ep_unpack(src.data_ptr(), b.block_bytes, w, c, h, k, b.rx.data_ptr(), b.rid.data_ptr(), b.rw.data_ptr(), st),
                       "ep unpack")
        if self._lf_out:
            yl = self.local_forward(b.rx, b.rid, b.rw, out=b.yl)
        else:
            yl = self.local_forward(b.rx, b.rid, b.rw)
        if out is None:
            out = torch.empty(m, h, dtype=x.dtype, device=x.device)
        if b.peer == "ll":   # partial rows back as flagged words, wait for this rank's own, sum in rank order: one launch
            _lib.check(lib.b200moe_ep_return_combine_ll(yl.data_ptr(), b.rid.data_ptr(), w, c, h, k, self.rank, per, b.peers_back, b.ll_back,
                                                        ids.data_ptr(), m, out.data_ptr(), b.calls.data_ptr(), b.status.data_ptr(), st), "ep return")
            return out
        if b.peer:   # partial rows back to their sources, wait for this rank's own, sum in rank order: one launch
            _lib.check(lib.b200moe_ep_return_combine(yl.data_ptr(), w, c, h, self.rank, b.back_y, b.back_flag, b.flags_back.data_ptr(),
                                                     b.calls.data_ptr(), b.status.data_ptr(), b.y.data_ptr(), m, out.data_ptr(), st), "ep return")
            return out
        if w == 1:
            y = yl
        else:
            dist.all_to_all_single(b.y.view(-1, h), yl.view(-1, h), group=self.group)
            y = b.y
        _lib.check(lib.b200moe_ep_combine(y.data_ptr(), m, h, w, c, out.data_ptr(), st), "ep combine")
        return out

    def status(self) -> None:
        """Synchronise and raise if a bounded wait of the peer-store exchange ran out (a peer's rows never arrived)."""
        for b in getattr(self, "_bufs", {}).values():
            if b.peer:
                v = int(b.status.item())
                if v:
                    b.status.zero_()
                    raise RuntimeError(f"expert-parallel exchange: rank {v - 1} did not deliver its rows within the wait limit")

    def _buffers(self, c: int, h: int, device, dtype):
        key = (c, h, str(device), dtype)
        bufs = self.__dict__.setdefault("_bufs", {})
        if key in bufs:
            return bufs[key]
        import ctypes as C
        from types import SimpleNamespace
        w, k = self.world, self.k
        block = c * (h * 2 + k * 8)
        block = (block + 255) // 256 * 256
        z = lambda *shape, dt: torch.zeros(*shape, dtype=dt, device=device)  # noqa: E731
        b = SimpleNamespace(block_bytes=block, peer=False, rx=None, rid=None, rw=None, y=None,
                            yl=z(w * c, h, dt=dtype), dst_flag=None)
        parr = lambda vals: (C.c_void_p * len(vals))(*vals)  # noqa: E731
        if self.transport in ("peer", "peer_fence"):
            try:
                if self.transport == "peer":
                    self._peer_ll_buffers(b, c, h, device, dtype, parr)
                else:
                    self._peer_buffers(b, c, h, device, dtype, parr)
            except Exception as ex:  # noqa: BLE001 - no peer mapping on this system: fall back to the NCCL transport, loudly
                import sys
                print(f"expert-parallel peer transport unavailable ({type(ex).__name__}: {ex}); using the NCCL exchange", file=sys.stderr)
                b.peer = False
        if self.transport in ("peer", "peer_fence") and self.world > 1:
            ok = torch.tensor([1 if b.peer else 0], dtype=torch.int32, device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
            if not int(ok.item()):
                b.peer = False
        if not b.peer:
            b.sbuf, b.rbuf = z(w, block, dt=torch.uint8), z(w, block, dt=torch.uint8)
            b.rx, b.rid, b.rw = z(w * c, h, dt=dtype), z(w * c, k, dt=torch.int32), z(w * c, k, dt=torch.float32)
            b.y = z(w, c, h, dt=dtype)
            base = b.sbuf.data_ptr()
            b.dst_x = parr([base + d * block for d in range(w)])
            b.dst_ids = parr([base + d * block + c * h * 2 for d in range(w)])
            b.dst_wts = parr([base + d * block + c * h * 2 + c * k * 4 for d in range(w)])
            b.dst_flag = None
        bufs[key] = b
        self._buf = b   # the most recent set (what tests and tools look at)
        return b

    def _peer_buffers(self, b, c, h, device, dtype, parr) -> None:
        """One symmetric allocation per rank: [rx | rid | rw | back | flags_in | flags_back], mapped into every peer."""
        import torch.distributed._symmetric_memory as symm
        w, k = self.world, self.k
        n_rx, n_id = w * c * h * 2, w * c * k * 4
        off_rid, off_rw, off_back = n_rx, n_rx + n_id, n_rx + 2 * n_id
        off_fin = off_back + w * c * h * 2
        off_fback = off_fin + 256
        total = off_fback + 256
        buf = symm.empty(total, dtype=torch.uint8, device=device)
        buf.zero_()
        hdl = symm.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
        torch.cuda.synchronize(device)
        hdl.barrier()
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        b.symm, b.handle = buf, hdl
        b.rx = buf[:n_rx].view(dtype).view(w * c, h)
        b.rid = buf[off_rid:off_rid + n_id].view(torch.int32).view(w * c, k)
        b.rw = buf[off_rw:off_rw + n_id].view(torch.float32).view(w * c, k)
        b.y = buf[off_back:off_back + w * c * h * 2].view(dtype).view(w, c, h)
        b.flags_in = buf[off_fin:off_fin + 4 * w].view(torch.int32)
        b.flags_back = buf[off_fback:off_fback + 4 * w].view(torch.int32)
        b.calls = torch.zeros(2, dtype=torch.int32, device=device)
        b.status = torch.zeros(1, dtype=torch.int32, device=device)
        r = self.rank
        # my block inside destination d's arrays starts at row r * c
        b.dst_x = parr([ptrs[d] + r * c * h * 2 for d in range(w)])
        b.dst_ids = parr([ptrs[d] + off_rid + r * c * k * 4 for d in range(w)])
        b.dst_wts = parr([ptrs[d] + off_rw + r * c * k * 4 for d in range(w)])
        b.dst_flag = parr([ptrs[d] + off_fin + 4 * r for d in range(w)])
        b.back_y = parr([ptrs[s] + off_back for s in range(w)])
        b.back_flag = parr([ptrs[s] + off_fback + 4 * r for s in range(w)])
        b.peer = True

    def _peer_ll_buffers(self, b, c, h, device, dtype, parr) -> None:
        """The flagged-word exchange: one symmetric allocation per rank, [receive area | return area + markers], mapped into
        every peer; the arrays the layer call reads (rx, rid, rw) are ordinary local tensors the dispatch kernel fills."""
        import torch.distributed._symmetric_memory as symm
        w, k = self.world, self.k
        words, hw = h // 2 + 2 * k, h // 2
        n_in, n_back = w * c * words * 8, (w * c * hw + w) * 8
        buf = symm.empty(n_in + n_back, dtype=torch.uint8, device=device)
        buf.zero_()
        hdl = symm.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
        torch.cuda.synchronize(device)
        hdl.barrier()
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        r = self.rank
        b.symm, b.handle = buf, hdl
        b.ll_in, b.ll_back = ptrs[r], ptrs[r] + n_in
        b.peers_in = parr([ptrs[d] + r * c * words * 8 for d in range(w)])            # my block inside rank d's receive area
        b.peers_back = parr([ptrs[s] + n_in + r * c * hw * 8 for s in range(w)])      # my block inside rank s's return area
        z = lambda *shape, dt: torch.zeros(*shape, dtype=dt, device=device)  # noqa: E731
        b.rx, b.rid, b.rw = z(w * c, h, dt=dtype), z(w * c, k, dt=torch.int32), z(w * c, k, dt=torch.float32)
        b.calls = torch.zeros(2, dtype=torch.int32, device=device)
        b.status = torch.zeros(1, dtype=torch.int32, device=device)
        b.peer = "ll"

    def _forward_fixed_torch(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, c: int) -> torch.Tensor:
        m, h = x.shape
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
