"""Expert-parallel harness around ``gmm``: experts are sharded across ranks,
token rows travel to the rank that owns their expert with one all-to-all
(dispatch), the local grouped GEMM runs, and results travel back (combine).

The reference has no multi-GPU code; this is the exchange step either side of
its operator for callers that shard experts (one process per GPU,
``torch.distributed``; NCCL over NVLink on GPUs, gloo on CPU for tests).

Layout after dispatch on a rank: rows grouped by local expert (the contiguous
layout ``gmm`` needs, grouped_gemm/ops_test.py:44-53), within an expert ordered
by source rank, within a source rank in that rank's (token, slot) order.

All split sizes are fixed when the plan is built (one small all-to-all of counts
plus one host read).  ``dispatch`` / ``combine`` themselves never synchronise
with the host, so a plan built once for a routing can be replayed every step.
"""
from dataclasses import dataclass
from typing import List

import torch
import torch.distributed as dist


@dataclass
class Plan:
    """Everything ``dispatch`` / ``combine`` need, for one routing."""
    world_size: int
    rank: int
    top_k: int
    num_tokens: int
    experts_per_rank: int
    send_order: torch.Tensor       # [tokens*top_k] flat (token*top_k+slot) ids, sorted by expert
    send_token: torch.Tensor       # token index of each sent row
    send_splits: List[int]         # rows to each destination rank
    recv_splits: List[int]         # rows from each source rank
    regroup: torch.Tensor          # received-row index for each row of the expert-grouped layout
    batch_sizes: torch.Tensor      # int64 [experts_per_rank], on the data device
    batch_sizes_host: List[int]

    @property
    def local_rows(self):
        return int(sum(self.recv_splits))


def build_plan(expert_ids, num_experts, group=None):
    """``expert_ids``: int64 [tokens, top_k], global expert id chosen for each
    slot of each local token.  Rank r owns experts
    [r*num_experts/W, (r+1)*num_experts/W).  Collective: every rank of ``group``
    must call it."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    assert num_experts % world == 0, "experts must divide evenly across ranks"
    per_rank = num_experts // world
    tokens, top_k = expert_ids.shape
    device = expert_ids.device
    flat = expert_ids.reshape(-1)
    # stable: rows of one expert keep (token, slot) order
    send_order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts).view(world, per_rank)  # [dest, local expert]
    if world > 1:
        recv_counts = torch.empty_like(counts)  # [source, local expert]
        dist.all_to_all_single(recv_counts, counts, group=group)
    else:
        recv_counts = counts.clone()
    counts_host = counts.cpu()
    recv_host = recv_counts.cpu()
    send_splits = [int(v) for v in counts_host.sum(1).tolist()]
    recv_splits = [int(v) for v in recv_host.sum(1).tolist()]
    # Received rows arrive as [source][local expert][row]; regroup to
    # [local expert][source][row].
    src_base = torch.zeros(world, dtype=torch.int64)
    src_base[1:] = torch.cumsum(torch.tensor(recv_splits[:-1], dtype=torch.int64), 0) if world > 1 else 0
    within = torch.cumsum(recv_host, 1) - recv_host  # start of expert e inside source s's block
    pieces = []
    for e in range(per_rank):
        for s in range(world):
            n = int(recv_host[s, e])
            if n:
                start = int(src_base[s] + within[s, e])
                pieces.append(torch.arange(start, start + n, dtype=torch.int64))
    regroup = torch.cat(pieces) if pieces else torch.zeros(0, dtype=torch.int64)
    batch_sizes_host = [int(v) for v in recv_host.sum(0).tolist()]
    return Plan(
        world_size=world, rank=rank, top_k=top_k, num_tokens=tokens, experts_per_rank=per_rank,
        send_order=send_order, send_token=torch.div(send_order, top_k, rounding_mode="floor"),
        send_splits=send_splits, recv_splits=recv_splits, regroup=regroup.to(device),
        batch_sizes=torch.tensor(batch_sizes_host, dtype=torch.int64, device=device),
        batch_sizes_host=batch_sizes_host)


def _exchange(rows, out_splits, in_splits, group):
    out = rows.new_empty((int(sum(out_splits)),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows, out_splits, in_splits, group=group)
    return out


def dispatch(x, plan, group=None):
    """[tokens, h] -> [local_rows, h]: each token's row is sent once per chosen
    expert and arrives grouped by local expert."""
    send = x.index_select(0, plan.send_token)
    recv = _exchange(send, plan.recv_splits, plan.send_splits, group) if plan.world_size > 1 else send
    return recv.index_select(0, plan.regroup)


def dispatch_rows(rows, plan, group=None):
    """[tokens*top_k, h] (one row per (token, slot), e.g. the gradient of a
    ``combine(reduce=False)`` output) -> [local_rows, h]."""
    send = rows.index_select(0, plan.send_order)
    recv = _exchange(send, plan.recv_splits, plan.send_splits, group) if plan.world_size > 1 else send
    return recv.index_select(0, plan.regroup)


def combine(y, plan, group=None, weights=None, reduce=True):
    """Inverse of ``dispatch``: [local_rows, h] -> per-slot rows back on the rank
    that owns the token.  ``reduce=True`` sums a token's ``top_k`` rows (scaled by
    ``weights`` [tokens, top_k] if given) into [tokens, h]; ``reduce=False``
    returns [tokens*top_k, h] in (token, slot) order."""
    ungrouped = torch.empty_like(y)
    ungrouped.index_copy_(0, plan.regroup, y)
    back = _exchange(ungrouped, plan.send_splits, plan.recv_splits, group) if plan.world_size > 1 else ungrouped
    slots = torch.empty_like(back)
    slots.index_copy_(0, plan.send_order, back)
    if not reduce:
        return slots
    slots = slots.view(plan.num_tokens, plan.top_k, -1)
    if weights is not None:
        slots = slots * weights.unsqueeze(-1).to(slots.dtype)
    return slots.sum(1)


def expert_parallel_step(x, w, grad_rows, plan, gmm_fn, group=None):
    """One forward + backward of an expert-parallel projection, the unit that
    benchmark configuration 5 times: dispatch, local forward, combine; dispatch of the
    output gradient, local dgrad and wgrad, combine of dgrad.

    ``w``: this rank's experts [experts_per_rank, h_in, h_out]; ``grad_rows``:
    gradient w.r.t. the per-slot output rows [tokens*top_k, h_out].
    ``gmm_fn(a, b, batch_sizes, trans_a, trans_b)`` is the local grouped GEMM
    (``grouped_gemm_b200.backend.gmm`` on GPUs).
    Returns (out_rows [tokens*top_k, h_out], dx [tokens, h_in], dw like w)."""
    a = dispatch(x, plan, group)
    c = gmm_fn(a, w, plan.batch_sizes, False, False)
    out_rows = combine(c, plan, group, reduce=False)
    g = dispatch_rows(grad_rows, plan, group)
    da = gmm_fn(g, w, plan.batch_sizes, False, True)
    dw = gmm_fn(a, g, plan.batch_sizes, True, False)
    dx = combine(da, plan, group, reduce=True)
    return out_rows, dx, dw


# ---------------------------------------------------------------------------
# Peer-memory exchange: one pass per exchange instead of gather + all-to-all +
# regroup.  Each rank writes its rows straight into the expert-grouped buffer
# of the rank that owns the expert (and, on the way back, straight into the
# token owner's slot-ordered buffer) with ``b200gmm_push_rows`` over NVLink.
# ---------------------------------------------------------------------------
def interleave_by_destination(dest, rank, world):
    """Permutation that deals items round-robin over their destinations.

    ``dest[i]`` is the destination rank of item i.  In the returned order the
    n-th items of all destinations come before any (n+1)-th item, and within one
    round the destinations follow each other as rank+1, rank+2, ... (mod world),
    so that a kernel walking the items in order sends to every destination at
    once and no two ranks start on the same receiver.  Items of one destination
    keep their relative order."""
    dest = dest.to(torch.int64)
    counts = torch.bincount(dest, minlength=world)
    # n-th item of its destination, without assuming the items are grouped by destination
    by_dest = torch.argsort(dest, stable=True)
    start = torch.cumsum(counts, 0) - counts
    nth = torch.empty_like(dest)
    nth[by_dest] = torch.arange(dest.numel(), device=dest.device) - start[dest[by_dest]]
    turn = (dest - rank - 1) % world
    return torch.argsort(nth * world + turn, stable=True)


class PeerExchange:
    """Plan + symmetric buffers for one routing.

    Buffers (all in one symmetric allocation per rank, same size on every rank):
      ``a_grouped``  [cap, h_in]   dispatch target, rows grouped by local expert
      ``g_grouped``  [cap, h_out]  dispatch target for output gradients
      ``out_slots``  [pairs, h_out] combine target, (token, slot) order
      ``da_slots``   [pairs, h_in]  combine target for dgrad rows
    ``cap`` is the largest number of rows any rank receives, ``pairs`` the largest
    tokens*top_k of any rank.  Rows of expert e on its owner are ordered by source
    rank, then by the source's (token, slot) order: the same layout the
    all-to-all path produces.
    """

    def __init__(self, expert_ids, num_experts, h_in, h_out, group=None, dtype=torch.bfloat16,
                 single_rank=False, interleave_destinations=True):
        from grouped_gemm_b200 import _capi

        self._lib = _capi.load()
        self._check = _capi.check
        # single_rank: every expert is local to this process (also the mode used
        # when torch.distributed is not initialised); buffers are ordinary tensors.
        single_rank = single_rank or not dist.is_initialized()
        if not single_rank:
            self.group = group if group is not None else dist.group.WORLD
            self.world = dist.get_world_size(self.group)
            self.rank = dist.get_rank(self.group)
        else:
            self.group, self.world, self.rank = None, 1, 0
        assert num_experts % self.world == 0, "experts must divide evenly across ranks"
        self.per_rank = num_experts // self.world
        self.num_tokens, self.top_k = expert_ids.shape
        self.h_in, self.h_out, self.dtype = h_in, h_out, dtype
        device = expert_ids.device
        self.device = device
        esize = torch.empty(0, dtype=dtype).element_size()
        assert (h_in * esize) % 16 == 0 and (h_out * esize) % 16 == 0

        flat = expert_ids.reshape(-1)
        counts = torch.bincount(flat, minlength=num_experts)
        all_counts = torch.empty(self.world, num_experts, dtype=counts.dtype, device=device)
        if self.world > 1:
            dist.all_gather_into_tensor(all_counts, counts.contiguous(), group=self.group)
        else:
            all_counts[0] = counts
        C = all_counts.cpu()                                   # [source rank, global expert]
        per_expert = C.sum(0)                                  # rows of each expert, all sources
        owner = torch.arange(num_experts) // self.per_rank
        # first row of expert e inside its owner's buffer, then of source s inside e
        expert_base = torch.zeros(num_experts, dtype=torch.int64)
        for d in range(self.world):
            sl = slice(d * self.per_rank, (d + 1) * self.per_rank)
            expert_base[sl] = torch.cumsum(per_expert[sl], 0) - per_expert[sl]
        before_me = C[: self.rank].sum(0) if self.rank > 0 else torch.zeros(num_experts, dtype=torch.int64)
        my_offset = (expert_base + before_me).to(device)       # where this rank's rows of expert e start
        rows_per_rank = [int(per_expert[d * self.per_rank:(d + 1) * self.per_rank].sum()) for d in range(self.world)]
        self.local_rows = rows_per_rank[self.rank]
        self.cap = max(max(rows_per_rank), 1)
        pairs = torch.tensor([self.num_tokens * self.top_k], device=device)
        if self.world > 1:
            dist.all_reduce(pairs, op=dist.ReduceOp.MAX, group=self.group)
        self.pairs_cap = int(pairs.item())
        self.batch_sizes_host = [int(v) for v in per_expert[self.rank * self.per_rank:(self.rank + 1) * self.per_rank]]
        self.batch_sizes = torch.tensor(self.batch_sizes_host, dtype=torch.int64, device=device)

        # items in expert-sorted order (stable: (token, slot) order inside an expert)
        order = torch.argsort(flat, stable=True)
        e_sorted = flat[order]
        my_start = (torch.cumsum(counts, 0) - counts)          # start of expert e among this rank's sorted items
        within = torch.arange(order.numel(), device=device) - my_start[e_sorted]
        item_rank = e_sorted // self.per_rank                                  # owner of the item's expert
        item_row = my_offset[e_sorted] + within                                # row in the owner's grouped buffer
        # The push kernels walk the items in order, all thread blocks side by side.  In
        # expert order that would send every rank's rows to rank 0 first, then to rank 1,
        # ...: all senders on one receiver's links at a time, and this rank's own rows
        # (no link at all) in a phase of their own.  So the items are dealt round-robin
        # over the destinations instead, each rank starting with its right-hand
        # neighbour: every stretch of items then goes to all destinations at once.
        if interleave_destinations and self.world > 1:
            mix = interleave_by_destination(item_rank, self.rank, self.world)
            order, item_rank, item_row = order[mix], item_rank[mix], item_row[mix]
        self.item_pair = order.to(torch.int32)                                 # (token*top_k + slot) of each item
        self.item_token = torch.div(order, self.top_k, rounding_mode="floor").to(torch.int32)
        self.item_rank = item_rank.to(torch.int32)
        self.item_row = item_row.to(torch.int64)
        self.n_items = int(order.numel())

        # one symmetric allocation, carved into the four buffers + the origin table
        def align(n):
            return (n + 255) // 256 * 256
        sizes = [self.cap * h_in * esize, self.cap * h_out * esize, self.pairs_cap * h_out * esize,
                 self.pairs_cap * h_in * esize, self.cap * 16, self.cap * h_in * esize]
        offs, total = [], 0
        for n in sizes:
            offs.append(total)
            total += align(n)
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self._symm = symm_mem.empty(total, dtype=torch.uint8, device=device)
            self._hdl = symm_mem.rendezvous(self._symm, self.group)
            bases = [int(p) for p in self._hdl.buffer_ptrs]
        else:
            self._symm = torch.empty(total, dtype=torch.uint8, device=device)
            self._hdl = None
            bases = [self._symm.data_ptr()]

        def table(off):
            return torch.tensor([b + off for b in bases], dtype=torch.int64, device=device)

        def view(off, rows, cols, dt):
            n = rows * cols * torch.empty(0, dtype=dt).element_size()
            return self._symm[off:off + n].view(dt).view(rows, cols)

        self._t_a, self._t_g, self._t_out, self._t_da, self._t_origin, self._t_a2 = (table(o) for o in offs)
        self.a_grouped = view(offs[0], self.cap, h_in, dtype)
        self.a_grouped2 = view(offs[5], self.cap, h_in, dtype)   # target of an activation dispatch sent a step ahead
        self.g_grouped = view(offs[1], self.cap, h_out, dtype)
        self.out_slots = view(offs[2], self.pairs_cap, h_out, dtype)
        self.da_slots = view(offs[3], self.pairs_cap, h_in, dtype)
        origin = view(offs[4], self.cap, 4, torch.int32)

        # Tell each owner where its rows came from: push (source rank, pair) records
        # along the dispatch route once; the way back reuses them.
        rec = torch.zeros(self.n_items, 4, dtype=torch.int32, device=device)
        rec[:, 0] = self.rank
        rec[:, 1] = self.item_pair
        self.barrier()
        self._push(rec, None, self.item_rank, self.item_row, self._t_origin)
        self.barrier()
        self.back_rank = origin[: self.local_rows, 0].contiguous()
        self.back_row = origin[: self.local_rows, 1].to(torch.int64).contiguous()
        # Final address of every grouped row on the rank that owns its token, for
        # the GEMMs that write their result straight there (step_fused).
        out_bases = self._t_out[self.back_rank.long()]
        da_bases = self._t_da[self.back_rank.long()]
        self.dest_out = (out_bases + self.back_row * (h_out * esize)).contiguous()
        self.dest_da = (da_bases + self.back_row * (h_in * esize)).contiguous()
        self._ws_bytes = _capi.workspace_bytes(self.per_rank)
        self._status = torch.zeros(1, dtype=torch.int32, device=device)
        # step_fused(..., timeline=True) leaves here the CUDA events that bracket its
        # phases (see phase_times)
        self._marks = None
        # step_fused(x_next=...): (the tensor whose rows were sent ahead, its version, buffer index)
        self._ahead = None
        self._cur = 0            # which a_grouped buffer step_fused reads

    # -- plumbing ---------------------------------------------------------------
    def barrier(self):
        """Every rank's earlier work on the current stream is complete, and visible
        to its peers, before any rank's later work starts (stream-ordered)."""
        if self.world > 1:
            self._hdl.barrier()

    def _push(self, src, src_row, dst_rank, dst_row, table, max_ctas=0):
        n_items = int(dst_rank.numel())
        row_bytes = src.shape[1] * src.element_size()
        rc = self._lib.b200gmm_push_rows(
            src.data_ptr(), row_bytes, n_items, 0 if src_row is None else src_row.data_ptr(),
            dst_rank.data_ptr(), dst_row.data_ptr(), table.data_ptr(), int(max_ctas),
            torch.cuda.current_stream(self.device).cuda_stream)
        self._check(rc, "b200gmm_push_rows")

    # -- exchanges --------------------------------------------------------------
    def dispatch(self, x):
        """[tokens, h_in] -> this rank's grouped rows [local_rows, h_in]."""
        self._ahead = None   # rows sent ahead by step_fused may sit in this buffer
        self._push(x, self.item_token, self.item_rank, self.item_row, self._t_a)
        self.barrier()
        return self.a_grouped[: self.local_rows]

    def dispatch_rows(self, rows):
        """[tokens*top_k, h_out] per-slot rows -> grouped rows [local_rows, h_out]."""
        self._push(rows, self.item_pair, self.item_rank, self.item_row, self._t_g)
        self.barrier()
        return self.g_grouped[: self.local_rows]

    def combine_rows(self, y):
        """Grouped rows [local_rows, h_out] -> per-slot rows on the token owners."""
        self._push(y, None, self.back_rank, self.back_row, self._t_out)
        self.barrier()
        return self.out_slots[: self.num_tokens * self.top_k]

    def combine_reduce(self, y):
        """Grouped rows [local_rows, h_in] -> [tokens, h_in], summed over a token's slots."""
        self._push(y, None, self.back_rank, self.back_row, self._t_da)
        self.barrier()
        return self._sum_slots(self.da_slots)

    def _sum_slots(self, slots):
        """[tokens * top_k, h] per-slot rows -> [tokens, h]: a token's rows added in
        fp32, rounded once (``b200gmm_sum_slots``)."""
        h = slots.shape[1]
        out = torch.empty(self.num_tokens, h, dtype=slots.dtype, device=self.device)
        if self.top_k > 8 or slots.dtype != torch.bfloat16:
            return slots[: self.num_tokens * self.top_k].view(self.num_tokens, self.top_k, h).sum(1)
        rc = self._lib.b200gmm_sum_slots(slots.data_ptr(), out.data_ptr(), self.num_tokens, self.top_k, h,
                                         torch.cuda.current_stream(self.device).cuda_stream)
        self._check(rc, "b200gmm_sum_slots")
        return out

    def step(self, x, w, grad_rows, gmm_fn):
        """Same unit of work as ``expert_parallel_step``, over peer memory: four
        row pushes, each followed by a barrier.  Starts with a barrier, so that
        whatever an earlier step still reads on any rank is done before this one
        overwrites the buffers."""
        self.barrier()
        a = self.dispatch(x)
        c = gmm_fn(a, w, self.batch_sizes, False, False)
        out_rows = self.combine_rows(c)
        g = self.dispatch_rows(grad_rows)
        da = gmm_fn(g, w, self.batch_sizes, False, True)
        dw = gmm_fn(a, g, self.batch_sizes, True, False)
        dx = self.combine_reduce(da)
        return out_rows, dx, dw

    def _gmm_scatter(self, a, w, dest, trans_b, push=None):
        """Local grouped GEMM whose epilogue writes row i to address dest[i].
        ``push`` = (src, src_row, dst_rank, dst_row, table): rows the same launch
        moves to their owners with its push warps while the product runs."""
        n = w.shape[1] if trans_b else w.shape[2]
        ws = torch.empty(self._ws_bytes, dtype=torch.uint8, device=self.device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        if push is None:
            rc = self._lib.b200gmm_run_scatter(
                a.data_ptr(), w.data_ptr(), dest.data_ptr(), None, 0,   # addresses in peer buffers: table built here
                self.batch_sizes.data_ptr(), 1,
                self.per_rank, a.shape[0], a.shape[1], n, 1 if trans_b else 0,
                ws.data_ptr(), self._ws_bytes, self._status.data_ptr(), stream)
            self._check(rc, "b200gmm_run_scatter")
            return
        src, src_row, dst_rank, dst_row, table = push
        rc = self._lib.b200gmm_run_scatter_push(
            a.data_ptr(), w.data_ptr(), dest.data_ptr(), None, 0,
            self.batch_sizes.data_ptr(), 1,
            self.per_rank, a.shape[0], a.shape[1], n, 1 if trans_b else 0,
            src.data_ptr(), src.shape[1] * src.element_size(), int(dst_rank.numel()),
            0 if src_row is None else src_row.data_ptr(), dst_rank.data_ptr(), dst_row.data_ptr(), table.data_ptr(),
            ws.data_ptr(), self._ws_bytes, self._status.data_ptr(), stream)
        self._check(rc, "b200gmm_run_scatter_push")

    def phase_times(self):
        """Milliseconds between the marks of the last ``step_fused(timeline=True)``
        on the stream (synchronises): how long each GEMM ran with whatever it
        waited for in front of it, the dispatches and the barriers."""
        if not self._marks:
            return {}
        torch.cuda.synchronize(self.device)
        names = [n for n, _ in self._marks]
        evs = [e for _, e in self._marks]
        return {f"{names[i]} -> {names[i + 1]}": evs[i].elapsed_time(evs[i + 1]) for i in range(len(evs) - 1)}

    def step_fused(self, x, w, grad_rows, gmm_fn, timeline=False, push_in_kernel=True, x_next=None):
        """``step`` with both combines folded into the GEMMs: the forward and the
        dgrad kernels send each result row from their epilogue straight into the
        token owner's buffer (over NVLink when the owner is another GPU), so no
        combine pass exists and the two dispatches are the only exchange passes.
        Same results as ``step``, bit for bit.

        ``push_in_kernel`` (default) moves the dispatches into the GEMM kernels as
        well: the forward kernel sends the gradient rows to the expert owners while
        its tensor cores work (``b200gmm_run_scatter_push``: one more thread per
        block issues bulk copies global -> shared -> peer), and given ``x_next``, the
        activations of the NEXT call, the dgrad kernel sends those (into a second
        buffer), so that the next call, if it is made with that same unmodified
        tensor, starts its forward product right after its entry barrier.  Every
        rank must make the same choice.  Measured on B200 against the two row pushes
        as kernels of their own: 3.7 % more throughput at 2 GPUs, 5.6 % at 4, 6.2 % at 8.

        Everything runs on the current stream, one kernel at a time.

        Cross-rank order: a barrier on entry (every rank has finished with the
        previous step's buffers), one after each dispatch (its rows have arrived),
        one at the end (the rows the epilogues sent have arrived)."""
        compute = torch.cuda.current_stream(self.device)
        pairs = self.num_tokens * self.top_k
        rows = self.local_rows
        marks = [] if timeline else None

        def mark(name):
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(compute)
                marks.append((name, ev))

        ahead, self._ahead = self._ahead, None
        sent_ahead = ahead is not None and ahead[0] is x and ahead[1] == x._version
        if sent_ahead:
            self._cur = ahead[2]
        a_buf, a_table = (self.a_grouped, self._t_a) if self._cur == 0 else (self.a_grouped2, self._t_a2)
        mark("start")
        self.barrier()                         # with rows sent ahead: they have arrived from every rank
        mark("entry barrier")
        if not sent_ahead:
            self._push(x, self.item_token, self.item_rank, self.item_row, a_table)
            self.barrier()
        mark("activations dispatched")
        a = a_buf[:rows]
        if push_in_kernel:
            self._gmm_scatter(a, w, self.dest_out, False,
                              push=(grad_rows, self.item_pair, self.item_rank, self.item_row, self._t_g))
            mark("forward")
        else:
            self._gmm_scatter(a, w, self.dest_out, False)
            mark("forward")
            self._push(grad_rows, self.item_pair, self.item_rank, self.item_row, self._t_g)
        self.barrier()                         # publishes the forward's rows and the gradient rows
        mark("gradient rows dispatched")
        g = self.g_grouped[:rows]
        if x_next is not None and push_in_kernel:
            nxt = 1 - self._cur
            self._gmm_scatter(g, w, self.dest_da, True,
                              push=(x_next, self.item_token, self.item_rank, self.item_row,
                                    self._t_a if nxt == 0 else self._t_a2))
            self._ahead = (x_next, x_next._version, nxt)
        else:
            self._gmm_scatter(g, w, self.dest_da, True)
        mark("dgrad")
        dw = gmm_fn(a, g, self.batch_sizes, True, False)
        mark("wgrad")
        self.barrier()                         # the rows both epilogues sent have arrived everywhere
        mark("final barrier")
        dx = self._sum_slots(self.da_slots)
        mark("top-k sum")
        self._marks = marks
        return self.out_slots[:pairs], dx, dw
