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
    BASELINE config 5 times: dispatch, local forward, combine; dispatch of the
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
