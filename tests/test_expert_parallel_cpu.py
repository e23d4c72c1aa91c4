"""Expert-parallel dispatch / combine bookkeeping on CPU ranks (gloo,
world_size 2), with the CPU oracle standing in for the local grouped GEMM.
Checks the sharded result against the same computation done unsharded."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import gmm_oracle

Z, TOKENS, TOPK, H_IN, H_OUT = 8, 48, 2, 16, 24


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _global_problem():
    g = torch.Generator().manual_seed(11)
    x = torch.randn(TOKENS, H_IN, generator=g).bfloat16()
    w = (torch.randn(Z, H_IN, H_OUT, generator=g) * 0.25).bfloat16()
    # distinct experts per token, skewed so some experts get nothing from a rank
    ids = torch.stack([torch.randperm(Z - 2, generator=g)[:TOPK] for _ in range(TOKENS)])
    grad = torch.randn(TOKENS * TOPK, H_OUT, generator=g).bfloat16()
    return x, w, ids, grad


def _oracle_fn(a, b, bs, trans_a, trans_b):
    return gmm_oracle.gmm(a, b, bs, trans_a=trans_a, trans_b=trans_b)


def _unsharded():
    """Same step with every expert local: sort slots by expert, loop, unsort."""
    x, w, ids, grad = _global_problem()
    flat = ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    bs = torch.bincount(flat, minlength=Z)
    a = x[order // TOPK]
    c = gmm_oracle.gmm(a, w, bs)
    out_rows = torch.empty_like(c)
    out_rows[order] = c
    g = grad[order]
    da = gmm_oracle.gmm(g, w, bs, trans_b=True)
    dw = gmm_oracle.gmm(a, g, bs, trans_a=True)
    slots = torch.empty_like(da)
    slots[order] = da
    dx = slots.view(TOKENS, TOPK, -1).float().sum(1)
    return out_rows, dx, dw


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from grouped_gemm_b200 import expert_parallel as ep
        x, w, ids, grad = _global_problem()
        per = TOKENS // world
        sl = slice(rank * per, (rank + 1) * per)
        zs = slice(rank * Z // world, (rank + 1) * Z // world)
        plan = ep.build_plan(ids[sl], Z)
        assert sum(plan.send_splits) == per * TOPK
        assert plan.local_rows == sum(plan.batch_sizes_host)
        # round trip: dispatch then combine(reduce=False) returns each slot's own row
        a = ep.dispatch(x[sl], plan)
        back = ep.combine(a, plan, reduce=False)
        assert torch.equal(back, x[sl].repeat_interleave(TOPK, 0))
        out_rows, dx, dw = ep.expert_parallel_step(
            x[sl], w[zs].contiguous(), grad[sl.start * TOPK:sl.stop * TOPK], plan, _oracle_fn)
        results[rank] = (out_rows, dx.float(), dw, plan.batch_sizes_host)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_step_matches_unsharded():
    world = 2
    port = _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        got = [results[r] for r in range(world)]
    out_rows, dx, dw = _unsharded()
    per = TOKENS // world
    _, _, ids, _ = _global_problem()
    for r in range(world):
        o, d, w_r, bs_host = got[r]
        assert torch.equal(o, out_rows[r * per * TOPK:(r + 1) * per * TOPK]), "forward rows differ"
        assert torch.allclose(d, dx[r * per:(r + 1) * per], rtol=1e-2, atol=1e-2)
        assert bs_host == torch.bincount(ids.reshape(-1), minlength=Z)[r * Z // world:(r + 1) * Z // world].tolist()
    # wgrad: each rank's rows arrive grouped by source rank, the unsharded run has them in
    # global order; the sums agree up to bf16 rounding of a different summation order
    dw_sharded = torch.cat([got[r][2] for r in range(world)])
    assert torch.allclose(dw_sharded.float(), dw.float(), rtol=2e-2, atol=2e-2)


def test_single_process_plan_is_identity_exchange():
    from grouped_gemm_b200 import expert_parallel as ep
    x, w, ids, grad = _global_problem()
    plan = ep.build_plan(ids, Z)
    assert plan.world_size == 1 and plan.send_splits == [TOKENS * TOPK]
    out_rows, dx, dw = ep.expert_parallel_step(x, w, grad, plan, _oracle_fn)
    want_rows, want_dx, want_dw = _unsharded()
    assert torch.equal(out_rows, want_rows)
    assert torch.equal(dw, want_dw)
    assert torch.allclose(dx.float(), want_dx, rtol=1e-2, atol=1e-2)


def test_interleave_by_destination_round_robin():
    """The order in which a row push walks its items: a permutation; the n-th items
    of all destinations before any (n+1)-th; inside a round the destinations follow
    as rank+1, rank+2, ...; items of one destination keep their order."""
    import torch
    from grouped_gemm_b200.expert_parallel import interleave_by_destination
    g = torch.Generator().manual_seed(7)
    for world, rank, n in ((2, 0, 11), (4, 1, 257), (8, 7, 1000), (4, 3, 0), (3, 2, 5)):
        dest = torch.randint(0, world, (n,), generator=g)
        if n > 20:
            dest[dest == 2 % world] = (rank + 1) % world       # one destination gets (almost) nothing
        mix = interleave_by_destination(dest, rank, world)
        assert sorted(mix.tolist()) == list(range(n))
        d = dest[mix].tolist()
        seen = [0] * world
        prev_key = -1
        for i, dst in zip(mix.tolist(), d):
            key = seen[dst] * world + (dst - rank - 1) % world   # (round, turn inside the round)
            assert key > prev_key
            prev_key = key
            seen[dst] += 1
        for r in range(world):                                   # stable inside a destination
            mine = [i for i in mix.tolist() if dest[i] == r]
            assert mine == sorted(mine)
        if n >= world and all(c > 0 for c in torch.bincount(dest, minlength=world).tolist()):
            assert d[:world] == [(rank + 1 + j) % world for j in range(world)]
