"""Peer-memory row exchange (b200gmm_push_rows + PeerExchange) on GPUs.

Single GPU: every expert local, rows only permuted; checked against the CPU
oracle run unsharded.  Two GPUs (skipped when the box has one): two NCCL ranks
as child processes; the peer path must equal the all-to-all path bit for bit and
match the unsharded oracle."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import gmm_oracle

pytestmark = pytest.mark.gpu

Z, TOKENS, TOPK, H_IN, H_OUT = 8, 96, 2, 64, 128


def _problem():
    g = torch.Generator().manual_seed(21)
    x = torch.randn(TOKENS, H_IN, generator=g).bfloat16()
    w = (torch.randn(Z, H_IN, H_OUT, generator=g) * 0.25).bfloat16()
    ids = torch.stack([torch.randperm(Z - 1, generator=g)[:TOPK] for _ in range(TOKENS)])  # one expert stays empty
    grad = torch.randn(TOKENS * TOPK, H_OUT, generator=g).bfloat16()
    return x, w, ids, grad


def _unsharded_oracle():
    x, w, ids, grad = _problem()
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
    return out_rows, slots.view(TOKENS, TOPK, -1).float().sum(1), dw


def _close(a, b, atol=2e-2):
    return torch.allclose(a.float().cpu(), b.float().cpu(), rtol=1e-2, atol=atol)


def test_push_rows_permutation_single_gpu():
    """The kernel alone: a permutation with repeated source rows into one buffer."""
    from grouped_gemm_b200 import _capi
    lib = _capi.load()
    torch.manual_seed(0)
    src = torch.randn(50, 72, device="cuda").bfloat16()          # 144-byte rows
    src_row = torch.randint(0, 50, (200,), device="cuda", dtype=torch.int32)
    dst_row = torch.randperm(200, device="cuda").to(torch.int64)
    dst = torch.zeros(200, 72, device="cuda", dtype=torch.bfloat16)
    table = torch.tensor([dst.data_ptr()], dtype=torch.int64, device="cuda")
    rank0 = torch.zeros(200, dtype=torch.int32, device="cuda")
    rc = lib.b200gmm_push_rows(src.data_ptr(), 144, 200, src_row.data_ptr(), rank0.data_ptr(),
                               dst_row.data_ptr(), table.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    want = torch.zeros_like(dst)
    want[dst_row] = src[src_row.long()]
    assert torch.equal(dst, want)
    # identity source rows, and the argument checks
    rc = lib.b200gmm_push_rows(src.data_ptr(), 144, 50, None, rank0.data_ptr(), dst_row.data_ptr(),
                               table.data_ptr(), 3, torch.cuda.current_stream().cuda_stream)   # three blocks only
    assert rc == 0
    assert torch.equal(dst[dst_row[:50]], src)
    assert lib.b200gmm_push_rows(src.data_ptr(), 100, 50, None, rank0.data_ptr(), dst_row.data_ptr(),
                                 table.data_ptr(), 0, None) == -1   # rows must be multiples of 16 bytes


@pytest.mark.parametrize("tokens,top_k,cols", [(1, 1, 8), (37, 2, 72), (1000, 4, 6144), (513, 8, 264), (0, 4, 64)])
def test_sum_slots_equals_fp32_sum(tokens, top_k, cols):
    """b200gmm_sum_slots: a token's top_k rows added in fp32 in slot order and rounded
    once; bit for bit what an fp32 sum followed by one rounding gives, also with
    values 2**20 apart in one sum."""
    from grouped_gemm_b200 import _capi
    lib = _capi.load()
    torch.manual_seed(tokens + top_k)
    slots = torch.randn(tokens * top_k, cols, device="cuda")
    if tokens:
        slots[::3] *= 1024.0
        slots[1::5] *= 2.0 ** -10
    slots = slots.bfloat16()
    out = torch.full((tokens, cols), 3.0, device="cuda", dtype=torch.bfloat16)
    rc = lib.b200gmm_sum_slots(slots.data_ptr() if tokens else 0, out.data_ptr() if tokens else 0, tokens, top_k, cols,
                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    want = torch.zeros(tokens, cols, device="cuda")
    for j in range(top_k):   # the same order of additions
        want += slots.view(tokens, top_k, cols)[:, j].float()
    assert torch.equal(out, want.bfloat16())
    assert lib.b200gmm_sum_slots(slots.data_ptr(), out.data_ptr(), tokens, 9, cols, 0) != 0       # top_k beyond the limit
    assert lib.b200gmm_sum_slots(slots.data_ptr(), out.data_ptr(), tokens, top_k, cols + 4, 0) != 0  # cols not a multiple of 8


def test_peer_exchange_single_rank_matches_oracle():
    from grouped_gemm_b200 import backend, expert_parallel as ep
    x, w, ids, grad = _problem()
    px = ep.PeerExchange(ids.cuda(), Z, H_IN, H_OUT, single_rank=True)
    assert px.batch_sizes_host == torch.bincount(ids.reshape(-1), minlength=Z).tolist()
    gmm_fn = lambda a, b, bs, ta, tb: backend.gmm(a, b, bs, trans_a=ta, trans_b=tb)
    # a dispatch followed by a combine returns every slot's own row
    back = px.combine_rows(px.dispatch_rows(grad.cuda()).clone())
    assert torch.equal(back.cpu(), grad)
    out_rows, dx, dw = px.step(x.cuda(), w.cuda(), grad.cuda(), gmm_fn)
    out_rows, dx, dw = out_rows.clone(), dx.clone(), dw.clone()
    xd, wd, gd = x.cuda(), w.cuda(), grad.cuda()
    for in_kernel, nxt in ((True, None), (False, None), (True, xd), (True, xd), (True, None)):
        o2, dx2, dw2 = px.step_fused(xd, wd, gd, gmm_fn, timeline=True, push_in_kernel=in_kernel, x_next=nxt)
        torch.cuda.synchronize()
        assert torch.equal(o2, out_rows) and torch.equal(dx2, dx) and torch.equal(dw2, dw)
    assert len(px.phase_times()) == 8  # nine marks, eight intervals
    # rows sent ahead are not used for a tensor that changed since, nor for another tensor
    px.step_fused(xd, wd, gd, gmm_fn, push_in_kernel=True, x_next=xd)
    xd.mul_(2.0)
    o3 = px.step_fused(xd, wd, gd, gmm_fn, push_in_kernel=True)[0].clone()
    torch.cuda.synchronize()
    want3 = px.step(xd, wd, gd, gmm_fn)[0]
    assert torch.equal(o3, want3) and not torch.equal(o3, out_rows)
    want_rows, want_dx, want_dw = _unsharded_oracle()
    assert _close(out_rows, want_rows) and _close(dx, want_dx, 5e-2) and _close(dw, want_dw, 5e-2)
    assert bool((dw[Z - 1] == 0).all())
    assert backend.device_status() == 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from grouped_gemm_b200 import backend, expert_parallel as ep
        x, w, ids, grad = _problem()
        per = TOKENS // world
        sl = slice(rank * per, (rank + 1) * per)
        zs = slice(rank * Z // world, (rank + 1) * Z // world)
        xl, wl, gl, il = x[sl].to(dev), w[zs].contiguous().to(dev), grad[sl.start * TOPK:sl.stop * TOPK].to(dev), ids[sl].to(dev)
        gmm_fn = lambda a, b, bs, ta, tb: backend.gmm(a, b, bs, trans_a=ta, trans_b=tb)
        plan = ep.build_plan(il, Z)
        o1, dx1, dw1 = ep.expert_parallel_step(xl, wl, gl, plan, gmm_fn)
        px = ep.PeerExchange(il, Z, H_IN, H_OUT)
        o2, dx2, dw2 = px.step(xl, wl, gl, gmm_fn)
        o2, dx2, dw2 = o2.clone(), dx2.clone(), dw2.clone()
        same = bool(torch.equal(o1, o2) and torch.equal(dw1, dw2) and torch.equal(dx1, dx2))
        # Replayed steps reuse the buffers, so the barriers must order them: every
        # iteration gets its own inputs and is compared with its own all-to-all
        # result (an overwrite by a rank that runs ahead would change the output).
        xs = [(xl.float() * (1 + 0.25 * i)).bfloat16() for i in range(5)]
        gs = [(gl.float() * (1 - 0.125 * i)).bfloat16() for i in range(5)]
        for mode in ("pushes", "fused", "fused-separate-push", "fused-ahead"):
            for i in range(4):
                want = ep.expert_parallel_step(xs[i], wl, gs[i], plan, gmm_fn)
                if mode == "pushes":
                    got = px.step(xs[i], wl, gs[i], gmm_fn)
                elif mode == "fused-ahead":   # iteration i announces the activations of iteration i + 1
                    got = px.step_fused(xs[i], wl, gs[i], gmm_fn, push_in_kernel=True, x_next=xs[i + 1])
                else:
                    got = px.step_fused(xs[i], wl, gs[i], gmm_fn, push_in_kernel=(mode == "fused"))
                got = [t.clone() for t in got]
                torch.cuda.synchronize()
                same = same and all(torch.equal(u, v) for u, v in zip(got, want))
        results[rank] = (same, o2.cpu(), dx2.float().cpu(), dw2.cpu(), backend.device_status(dev))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_peer_exchange_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port = 2, _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        got = [results[r] for r in range(world)]
    want_rows, want_dx, want_dw = _unsharded_oracle()
    per = TOKENS // world
    for r in range(world):
        same, o, dx, dw, status = got[r]
        assert same, "peer-memory path differs from the all-to-all path"
        assert status == 0
        assert _close(o, want_rows[r * per * TOPK:(r + 1) * per * TOPK])
        assert _close(dx, want_dx[r * per:(r + 1) * per], 5e-2)
    assert _close(torch.cat([got[r][3] for r in range(world)]), want_dw, 5e-2)
