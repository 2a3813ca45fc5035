"""CPU test of the expert-parallel exchange (world size 2, gloo): each rank computes the (token, rank) rows of the
experts it owns with the FP oracle, zeros elsewhere; an all-reduce (sum) must reproduce the single-rank buffer bit
for bit, and the combine on top of it must equal the single-rank layer output."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from qwental_b200 import ep, synth

E, D, I, TOPK, B = 16, 256, 256, 4, 6


def rows_for(x, ids, gate, up, down, lo, hi, orc):
    """fp32 rows [B][TOPK][D] of the experts in [lo, hi), zeros elsewhere (what moe_dn writes on one rank)."""
    out = np.zeros((B, TOPK, D), np.float32)
    xf = x.astype(np.float32)
    for t in range(B):
        for k in range(TOPK):
            e = int(ids[t, k])
            if lo <= e < hi:
                g = orc.qmv_cpu(21, gate[e], D, xf[t:t + 1], 1)[0][0]
                u = orc.qmv_cpu(21, up[e], D, xf[t:t + 1], 1)[0][0]
                h = (g / (1 + np.exp(-g)) * u).astype(np.float32)
                out[t, k] = orc.qmv_cpu(21, down[e], I, h[None], 1)[0][0]
    return out


def make_inputs():
    from oracle import oracle as orc
    rng = np.random.default_rng(0)
    x = synth.acts_fp16(rng, B, D)
    Wr = (rng.standard_normal((E, D)) * 0.02).astype(np.float16)
    gate = synth.iq3s_rows(rng, E * I, D, 2.0 ** -5).reshape(E, I, -1)
    up = synth.iq3s_rows(rng, E * I, D, 2.0 ** -5).reshape(E, I, -1)
    down = synth.iq3s_rows(rng, E * D, I, 2.0 ** -5).reshape(E, D, -1)
    ids, w = orc.topk(orc.router_canon(Wr, x), TOPK)
    return orc, x, ids, w, gate, up, down


def worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc, x, ids, w, gate, up, down = make_inputs()  # replicated, deterministic: the router needs no exchange
        lo, hi = ep.expert_range(E, rank, world)
        mine = rows_for(x, ids, gate, up, down, lo, hi, orc)
        assert np.all(mine[~((ids >= lo) & (ids < hi))] == 0)
        t = torch.from_numpy(mine.copy())
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        full = rows_for(x, ids, gate, up, down, 0, E, orc)
        ok = np.array_equal(t.numpy().view(np.uint32), full.view(np.uint32))
        comb = (t.numpy() * w[:, :, None]).sum(1)
        ok2 = np.array_equal(comb, (full * w[:, :, None]).sum(1))
        q.put((rank, ok, ok2, int(((ids >= lo) & (ids < hi)).sum())))
    finally:
        dist.destroy_process_group()


def shard_worker(rank, world, port, q):
    """Slot sharding: every rank produces the rows of the slots it owns (here a deterministic function of slot and token),
    in the shared device order; summing zero-padded buffers stands in for the peer stores of the out-projection."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sids = np.array([5, 0, 2, 7, 4, 9, 1], np.int32)
        toks = np.arange(len(sids), dtype=np.int64) * 3 + 1
        perm, lo, hi = ep.row_order(sids, world, rank)
        full = np.stack([np.full(8, float(sids[i] * 100 + toks[i]), np.float32) for i in perm])  # device order, all rows
        mine = np.zeros_like(full)
        assert all(sids[perm[j]] % world == rank for j in range(lo, hi))
        mine[lo:hi] = full[lo:hi]
        t = torch.from_numpy(mine.copy())
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        allperm = [torch.zeros(len(sids), dtype=torch.int32) for _ in range(world)]
        dist.all_gather(allperm, torch.from_numpy(perm.copy()))
        same_order = all(np.array_equal(p.numpy(), perm) for p in allperm)
        back = np.empty_like(full)
        back[perm] = t.numpy()  # the caller's order
        want = np.stack([np.full(8, float(sids[i] * 100 + toks[i]), np.float32) for i in range(len(sids))])
        q.put((rank, bool(np.array_equal(back, want)), same_order, lo, hi))
    finally:
        dist.destroy_process_group()


def test_slot_sharded_rows_gather_to_the_full_batch_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=shard_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    assert all(r[1] and r[2] for r in res)
    assert res[0][3] == 0 and res[0][4] == res[1][3] and res[1][4] == 7 and res[0][4] == 3  # slots 0, 2, 4 are rank 0's


def test_row_order_edge_cases():
    perm, lo, hi = ep.row_order([3, 1, 5], 2, 0)  # all slots odd: rank 0 owns no row
    assert (lo, hi) == (0, 0) and perm.tolist() == [0, 1, 2]
    perm, lo, hi = ep.row_order([3, 1, 5], 2, 1)
    assert (lo, hi) == (0, 3)
    perm, lo, hi = ep.row_order([6, 1, 4, 3], 1, 0)  # one rank: the caller's order
    assert perm.tolist() == [0, 1, 2, 3] and (lo, hi) == (0, 4)
    perm, lo, hi = ep.row_order([6, 1, 4, 3, 8], 4, 0)  # stable within a rank: slots 4 and 8 keep their order
    assert perm.tolist() == [2, 4, 1, 0, 3] and (lo, hi) == (0, 2)
    with pytest.raises(ValueError):
        ep.row_order([1], 2, 2)


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_expert_ranges_partition():
    for n in (1, 2, 4, 8):
        r = [ep.expert_range(512, k, n) for k in range(n)]
        assert r[0][0] == 0 and r[-1][1] == 512 and all(r[i][1] == r[i + 1][0] for i in range(n - 1))
    with pytest.raises(ValueError):
        ep.expert_range(10, 0, 3)


@pytest.mark.timeout(180)
def test_allreduce_of_owned_rows_is_bit_identical_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=150) for _ in procs]
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    assert all(ok and ok2 for _, ok, ok2, _ in res)
    assert sum(n for _, _, _, n in res) == B * TOPK
