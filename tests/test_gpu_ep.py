"""Expert-parallel decode step on 2 GPUs (skipped with fewer): experts sharded over the ranks, everything else
replicated.  Two exchanges are covered: one NCCL all-reduce per MoE layer, and the fused one (the down projection
stores its rows into every rank's buffer over NVLink and the next norm waits on sequence flags).  With the fused exchange
on full-size layer shapes the slots are sharded too: attention and Gated DeltaNet run only on the rank that owns a slot and
the out-projection's rows are gathered the same way -- covered with rows on both ranks and with a step in which one rank
owns no row at all.  The logits of every rank must be bit-identical to the single-GPU step (each exchanged row has exactly
one contributor)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CTX = {0: 300, 2: 17, 5: 700}
SIDS, TOKS = [0, 2, 5], [5, 9, 33]


def _cfg(fused, **kw):
    from qwental_b200.engine import tiny_cfg, wide_cfg
    return wide_cfg(**kw) if fused else tiny_cfg(**kw)


def _steps(eng):
    for s, n in CTX.items():
        eng.seed_slot(s, n, 1000 + s)
    l1, _ = eng.step(SIDS, TOKS)
    l2, _ = eng.step(SIDS, list(l1.argmax(1).astype(np.int32)))
    l3, _ = eng.step([2, 0], [7, 8])  # even slots only: with two ranks and slot sharding rank 1 owns no row of this step
    ids, _ = eng.decode_greedy(SIDS, TOKS, 3)
    eng.gpu.L.qw_gpu_set_graphs(eng.gpu.g, True)  # the same chain replayed as CUDA graphs (flag waits inside the graph)
    try:
        ids_g, _ = eng.decode_greedy(SIDS, [1, 2, 3], 4)
    finally:
        eng.gpu.L.qw_gpu_set_graphs(eng.gpu.g, False)
    return l1, l2, l3, ids, ids_g


def _worker(rank, world, uid, q, up, down):
    os.environ["QW_CUDA_DEVICE"] = str(rank)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from qwental_b200.engine import Engine
    from qwental_b200.gpu import Gpu
    gpu = Gpu()
    eng = Engine(gpu, _cfg(uid is None, ep_rank=rank, ep_size=world))
    if uid is not None:
        eng.ep_init(uid)
    else:  # fused exchange: the parent gathers the buffer handles and hands the list back
        up.put((rank, eng.ep_export()))
        eng.ep_connect(down.get(timeout=120))
    q.put((rank,) + _steps(eng))
    down.get(timeout=120)  # nobody unmaps or frees an exchange buffer before every rank has finished stepping
    eng.close()
    gpu.close()


@pytest.mark.parametrize("fused", [False, True])
def test_expert_parallel_step_bit_identical_to_single_gpu(fused):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from qwental_b200.engine import Engine, ep_unique_id
    from qwental_b200.gpu import Gpu
    uid = None if fused else ep_unique_id()
    ctx = mp.get_context("spawn")
    q, up = ctx.Queue(), ctx.Queue()
    down = [ctx.Queue() for _ in range(2)]
    procs = [ctx.Process(target=_worker, args=(r, 2, uid, q, up, down[r])) for r in range(2)]
    for p in procs:
        p.start()
    if fused:
        hs = dict(up.get(timeout=240) for _ in procs)
        for d in down:
            d.put([hs[0], hs[1]])
    res = sorted((q.get(timeout=240) for _ in procs), key=lambda r: r[0])
    for d in down:
        d.put("done")
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    gpu = Gpu()
    eng = Engine(gpu, _cfg(fused))
    ref = _steps(eng)
    eng.close()
    gpu.close()
    for r in res:
        for got, want in zip(r[1:4], ref[:3]):
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), r[0]
        assert np.array_equal(r[4], ref[3]) and np.array_equal(r[5], ref[4]), r[0]


def test_missing_peer_is_reported_not_waited_for_forever():
    """Failure detection without a fault: the kernel that consumes exchanged rows waits for every rank's sequence flag for a
    bounded time (about 2 s).  Here rank 1's flag never advances (nothing sets it -- the situation after a peer process has
    died between steps): the wait runs out, the batch ends with an error that names the bounded wait, and the device and
    the library stay usable.  One GPU is enough."""
    import time
    from qwental_b200.gpu import Gpu, GpuError
    gpu = Gpu()
    try:
        D, nb = 2048, 4
        rng = np.random.default_rng(0)
        h = gpu.buf_from(rng.standard_normal((nb, D)).astype(np.float32))
        delta = gpu.buf_from(rng.standard_normal((nb, D)).astype(np.float16))
        w = gpu.buf_from(np.ones(D, np.float32))
        x = gpu.buf(nb * D * 2).zero()
        flags = gpu.buf_from(np.array([1, 0, 0, 0, 0, 0, 0, 0], np.uint32))  # rank 0 published step 1, rank 1 never does
        seq = gpu.buf_from(np.array([1, 0], np.uint32))
        k = gpu.compile("add_rmsnorm", "add_rmsnorm_epx_t", ADD=1, EPX=2)
        args = np.array([nb, D], np.uint32)
        t0 = time.time()
        with pytest.raises(GpuError, match="bounded wait"):
            gpu.batch().kernel(k).buf(0, h).buf(1, delta).buf(2, w).buf(3, x).bytes(4, args).buf(7, flags).buf(8, seq).dispatch((nb,), (256,)).end()
        assert 1.0 < time.time() - t0 < 10.0
        # the same kernel completes at once when both ranks have published, and the device is still fine
        flags.upload(np.array([1, 1, 0, 0, 0, 0, 0, 0], np.uint32))
        gpu.batch().kernel(k).buf(0, h).buf(1, delta).buf(2, w).buf(3, x).bytes(4, args).buf(7, flags).buf(8, seq).dispatch((nb,), (256,)).end()
        assert np.isfinite(x.download(np.float16, nb * D).astype(np.float32)).all()
    finally:
        gpu.close()
