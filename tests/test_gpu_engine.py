"""GPU parity of the full decode step through the engine C ABI (benchmark config 4 at two reduced model sizes, so
the FP64 oracle finishes in seconds: "tiny" shrinks every dimension, "wide" keeps the full-size layer shapes and with
them the kernel variants of the benchmark model): logits within fp16 tolerance of the chained FP64 reference with top-1
agreement, chosen experts identical, batched rows bit-identical to each slot alone, chained greedy decode equal to
step-by-step decode, CUDA-graph replay equal to plain launches."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    from qwental_b200.gpu import Gpu
    g = Gpu()
    yield g
    g.close()


@pytest.fixture(scope="module", params=["tiny", "wide"])
def eng(gpu, request):
    from qwental_b200.engine import Engine, tiny_cfg, wide_cfg
    e = Engine(gpu, tiny_cfg() if request.param == "tiny" else wide_cfg())
    yield e
    e.close()


CTX = {0: 300, 3: 5, 5: 777, 6: 255}


def seed_all(eng):
    for sid, n in CTX.items():
        eng.seed_slot(sid, n, 1000 + sid)


def test_step_logits_match_fp64_reference(eng):
    from oracle.model_ref import RefModel
    seed_all(eng)
    ref = RefModel(eng.cfg, eng)
    sids = [0, 3, 5, 6]
    toks = [7, 100, 511, 0]
    states = {s: ref.read_slot(eng, s) for s in sids}
    logits, ms = eng.step(sids, toks)
    assert ms > 0 and logits.shape == (4, eng.cfg.vocab) and np.isfinite(logits).all()
    h = eng.tap("h", 0, np.float32).reshape(4, -1)
    for i, s in enumerate(sids):
        dev_ids = [eng.tap("sel", l, np.uint8)[16:16 + 64 * 16 * 4].view(np.int32).reshape(64, 16)[i, :eng.cfg.topk] for l in range(eng.cfg.layers)]
        lg, hh, chosen = ref.step(states[s], toks[i], ids_by_layer=dev_ids)
        scale = np.abs(lg).max()
        assert np.abs(logits[i] - lg).max() < 2e-2 * scale, (s, np.abs(logits[i] - lg).max(), scale)
        assert int(logits[i].argmax()) == int(lg.argmax())
        assert eng.pos(s) == CTX[s] + 1
    # the slot state the device left behind matches the reference's (KV append, GDN state)
    for s in sids:
        after = ref.read_slot(eng, s)
        assert np.abs(after["S"] - states[s]["S"]).max() < 1e-3 * max(1.0, np.abs(states[s]["S"]).max())
        p = CTX[s]
        assert np.abs(after["kv"][:, :, :, p].astype(np.float64) - states[s]["kv"][:, :, :, p].astype(np.float64)).max() < 2e-2


def test_batched_rows_bit_identical_to_alone(eng):
    sids, toks = [0, 3, 5, 6], [11, 12, 13, 14]
    seed_all(eng)
    lb, _ = eng.step(sids, toks)
    for i, s in enumerate(sids):
        seed_all(eng)
        la, _ = eng.step([s], [toks[i]])
        assert np.array_equal(la[0].view(np.uint32), lb[i].view(np.uint32)), s
    # order of rows does not matter either
    seed_all(eng)
    lp, _ = eng.step([6, 0], [14, 11])
    assert np.array_equal(lp[0].view(np.uint32), lb[3].view(np.uint32)) and np.array_equal(lp[1].view(np.uint32), lb[0].view(np.uint32))


def test_greedy_chain_equals_stepwise_and_graph_replay(eng, gpu):
    sids, toks = [0, 5], [3, 4]
    seed_all(eng)
    ids_chain, _ = eng.decode_greedy(sids, toks, 4)
    seed_all(eng)
    cur = list(toks)
    for k in range(4):
        ids, _ = eng.step_greedy(sids, cur)
        assert np.array_equal(ids, ids_chain[k])
        cur = list(ids)
    # logits path gives the same arg-max (ties -> lowest id)
    seed_all(eng)
    lg, _ = eng.step(sids, toks)
    assert np.array_equal(lg.argmax(1).astype(np.int32), ids_chain[0])
    gpu.L.qw_gpu_set_graphs(gpu.g, True)
    try:
        seed_all(eng)
        ids_graph, _ = eng.decode_greedy(sids, toks, 4)
    finally:
        gpu.L.qw_gpu_set_graphs(gpu.g, False)
    assert np.array_equal(ids_graph, ids_chain)


def test_slot_errors_and_accounting(eng):
    from qwental_b200.gpu import GpuError
    seed_all(eng)
    with pytest.raises(GpuError):
        eng.step([0, 0], [1, 2])            # the same slot twice
    with pytest.raises(GpuError):
        eng.step([1], [1])                  # slot never seeded
    with pytest.raises(GpuError):
        eng.step([0], [eng.cfg.vocab])      # token out of range
    with pytest.raises(GpuError):
        eng.step([], [])                    # an empty batch
    with pytest.raises(GpuError):
        eng.step(list(range(65)), [0] * 65) # more rows than QW_PAR_MAX
    eng.seed_slot(7, eng.cfg.max_ctx - 1, 9)  # the last position that fits
    eng.step([7], [1])
    with pytest.raises(GpuError):
        eng.step([7], [1])                  # one more would exceed max_ctx
    eng.finish(7)
    lg, _ = eng.step([0, 3], [1, 2])        # the engine is still usable
    b = eng.step_bytes()
    c = eng.cfg
    assert b.ctx_tokens == (CTX[0] + 1) + (CTX[3] + 1)
    assert 1 <= b.unique_experts_sum <= c.layers * 2 * c.topk
    assert b.total == pytest.approx(b.moe + b.dense + b.lm_head + b.kv + b.gdn_state + b.other)
    assert eng.mem() > 0 and eng.cost(2) > 0
    assert eng.pick(busy=0b1111111) == 7
    eng.finish(3)
    assert eng.pos(3) == -1 and eng.pick(busy=0) in (1, 2, 3, 4, 7)


@pytest.mark.parametrize("attn_every", [4, 1])
def test_fresh_engines_agree_bit_for_bit(gpu, attn_every):
    """Two engines opened one after the other (so the second one's buffers hold the first one's leftovers) produce the
    same logits, bit for bit, with dependent launch on: a kernel that read its predecessor's output too early, or through a
    non-coherent path, shows up here as run-to-run noise."""
    from qwental_b200.engine import Engine, wide_cfg
    outs = []
    for _ in range(3):
        e = Engine(gpu, wide_cfg(layers=2, attn_every=attn_every))
        for sid, n in CTX.items():
            e.seed_slot(sid, n, 1000 + sid)
        lg, _ = e.step([0, 3, 5, 6], [7, 100, 511, 0])
        lg2, _ = e.step([0, 5], [1, 2])
        outs.append((lg.copy(), lg2.copy()))
        e.close()
    for a, b2 in outs[1:]:
        assert np.array_equal(a.view(np.uint32), outs[0][0].view(np.uint32))
        assert np.array_equal(b2.view(np.uint32), outs[0][1].view(np.uint32))


def test_full_batch_of_64_rows_matches_each_slot_alone(gpu):
    """The largest batch the step accepts (QW_PAR_MAX = 64 rows, contexts straddling page boundaries): a sample of its rows
    is bit-identical to the same slots stepped alone, on both model sizes' kernel variants."""
    from qwental_b200.engine import Engine, tiny_cfg, wide_cfg
    for cfg in (tiny_cfg(max_slots=64, max_ctx=1024), wide_cfg(max_slots=64, max_ctx=1024, layers=2)):
        e = Engine(gpu, cfg)
        ctx = {s: [1, 255, 256, 257, 511, 512, 700, 33][s % 8] + s for s in range(64)}

        def seed():
            for s, n in ctx.items():
                e.seed_slot(s, n, 5000 + s)
        seed()
        sids = list(range(63, -1, -1))
        toks = [(s * 37 + 11) % cfg.vocab for s in sids]
        lb, _ = e.step(sids, toks)
        assert np.isfinite(lb).all()
        for i in (0, 7, 31, 40, 63):
            seed()
            la, _ = e.step([sids[i]], [toks[i]])
            assert np.array_equal(la[0].view(np.uint32), lb[i].view(np.uint32)), (cfg.hidden, sids[i])
        e.close()


def test_benchmark_layer_shapes_match_fp64_reference(gpu):
    """Four layers of the benchmark model itself (hidden 2048, 512 experts with top-10, 151 936-token vocabulary; three
    Gated DeltaNet layers and one attention layer) against the chained FP64 reference: logits within tolerance, top-1
    equal, chosen experts taken from the device and checked to be the reference's own top-10 wherever its margin is clear."""
    from oracle.model_ref import RefModel
    from qwental_b200.engine import Engine, default_cfg
    e = Engine(gpu, default_cfg(layers=4, max_slots=4, max_ctx=2048, kv_pages=0, seed=3))
    try:
        ctx = {0: 700, 2: 255, 3: 40}
        for sid, n in ctx.items():
            e.seed_slot(sid, n, 2000 + sid)
        ref = RefModel(e.cfg, e)
        sids, toks = [3, 0, 2], [11, 150000, 77]
        states = {s: ref.read_slot(e, s) for s in sids}
        logits, _ = e.step(sids, toks)
        assert np.isfinite(logits).all()
        for i, s in enumerate(sids):
            dev_ids = [e.tap("sel", l, np.uint8)[16:16 + 64 * 16 * 4].view(np.int32).reshape(64, 16)[i, :e.cfg.topk] for l in range(e.cfg.layers)]
            lg, hh, chosen = ref.step(states[s], toks[i], ids_by_layer=dev_ids)
            scale = np.abs(lg).max()
            assert np.abs(logits[i] - lg).max() < 2e-2 * scale, (s, np.abs(logits[i] - lg).max(), scale)
            assert int(logits[i].argmax()) == int(lg.argmax())
    finally:
        e.close()


def test_prefill_is_the_decode_path_token_by_token(gpu):
    """qw_engine_par_prefill feeds a prompt through the decode step: prefill(p) equals prefill(p[:-1]) followed by one
    step of p[-1], bit for bit; the result does not depend on the slot; a slot that was in use is emptied first; a
    prefilled slot steps together with a seeded one exactly as it steps alone."""
    from qwental_b200.engine import Engine, tiny_cfg
    from qwental_b200.gpu import GpuError
    e = Engine(gpu, tiny_cfg())
    try:
        prompt = [5, 17, 300, 4, 4, 511, 0, 260, 33]
        full = e.prefill(1, prompt)
        assert e.pos(1) == len(prompt) and np.isfinite(full).all()
        part = e.prefill(4, prompt[:-1])
        lg, _ = e.step([4], [prompt[-1]])
        assert np.array_equal(lg[0].view(np.uint32), full.view(np.uint32))
        e.seed_slot(2, 300, 77)  # slot 2 in use with other contents: prefill starts it over
        again = e.prefill(2, prompt)
        assert np.array_equal(again.view(np.uint32), full.view(np.uint32)) and e.pos(2) == len(prompt)
        a, _ = e.step([1], [9])
        e.prefill(1, prompt)
        e.seed_slot(6, 500, 5)
        b, _ = e.step([6, 1], [3, 9])
        assert np.array_equal(b[1].view(np.uint32), a[0].view(np.uint32))
        with pytest.raises(GpuError):
            e.prefill(0, [e.cfg.vocab])
        with pytest.raises(GpuError):
            e.prefill(99, [1])
    finally:
        e.close()


def test_benchmark_engine_full_depth_batched_equals_alone_and_graph_replay(gpu):
    """The benchmark engine itself -- all 48 layers, the 16 ragged conversations bench.py steps (contexts log-uniform in
    1K..48K, the same seeds) -- needs no oracle for the reference's own guarantee (src/engine.c:7977-7986,
    tools/run.c:217-229): three rows of the 16-row step are bit-identical to the same slots stepped alone, and the step
    replayed as a CUDA graph gives the bytes of the plain launches."""
    from qwental_b200 import synth
    from qwental_b200.engine import Engine, default_cfg
    B = 16
    ctx = synth.ragged_contexts(np.random.default_rng(0), B)
    pages = int(sum((int(n) + 64 + 256) // 256 + 1 for n in ctx))
    e = Engine(gpu, default_cfg(max_slots=B, max_ctx=int(ctx.max()) + 1024, kv_pages=pages, seed=0))
    try:
        def seed(rows):
            for s in rows:
                e.seed_slot(s, int(ctx[s]), 100 + s)
        sids = np.arange(B, dtype=np.int32)
        toks = (np.arange(B, dtype=np.int32) * 7919) % e.cfg.vocab
        seed(range(B))
        lb, _ = e.step(sids, toks)
        assert np.isfinite(lb).all()
        longest, shortest = int(np.argmax(ctx)), int(np.argmin(ctx))
        for r in sorted({longest, shortest, 7}):
            seed([r])
            la, _ = e.step([r], [toks[r]])
            assert np.array_equal(la[0].view(np.uint32), lb[r].view(np.uint32)), (r, int(ctx[r]))
        gpu.L.qw_gpu_set_graphs(gpu.g, True)
        try:
            seed(range(B))
            e.step(sids, toks)        # records the graph
            seed(range(B))
            lg, _ = e.step(sids, toks)  # replays it
        finally:
            gpu.L.qw_gpu_set_graphs(gpu.g, False)
        assert np.array_equal(lg.view(np.uint32), lb.view(np.uint32))
    finally:
        e.close()
