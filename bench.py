#!/usr/bin/env python3
"""Benchmark of the batched decode step: decode tokens/s at 16 ragged slots of the full 48-layer
Qwen3-Next-80B-A3B-shaped model with random-init IQ3_S weights (Q8_0 lm_head), greedy sampling.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--slots 16] [--impl reference]

One "step" advances every slot by one token.  Prints ONE JSON line (rank 0):
  value     tokens/s of K chained greedy steps with all inputs resident in HBM (device-timed, CUDA events on the
            engine's stream, max over ranks)
  e2e       the same metric through the public C-ABI call qw_engine_par_step_greedy with host token ids in and
            host sampled ids out every step
  roofline  the dominant kernel (the MoE expert FFN: IQ3_S gate/up/down matvecs over the gathered experts): algorithmic
            bytes per launch / mean launch duration (CUDA events around every dispatch, qw_profile_*), against the
            measured HBM copy bandwidth of MEASURED_PEAKS.json; copy_ceiling_gbs = the same launch with the decode taken
            out (the staged copies only), timed the same way
  sustained the same chained steps repeated for a few seconds, with the SM clock seen meanwhile
  slots64   the same step at 64 active slots (1 GPU)
  cpu_baseline  the CPU oracle (block decode + fp32 dot on all host cores, numpy attention / GDN) timed on a
            bounded sample of the same step and scaled to a whole step
With --gpus N > 1 (launched by torchrun) the experts are sharded over the ranks (expert parallel) and the
attention / GDN / dense parts are replicated: the same 16 slots, so scaling is "strong".
--impl reference times the CPU implementation alone (no GPU kernels).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tok/s at 16 ragged slots"
UNIT = "tokens/s"
CFG = dict(hidden=2048, layers=48, attn_every=4, vocab=151936, experts=512, topk=10, expert_inter=512, qh=16, kvh=2, hd=256, hk=16, hv=32)


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s)"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, dev: int):
        self.dev, self.rows, self.proc = dev, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.dev), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------------------- CPU arm
def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


def cpu_step_sample(nslots: int, ctx: np.ndarray, seed: int = 0):
    """Times the CPU implementation of one decode step on a bounded sample and scales it to the whole step.

    Sample: ONE GDN-type layer and ONE attention-type layer (input/output projections, the recurrent or attention
    core for every slot, the MoE block with the experts a seeded router actually picks) plus the lm_head rows of
    1/8 of the vocabulary.  Whole step = 36 x GDN layer + 12 x attention layer + 8 x lm_head sample.
    Matvecs: oracle/qw_oracle.c orc_qmv_cpu (decode each row to fp32 as tools/dqcpu.c does, then an fp32 dot) on
    all host cores; the Q8_0 rows go through the reference's own src/ggml_dq.c when oracle/_ref is built.
    Attention / GDN cores: the numpy FP64 restatements of bench/qsa.c:181-200 and bench/gdn_decode.c:74-85."""
    from oracle import oracle as orc
    from qwental_b200 import synth
    c = CFG
    D, I, E, TOPK = c["hidden"], c["expert_inter"], c["experts"], c["topk"]
    rng = np.random.default_rng(seed)
    x = synth.acts_fp16(rng, nslots, D)
    xf = x.astype(np.float32)
    cores = host_threads()  # asked for explicitly: a launcher may have set OMP_NUM_THREADS=1 for its ranks
    t = {}

    def mv(W, K, xin):
        return orc.qmv_cpu(21, W, K, xin, cores)[0]

    # ---- MoE block (same for both layer types)
    Wr = (rng.standard_normal((E, D)) * 0.02).astype(np.float16)
    lg = orc.router_canon(Wr, x)
    ids, w = orc.topk(lg, TOPK)
    uniq = np.unique(ids)
    gate = {int(e): synth.iq3s_rows(rng, I, D, 1 / 64) for e in uniq}
    up = {int(e): synth.iq3s_rows(rng, I, D, 1 / 64) for e in uniq}
    down = {int(e): synth.iq3s_rows(rng, D, I, 1 / 32) for e in uniq}
    sh = (synth.iq3s_rows(rng, I, D, 1 / 64), synth.iq3s_rows(rng, I, D, 1 / 64), synth.iq3s_rows(rng, D, I, 1 / 32))
    t0 = time.perf_counter()
    out = np.zeros((nslots, D), np.float32)
    for e in uniq:
        toks = np.nonzero((ids == e).any(1))[0]
        g, u = mv(gate[int(e)], D, xf[toks]), mv(up[int(e)], D, xf[toks])
        h = (g / (1 + np.exp(-g)) * u).astype(np.float32)
        p = mv(down[int(e)], I, h)
        for j, tk in enumerate(toks):
            out[tk] += w[tk, list(ids[tk]).index(e)] * p[j]
    g, u = mv(sh[0], D, xf), mv(sh[1], D, xf)
    out += mv(sh[2], I, (g / (1 + np.exp(-g)) * u).astype(np.float32))
    t["moe"] = time.perf_counter() - t0
    # ---- GDN-type layer: in-proj 12352 x 2048, out-proj 2048 x 4096, recurrence for every slot
    Win, Wout = synth.iq3s_rows(rng, 12352, D, 1 / 64), synth.iq3s_rows(rng, D, 4096, 1 / 128)
    S = (rng.standard_normal((nslots, 32, 128, 128)) * 0.1)
    t0 = time.perf_counter()
    proj = mv(Win, D, xf)
    for s in range(nslots):
        q, k, v = proj[s, :2048].reshape(16, 128), proj[s, 2048:4096].reshape(16, 128), proj[s, 4096:8192].reshape(32, 128)
        S[s], _, y = orc.gdn_step_ref(S[s], q, k, v, -np.ones(32) * 0.5, np.full(32, 0.5), proj[s, 8192:12288].reshape(32, 128), np.ones(128),
                                      np.arange(32) % 16)
    mv(Wout, 4096, np.ascontiguousarray(proj[:, :4096]))
    t["gdn_layer"] = time.perf_counter() - t0
    # ---- attention-type layer: qkv 9216 x 2048, o 2048 x 4096, attention over every slot's context
    Wqkv, Wo = synth.iq3s_rows(rng, 9216, D, 1 / 64), synth.iq3s_rows(rng, D, 4096, 1 / 128)
    kvs = [(rng.standard_normal((int(n), 2, 256)).astype(np.float16), rng.standard_normal((int(n), 2, 256)).astype(np.float16)) for n in ctx]
    t0 = time.perf_counter()
    qkv = mv(Wqkv, D, xf).astype(np.float16)
    for s in range(nslots):
        orc.attn_ref(qkv[s, :8192].reshape(16, 512)[:, :256], kvs[s][0], kvs[s][1], qkv[s, :8192].reshape(16, 512)[:, 256:])
    mv(Wo, 4096, np.ascontiguousarray(qkv[:, :4096].astype(np.float32)))
    t["attn_layer"] = time.perf_counter() - t0
    # ---- lm_head sample: 1/8 of the vocabulary, Q8_0
    V8 = c["vocab"] // 8
    Wl = synth.q8_0_rows(rng, V8, D)
    kind = "port"
    t0 = time.perf_counter()
    if os.path.exists(orc.REF_LIB):
        orc.ref_dq_q8_0_rows(Wl[:2048], D)  # the reference's own decoder on a slice (single thread, its only CPU code on this path)
        kind = "port (+ reference ggml_dq.c for a Q8_0 slice)"
    orc.qmv_cpu(8, Wl, D, xf, cores)
    t["lm_head_eighth"] = time.perf_counter() - t0
    step = 36 * (t["gdn_layer"] + t["moe"]) + 12 * (t["attn_layer"] + t["moe"]) + 8 * t["lm_head_eighth"]
    sample = ("1 GDN layer + 1 attention layer + MoE block (%d distinct experts) + 1/8 of lm_head, %d slots; "
              "scaled x36 / x12 / x8 to a step; sample took %.1f s") % (len(uniq), nslots, sum(t.values()))
    return nslots / step, cores, kind, sample, t


def workload_config(layers, slots, ctx_sum, world, graphs, ep="nccl"):
    return {"workload": "full %d-layer Qwen3-Next-80B-A3B-shaped decode step, %d ragged slots (contexts log-uniform 1K-48K, sum %d tokens), "
                        "IQ3_S weights, Q8_0 lm_head, greedy" % (layers, slots, ctx_sum),
            "parallelism": ("ep%d (experts sharded, attention and Gated DeltaNet sharded by slot with conversations placed on the least "
                            "loaded rank, rest replicated; exchange: peer stores fused into the down and out projections)" % world
                            if ep == "fused" else
                            "ep%d (experts sharded, rest replicated; exchange: NCCL all-reduce)" % world) if world > 1 else "1 GPU",
            "l2": "inputs larger than L2 (weights 35 GB, KV and state several GB per step)", "cuda_graphs": bool(graphs)}


def cpu_baseline_avg(nslots, ctx, reps=3, min_seconds=10.0):
    """Mean over at least `reps` samples and at least `min_seconds` of CPU work (bounded at 12 samples)."""
    vals, last, t0 = [], None, time.time()
    i = 0
    while i < reps or (time.time() - t0 < min_seconds and i < 12):
        last = cpu_step_sample(nslots, ctx, seed=i)
        vals.append(last[0])
        i += 1
    reps = i
    v, cores, kind, sample, _ = last
    return float(np.mean(vals)), cores, kind, sample + " (mean of %d samples)" % reps


def run_reference(args):
    """The CPU implementation alone: W untimed and K timed steps, each step one bounded sample of the workload (see
    cpu_step_sample) scaled to a whole decode step; value = slots / mean scaled step time over the K timed samples."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from qwental_b200 import synth
    ctx = synth.ragged_contexts(np.random.default_rng(0), args.slots)
    K, W = max(1, args.steps), max(0, args.warmup)
    for i in range(W):
        cpu_step_sample(args.slots, ctx, seed=1000 + i)
    vals, spent, last = [], 0.0, None
    t0 = time.time()
    for i in range(K):
        last = cpu_step_sample(args.slots, ctx, seed=i)
        vals.append(args.slots / last[0])  # scaled seconds per step
        spent += sum(last[4].values())
    _, cores, kind, sample, _ = last
    step_s = float(np.mean(vals))
    v = args.slots / step_s
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": K, "warmup": W,
        "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(48, args.slots, int(ctx.sum()), 1, True),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": sample + " (each of the %d timed steps is one such sample; %.1f s of CPU work measured, %.1f s wall)" % (K, spent, time.time() - t0)},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ----------------------------------------------------------------------------------------------------------- GPU arm
CHAIN_FIXTURE = os.path.join(ROOT, "tests", "golden", "greedy_chain_16slots.npz")
CHAIN_STEPS = 64  # steps of the seeded greedy chain kept in the fixture


def place_contexts(ctx, world):
    """Placement as a scheduler would do it when slot s is served by rank s mod N: the same conversations, each put into a free
    slot of the rank that holds the fewest context tokens so far (longest first).  With one rank nothing changes."""
    if world <= 1:
        return ctx
    B = len(ctx)
    placed, load, free = np.zeros(B, ctx.dtype), np.zeros(world), [list(range(r, B, world)) for r in range(world)]
    for c in sorted(ctx.tolist(), reverse=True):
        r = min((q for q in range(world) if free[q]), key=lambda q: load[q])
        placed[free[r].pop(0)] = c
        load[r] += c
    return placed


def profile_step(gpu, eng, sids, cur):
    """One step with CUDA events around every dispatch (graphs off): {kernel name: [durations in us]}."""
    import ctypes as C
    gpu.L.qw_gpu_set_graphs(gpu.g, False)
    gpu.L.qw_profile_enable(gpu.g, True)
    nxt, _ = eng.step_greedy(sids, cur)
    per = {}
    for i in range(gpu.L.qw_profile_count(gpu.g)):
        us = C.c_double()
        nm = gpu.L.qw_profile_get(gpu.g, i, C.byref(us)).decode()
        per.setdefault(nm, []).append(us.value)
    gpu.L.qw_profile_enable(gpu.g, False)
    return per, nxt


def ncu_traffic_ratio():
    """dram bytes / algorithmic bytes of one launch of the expert FFN kernel, from the tracked ncu summary (a line
    'dram_bytes_per_launch: X  algorithmic_bytes_per_launch: Y'); None when no such capture is recorded."""
    import re
    try:
        txt = open(os.path.join(ROOT, "profiles", "moe_ffn_16slots_ncu.md")).read()
        m = re.search(r"dram_bytes_per_launch:\s*([0-9.eE+]+)\s+algorithmic_bytes_per_launch:\s*([0-9.eE+]+)", txt)
        return float(m.group(1)) / float(m.group(2)) if m else None
    except Exception:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--slots", type=int, default=16)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=48, help="(debug) fewer layers; a number measured with fewer layers is not a benchmark value")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--graphs", type=int, default=1)
    ap.add_argument("--ep", default="fused", choices=["nccl", "fused"],
                    help="expert-parallel exchange at N > 1: one NCCL all-reduce per layer, or peer stores fused into the down projection")
    ap.add_argument("--sustain", type=float, default=3.0, help="seconds of back-to-back chained steps for the sustained figure (0: skip)")
    ap.add_argument("--slots-big", type=int, default=64, help="second leg at this many slots on 1 GPU (0: skip)")
    ap.add_argument("--place-as", type=int, default=0, help="(1 GPU) lay the conversations out as the N-GPU run does: the chain then equals that run's")
    ap.add_argument("--write-chain", default="", help="(1 GPU) record the first %d steps of the seeded greedy chain under this key of the fixture and exit" % CHAIN_STEPS)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("QW_CUDA_DEVICE", str(local))
    import torch
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from qwental_b200 import synth
    from qwental_b200.engine import Engine, default_cfg, ep_unique_id
    from qwental_b200.gpu import Gpu

    B, K, W = args.slots, args.steps, max(3, args.warmup)
    place = world if world > 1 else max(1, args.place_as)
    ctx = place_contexts(synth.ragged_contexts(np.random.default_rng(0), B), place)
    BB = args.slots_big if (world == 1 and args.slots_big > B and not args.write_chain) else 0
    ctx_big = np.concatenate([ctx, synth.ragged_contexts(np.random.default_rng(1), BB)[B:]]) if BB else ctx
    peak, peak_src = measured_peak_gbs()
    est_ms = 8.0  # only to size the KV reservation of the sustained leg
    sustain_steps = int(args.sustain * 1e3 / est_ms * 2) if args.sustain > 0 else 0
    nsteps_total = 3 * (K + W) + 16 + sustain_steps + CHAIN_STEPS
    pages = int(sum((int(n) + nsteps_total + 256) // 256 + 1 for n in ctx_big))
    cfg = default_cfg(max_slots=max(B, BB), max_ctx=int(ctx_big.max()) + nsteps_total + 512, kv_pages=pages, ep_rank=rank, ep_size=world, seed=0, layers=args.layers)
    gpu = Gpu()
    eng = Engine(gpu, cfg)
    if world > 1:
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            idt.copy_(torch.frombuffer(bytearray(ep_unique_id()), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        eng.ep_init(bytes(idt.cpu().numpy().tobytes()))
        if args.ep == "fused":
            # every rank must take the same branch: agree on the outcome of the export before connecting
            try:
                mine = torch.frombuffer(bytearray(eng.ep_export()), dtype=torch.uint8).cuda()
                okf = torch.ones(1, device="cuda")
            except Exception as ex:  # e.g. no peer access between the GPUs: keep the NCCL exchange
                print("rank %d: fused exchange unavailable (%s), using the NCCL all-reduce" % (rank, ex), file=sys.stderr)
                mine, okf = torch.zeros(64, dtype=torch.uint8, device="cuda"), torch.zeros(1, device="cuda")
            dist.all_reduce(okf, op=dist.ReduceOp.MIN)
            if okf.item() > 0:
                allh = [torch.zeros(64, dtype=torch.uint8, device="cuda") for _ in range(world)]
                dist.all_gather(allh, mine)
                eng.ep_connect([bytes(t.cpu().numpy().tobytes()) for t in allh])
            else:
                args.ep = "nccl"
            dist.barrier()
    for s in range(len(ctx_big)):
        eng.seed_slot(s, int(ctx_big[s]), 100 + s)
    gpu.L.qw_gpu_set_graphs(gpu.g, bool(args.graphs))
    sids = np.arange(B, dtype=np.int32)
    toks = (np.arange(B, dtype=np.int32) * 7919) % cfg.vocab
    stream = torch.cuda.ExternalStream(int(gpu.L.qw_gpu_stream_handle(gpu.g, 0)))

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    if args.write_chain:  # fixture generation: the first CHAIN_STEPS steps of the chain every run below walks
        ids, _ = eng.decode_greedy(sids, toks, CHAIN_STEPS)
        old = dict(np.load(CHAIN_FIXTURE)) if os.path.exists(CHAIN_FIXTURE) else {}
        old[args.write_chain] = ids.astype(np.int32)
        np.savez_compressed(CHAIN_FIXTURE, **old)
        print(json.dumps({"wrote": CHAIN_FIXTURE, "key": args.write_chain, "steps": CHAIN_STEPS, "layers": cfg.layers}))
        eng.close()
        gpu.close()
        return

    # ---- warm-up (also builds the CUDA graphs of both step forms)
    chain = []
    ids, _ = eng.decode_greedy(sids, toks, W)
    chain.append(ids)
    cur = ids[-1]
    for _ in range(W):
        cur, _ = eng.step_greedy(sids, cur)
        chain.append(cur[None])

    # ---- timed region 1: K chained steps, inputs resident in HBM (weights 35 GB + KV: far larger than L2)
    sampler = ClockSampler(local)
    sampler.start()
    sync_all()
    l0 = gpu.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    ids, _ = eng.decode_greedy(sids, cur, K)
    e1.record(stream)
    sync_all()
    launches = gpu.launches() - l0
    dev_ms = e0.elapsed_time(e1)
    chain.append(ids)
    cur = ids[-1]
    # ---- timed region 2: K steps through the public call, host ids in / host ids out each step
    sync_all()
    t0 = time.perf_counter()
    for _ in range(K):
        cur, _ = eng.step_greedy(sids, cur)
        chain.append(cur[None])
    sync_all()
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    if dist is not None:
        tt = torch.tensor([dev_ms, e2e_wall_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dev_ms, e2e_wall_ms = float(tt[0]), float(tt[1])

    # ---- the chain so far against the committed single-GPU chain of the same seed and placement; all ranks must agree
    chain = np.concatenate(chain)
    ids_match = None
    if os.path.exists(CHAIN_FIXTURE) and cfg.layers == 48 and B == 16:
        fx = np.load(CHAIN_FIXTURE)
        key = "place%d" % place
        if key in fx.files:
            n = min(len(chain), fx[key].shape[0])
            ids_match = bool(np.array_equal(chain[:n], fx[key][:n]))
    if dist is not None:
        mine = torch.from_numpy(chain.astype(np.int32)).cuda()
        alls = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(alls, mine)
        same = all(bool(torch.equal(alls[0], a)) for a in alls)
        ids_match = (ids_match and same) if ids_match is not None else (None if same else False)

    # ---- sustained: the same chained steps back to back for a few seconds, SM clock sampled meanwhile
    sustained = None
    if sustain_steps > 0:
        smp = ClockSampler(local)
        smp.start()
        sync_all()
        done, t0s = 0, time.perf_counter()
        es, ee = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        es.record(stream)
        while time.perf_counter() - t0s < args.sustain and done + K <= sustain_steps:
            ids, _ = eng.decode_greedy(sids, cur, K)
            cur = ids[-1]
            done += K
        ee.record(stream)
        sync_all()
        sms = es.elapsed_time(ee)
        ck = smp.stop()
        if dist is not None:
            tt = torch.tensor([sms], dtype=torch.float64, device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            sms = float(tt[0])
        if done:
            sustained = {"value": B * done / (sms * 1e-3), "unit": UNIT, "steps": done, "seconds": sms * 1e-3, "ms_per_step": sms / done,
                         "sm_mhz": ck.get("sm_mhz"), "reasons": ck.get("reasons"), "clock_samples": ck.get("samples"),
                         "ms_per_step_x_sm_ghz": (sms / done) * (ck["sm_mhz"] / 1e3) if ck.get("sm_mhz") else None}

    # ---- per-kernel durations (CUDA events around every dispatch) and algorithmic bytes of the last step
    per, cur = profile_step(gpu, eng, sids, cur)
    sb = eng.step_bytes()
    fused = "moe_ffn" in per or "moe_ffn_epx" in per
    kname = "moe_ffn" if "moe_ffn" in per else "moe_ffn_epx" if fused else "moe_gu"
    experts_per_launch = sb.unique_experts_sum / cfg.layers + (1 if rank == 0 else 0)
    iq3x = fused and sb.moe_iq3s > 0 and abs(sb.moe - sb.moe_iq3s) > 1  # experts re-coded into the kernel's own layout (136 B / 256 weights)
    iq3s_bytes = experts_per_launch * (3 if fused else 2) * cfg.expert_inter * (cfg.hidden // 256 * 110)
    gu_bytes = experts_per_launch * ((cfg.expert_inter // 64) * (cfg.hidden // 512) + (cfg.hidden // 128) * (cfg.expert_inter // 512)) * 128 * 272 if iq3x else iq3s_bytes
    gu_us = float(np.mean(per.get(kname, [float("nan")])))
    achieved = gu_bytes / (gu_us * 1e-6) / 1e9
    ratio = ncu_traffic_ratio() if fused else None
    tot_us = sum(sum(v) for v in per.values())
    shares = {k: round(sum(v) / tot_us, 4) for k, v in sorted(per.items(), key=lambda kv: -sum(kv[1]))}
    kernel_us = {k: [len(v), round(float(np.mean(v)), 2)] for k, v in sorted(per.items(), key=lambda kv: -sum(kv[1]))}
    # the copy-only twin of the expert FFN kernel in its place: what the staging pipeline alone sustains on the same experts
    copy_gbs = None
    if fused and world == 1 and eng.L.qw_engine_set_moe_probe(eng.e, 1) == 0:
        perp, cur = profile_step(gpu, eng, sids, cur)
        eng.L.qw_engine_set_moe_probe(eng.e, 0)
        sbp = eng.step_bytes()
        pb = gu_bytes / experts_per_launch * (sbp.unique_experts_sum / cfg.layers + 1)
        pu = float(np.mean(perp.get("moe_ffn_copy_probe", [float("nan")])))
        copy_gbs = pb / (pu * 1e-6) / 1e9
    gpu.L.qw_gpu_set_graphs(gpu.g, bool(args.graphs))
    step_bytes_max = sb.total
    if dist is not None:  # every rank moves its own experts, KV pages and recurrent state: the slowest rank bounds the step
        tt = torch.tensor([sb.total], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        step_bytes_max = float(tt[0])

    # ---- 64 active slots (1 GPU): the first 16 are the same conversations
    big = None
    if BB:
        sb_ids = np.arange(BB, dtype=np.int32)
        tb = np.concatenate([cur, (np.arange(B, BB, dtype=np.int32) * 7919) % cfg.vocab]).astype(np.int32)
        ids, _ = eng.decode_greedy(sb_ids, tb, W)
        sync_all()
        eb0, eb1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        eb0.record(stream)
        ids, _ = eng.decode_greedy(sb_ids, ids[-1], K)
        eb1.record(stream)
        sync_all()
        bms = eb0.elapsed_time(eb1)
        sbb = eng.step_bytes()
        big = {"slots": BB, "value": BB * K / (bms * 1e-3), "unit": UNIT, "ms_per_step": bms / K, "ctx_tokens": int(sbb.ctx_tokens),
               "unique_experts_per_layer": sbb.unique_experts_sum / cfg.layers, "step_bytes": sbb.total,
               "step_frac_of_hbm_roofline": sbb.total / (peak * 1e9) * 1e3 / (bms / K)}

    if rank == 0:
        value = B * K / (dev_ms * 1e-3)
        e2e = B * K / (e2e_wall_ms * 1e-3)
        step_roof_ms = step_bytes_max / (peak * 1e9) * 1e3
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": dev_ms / K,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16 x int (IQ3_S / Q8_0 weights), f32 accumulate",
            "data": "synthetic",
            "config": workload_config(cfg.layers, B, int(ctx.sum()), world, args.graphs, args.ep),
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": 3 * 64 * 4, "d2h_bytes_per_step": B * 4, "ms_per_step": e2e_wall_ms / K},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": kname + (" (IQ3_S gate/up + down matvecs over the gathered experts, one launch per layer)" if fused
                                                               else " (IQ3_S gate/up matvec over gathered experts)"),
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": gu_bytes * ratio if ratio else None,
                         "traffic_source": "ncu dram bytes of one launch (tracked summary under profiles/), scaled by algorithmic bytes" if ratio
                                           else "no ncu capture of this kernel recorded",
                         "peak_source": peak_src, "bytes_per_launch": gu_bytes, "us_per_launch": gu_us, "copy_ceiling_gbs": copy_gbs,
                         "weight_format": "IQ3X (the IQ3_S experts re-coded losslessly at load time, 136 bytes per 256 weights)" if iq3x else "IQ3_S (110 bytes per 256 weights)",
                         "iq3s_equivalent_gbs": iq3s_bytes / (gu_us * 1e-6) / 1e9},
            "step_bytes": {"total": step_bytes_max, "moe": sb.moe, "moe_in_iq3s_bytes": sb.moe_iq3s, "dense": sb.dense, "lm_head": sb.lm_head, "kv": sb.kv, "gdn_state": sb.gdn_state,
                           "scope": "one rank (the largest over ranks in total)" if world > 1 else "the GPU",
                           "unique_experts_per_layer": sb.unique_experts_sum / cfg.layers, "ctx_tokens": int(sb.ctx_tokens),
                           "step_roofline_ms": step_roof_ms, "step_frac_of_hbm_roofline": step_roof_ms / (dev_ms / K),
                           "frac_of_nominal_8TBs": step_bytes_max / 8e12 * 1e3 / (dev_ms / K)},
            "kernel_time_shares": shares, "kernel_us": kernel_us,
            "ids_match_single_gpu": ids_match,
        }
        if sustained:
            out["sustained"] = sustained
        if big:
            out["slots64" if BB == 64 else "slots_big"] = big
        if world == 1 and not args.no_cpu:
            v, cores, kind, sample = cpu_baseline_avg(B, ctx)
            out["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample}
        print(json.dumps(out))
    if dist is not None:
        dist.barrier()  # nobody unmaps or frees an exchange buffer while another rank may still be stepping
    eng.close()
    gpu.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
