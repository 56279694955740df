#!/usr/bin/env python
"""Benchmark of the speculative-decode (MTP) step on seeded random-init Gemma-4-architecture GGUFs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config b12|e4b|tiny] [--depth D] [--p P] [--mtp-n M]

One "step" is one MTP round at batch 1: M-1 draft-head forwards, one M-token verify forward of
the target (every weight streamed once), greedy acceptance and position advance -- all on the
device, rounds back to back with no host synchronisation.  Drafts are the draft head's cost plus
oracle-replayed tokens: the head runs, then its tokens are replaced by ones that match the
recorded plain-greedy stream with probability p, because a random-init head accepts ~nothing.

  value      tokens emitted per second over K rounds, device-timed (CUDA events on the engine's
             stream), inputs resident in HBM; whole job = sum over ranks / max rank time
  e2e        the same metric through the reference-shaped blocking C API (mtp_draft,
             mtp_draft_chain, model_forward_spec): every call uploads its tokens and position
             and downloads its result, host clock
  roofline   the weight-streaming matmul kernel timed alone over one verify step's matrices
             (cold: 6.6 GB >> L2): algorithmic q4 bytes / device time vs the measured HBM peak
  cpu_baseline  the reference's own CPU backend (oracle/_ref) on the same file, plain greedy
             decode, a bounded sample of tokens on the host cores

N > 1 (torchrun): one independent replica per GPU, own session seed, no collective on the data
path; a gloo barrier brackets the timed region and the max time over ranks is used.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

RANK = int(os.environ.get("RANK", "0"))
LOCAL_RANK = int(os.environ.get("LOCAL_RANK", "0"))
WORLD = int(os.environ.get("WORLD_SIZE", "1"))
if WORLD > 1 and "LG_B200_VISIBLE_SET" not in os.environ:
    # one GPU per process, fixed before any CUDA runtime initialises (the library and torch each
    # carry their own runtime; both must see the same single device)
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    devs = vis.split(",") if vis else [str(i) for i in range(64)]
    os.environ["CUDA_VISIBLE_DEVICES"] = devs[LOCAL_RANK % len(devs)]
    os.environ["LG_B200_VISIBLE_SET"] = "1"

import numpy as np  # noqa: E402

CACHE = os.environ.get("LG_B200_CACHE", "/tmp/lg_b200_cache")
# dram__bytes_read+write / algorithmic bytes of the matmul kernel, from profiles/gemv_e4b_gateup_ncu.md
DRAM_TRAFFIC_RATIO = 37.793024 / 37.748736


def shapes(name):
    s = importlib.import_module("little-gemma_b200.synth")
    return {"b12": (s.B12, s.B12_HEAD, "12B-class q4_0"), "e4b": (s.E4B, s.E4B_HEAD, "E4B-class q4_0"),
            "tiny": (s.TINY, s.TINY_HEAD, "tiny q4_0")}[name]


def ensure_files(cfg, device, layers=0):
    """Seeded model files under CACHE (rank 0 writes; big ones are generated on the GPU)."""
    s = importlib.import_module("little-gemma_b200.synth")
    t, h, _ = shapes(cfg)
    tag = cfg
    if layers > 0:
        import dataclasses
        t = dataclasses.replace(t, n_layer=layers)
        tag = f"{cfg}_l{layers}"
    dev = device if t.weight_bytes() > (1 << 28) else "cpu"
    tp = s.cached(CACHE, f"{tag}_seed0_{dev}.gguf", s.write_target, t, 0, dev)
    hp = s.cached(CACHE, f"{tag}_head_seed1_{dev}.gguf", s.write_head, h, t, 1, dev)
    return tp, hp


class ClockSampler:
    """nvidia-smi sampled in the background during a timed region."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.p = None

    def start(self):
        try:
            idx = os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or "0"
            self.p = subprocess.Popen(["nvidia-smi", "-i", idx, f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.p = None

    def stop(self):
        if not self.p:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.p.terminate()
        out, _ = self.p.communicate(timeout=5)
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            try:
                sm.append(float(f[0])); mx = max(mx, float(f[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_reference_run(tp, n_tokens, warm=1):
    """Plain greedy decode of the reference CPU backend on the host cores; returns (tok/s, dict)."""
    from oracle import pyref
    kind = "reference" if os.path.exists(pyref.ref_lib_path(4)) else "port"
    if kind == "port":
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "port"])
    # all host cores (torchrun pins OMP_NUM_THREADS=1 for its workers; the CPU baseline is not one of them)
    cores = int(os.environ.get("LG_CPU_THREADS", os.cpu_count() or 1))
    os.environ["OMP_NUM_THREADS"] = str(cores)
    o = (pyref.RefOracle if kind == "reference" else pyref.PortOracle)(tp, None, 64, False, 4)
    tok, pos = 1, 0
    for _ in range(warm):
        tok = o.next(tok, pos); pos += 1
    t0 = time.perf_counter()
    for _ in range(n_tokens):
        tok = o.next(tok, pos); pos += 1
    dt = time.perf_counter() - t0
    o.close()
    return n_tokens / dt, {"kind": kind, "cores": int(os.environ["OMP_NUM_THREADS"]),
                           "sample": f"{n_tokens} plain greedy tokens at depth<{pos} after {warm} warm-up, OpenMP over rows"}


def kv_bytes_step(t, depth, M):
    """f16 K and V rows one verify step reads (each row once) and writes."""
    per_pos = 4 * t.n_head_kv * t.head_dim
    own = t.n_layer - t.shared_kv_layers
    rd = sum(per_pos * (min(depth + M, t.window) if t.is_local(l) else depth + M) for l in range(t.n_layer))
    return rd + M * per_pos * own


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="b12", choices=["b12", "e4b", "tiny"])
    ap.add_argument("--depth", type=int, default=1024)
    ap.add_argument("--p", type=float, default=0.8)
    ap.add_argument("--mtp-n", type=int, default=4)
    ap.add_argument("--cpu-tokens", type=int, default=4)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--profile-step", action="store_true",
                    help="short path for profilers: load, prefill, W warm-up rounds, K rounds, exit")
    ap.add_argument("--profile-prefill", type=int, default=None, metavar="CLASSES",
                    help="short path for profilers: load, model_prefill of 512 tokens, 3 wide prompt blocks of 256 tokens "
                         "restricted to kernel classes (4 = gate/up matmul, 1023 = everything), exit")
    ap.add_argument("--layers", type=int, default=0, help="cut the model to this many layers (small profiling cases)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    t_shape, h_shape, label = shapes(a.config)
    if a.layers > 0:
        import dataclasses
        t_shape = dataclasses.replace(t_shape, n_layer=a.layers)
        label += f" cut to {a.layers} layers"
    M = a.mtp_n
    workload = (f"{label}, batch 1, MTP K={M - 1} (verify width {M}), KV depth {a.depth}, "
                f"oracle-replayed drafts p={a.p}, greedy")
    base = {"metric": "MTP decode tok/s (batch 1)", "unit": "tok/s", "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
            "config": {"workload": workload, "weights": "seeded N(0,0.02) q4_0", "l2": "inputs larger than L2 (weights >> 126 MB)"}}

    # ---------------------------------------------------------------- reference arm (CPU)
    if a.impl == "reference":
        if RANK != 0:
            return
        import torch
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        tp, hp = ensure_files(a.config, dev, a.layers)
        n = max(1, min(a.steps, a.cpu_tokens))
        tps, info = cpu_reference_run(tp, n, warm=min(a.warmup, 1))
        line = dict(base, impl="reference", value=tps, ms_per_step=1e3 / tps, dtype="f32",
                    cpu_baseline=dict(info, value=tps, unit="tok/s"),
                    e2e={"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    gpu_launches=0)
        line["config"] = dict(line["config"], note="reference CPU backend, plain greedy decode (its MTP path runs the "
                              "same forwards sequentially); a step is one token; bounded sample")
        print(json.dumps(line), flush=True)
        return

    # ---------------------------------------------------------------- our arm (GPU)
    import torch
    import torch.distributed as dist
    if WORLD > 1:
        dist.init_process_group("gloo", rank=RANK, world_size=WORLD)
    torch.cuda.set_device(0)
    lg = importlib.import_module("little-gemma_b200")
    synth = importlib.import_module("little-gemma_b200.synth")
    build = importlib.import_module("little-gemma_b200.build")
    if RANK == 0:
        build.build()
        ensure_files(a.config, "cuda", a.layers)
    if WORLD > 1:
        dist.barrier()
    tp, hp = ensure_files(a.config, "cuda", a.layers)
    torch.cuda.empty_cache()

    V = t_shape.n_vocab
    n_gen = (a.steps + a.warmup + 4) * M + 8
    max_seq = a.depth + n_gen + 64
    sess = lg.Session(tp, hp, max_seq, mtp_n=M)
    stream = torch.cuda.ExternalStream(sess.stream())
    prompt = synth.prompt_ids(a.depth, V, seed=100 + RANK)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def barrier():
        torch.cuda.synchronize()
        if WORLD > 1:
            dist.barrier()

    # prompt -> cache, first token.  Every timed phase below starts from this state again: a phase
    # may run past the sliding-window rings' length, after which rewinding the position would read
    # rows that later positions have overwritten.
    def restart():
        sess.prefill(prompt[:-1], 0)
        return sess.next(int(prompt[-1]), a.depth - 1)

    if a.profile_prefill is not None:
        sess.prefill(synth.prompt_ids(min(512, max_seq - 8), V, seed=300), 0)
        n_l = 0
        for _ in range(3):
            n_l = sess.prefill_pass(256, a.profile_prefill)
        torch.cuda.synchronize()
        print(json.dumps({"profile_prefill": a.profile_prefill, "launches_per_block": n_l, "config": base["config"]}), flush=True)
        sess.close()
        return

    first = restart()
    pos0 = a.depth

    if a.profile_step:
        sess.set_replay(np.zeros(n_gen + 8, dtype=np.int32))
        sess.rounds_begin(first, pos0, 1)
        sess.rounds_enqueue(M, 2, a.warmup)
        sess.rounds_collect(1, 0)
        e0, e1 = ev(), ev()
        e0.record(stream)
        sess.rounds_enqueue(M, 2, a.steps)
        e1.record(stream)
        e1.synchronize()
        print(json.dumps({"profile_step": True, "ms_per_round": e0.elapsed_time(e1) / a.steps,
                          "launches_per_round": sess.round_launches(), "config": base["config"]}), flush=True)
        sess.close()
        return

    # the plain-greedy stream the drafts are replayed from (device-resident plain decode)
    sess.rounds_begin(first, pos0, 1)
    sess.rounds_enqueue(1, 0, n_gen, use_head=False)
    plain, st = sess.rounds_collect(1, n_gen)
    greedy = np.concatenate([[first], plain]).astype(np.int32)
    replay = synth.replay_drafts(greedy, V, a.p, seed=7 + RANK)
    sess.set_replay(replay)

    # warm-up rounds (graph capture happens here), then K timed rounds
    restart()
    sess.rounds_begin(first, pos0, 1)
    sess.rounds_enqueue(M, 2, a.warmup)
    _, st_w = sess.rounds_collect(1, 0)
    launches_per_round = sess.round_launches()
    clk = ClockSampler()
    barrier()
    clk.start()
    e0, e1 = ev(), ev()
    e0.record(stream)
    sess.rounds_enqueue(M, 2, a.steps)
    e1.record(stream)
    e1.synchronize()
    barrier()
    clocks = clk.stop()
    ms = e0.elapsed_time(e1)
    toks, st = sess.rounds_collect(1, st_w["n_emitted"] + a.steps * M)
    emitted = st["n_emitted"] - st_w["n_emitted"]
    got = np.concatenate([[first], toks])[:st["n_emitted"]]
    identical = bool(np.array_equal(got, greedy[:len(got)]))
    accept = (st["n_accept"] - st_w["n_accept"]) / max(1, st["n_draft"] - st_w["n_draft"])

    # plain decode (verify width 1) for context
    restart()
    sess.rounds_begin(first, pos0, 1)
    sess.rounds_enqueue(1, 0, a.warmup, use_head=False)
    sess.rounds_collect(1, 0)
    p0, p1 = ev(), ev()
    p0.record(stream)
    sess.rounds_enqueue(1, 0, a.steps, use_head=False)
    p1.record(stream)
    p1.synchronize()
    plain_ms = p0.elapsed_time(p1) / a.steps

    # verify step alone (no draft head) at width M
    restart()
    sess.rounds_begin(first, pos0, 1)
    sess.rounds_enqueue(M, 2, a.warmup, use_head=False)
    sess.rounds_collect(1, 0)
    v0, v1 = ev(), ev()
    v0.record(stream)
    sess.rounds_enqueue(M, 2, a.steps, use_head=False)
    v1.record(stream)
    v1.synchronize()
    verify_ms = v0.elapsed_time(v1) / a.steps

    # the streaming matmul kernel alone: all matrices of one verify step, cold, event-timed
    reps = 10
    n_mm = sess.matmul_pass(M)
    torch.cuda.synchronize()
    m0, m1 = ev(), ev()
    m0.record(stream)
    for _ in range(reps):
        sess.matmul_pass(M)
    m1.record(stream)
    m1.synchronize()
    mm_ms = m0.elapsed_time(m1) / reps
    W = t_shape.weight_bytes() - int(t_shape.n_embd * t_shape.ple * t_shape.n_layer * 0.5625)  # proj table is gathered, not multiplied

    # the prompt pass: model_prefill of a 929-token prompt (host call, wall clock, synchronised), and the
    # wide tcgen05 matmuls of one 256-token block over all layers, event-timed, against the tensor peak
    prefill_rec = None
    n_pf = min(929, max_seq - 8)
    pf_prompt = synth.prompt_ids(n_pf, V, seed=300 + RANK)
    sess.prefill(pf_prompt, 0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    sess.prefill(pf_prompt, 0)
    torch.cuda.synchronize()
    pf_s = time.perf_counter() - t0
    prefill_rec = {"tokens": n_pf, "ms": pf_s * 1e3, "tok_s": n_pf / pf_s}
    if sess.prefill_pass(256, 0) > 0:
        torch.cuda.synchronize()
        g0, g1 = ev(), ev()
        g0.record(stream)
        for _ in range(5):
            n_pf_mm = sess.prefill_pass(256, 0)
        g1.record(stream)
        g1.synchronize()
        pf_mm_ms = g0.elapsed_time(g1) / 5
        ne_, H_, Hkv_, hd_, L_, nff_ = (t_shape.n_embd, t_shape.n_head, t_shape.n_head_kv, t_shape.head_dim, t_shape.n_layer,
                                        t_shape.n_ff)
        layer_params = L_ * (ne_ * (H_ + 2 * Hkv_) * hd_ + H_ * hd_ * ne_ + 3 * ne_ * nff_)
        tfl = 2.0 * layer_params * 256 / (pf_mm_ms * 1e-3) / 1e12
        prefill_rec["matmul_block"] = {"bound": "tensor", "kernel": "lg_pf_gemm_kernel (tcgen05, f16 operands, f32 accumulate)",
                                       "tokens": 256, "launches": n_pf_mm, "ms": pf_mm_ms, "achieved": tfl, "unit": "TFLOP/s"}

    # end to end through the blocking reference-shaped API
    e2e_rounds = max(20, a.steps // 3)
    restart()
    sess.rounds_host(first, pos0, 1, 8 * M, 4, 3, replay)                       # warm the per-call graphs
    restart()
    barrier()
    t0 = time.perf_counter()
    toks_h, st_h = sess.rounds_host(first, pos0, 1, n_gen, e2e_rounds, 3, replay)
    torch.cuda.synchronize()
    dt_h = time.perf_counter() - t0
    e2e_tps = len(toks_h) / dt_h
    identical = identical and bool(np.array_equal(toks_h, greedy[1:1 + len(toks_h)]))
    h2d = (M - 1) * 12 + (1 + M) * 4
    d2h = (M - 1) * 4 + 36 + 4

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s"
    kvb = kv_bytes_step(t_shape, a.depth, M)
    mm_gbs = W / (mm_ms * 1e-3) / 1e9
    if prefill_rec and "matmul_block" in prefill_rec:
        tpeak = float(peaks.get("bf16_tflops_sustained", 1400.0))
        prefill_rec["matmul_block"].update(peak=tpeak, frac=prefill_rec["matmul_block"]["achieved"] / tpeak,
                                           peak_source=("measured (MEASURED_PEAKS.json bf16_tflops_sustained: the pass is a few ms of "
                                                        "back-to-back launches)" if peaks else "fallback 1400 TFLOP/s sustained"))

    # aggregate over replicas
    my = torch.tensor([float(emitted), float(ms), float(len(toks_h)), float(dt_h), float(identical)], dtype=torch.float64)
    if WORLD > 1:
        allv = [torch.zeros_like(my) for _ in range(WORLD)]
        dist.all_gather(allv, my)
    else:
        allv = [my]
    from importlib import import_module
    agg = import_module("little-gemma_b200.replicas").aggregate([v.tolist() for v in allv])

    cpu = None
    if RANK == 0 and WORLD == 1 and not a.no_cpu:
        try:
            tps, info = cpu_reference_run(tp, a.cpu_tokens)
            cpu = dict(info, value=tps, unit="tok/s")
        except Exception as ex:  # the checker is optional for the timing itself
            cpu = {"value": None, "unit": "tok/s", "kind": "unavailable", "cores": 0, "sample": repr(ex)}

    if RANK == 0:
        line = dict(base, impl="ours", value=agg["tok_s"], ms_per_step=agg["max_ms"] / a.steps, dtype="int8",
                    clocks=clocks, gpu_launches=int(launches_per_round * a.steps),
                    e2e={"value": agg["e2e_tok_s"], "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                         "rounds": e2e_rounds, "host_syncs_per_round": M},
                    roofline={"bound": "hbm", "kernel": "lg_gemv_kernel", "achieved": mm_gbs, "peak": peak, "unit": "GB/s",
                              "frac": mm_gbs / peak, "traffic": int(W * DRAM_TRAFFIC_RATIO), "peak_source": peak_src,
                              "traffic_note": "dram read+write bytes of the matmul pass: ncu capture of the E4B-class gate/up "
                                              "launch (37.793 MB moved for 37.749 MB of q4_0) scaled by weight bytes; writes 0",
                              "algorithmic_bytes": W, "launches": n_mm, "ms": mm_ms,
                              "frac_of_8TBs": mm_gbs / 8000.0},
                    cpu_baseline=cpu, prefill=prefill_rec)
        line["config"] = dict(line["config"], mtp_n=M, depth=a.depth, p=a.p, launches_per_round=int(launches_per_round),
                              tokens_per_round=emitted / a.steps, acceptance=accept,
                              stream_identical_to_plain_greedy=bool(agg["identical"]),
                              plain_decode_ms=plain_ms, plain_decode_tok_s=1e3 / plain_ms,
                              verify_step_ms=verify_ms,
                              verify_step_gbs=(W + kvb) / (verify_ms * 1e-3) / 1e9,
                              verify_step_frac_measured=(W + kvb) / (verify_ms * 1e-3) / 1e9 / peak,
                              verify_step_frac_8TBs=(W + kvb) / (verify_ms * 1e-3) / 1e9 / 8000.0,
                              weight_bytes=W, kv_bytes_step=kvb)
        print(json.dumps(line), flush=True)
    sess.close()
    if WORLD > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
