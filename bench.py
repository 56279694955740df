#!/usr/bin/env python
"""Benchmark of the speculative-decode (MTP) step on seeded random-init Gemma-4-architecture GGUFs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config b12|b12k|e4b|tiny|c5] [--depth D] [--p P] [--mtp-n M]
    python bench.py --sweep e4b|b12|b12k [--sweep-out FILE.md]

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
  roofline   the dominant kernel (the small-M weight matmul, in the epilogue variants the step
             runs) over one verify step's matrices, replayed alone and cold (6.6 GB >> L2):
             algorithmic q4 bytes / device time vs the measured HBM peak; `step_frac` is the whole
             verify step (weights + cache rows) / its device time vs the same peak
  cpu_baseline  the reference's own CPU backend (oracle/_ref) on the same file, plain greedy
             decode, a bounded sample of tokens on the host cores

--config c5 is the serving workload of the plan: a 2048-token prompt and 1024 generated tokens at
p = 0.7 per session (K is then the number of rounds that took).  --sweep runs the plan's tables for
one model (KV depth x verify width x acceptance) and writes them as markdown.

N > 1 (torchrun): one independent replica per GPU, own prompt seed, no collective on the data
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
if "reference" in sys.argv:
    # The CPU arm wants every host core.  A launcher may have exported OMP_NUM_THREADS=1 for its workers
    # (torchrun does); OpenMP runtimes read it when they are loaded, so it is replaced before anything loads one.
    os.environ["OMP_NUM_THREADS"] = os.environ.get("LG_CPU_THREADS", str(os.cpu_count() or 1))
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
    import dataclasses
    b12k = dataclasses.replace(s.B12, wtype=s.Q4_K)
    return {"b12": (s.B12, s.B12_HEAD, "12B-class q4_0"), "e4b": (s.E4B, s.E4B_HEAD, "E4B-class q4_0"),
            "b12k": (b12k, s.B12_HEAD, "12B-class q4_K"), "c5": (s.B12, s.B12_HEAD, "12B-class q4_0"),
            "tiny": (s.TINY, s.TINY_HEAD, "tiny q4_0")}[name]


def ensure_files(cfg, device, layers=0):
    """Seeded model files under CACHE (rank 0 writes; big ones are generated on the GPU)."""
    s = importlib.import_module("little-gemma_b200.synth")
    t, h, _ = shapes(cfg)
    tag = "b12" if cfg == "c5" else cfg
    if layers > 0:
        import dataclasses
        t = dataclasses.replace(t, n_layer=layers)
        tag = f"{tag}_l{layers}"
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
                                       "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            time.sleep(0.15)            # let the first samples land before the timed region opens
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
    want = int(os.environ.get("LG_CPU_THREADS", os.cpu_count() or 1))
    o = (pyref.RefOracle if kind == "reference" else pyref.PortOracle)(tp, None, 64, False, 4)
    cores = o.set_threads(want)          # what the checker's OpenMP runtime will really use (not the environment's word)
    tok, pos = 1, 0
    for _ in range(warm):
        tok = o.next(tok, pos); pos += 1
    t0 = time.perf_counter()
    for _ in range(n_tokens):
        tok = o.next(tok, pos); pos += 1
    dt = time.perf_counter() - t0
    o.close()
    return n_tokens / dt, {"kind": kind, "cores": cores,
                           "sample": f"{n_tokens} plain greedy tokens at depth<{pos} after {warm} warm-up, OpenMP over rows"}


def kv_bytes_step(t, depth, M):
    """f16 K and V rows one verify step reads (each row once) and writes."""
    own = t.n_layer - t.shared_kv_layers
    rd = sum(4 * t.n_head_kv * t.hd(l) * (min(depth + M, t.window) if t.is_local(l) else depth + M) for l in range(t.n_layer))
    return rd + M * sum(4 * t.n_head_kv * t.hd(l) for l in range(own))


def matmul_weight_bytes(t):
    """q4 bytes the matmuls of one verify step stream (the per-layer token table is gathered, not multiplied)."""
    return t.weight_bytes() - int(t.n_embd * t.ple * t.n_layer * 0.5625)


class Runner:
    """One loaded session at a fixed KV depth plus the timing helpers shared by the default line and the sweeps."""

    def __init__(self, lg, synth, torch, tp, hp, t_shape, depth, n_gen, mtp_n, seed):
        self.lg, self.synth, self.torch, self.t = lg, synth, torch, t_shape
        self.depth, self.n_gen = depth, n_gen
        self.max_seq = depth + n_gen + 64
        self.sess = lg.Session(tp, hp, self.max_seq, mtp_n=mtp_n)
        self.stream = torch.cuda.ExternalStream(self.sess.stream())
        self.prompt = synth.prompt_ids(depth, t_shape.n_vocab, seed=seed)
        self.first = self.restart()
        self.greedy = None

    def ev(self):
        return self.torch.cuda.Event(enable_timing=True)

    # prompt -> cache, first token.  Every timed phase starts from this state again: a phase may run past the
    # sliding-window rings' length, after which rewinding the position would read rows that later positions overwrote.
    def restart(self):
        self.sess.prefill(self.prompt[:-1], 0)
        return self.sess.next(int(self.prompt[-1]), self.depth - 1)

    def plain_stream(self):
        """The plain-greedy stream the drafts are replayed from (device-resident plain decode)."""
        s = self.sess
        s.rounds_begin(self.first, self.depth, 1)
        if s.rounds_enqueue(1, 0, self.n_gen, use_head=False) != 0:
            raise RuntimeError("plain decode rounds refused")
        plain, _ = s.rounds_collect(1, self.n_gen)
        self.greedy = np.concatenate([[self.first], plain]).astype(np.int32)
        return self.greedy

    def timed_rounds(self, M, mode, steps, warmup, use_head, sampler=None, barrier=None):
        """Warm-up rounds (graph capture happens there), then `steps` rounds between two events on the engine's stream."""
        s = self.sess
        self.restart()
        s.rounds_begin(self.first, self.depth, 1)
        if s.rounds_enqueue(M, mode, warmup, use_head=use_head) != 0:
            raise RuntimeError("rounds refused")
        _, st_w = s.rounds_collect(1, 0)
        if barrier:
            barrier()
        if sampler:
            sampler.start()
        e0, e1 = self.ev(), self.ev()
        e0.record(self.stream)
        if s.rounds_enqueue(M, mode, steps, use_head=use_head) != 0:
            raise RuntimeError("rounds refused")
        e1.record(self.stream)
        e1.synchronize()
        if barrier:
            barrier()
        clocks = sampler.stop() if sampler else None
        ms = e0.elapsed_time(e1)
        toks, st = s.rounds_collect(1, st_w["n_emitted"] + steps * M)
        emitted = st["n_emitted"] - st_w["n_emitted"]
        got = np.concatenate([[self.first], toks])[:st["n_emitted"]]
        identical = self.greedy is None or bool(np.array_equal(got, self.greedy[:len(got)]))
        accept = (st["n_accept"] - st_w["n_accept"]) / max(1, st["n_draft"] - st_w["n_draft"])
        return {"ms": ms, "emitted": emitted, "identical": identical, "accept": accept, "clocks": clocks}

    def close(self):
        self.sess.close()


def sweep(a, lg, synth, torch):
    """The plan's tables for one model: KV depth x verify width x acceptance; markdown to --sweep-out."""
    cfg = a.sweep
    t_shape, h_shape, label = shapes(cfg)
    tp, hp = ensure_files(cfg, "cuda")
    depths = [int(x) for x in a.sweep_depths.split(",")]
    widths = [int(x) for x in a.sweep_widths.split(",")]
    ps = [float(x) for x in a.sweep_p.split(",")]
    steps, warm = max(a.steps // 6, 30), 4
    peaks = load_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    W = matmul_weight_bytes(t_shape)
    rows, lines = [], []
    for depth in depths:
        n_gen = (steps + warm + 4) * max(widths) + 8
        r = Runner(lg, synth, torch, tp, hp, t_shape, depth, n_gen, max(widths), seed=100)
        greedy = r.plain_stream()
        for M in widths:
            # the verify step alone (no draft head), then rounds with the head at each acceptance
            r.sess.set_replay(synth.replay_drafts(greedy, t_shape.n_vocab, 1.0, seed=7))
            v = r.timed_rounds(M, 2 if M > 1 else 0, steps, warm, use_head=False)
            verify_ms = v["ms"] / steps
            kvb = kv_bytes_step(t_shape, depth, M)
            for p in (ps if M > 1 else [None]):
                if p is None:
                    rec = {"tok_s": v["emitted"] / (v["ms"] * 1e-3), "ms_round": verify_ms, "tokens_round": 1.0, "identical": v["identical"]}
                else:
                    r.sess.set_replay(synth.replay_drafts(greedy, t_shape.n_vocab, p, seed=7))
                    m = r.timed_rounds(M, 2, steps, warm, use_head=True)
                    rec = {"tok_s": m["emitted"] / (m["ms"] * 1e-3), "ms_round": m["ms"] / steps,
                           "tokens_round": m["emitted"] / steps, "identical": m["identical"]}
                rec.update(config=cfg, depth=depth, M=M, p=p, verify_ms=verify_ms,
                           verify_gbs=(W + kvb) / (verify_ms * 1e-3) / 1e9, verify_frac=(W + kvb) / (verify_ms * 1e-3) / 1e9 / peak)
                rows.append(rec)
                print(json.dumps({"sweep": rec}), flush=True)
        r.close()
    lines.append(f"# Sweep: {label}, batch 1, device-resident rounds ({steps} timed rounds per cell)\n")
    lines.append(f"Command: `python bench.py --sweep {cfg} --sweep-depths {a.sweep_depths} --sweep-widths {a.sweep_widths} "
                 f"--sweep-p {a.sweep_p} --steps {a.steps}`.  CUDA events on the engine's stream; verify step = weights "
                 f"({W / 1e9:.3f} GB) + cache rows over its device time, against the measured copy peak {peak:.0f} GB/s.  "
                 f"M = verify width (M = 1 is plain decode, no drafts); p = probability that a replayed draft matches.\n")
    lines.append("| depth | M | p | tok/s | ms/round | tokens/round | verify ms | verify GB/s | of measured peak | stream = plain greedy |")
    lines.append("|---:|---:|---:|---:|---:|---:|---:|---:|---:|:---:|")
    for x in rows:
        lines.append(f"| {x['depth']} | {x['M']} | {'-' if x['p'] is None else x['p']} | {x['tok_s']:.1f} | {x['ms_round']:.3f} | "
                     f"{x['tokens_round']:.2f} | {x['verify_ms']:.3f} | {x['verify_gbs']:.0f} | {x['verify_frac']:.3f} | "
                     f"{'yes' if x['identical'] else 'NO'} |")
    if a.sweep_prefill:
        r = Runner(lg, synth, torch, tp, hp, t_shape, 16, 1024, 4, seed=100)
        pf = time_prefill(r, synth, torch, t_shape, peaks)
        r.close()
        print(json.dumps({"sweep_prefill": pf}), flush=True)
        lines.append(f"\nPrompt pass of {pf['tokens']} uniform-random tokens (model_prefill, host clock, synchronised): "
                     f"{pf['ms']:.1f} ms = {pf['tok_s']:.0f} tok/s" +
                     (f"; the tcgen05 layer matmuls of one 256-token block: {pf['matmul_block']['ms']:.2f} ms = "
                      f"{pf['matmul_block']['achieved']:.0f} TFLOP/s = {pf['matmul_block']['frac']:.3f} of the measured sustained "
                      f"bf16 peak." if "matmul_block" in pf else "."))
    out = a.sweep_out or os.path.join(ROOT, "gpurun_out", f"sweep_{cfg}.md")
    os.makedirs(os.path.dirname(out), exist_ok=True)
    with open(out, "w") as f:
        f.write("\n".join(lines) + "\n")


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        return {}


def time_prefill(r, synth, torch, t_shape, peaks):
    """model_prefill of a 929-token prompt (host call, wall clock, synchronised) and the wide tcgen05 matmuls of one
    256-token block over all layers, event-timed, against the tensor peak."""
    sess = r.sess
    n_pf = min(929, r.max_seq - 8)
    pf_prompt = synth.prompt_ids(n_pf, t_shape.n_vocab, seed=300 + RANK)
    sess.prefill(pf_prompt, 0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    sess.prefill(pf_prompt, 0)
    torch.cuda.synchronize()
    pf_s = time.perf_counter() - t0
    rec = {"tokens": n_pf, "ms": pf_s * 1e3, "tok_s": n_pf / pf_s}
    if sess.prefill_pass(256, 0) > 0:
        torch.cuda.synchronize()
        g0, g1 = r.ev(), r.ev()
        g0.record(r.stream)
        for _ in range(5):
            n_pf_mm = sess.prefill_pass(256, 0)
        g1.record(r.stream)
        g1.synchronize()
        pf_mm_ms = g0.elapsed_time(g1) / 5
        ne_, H_, Hkv_, nff_ = t_shape.n_embd, t_shape.n_head, t_shape.n_head_kv, t_shape.n_ff
        layer_params = sum(ne_ * (H_ + 2 * Hkv_) * t_shape.hd(l) + H_ * t_shape.hd(l) * ne_ + 3 * ne_ * nff_ for l in range(t_shape.n_layer))
        tfl = 2.0 * layer_params * 256 / (pf_mm_ms * 1e-3) / 1e12
        tpeak = float(peaks.get("bf16_tflops_sustained", 1400.0))
        rec["matmul_block"] = {"bound": "tensor", "kernel": "lg_pf_gemm_kernel (tcgen05, f16 operands, f32 accumulate)",
                               "tokens": 256, "launches": n_pf_mm, "ms": pf_mm_ms, "achieved": tfl, "unit": "TFLOP/s",
                               "peak": tpeak, "frac": tfl / tpeak,
                               "peak_source": ("measured (MEASURED_PEAKS.json bf16_tflops_sustained: the pass is a few ms of "
                                               "back-to-back launches)" if peaks else "fallback 1400 TFLOP/s sustained")}
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="b12", choices=["b12", "b12k", "e4b", "tiny", "c5"])
    ap.add_argument("--depth", type=int, default=None)
    ap.add_argument("--p", type=float, default=None)
    ap.add_argument("--mtp-n", type=int, default=4)
    ap.add_argument("--cpu-tokens", type=int, default=4)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--sweep", default=None, choices=["e4b", "b12", "b12k", "tiny"],
                    help="run the depth x width x acceptance tables of one model instead of the benchmark line")
    ap.add_argument("--sweep-depths", default="1024,8192,32768")
    ap.add_argument("--sweep-widths", default="1,2,4,5,8")
    ap.add_argument("--sweep-p", default="0,0.5,0.8,1")
    ap.add_argument("--sweep-prefill", action="store_true", help="with --sweep: also time the 929-token prompt pass")
    ap.add_argument("--sweep-out", default=None)
    ap.add_argument("--profile-step", action="store_true",
                    help="short path for profilers: load, prefill, W warm-up rounds, K rounds, exit")
    ap.add_argument("--profile-prefill", type=int, default=None, metavar="CLASSES",
                    help="short path for profilers: load, model_prefill of 512 tokens, 3 wide prompt blocks of 256 tokens "
                         "restricted to kernel classes (4 = gate/up matmul, 1023 = everything), exit")
    ap.add_argument("--layers", type=int, default=0, help="cut the model to this many layers (small profiling cases)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    c5 = a.config == "c5"
    if a.depth is None:
        a.depth = 2048 if c5 else 1024
    if a.p is None:
        a.p = 0.7 if c5 else 0.8
    t_shape, h_shape, label = shapes(a.config)
    if a.layers > 0:
        import dataclasses
        t_shape = dataclasses.replace(t_shape, n_layer=a.layers)
        label += f" cut to {a.layers} layers"
    M = a.mtp_n
    workload = (f"{label}, batch 1, MTP K={M - 1} (verify width {M}), KV depth {a.depth}, "
                f"oracle-replayed drafts p={a.p}, greedy")
    if c5:
        workload = (f"{label}, one session per GPU: {a.depth}-token uniform-random prompt (own seed), 1024 generated tokens, "
                    f"MTP K={M - 1} (verify width {M}), oracle-replayed drafts p={a.p}, greedy")
    wdesc = "seeded q4_K super-blocks (uniform scale bytes)" if a.config == "b12k" else "seeded N(0,0.02) q4_0"
    base = {"metric": "MTP decode tok/s (batch 1)", "unit": "tok/s", "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
            "config": {"workload": workload, "weights": wdesc, "l2": "inputs larger than L2 (weights >> 126 MB)",
                       "mtp_n": M, "depth": a.depth, "p": a.p}}

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
        line["note"] = ("reference CPU backend, plain greedy decode (its MTP path runs the same forwards sequentially); "
                        "a step is one token; bounded sample")
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
    if a.sweep:
        sweep(a, lg, synth, torch)
        return
    if RANK == 0:
        ensure_files(a.config, "cuda", a.layers)
    if WORLD > 1:
        dist.barrier()
    tp, hp = ensure_files(a.config, "cuda", a.layers)
    torch.cuda.empty_cache()

    def barrier():
        torch.cuda.synchronize()
        if WORLD > 1:
            dist.barrier()

    V = t_shape.n_vocab
    n_gen = (1024 + 64) if c5 else (a.steps + a.warmup + 4) * M + 8
    r = Runner(lg, synth, torch, tp, hp, t_shape, a.depth, n_gen, M, seed=100 + RANK)
    sess, stream, first, pos0 = r.sess, r.stream, r.first, a.depth

    if a.profile_prefill is not None:
        sess.prefill(synth.prompt_ids(min(512, r.max_seq - 8), V, seed=300), 0)
        n_l = 0
        for _ in range(3):
            n_l = sess.prefill_pass(256, a.profile_prefill)
        torch.cuda.synchronize()
        print(json.dumps({"profile_prefill": a.profile_prefill, "launches_per_block": n_l, "config": base["config"]}), flush=True)
        r.close()
        return

    if a.profile_step:
        sess.set_replay(np.zeros(n_gen + 8, dtype=np.int32))
        sess.rounds_begin(first, pos0, 1)
        sess.rounds_enqueue(M, 2, a.warmup)
        sess.rounds_collect(1, 0)
        e0, e1 = r.ev(), r.ev()
        e0.record(stream)
        sess.rounds_enqueue(M, 2, a.steps)
        e1.record(stream)
        e1.synchronize()
        print(json.dumps({"profile_step": True, "ms_per_round": e0.elapsed_time(e1) / a.steps,
                          "launches_per_round": sess.round_launches(), "config": base["config"]}), flush=True)
        r.close()
        return

    # every replica replays with the same hit pattern (seed 7): tokens per round then agree across ranks and the scaling
    # figure measures the machine, not differing Bernoulli draws
    greedy = r.plain_stream()
    replay = synth.replay_drafts(greedy, V, a.p, seed=7)
    sess.set_replay(replay)

    clk = ClockSampler()
    if c5:
        # the serving workload: rounds until 1024 tokens are out; timed as the sum of the enqueue..drain intervals
        r.restart()
        sess.rounds_begin(first, pos0, 1)
        sess.rounds_enqueue(M, 2, a.warmup)
        sess.rounds_collect(1, 0)
        r.restart()
        sess.rounds_begin(first, pos0, 1)
        barrier()
        clk.start()
        ms, rounds, st = 0.0, 0, {"n_emitted": 1, "n_draft": 0, "n_accept": 0}
        while st["n_emitted"] < 1025:
            k = (1025 - st["n_emitted"] + M - 1) // M
            e0, e1 = r.ev(), r.ev()
            e0.record(stream)
            sess.rounds_enqueue(M, 2, k)
            e1.record(stream)
            e1.synchronize()
            ms += e0.elapsed_time(e1)
            rounds += k
            _, st = sess.rounds_collect(1, 0)
        barrier()
        clocks = clk.stop()
        toks, st = sess.rounds_collect(1, st["n_emitted"])
        emitted = st["n_emitted"] - 1
        got = np.concatenate([[first], toks])[:st["n_emitted"]]
        identical = bool(np.array_equal(got, greedy[:len(got)]))
        accept = st["n_accept"] / max(1, st["n_draft"])
        a.steps = rounds
        base["steps"] = rounds
    else:
        m = r.timed_rounds(M, 2, a.steps, a.warmup, use_head=True, sampler=clk, barrier=barrier)
        ms, emitted, identical, accept, clocks = m["ms"], m["emitted"], m["identical"], m["accept"], m["clocks"]
    launches_per_round = sess.round_launches()

    # plain decode (verify width 1) and the verify step alone (no draft head) at width M, for context
    k_ctx = min(a.steps, 200)
    plain_ms = r.timed_rounds(1, 0, k_ctx, a.warmup, use_head=False)["ms"] / k_ctx
    verify_ms = r.timed_rounds(M, 2, k_ctx, a.warmup, use_head=False)["ms"] / k_ctx

    # the dominant kernel alone: all matrices of one verify step, cold, event-timed -- in the epilogue variants the step
    # runs (classes 0), and as plain store-epilogue kernels (classes 63) for comparison
    def mm_pass(classes):
        n = sess.matmul_pass(M, classes)
        torch.cuda.synchronize()
        m0, m1 = r.ev(), r.ev()
        m0.record(stream)
        for _ in range(10):
            sess.matmul_pass(M, classes)
        m1.record(stream)
        m1.synchronize()
        return n, m0.elapsed_time(m1) / 10
    n_mm, mm_ms = mm_pass(0)
    _, mm_plain_ms = mm_pass(63)
    W = matmul_weight_bytes(t_shape)
    # ... and the ONE kernel with the largest share of the step: the gate/up matmul with its GeGLU epilogue, one launch per
    # layer, replayed back to back (class 4, in the variant the step runs); bytes per launch = the layer's gate + up matrices
    n_gu, gu_ms = mm_pass(1024 + 4)
    gu_bytes = int(2 * t_shape.n_ff * t_shape.n_embd * 0.5625)
    gu_us = gu_ms * 1e3 / max(n_gu, 1)
    gu_gbs = gu_bytes / (gu_us * 1e-6) / 1e9

    peaks = load_peaks()
    prefill_rec = time_prefill(r, synth, torch, t_shape, peaks)

    # end to end through the blocking reference-shaped API
    e2e_rounds = max(20, a.steps // 3)
    r.restart()
    sess.rounds_host(first, pos0, 1, 8 * M, 4, 3, replay)                       # warm the per-call graphs
    r.restart()
    barrier()
    syncs0 = sess.host_syncs()
    t0 = time.perf_counter()
    toks_h, st_h = sess.rounds_host(first, pos0, 1, n_gen, e2e_rounds, 3, replay)
    torch.cuda.synchronize()
    dt_h = time.perf_counter() - t0
    syncs_per_round = (sess.host_syncs() - syncs0) / e2e_rounds
    identical = identical and bool(np.array_equal(toks_h, greedy[1:1 + len(toks_h)]))
    # per round the blocking calls upload the round state once and download its record once (both sizeof(LgRoundState) = 96 B)
    # plus the 4-byte status word; the per-call form (LG_LAZY_ROUND=0) moves (M-1)*12 + (1+M)*4 up and (M-1)*4 + 40 down
    h2d = 96 if syncs_per_round < 1.5 else (M - 1) * 12 + (1 + M) * 4
    d2h = 100 if syncs_per_round < 1.5 else (M - 1) * 4 + 36 + 4

    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s"
    kvb = kv_bytes_step(t_shape, a.depth, M)
    mm_gbs = W / (mm_ms * 1e-3) / 1e9
    step_gbs = (W + kvb) / (verify_ms * 1e-3) / 1e9

    # aggregate over replicas
    my = torch.tensor([float(emitted), float(ms), float(len(toks_h)), float(dt_h), float(identical)], dtype=torch.float64)
    if WORLD > 1:
        allv = [torch.zeros_like(my) for _ in range(WORLD)]
        dist.all_gather(allv, my)
    else:
        allv = [my]
    agg = importlib.import_module("little-gemma_b200.replicas").aggregate([v.tolist() for v in allv])

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
                         "rounds": e2e_rounds, "host_syncs_per_round": syncs_per_round},
                    roofline={"bound": "hbm",
                              "kernel": "lg_gemv_kernel<4, NP, q4, GeGLU>: the gate/up matmul, the step's dominant kernel (23 % of its "
                                        "kernel time), one launch per layer timed back to back",
                              "achieved": gu_gbs, "peak": peak, "unit": "GB/s", "frac": gu_gbs / peak,
                              "traffic": int(gu_bytes * DRAM_TRAFFIC_RATIO), "peak_source": peak_src,
                              "traffic_note": "dram read+write bytes per launch: ncu capture of the E4B-class gate/up launch "
                                              "(37.793 MB moved for 37.749 MB of q4_0) scaled by the launch's weight bytes; writes 0",
                              "algorithmic_bytes": gu_bytes, "launches": n_gu, "us_per_launch": gu_us,
                              "frac_of_8TBs": gu_gbs / 8000.0,
                              # every weight matmul of one verify step replayed alone, in the epilogue variants the step runs
                              "all_matmuls": {"algorithmic_bytes": W, "launches": n_mm, "ms": mm_ms, "achieved": mm_gbs,
                                              "frac": mm_gbs / peak, "plain_store_variants_ms": mm_plain_ms},
                              # the whole verify step (weights + cache rows over its device time): the number the kernels add up to
                              "step_ms": verify_ms, "step_bytes": W + kvb, "step_achieved": step_gbs,
                              "step_frac": step_gbs / peak, "step_frac_of_8TBs": step_gbs / 8000.0},
                    cpu_baseline=cpu, prefill=prefill_rec)
        line["detail"] = dict(launches_per_round=int(launches_per_round),
                              tokens_per_round=emitted / a.steps, acceptance=accept,
                              stream_identical_to_plain_greedy=bool(agg["identical"]),
                              plain_decode_ms=plain_ms, plain_decode_tok_s=1e3 / plain_ms,
                              verify_step_ms=verify_ms,
                              verify_step_gbs=step_gbs,
                              verify_step_frac_measured=step_gbs / peak,
                              verify_step_frac_8TBs=step_gbs / 8000.0,
                              weight_bytes=W, kv_bytes_step=kvb)
        print(json.dumps(line), flush=True)
    r.close()
    if WORLD > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
