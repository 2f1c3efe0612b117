#!/usr/bin/env python3
"""Benchmark of the decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload decode|gemv|attend]

The default workload is the headline configuration: one greedy decode step of the Gemma-4-E4B-shaped random-init Q8
model (35 layers, width 2048, FFN 16384, vocabulary 262144) with the context pre-filled to 2048 positions, the whole
step replayed as a CUDA graph.  A "step" is one token.  With N > 1 (under torchrun) every rank runs an independent
replica on its own GPU (decode is single-request and does not shard; no collective is on the data path) and the
value is the sum over replicas divided by the slowest replica's time.

Prints ONE JSON line.  `value` is tokens/s with everything resident on the device; `e2e` is the same loop driven
through tb_decoder_step with the token crossing the host boundary in both directions every step; `roofline` times
the dominant kernel (the gate/up projection, 16384x2 rows of 2048 int8 weights plus scales) alone over all layers'
matrices; `cpu_baseline` is the CPU oracle on the same model (reported, not a target).  The metric names prefill
tokens/s beside decode tokens/s, so the default line also carries `prefill` (configs[3]: a prompt of 2048 tokens), and
`gemv`, `attend`, `encoder` (configs[0], [1], [4]) as sub-objects with their own rooflines, and `switch` (the model's
return from the host-RAM tier, as the reference's benches/switch.rs times it); `--workload X` runs one of them alone
with more repetitions.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 20251
CONTEXT_FILLED = 2048
CONTEXT = 4096
HBM_SPEC_GBS = 8000.0  # the denominator the benchmark definition fixes
MIN_TIMED_MS = 250.0  # the decode loop is repeated until this much has been timed; the median repetition is reported
GATEUP_TRAFFIC_SHAPE = (32768, 2048)  # the shape that capture was taken on
GATEUP_TRAFFIC = 72_201_216  # bytes per launch of the gate/up kernel under ncu (dram read + write), profiles/gemv_q8_kernel__gate_up_32768x2048.md


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ---------------------------------------------------------------------------------------------------------------------
# distributed plumbing: barrier and max over ranks (replicas only)
# ---------------------------------------------------------------------------------------------------------------------

class Ranks:
    def __init__(self, gpus: int):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group(backend="gloo", rank=self.rank, world_size=self.world)
            self.dist = dist

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def max(self, v: float) -> float:
        if not self.dist:
            return v
        import torch

        t = torch.tensor([v], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t[0])

    def sum(self, v: float) -> float:
        if not self.dist:
            return v
        import torch

        t = torch.tensor([v], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t[0])

    def close(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------------
# clocks during the timed region
# ---------------------------------------------------------------------------------------------------------------------

class Clocks:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu: int):
        self.proc, self.path = None, None
        exe = shutil.which("nvidia-smi")
        if exe:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen([exe, "-i", str(gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)

    def stop(self):
        if not self.proc:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                try:
                    rows.append((float(parts[0]), float(parts[1]), parts[3:7]))
                except ValueError:
                    pass
        os.unlink(self.path)
        if not rows:
            return None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for _, _, flags in rows for n, f in zip(names, flags) if f.lower().startswith("active")})
        return {"sm_mhz": statistics.median(r[0] for r in rows), "sm_max_mhz": rows[0][1], "reasons": reasons, "samples": len(rows)}


# ---------------------------------------------------------------------------------------------------------------------
# CPU oracle legs
# ---------------------------------------------------------------------------------------------------------------------

def cpu_decode(cfg, steps_wanted: int, budget_s: float, gpu_tokens=None, weight_bits: int = 8):
    """The CPU oracle's decode step on the same seeded model and pre-filled cache; returns tokens/s and what ran."""
    import oracle
    from oracle.model import OracleModel

    cores = oracle.lib().tbo_threads()
    t0 = time.time()
    model = OracleModel(cfg, SEED, context=CONTEXT, chunk=0, weight_bits=weight_bits)
    model.fill_cache(SEED + 1)
    build_s = time.time() - t0
    token, times, tokens, gaps = 1, [], [], []
    for i in range(steps_wanted):
        t = time.time()
        token, logits, _ = model.step(token, CONTEXT_FILLED + i, want_logits=True)
        times.append(time.time() - t)
        tokens.append(int(token))
        top = np.sort(logits)[-2:]
        gaps.append(float((top[1] - top[0]) / np.abs(logits).max()))  # top-2 gap relative to the largest logit
        if gpu_tokens is not None and i < len(gpu_tokens) and int(gpu_tokens[i]) != token:
            token = int(gpu_tokens[i])  # keep both on the same sequence after a near-tie
        if sum(times) > budget_s:
            break
    per = statistics.median(times)
    agree = None
    if gpu_tokens is not None:
        # the picks must agree wherever the CPU's top-2 gap clears the tolerance of the logits (2e-3 of the largest)
        agree = all(int(g) == t or gap < 4e-3 for g, t, gap in zip(gpu_tokens, tokens, gaps))
    return {"value": 1.0 / per, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{len(times)} full decode steps (35 layers + LM head, context {CONTEXT_FILLED}) of the same seeded model; median step {per * 1e3:.1f} ms; "
                      f"model generation {build_s:.1f} s not timed",
            "tokens": tokens, "top2_gap_rel": gaps, "tokens_match_gpu": agree}, tokens


# ---------------------------------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------------------------------

def bench_decode(args, ranks: Ranks):
    import tachyon_b200 as tb

    ctx = tb.Context(ranks.local)
    cfg = tb.gemma4_e4b_shape(layers=args.layers)
    bits = 4 if args.weights == "q4" else 8
    dec = tb.Decoder(ctx, cfg, context=CONTEXT, chunk=0, keep_logits=False, fused=args.fused, weight_bits=bits)
    dec.fill_random(SEED)
    dec.build()
    K, W = args.steps, args.warmup
    launches_per_step = dec.step_launches

    def fresh():
        dec.fill_cache(SEED + 1, CONTEXT_FILLED)

    # ---- device-resident: K chained graph replays, repeated until at least a quarter of a second has been timed ----
    fresh()
    weight_bytes, cache_bytes = dec.step_bytes()
    dec.run(1, W, want_tokens=False)
    ctx.sync()
    room = CONTEXT - CONTEXT_FILLED - W  # positions left before the context is full
    e0, e1 = ctx.event(), ctx.event()
    e0.record()
    dec.run(1, min(K, room), want_tokens=False)
    e1.record()
    e1.sync()
    est_ms = max(e0.elapsed_ms(e1), 1e-3) * K / min(K, room)
    repeats = max(1, min(64, int(np.ceil(MIN_TIMED_MS / est_ms))))
    fresh()
    dec.run(1, W, want_tokens=False)
    ctx.sync()
    ranks.barrier()
    clocks = Clocks(ranks.local) if ranks.rank == 0 else None
    runs, used = [], W
    for _ in range(repeats):
        if used + K > CONTEXT - CONTEXT_FILLED:  # start again from the pre-filled context (not timed)
            fresh()
            dec.run(1, W, want_tokens=False)
            ctx.sync()
            used = W
        e0.record()
        dec.run(1, K, want_tokens=False)  # continues from the state before; weights (4.7 GB) exceed L2 by 37x
        e1.record()
        e1.sync()
        runs.append(e0.elapsed_ms(e1))
        used += K
    ms = statistics.median(runs)
    ranks.barrier()
    ms_max = ranks.max(ms)
    if ctx.status() != 0:
        raise RuntimeError("a kernel reported a bounded wait that ran out")

    # ---- end to end: the token crosses the host boundary both ways every step ----
    fresh()
    token = 1
    for _ in range(W):
        token = dec.step(token)
    ranks.barrier()
    e2e_runs, used = [], W
    for _ in range(repeats):
        if used + K > CONTEXT - CONTEXT_FILLED:
            fresh()
            token = 1
            for _ in range(W):
                token = dec.step(token)
            used = W
        t0 = time.perf_counter()
        e0.record()
        for _ in range(K):
            token = dec.step(token)
        e1.record()
        e1.sync()
        e2e_runs.append(max(e0.elapsed_ms(e1), (time.perf_counter() - t0) * 1e3))
        used += K
    e2e_ms = statistics.median(e2e_runs)
    e2e_ms_max = ranks.max(e2e_ms)
    clk = clocks.stop() if clocks else None

    # ---- greedy tokens for the parity note: first steps after the pre-fill ----
    fresh()
    gpu_tokens = [int(t) for t in dec.run(1, 4)]

    # ---- the dominant kernel alone: gate/up projection over every layer's matrix in turn (2.5 GB > L2) ----
    roof = kernel_roofline(ctx, cfg, W, K) if ranks.rank == 0 else None
    dec.close()
    ctx.trim()  # the decoder's memory back to the system, not only to this context's pool

    n = ranks.world
    value = n * K / (ms_max / 1e3)
    step_bytes = weight_bytes + cache_bytes
    peak, how = measured_peak_gbs()
    line = {
        "metric": "decode_tokens_per_second", "value": value, "unit": "tok/s", "n_gpus": n, "steps": K, "warmup": W,
        "ms_per_step": ms_max / K, "repeats": repeats, "timed_ms": sum(runs), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": ("int4 (the reference's Q4)" if bits == 4 else "int8") + " weights x f32 activations, f32 accumulate",
        "data": "synthetic", "impl": "ours",
        "config": {"workload": ("configs[2]" if cfg.layers == 35 else f"a {cfg.layers}-layer cut (for profiling) of configs[2]") + ": full decode step, Gemma-4-E4B-shape " + ("Q4 (the reference's converted format; not the configuration the metric is quoted on)" if bits == 4 else "Q8")
                   + ", batch 1, context pre-filled to 2048, greedy",
                   "step": "CUDA graph replay; " + ("one persistent kernel per step" if args.fused else "one launch per phase, programmatic dependent launch"),
                   "layers": cfg.layers, "hidden": cfg.hidden, "ffn": cfg.ffn, "vocab": cfg.vocab, "parallelism": f"{n} independent replicas",
                   "l2": f"inputs exceed L2: {weight_bytes / 1e9:.2f} GB of weights streamed per step",
                   "timing": f"{repeats} repetitions of {K} chained steps, CUDA events on the library's stream; the median repetition is reported"},
        "e2e": {"value": n * K / (e2e_ms_max / 1e3), "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4,
                "api": "tb_decoder_step: host token in, graph replay, sampled token read from pinned memory"},
        "gpu_launches": K * launches_per_step * repeats,
        "step_bytes": {"weights": weight_bytes, "kv_cache": cache_bytes},
        "step_hbm": {"achieved_gbs": step_bytes / (ms_max / K / 1e3) / 1e9, "frac_of_8tbs": step_bytes / (ms_max / K / 1e3) / 1e9 / HBM_SPEC_GBS,
                     "frac_of_measured_copy": step_bytes / (ms_max / K / 1e3) / 1e9 / peak, "peak_source": how},
        "roofline": roof, "clocks": clk, "first_tokens": gpu_tokens,
    }
    return line, cfg, gpu_tokens


def kernel_roofline(ctx, cfg, warmup: int, steps: int, matrices: int = 0):
    """Times the gate/up projection kernel (norm prologue, GeGLU epilogue) back to back over `layers` distinct matrices."""
    import tachyon_b200 as tb

    rows, cols, layers = 2 * cfg.ffn, cfg.hidden, matrices or cfg.layers
    lib = ctx.lib
    w = ctx.alloc(layers * rows * cols)
    s = ctx.alloc(layers * rows * (cols // 32) * 2)
    tb.check(lib.tb_fill_codes(ctx.handle, 3, 1, w.ptr, layers * rows * cols))
    tb.check(lib.tb_fill_scales(ctx.handle, 3, 2, s.ptr, layers * rows * (cols // 32), 0.02 / 127))
    h, y, w1, w2 = (ctx.upload(np.random.default_rng(i).uniform(0.5, 1.5, cols).astype(np.float32)) for i in range(4))
    hout, out = ctx.zeros(cols * 4), ctx.zeros(rows * 2)
    import ctypes as C

    def launch(i):
        wi = C.c_void_p(w.ptr + (i % layers) * rows * cols)
        si = C.c_void_p(s.ptr + (i % layers) * rows * (cols // 32) * 2)
        tb.check(lib.tb_gemv_q8_norm(ctx.handle, wi, si, h.ptr, y.ptr, w1.ptr, w2.ptr, 1e-6, 1.0, hout.ptr, out.ptr, rows, cols, 1))

    n = steps if matrices else max(steps, 64)
    for i in range(max(warmup, 3) * (1 if matrices else 4)):
        launch(i)
    ctx.sync()
    e0, e1 = ctx.event(), ctx.event()
    e0.record()
    for i in range(n):
        launch(i)
    e1.record()
    e1.sync()
    us = e0.elapsed_ms(e1) * 1e3 / n
    alg = rows * cols + rows * (cols // 32) * 2 + 4 * cols * 4 + rows // 2 * 4  # weights, scales, h/y/w1/w2, output
    peak, how = measured_peak_gbs()
    achieved = alg / (us * 1e-6) / 1e9
    for b in (w, s):
        b.free()
    return {"kernel": "gemv_q8_kernel<1, X_NORM, EPI_GEGLU> (gate/up projection)", "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "frac_of_8tbs": achieved / HBM_SPEC_GBS, "peak_source": how,
            "traffic": GATEUP_TRAFFIC if (rows, cols) == GATEUP_TRAFFIC_SHAPE else None,
            "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of this kernel and shape under ncu (profiles/gemv_q8_kernel__gate_up_32768x2048.md)",
            "bytes_per_launch": alg, "us_per_launch": us, "launches_timed": n,
            "how": f"back-to-back launches cycling over {layers} distinct matrices ({layers * rows * cols / 1e9:.1f} GB), CUDA events on the launching stream"}


def bench_gateup(args, ranks: Ranks):
    """The dominant kernel alone on few matrices (default 4 x 71 MB, larger than L2): the case small enough to capture."""
    import tachyon_b200 as tb

    ctx = tb.Context(ranks.local)
    roof = kernel_roofline(ctx, tb.gemma4_e4b_shape(), args.warmup, args.steps, matrices=min(args.copies, 35))
    return {"metric": "gate_up_gemv_gbs", "value": roof["achieved"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": roof["us_per_launch"] / 1e3, "higher_is_better": True, "dtype": "int8 weights x f32 activations, f32 accumulate", "data": "synthetic",
            "impl": "ours", "config": {"workload": "gate/up projection of configs[2] alone: norm prologue, 32768 x 2048 Q8, GeGLU epilogue"},
            "gpu_launches": args.steps, "roofline": roof}


def bench_gemv(args, ranks: Ranks):
    """configs[0]: the single Q8 GEMV, x f16 [2048], W [16384, 2048], y f16; cycles over 64 weight copies (2.3 GB)."""
    import ctypes as C

    import tachyon_b200 as tb

    ctx = tb.Context(ranks.local)
    rows, cols, copies = args.rows, args.cols, args.copies
    lib = ctx.lib
    f16w = args.weights == "f16"
    if f16w:
        copies = min(copies, 32)  # 67 MB a copy
        w = ctx.alloc(copies * rows * cols * 2)
        tb.check(lib.tb_fill_gauss_f16(ctx.handle, 3, 1, w.ptr, copies * rows * cols, 0.02))
    else:
        w, s = ctx.alloc(copies * rows * cols), ctx.alloc(copies * rows * (cols // 32) * 2)
        tb.check(lib.tb_fill_codes(ctx.handle, 3, 1, w.ptr, copies * rows * cols))
        tb.check(lib.tb_fill_scales(ctx.handle, 3, 2, s.ptr, copies * rows * (cols // 32), 0.02 / 127))
    x = ctx.upload(np.random.default_rng(0).standard_normal(cols).astype(np.float16))
    y = ctx.zeros(rows * 2)

    def launch(i):
        if f16w:
            tb.check(lib.tb_gemv_f16(ctx.handle, C.c_void_p(w.ptr + (i % copies) * rows * cols * 2), x.ptr, tb.F16, y.ptr, tb.F16, rows, cols))
        else:
            tb.check(lib.tb_gemv_q8(ctx.handle, C.c_void_p(w.ptr + (i % copies) * rows * cols), C.c_void_p(s.ptr + (i % copies) * rows * (cols // 32) * 2), x.ptr,
                                    tb.F16, y.ptr, tb.F16, rows, cols))

    for i in range(args.warmup):
        launch(i)
    ctx.sync()
    e0, e1 = ctx.event(), ctx.event()
    e0.record()
    for i in range(args.steps):
        launch(i)
    e1.record()
    e1.sync()
    us = e0.elapsed_ms(e1) * 1e3 / args.steps
    alg = (rows * cols * 2 if f16w else rows * cols + rows * (cols // 32) * 2) + cols * 2 + rows * 2
    peak, how = measured_peak_gbs()
    return {"metric": "gemv_f16_gbs" if f16w else "gemv_q8_gbs", "value": alg / us / 1e3, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": us / 1e3, "higher_is_better": True, "dtype": ("f16" if f16w else "int8") + " x f16 -> f16, f32 accumulate", "data": "synthetic", "impl": "ours",
            "config": {"workload": f"configs[0]: {'f16' if f16w else 'Q8'} GEMV {rows}x{cols}, {copies} weight copies cycled"}, "gpu_launches": args.steps,
            "roofline": {"bound": "hbm", "achieved": alg / us / 1e3, "peak": peak, "unit": "GB/s", "frac": alg / us / 1e3 / peak, "frac_of_8tbs": alg / us / 1e3 / HBM_SPEC_GBS,
                         "peak_source": how, "traffic": None, "bytes_per_launch": alg, "us_per_launch": us}}


def bench_gemv_q4(args, ranks: Ranks):
    """The reference's own GEMV on its own formats (benches/gemv.rs): Q4 W [16384, 2048] x Q8 x -> f32; 64 weight copies."""
    import ctypes as C

    import tachyon_b200 as tb

    ctx = tb.Context(ranks.local)
    rows, cols, copies = args.rows, args.cols, args.copies
    lib = ctx.lib
    wb, sb = rows * cols // 2, rows * (cols // 64) * 2
    w, s = ctx.alloc(copies * wb), ctx.alloc(copies * sb)
    tb.check(lib.tb_fill_codes(ctx.handle, 3, 1, w.ptr, copies * wb))  # any byte is two valid nibbles
    tb.check(lib.tb_fill_scales(ctx.handle, 3, 2, s.ptr, copies * sb // 2, 0.02 / 8))
    x = ctx.upload(np.random.default_rng(0).standard_normal(cols).astype(np.float32))
    q, pairs, y = ctx.zeros(cols), ctx.zeros(cols // 32 * 8), ctx.zeros(rows * 4)
    ctx.quant_q8(x, cols, q, pairs)

    def launch(i):
        tb.check(lib.tb_gemv_q4(ctx.handle, C.c_void_p(w.ptr + (i % copies) * wb), C.c_void_p(s.ptr + (i % copies) * sb), q.ptr, pairs.ptr, y.ptr, rows, cols))

    for i in range(args.warmup):
        launch(i)
    ctx.sync()
    e0, e1 = ctx.event(), ctx.event()
    e0.record()
    for i in range(args.steps):
        launch(i)
    e1.record()
    e1.sync()
    us = e0.elapsed_ms(e1) * 1e3 / args.steps
    alg = wb + sb + cols + cols // 32 * 8 + rows * 4
    peak, how = measured_peak_gbs()
    return {"metric": "gemv_q4_gbs", "value": alg / us / 1e3, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": us / 1e3,
            "higher_is_better": True, "dtype": "int4 x int8 -> f32 (dp4a, f32 scale steps)", "data": "synthetic", "impl": "ours",
            "config": {"workload": f"the reference's gemv_q4 {rows}x{cols} (Q4 weights, Q8 activations), {copies} weight copies cycled"}, "gpu_launches": args.steps,
            "roofline": {"bound": "hbm", "achieved": alg / us / 1e3, "peak": peak, "unit": "GB/s", "frac": alg / us / 1e3 / peak, "frac_of_8tbs": alg / us / 1e3 / HBM_SPEC_GBS,
                         "peak_source": how, "traffic": None, "bytes_per_launch": alg, "us_per_launch": us}}


def bench_attend(args, ranks: Ranks):
    """configs[1]: decode attention, 8 query / 2 kv heads of 256 over an f16 cache of 4096; global and sliding-512."""
    import tachyon_b200 as tb

    ctx = tb.Context(ranks.local)
    heads, kv, d, cap, copies = 8, 2, 256, 4096, args.copies
    lib = ctx.lib
    kc, vc = ctx.alloc(copies * kv * cap * d * 2), ctx.alloc(copies * kv * cap * d * 2)
    tb.check(lib.tb_fill_gauss_f16(ctx.handle, 1, 1, kc.ptr, copies * kv * cap * d, 1.0))
    tb.check(lib.tb_fill_gauss_f16(ctx.handle, 1, 2, vc.ptr, copies * kv * cap * d, 1.0))
    qkv = ctx.upload(np.random.default_rng(0).standard_normal((heads + 2 * kv) * d).astype(np.float32))
    pos = ctx.upload(np.array([cap - 1], np.uint32))
    out, count = ctx.zeros(heads * d * 2), ctx.zeros(16)
    results = {}
    for name, window, splits in (("global_4096", 4096, 64), ("sliding_512", 512, 16)):
        part = ctx.zeros(ctx.attend_scratch_bytes(heads, kv, splits))
        args_list = [tb.Attend(qkv=qkv.ptr, k_cache=kc.ptr + i * kv * cap * d * 2, v_cache=vc.ptr + i * kv * cap * d * 2, pos=pos.ptr, cap=cap, window=window,
                               fresh=0, heads=heads, kv_heads=kv, scale=1 / 16.0, eps=1e-6, partial=part.ptr, count=count.ptr, splits=splits, out=out.ptr,
                               out_dtype=tb.F16) for i in range(copies)]
        for i in range(args.warmup):
            ctx.attend_decode(args_list[i % copies])
        ctx.sync()
        e0, e1 = ctx.event(), ctx.event()
        e0.record()
        for i in range(args.steps):
            ctx.attend_decode(args_list[i % copies])
        e1.record()
        e1.sync()
        us = e0.elapsed_ms(e1) * 1e3 / args.steps
        alg = 2 * kv * window * d * 2 + heads * d * 4 + heads * d * 2
        results[name] = {"us_per_launch": us, "bytes_per_launch": alg, "achieved_gbs": alg / us / 1e3}
    peak, how = measured_peak_gbs()
    g = results["global_4096"]
    return {"metric": "attend_decode_us", "value": g["us_per_launch"], "unit": "us", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": g["us_per_launch"] / 1e3, "higher_is_better": False, "dtype": "f16 cache; f32 queries and probabilities as two f16 parts on mma.sync, f32 accumulate", "data": "synthetic", "impl": "ours",
            "config": {"workload": f"configs[1]: decode attention 8q/2kv x 256 over 4096 positions, {copies} cache copies cycled", "variants": results},
            "gpu_launches": 2 * args.steps,
            "roofline": {"bound": "hbm", "achieved": g["achieved_gbs"], "peak": peak, "unit": "GB/s", "frac": g["achieved_gbs"] / peak, "peak_source": how, "traffic": None}}


def measured_peak_tflops():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            j = json.load(f)
        return float(j["bf16_tflops"]), float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), "measured"
    except Exception:
        return 1590.0, 1400.0, "fallback"


def bench_gemm(args, ranks: Ranks):
    """configs[3]'s GEMM shapes alone: M tokens x K -> N on the tensor cores (tcgen05).  --weights q8: the codes are converted in
    the operand path (tb_gemm_q8); --weights f16: the product reads the codes' f16 copy by TMA (tb_dequant_f16 once, then
    tb_gemm_f16: what the decoder's prefill and the encoder run).  --mode is the output mode (0 f32, 1 f16, 2 gated GELU ...)."""
    import tachyon_b200 as tb

    ctx = tb.Context(ranks.local)
    m, n, k, mode = args.tokens, args.rows, args.cols, args.mode
    lib = ctx.lib
    w, s = ctx.alloc(n * k), ctx.alloc(n * (k // 32) * 2)
    tb.check(lib.tb_fill_codes(ctx.handle, 3, 1, w.ptr, n * k))
    tb.check(lib.tb_fill_scales(ctx.handle, 3, 2, s.ptr, n * (k // 32), 0.02 / 127))
    a = ctx.upload(np.random.default_rng(0).standard_normal((m, k)).astype(np.float16))
    out = ctx.zeros(m * n * 4)
    if args.weights == "f16":
        copy = ctx.alloc(n * k * 2)
        ctx.dequant_f16(w, s, n, k, 8, copy)
        run = lambda: ctx.gemm_f16(copy, a, m, n, k, out, mode)
    else:
        run = lambda: ctx.gemm_q8(w, s, a, m, n, k, out, mode)
    for _ in range(args.warmup):
        run()
    ctx.sync()
    e0, e1 = ctx.event(), ctx.event()
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    e1.sync()
    us = e0.elapsed_ms(e1) * 1e3 / args.steps
    tf = 2.0 * m * n * k / (us * 1e-6) / 1e12
    burst, sustained, how = measured_peak_tflops()
    kind = "f16 copy of the int8 weights read by TMA" if args.weights == "f16" else "int8 weights -> f16 in the operand path"
    return {"metric": "gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": us / 1e3,
            "higher_is_better": True, "dtype": kind + ", f16 activations, f32 accumulate (tcgen05)", "data": "synthetic", "impl": "ours",
            "config": {"workload": f"configs[3] GEMM: M={m} K={k} N={n}, output mode {mode}, weights {args.weights}"}, "gpu_launches": args.steps,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": burst, "unit": "TFLOP/s", "frac": tf / burst, "peak_source": how, "traffic": None,
                         "flops_per_launch": 2.0 * m * n * k, "us_per_launch": us}}


def bench_switch(args, ranks: Ranks):
    """A model's return from the host-RAM tier (the reference's benches/switch.rs, host_tier: E4B parked, then resumed): seconds
    and GB/s of its weights for tb_parked_resume (device memory taken, one copy over the link, buffers laid out, the step's
    graphs recorded, the prefill copy written), beside a plain copy of 1 GiB of pinned memory into device memory in use."""
    import tachyon_b200 as tb

    ctx = tb.Context(ranks.local)
    cfg = tb.gemma4_e4b_shape(layers=args.layers)
    dec = tb.Decoder(ctx, cfg, context=CONTEXT, chunk=512, keep_logits=False)
    dec.fill_random(SEED)
    dec.build()
    tok = dec.step(7)
    weights = dec.parked_bytes()
    t0 = time.perf_counter()
    parked = dec.park()
    first_park = time.perf_counter() - t0
    back, parks = [], []
    for _ in range(max(args.steps, 1) if args.steps <= 16 else 5):
        t0 = time.perf_counter()
        dec = parked.resume()
        back.append(time.perf_counter() - t0)
        assert dec.step(7) == tok, "the resumed model answers as before"
        t0 = time.perf_counter()
        parked = dec.park()
        parks.append(time.perf_counter() - t0)
    parked.close()
    ctx.trim()
    # the link alone: 1 GiB of pinned memory into device memory that is already in use
    n = 1 << 30
    hb, db = ctx.alloc_host(n), ctx.alloc(n)
    hb.array[:] = 1
    copies = []
    for _ in range(4):
        t0 = time.perf_counter()
        tb.check(ctx.lib.tb_upload(ctx.handle, db.ptr, hb.host, n))
        ctx.sync()
        copies.append(time.perf_counter() - t0)
    link = n / min(copies[1:]) / 1e9
    sec = statistics.median(back)
    return {"metric": "resume_from_host_tier_gb_per_second", "value": weights / sec / 1e9, "unit": "GB/s", "n_gpus": 1, "steps": len(back), "warmup": 0,
            "ms_per_step": sec * 1e3, "higher_is_better": True, "dtype": "u8", "data": "synthetic", "impl": "ours",
            "config": {"workload": f"the benchmark's decoder ({args.layers} layers, {weights} B of weights) parked in pinned host memory and resumed (tb_decoder_park / tb_parked_resume)"},
            "gpu_launches": None, "first_park_s": first_park, "park_with_kept_copy_s": statistics.median(parks), "resume_s": sec,
            "link_gb_per_second": link, "fraction_of_link": weights / sec / 1e9 / link}


def bench_load(args, ranks: Ranks):
    """The disk tier's way into VRAM (the reference's benches/load.rs: a .wpk streamed into device memory): the benchmark's decoder
    written as a converted model's weights.wpk (random codes, the file then in the page cache), and tb_decoder_load_wpk timed with
    the reader threads and with the reads on the calling thread, unchecked and with every tensor's CRC32C checked."""
    import shutil
    import tempfile

    import tachyon_b200 as tb

    ctx = tb.Context(ranks.local)
    cfg = tb.gemma4_e4b_shape(layers=args.layers)
    h, q = cfg.hidden, (cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim
    rng = np.random.default_rng(SEED)
    block = rng.integers(-127, 128, 1 << 26, dtype=np.int8)
    scales = np.full(1 << 24, 0.02 / 127.0, np.float16)
    d = tempfile.mkdtemp(prefix="tachyon_b200_load_", dir=os.environ.get("TACHYON_B200_BENCH_DIR"))
    path = os.path.join(d, "weights.wpk")
    try:
        with tb.WpkWriter(path) as w:
            def mat(name, rows, cols):
                n = rows * cols
                codes = block[:n] if n <= block.size else np.tile(block, -(-n // block.size))[:n]
                w.add(name + ".w", "i8", [rows, cols], codes)
                w.add(name + ".s", "f16", [rows, cols // 32], scales[: rows * cols // 32])

            mat("embed", cfg.vocab, h)
            w.add("norm", "f32", [h], np.ones(h, np.float32))
            for l in range(cfg.layers):
                mat(f"{l}.qkv", q, h), mat(f"{l}.o", h, cfg.heads * cfg.head_dim), mat(f"{l}.gate_up", 2 * cfg.ffn, h), mat(f"{l}.down", h, cfg.ffn)
                for name, n in (("q_norm", cfg.head_dim), ("k_norm", cfg.head_dim), ("input_layernorm", h), ("post_attention_layernorm", h),
                                ("pre_feedforward_layernorm", h), ("post_feedforward_layernorm", h), ("layer_scalar", 1)):
                    w.add(f"{l}.{name}", "f32", [n], np.ones(n, np.float32))
        size = os.path.getsize(path)
        times = {}
        tok = None
        for readers, verify in ((8, False), (0, False), (8, True), (0, True), (4, False), (16, False), (8, False)):
            os.environ["TACHYON_B200_LOAD_READERS"] = str(readers)
            dec = tb.Decoder(ctx, cfg, context=CONTEXT, chunk=512, keep_logits=False, prefill_copy=1)
            ctx.sync()
            t0 = time.perf_counter()
            dec.load_wpk(path, verify=verify)
            ctx.sync()
            times.setdefault((readers, verify), []).append(time.perf_counter() - t0)
            dec.build()
            got = dec.step(7)
            assert tok is None or got == tok, "every way of loading gives the same model"
            tok = got
            dec.close()
        os.environ.pop("TACHYON_B200_LOAD_READERS", None)
        ctx.trim()
    finally:
        shutil.rmtree(d, ignore_errors=True)
    sec = min(times[(8, False)])
    return {"metric": "load_from_disk_tier_gb_per_second", "value": size / sec / 1e9, "unit": "GB/s", "n_gpus": 1, "steps": len(times[(8, False)]), "warmup": 0,
            "ms_per_step": sec * 1e3, "higher_is_better": True, "dtype": "u8", "data": "synthetic", "impl": "ours",
            "config": {"workload": f"the benchmark's decoder ({args.layers} layers) as a weights.wpk of {size} B in the page cache, read into VRAM by tb_decoder_load_wpk (eight reader threads, pieces of 16 MiB, twelve pinned slots)"},
            "gpu_launches": None, "streamed_s": sec, "on_the_calling_thread_s": min(times[(0, False)]), "streamed_checked_s": min(times[(8, True)]),
            "on_the_calling_thread_checked_s": min(times[(0, True)]), "four_readers_s": min(times[(4, False)]), "sixteen_readers_s": min(times[(16, False)])}


def bench_token(args, ranks: Ranks):
    """The tokenizer on the host (the reference's benches/token.rs): the fixture's strings (a thousand texts of the reference's
    multilingual set, 200 KB) through tb_tokenizer_encode with the small Gemma-shaped vocabulary, and the ids back through the
    detokenizer; one thread."""
    import ctypes as C

    import tachyon_b200 as tb

    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tests", "golden", "token")
    tok = tb.Tokenizer.from_json(open(os.path.join(golden, "toy.json"), "rb").read())
    texts = [json.loads(line).encode("utf-8") for line in open(os.path.join(golden, "strings.jsonl"), encoding="utf-8")]
    ids = np.empty(max(len(t) for t in texts) + 16, np.uint32)
    n = C.c_size_t(0)
    rounds, tokens, nbytes = max(args.steps, 3), 0, sum(len(t) for t in texts)
    best = float("inf")
    for _ in range(rounds):
        tokens = 0
        t0 = time.perf_counter()
        for t in texts:
            tb.check(tok.lib.tb_tokenizer_encode(tok.handle, t, len(t), ids.ctypes.data, ids.size, C.byref(n)))
            tokens += n.value
        best = min(best, time.perf_counter() - t0)
    tok.close()
    return {"metric": "tokenizer_encode_mb_per_second", "value": nbytes / best / 1e6, "unit": "MB/s", "n_gpus": 0, "steps": rounds, "warmup": 0, "ms_per_step": best * 1e3,
            "higher_is_better": True, "dtype": "u8", "data": "fixture", "impl": "ours", "config": {"workload": f"{len(texts)} fixture strings, {nbytes} B, {tokens} tokens, one host thread"},
            "gpu_launches": 0, "tokens_per_second": tokens / best}


def bench_flash(args, ranks: Ranks):
    """configs[3]'s attention alone: 2048 tokens x 8 query / 2 kv heads of 256 over the cache ring, sliding 512 and global."""
    import tachyon_b200 as tb

    ctx = tb.Context(ranks.local)
    heads, kv, d, T, cap = 8, 2, 256, args.tokens, 4096
    lib = ctx.lib
    kc, vc, q = ctx.alloc(kv * cap * d * 2), ctx.alloc(kv * cap * d * 2), ctx.alloc(T * heads * d * 2)
    tb.check(lib.tb_fill_gauss_f16(ctx.handle, 1, 1, kc.ptr, kv * cap * d, 1.0))
    tb.check(lib.tb_fill_gauss_f16(ctx.handle, 1, 2, vc.ptr, kv * cap * d, 1.0))
    tb.check(lib.tb_fill_gauss_f16(ctx.handle, 1, 3, q.ptr, T * heads * d, 0.09))  # scale * log2(e) folded in: scores ~N(0, 1.4)
    out = ctx.zeros(T * heads * d * 2)
    results = {}
    for name, window in (("sliding_512", 512), ("global", cap)):
        for _ in range(args.warmup):
            ctx.prefill_attend(q, kc, vc, out, T, 0, cap, window, heads, kv, d)
        ctx.sync()
        e0, e1 = ctx.event(), ctx.event()
        e0.record()
        for _ in range(args.steps):
            ctx.prefill_attend(q, kc, vc, out, T, 0, cap, window, heads, kv, d)
        e1.record()
        e1.sync()
        us = e0.elapsed_ms(e1) * 1e3 / args.steps
        keys = sum(min(t + 1, window) for t in range(T))  # keys each token's heads see
        flops = 4.0 * keys * heads * d
        results[name] = {"us_per_launch": us, "flops_per_launch": flops, "achieved_tflops": flops / us / 1e6}
    burst, sustained, how = measured_peak_tflops()
    g = results["sliding_512"]
    return {"metric": "prefill_attention_us", "value": g["us_per_launch"], "unit": "us", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": g["us_per_launch"] / 1e3, "higher_is_better": False, "dtype": "f16 mma.sync, f32 softmax and sums", "data": "synthetic", "impl": "ours",
            "config": {"workload": f"configs[3] prefill attention: {T} tokens, 8 query / 2 kv heads of 256, sliding window 512 (and global)"},
            "gpu_launches": args.steps, "cases": results,
            "roofline": {"bound": "tensor", "achieved": g["achieved_tflops"], "peak": burst, "unit": "TFLOP/s", "frac": g["achieved_tflops"] / burst,
                         "peak_source": how, "traffic": None, "flops_per_launch": g["flops_per_launch"], "us_per_launch": g["us_per_launch"]}}


def bench_prefill(args, ranks: Ranks):
    """configs[3]: one prompt of 2048 token ids through the 35-layer model; the last token goes through the decode step."""
    import tachyon_b200 as tb

    ctx = tb.Context(ranks.local)
    cfg = tb.gemma4_e4b_shape()
    T = args.tokens
    dec = tb.Decoder(ctx, cfg, context=CONTEXT, chunk=args.chunk, keep_logits=False, weight_bits=4 if args.weights == "q4" else 8)
    dec.fill_random(SEED)
    dec.build()
    prompt = np.array([(i * 7919 + 13) % cfg.vocab for i in range(T)], np.uint32)  # the reference's prompt (benches/generate.rs:47)
    times, dev_times, first = [], [], None
    e0, e1 = ctx.event(), ctx.event()
    for it in range(args.warmup + args.steps):
        dec.reset()
        ctx.sync()
        ranks.barrier()
        t0 = time.perf_counter()
        e0.record()
        dec.prefill(prompt[:-1])
        tok = dec.step(int(prompt[-1]))
        e1.record()
        e1.sync()
        dt = time.perf_counter() - t0
        first = tok if first is None else first
        assert tok == first, "prefill is deterministic"
        if it >= args.warmup:
            times.append(dt)
            dev_times.append(e0.elapsed_ms(e1))
    ms = statistics.median(times) * 1e3
    ms_max = ranks.max(ms)
    dev_ms_max = ranks.max(statistics.median(dev_times))
    # arithmetic of the prompt (the last layer stops after its cache writes; its query/key/value product still runs)
    per_layer = (cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim * cfg.hidden + cfg.hidden * cfg.heads * cfg.head_dim + 3 * cfg.ffn * cfg.hidden
    flops = 2.0 * (T - 1) * (per_layer * (cfg.layers - 1) + (cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim * cfg.hidden)
    burst, sustained, how = measured_peak_tflops()
    tf = flops / (ms_max * 1e-3) / 1e12
    dec.close()
    ctx.trim()  # the decoder's memory back to the system, not only to this context's pool
    n = ranks.world
    return {"metric": "prefill_tokens_per_second", "value": n * T / (ms_max / 1e3), "unit": "tok/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": ("int4" if args.weights == "q4" else "int8") + " weights as their f16 values (a copy made once, read by TMA), f16 activations, f32 accumulate (tcgen05); f16/f32 flash attention", "data": "synthetic", "impl": "ours",
            "config": {"workload": f"configs[3]: prefill of {T} token ids, Gemma-4-E4B-shape {args.weights.upper()}, chunks of {args.chunk}, last token through the decode step; tb_settings.prefill_copy automatic (TACHYON_B200_PREFILL_COPY=0: codes converted in the loop)",
                       "timing": "host wall clock around tb_decoder_prefill + tb_decoder_step (token ids cross from host memory)"},
            "gpu_launches": None, "first_token": int(first), "device_ms": dev_ms_max,
            "e2e": {"value": n * T / (ms_max / 1e3), "unit": "tok/s", "h2d_bytes_per_step": T * 4, "d2h_bytes_per_step": 4,
                    "api": "tb_decoder_prefill + tb_decoder_step: host token ids in, first generated token out"},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": sustained, "unit": "TFLOP/s", "frac": tf / sustained, "peak_source": how + " (sustained)",
                         "frac_of_burst": tf / burst, "traffic": None, "gemm_flops": flops}}


def encoder_batch(cfg_vocab: int, sequences: int = 64, seed: int = 5):
    rng = np.random.default_rng(seed)
    lens = rng.integers(16, 513, sequences)
    return [rng.integers(0, cfg_vocab, int(n)).astype(np.uint32) for n in lens]


def bench_encoder(args, ranks: Ranks):
    """configs[4]: 64 sequences of 16..512 tokens, packed without padding, through the Granite-311m-shaped encoder."""
    import tachyon_b200 as tb

    ctx = tb.Context(ranks.local)
    cfg = tb.granite_311m_shape()
    seqs = encoder_batch(cfg.vocab, 64, 5 + ranks.rank)  # disjoint batches per replica
    tokens = int(sum(len(q) for q in seqs))
    enc = tb.Encoder(ctx, cfg, tokens=32768, sequences=64)
    enc.fill_random(SEED)
    for _ in range(args.warmup):
        out = enc.embed(seqs)
    ranks.barrier()
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        out = enc.embed(seqs)  # ids cross from host memory, embeddings come back to it
        times.append(time.perf_counter() - t0)
    ms = statistics.median(times) * 1e3
    ms_max = ranks.max(ms)
    assert np.allclose(np.linalg.norm(out, axis=1), 1.0, atol=1e-4)
    h, inter, L = cfg.hidden, cfg.inter, cfg.layers
    flops = 2.0 * tokens * L * (3 * h * h + h * h + 2 * h * inter)
    burst, sustained, how = measured_peak_tflops()
    tf = flops / (ms_max * 1e-3) / 1e12
    n = ranks.world
    enc.close()
    return {"metric": "encoder_sequences_per_second", "value": n * 64 / (ms_max / 1e3), "unit": "seq/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 weights as their f16 values (a copy made once, read by TMA), f16 activations, f32 accumulate (tcgen05); f16/f32 attention", "data": "synthetic", "impl": "ours",
            "config": {"workload": f"configs[4]: 64 sequences of 16..512 tokens ({tokens} tokens packed), Granite-311m shape, plain GELU FFN 3072, mean pooling, 256 dims",
                       "parallelism": f"{n} independent replicas on disjoint batches", "timing": "host wall clock around tb_encoder_embed (host ids in, host embeddings out)"},
            "e2e": {"value": n * 64 / (ms_max / 1e3), "unit": "seq/s", "h2d_bytes_per_step": tokens * 8 + 64 * 8, "d2h_bytes_per_step": 64 * 256 * 4},
            "gpu_launches": args.steps * (2 + L * 9),
            "roofline": {"bound": "tensor", "achieved": tf, "peak": burst, "unit": "TFLOP/s", "frac": tf / burst, "peak_source": how, "traffic": None, "gemm_flops": flops}}


def brief(line):
    """What a sub-object of the default line keeps of a workload's own line."""
    keep = ("metric", "value", "unit", "ms_per_step", "steps", "warmup", "higher_is_better", "dtype", "device_ms", "e2e", "roofline", "cases", "gpu_launches")
    out = {k: line[k] for k in keep if k in line}
    out["workload"] = line["config"]["workload"]
    if "variants" in line["config"]:
        out["variants"] = line["config"]["variants"]
    return out


def reference_arm(args, ranks: Ranks):
    """The reference's implementation of the path, on the host cores.  The reference (Rust + generated PTX) cannot be
    built in this environment, so this arm times the CPU oracle's restatement of its decode step on the same model."""
    if ranks.rank != 0:
        return None
    import tachyon_b200 as tb  # only for the configuration struct

    cfg = tb.gemma4_e4b_shape()
    base, _ = cpu_decode(cfg, max(1, min(args.steps, 16)), 120.0)
    v = base["value"]
    return {"metric": "decode_tokens_per_second", "value": v, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 / v, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 weights x f32 activations, f32 accumulate",
            "data": "synthetic", "impl": "reference",
            "config": {"workload": "configs[2]: full decode step, Gemma-4-E4B-shape Q8, batch 1, context pre-filled to 2048, greedy",
                       "step": "CPU restatement of the reference's decode step, all host cores"},
            "cpu_baseline": base, "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "gemv", "gemv_q4", "gateup", "attend", "gemm", "flash", "prefill", "encoder", "switch", "load", "token"])
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--cols", type=int, default=2048)
    ap.add_argument("--copies", type=int, default=64)
    ap.add_argument("--mode", type=int, default=0, help="gemm workload: the product's output mode (TB_GEMM_*)")
    ap.add_argument("--layers", type=int, default=35, help="decode workload: layers of the model (35 is the benchmark's; fewer for a profiler capture)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="decode workload: skip the prefill / encoder / single-kernel sub-objects")
    ap.add_argument("--weights", default="q8", choices=["q8", "q4", "f16"], help="gemv workload: Q8 or f16 weights; decode and prefill workloads: the benchmark's Q8 matrices, or the reference's converted Q4 format")
    ap.add_argument("--fused", action="store_true", help="decode with the single persistent step kernel instead of one launch per phase")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    ranks = Ranks(args.gpus)
    try:
        if args.impl == "reference":
            line = reference_arm(args, ranks)
        elif args.workload == "gemv":
            line = bench_gemv(args, ranks) if ranks.rank == 0 else None
        elif args.workload == "gateup":
            line = bench_gateup(args, ranks) if ranks.rank == 0 else None
        elif args.workload == "gemv_q4":
            line = bench_gemv_q4(args, ranks) if ranks.rank == 0 else None
        elif args.workload == "attend":
            line = bench_attend(args, ranks) if ranks.rank == 0 else None
        elif args.workload == "flash":
            line = bench_flash(args, ranks) if ranks.rank == 0 else None
        elif args.workload == "gemm":
            line = bench_gemm(args, ranks) if ranks.rank == 0 else None
        elif args.workload == "prefill":
            line = bench_prefill(args, ranks)
        elif args.workload == "encoder":
            line = bench_encoder(args, ranks)
        elif args.workload == "switch":
            line = bench_switch(args, ranks) if ranks.rank == 0 else None
        elif args.workload == "load":
            line = bench_load(args, ranks) if ranks.rank == 0 else None
        elif args.workload == "token":
            line = bench_token(args, ranks) if ranks.rank == 0 else None
        else:
            line, cfg, gpu_tokens = bench_decode(args, ranks)
            if not args.no_extras:
                # The rest of the metric and the other configurations, each a short run of its own workload: prefill and the
                # encoder on every replica, the single kernels on rank 0.
                sub = argparse.Namespace(**vars(args))
                sub.steps, sub.warmup = 5, 3
                line["prefill"] = brief(bench_prefill(sub, ranks))
                line["encoder"] = brief(bench_encoder(sub, ranks))
                if ranks.rank == 0:
                    sub.steps, sub.warmup = 256, 16
                    line["gemv"] = brief(bench_gemv(sub, ranks))
                    line["attend"] = brief(bench_attend(sub, ranks))
                    if ranks.world == 1 and args.layers == 35:  # one replica only: pinned host memory for a whole model
                        sub.steps = 3
                        sw = bench_switch(sub, ranks)
                        line["switch"] = {k: sw[k] for k in ("metric", "value", "unit", "resume_s", "first_park_s", "park_with_kept_copy_s", "link_gb_per_second", "fraction_of_link")}
                        line["switch"]["workload"] = sw["config"]["workload"]
                        try:  # the disk tier's way in: needs 5 GB of temporary files; left out where there is no room for them
                            if shutil.disk_usage(tempfile.gettempdir()).free > (12 << 30):
                                ld = bench_load(sub, ranks)
                                line["load"] = {k: ld[k] for k in ("metric", "value", "unit", "streamed_s", "on_the_calling_thread_s", "streamed_checked_s")}
                                line["load"]["workload"] = ld["config"]["workload"]
                        except (OSError, RuntimeError) as err:
                            line["load"] = {"unavailable": str(err)[:200]}
            if ranks.rank == 0 and ranks.world == 1 and not args.no_cpu:
                line["cpu_baseline"], _ = cpu_decode(cfg, 4, 30.0, gpu_tokens, 4 if args.weights == "q4" else 8)
            elif ranks.rank == 0:
                line["cpu_baseline"] = None
        if ranks.rank == 0 and line is not None:
            print(json.dumps(line), flush=True)
    finally:
        ranks.close()


if __name__ == "__main__":
    main()
