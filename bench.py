"""Benchmark of the hot path: batch-1 greedy decode of the synthetic
TinyLlama-shaped Q4_K_M model (benchmark configuration 1).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one decode token (one pass of the forward path). `value` is tokens/s with
everything resident in HBM (device-side greedy loop, CUDA-graph replays, device
timing); `e2e` is the same metric through the host-facing call (token id in, logits
out to host memory, host argmax, every step). With --gpus N > 1 (one rank per GPU,
launched by torchrun) each rank decodes its own replica: the model does not shard
(its FFN width is not a multiple of 4 super-blocks), so scaling is weak and there is
no data-path collective.

`--impl reference` times the reference's CPU implementation of the same path on the
host cores: the C++ restatement in oracle/ (the reference itself is Rust and no Rust
toolchain exists here), with the reference's default thread count min(cores, 8).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as graft  # noqa: E402

METRIC = "decode_tokens_per_s"
UNIT = "tok/s"
PROMPT_SEED, PROMPT_LEN = 7, 6
N_CTX = 2048


def measured_peak_gbs() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs
    (read-only queries)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80, "sw_power_cap": 0x4}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        if self.nv:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._t:
            self._t.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


L2_BYTES = 126 * 1024 * 1024
KINDS = {"f32": 0, "f16": 1, "bf16": 2, "q4_0": 3, "q5_0": 4, "q8_0": 5, "q4_k": 6, "q5_k": 7, "q6_k": 8}


def _synth_matrix(pkg, kind: int, rows: int, cols: int, seed: int) -> np.ndarray:
    """Seeded random blocks of one quant type, every field of the layout filled uniformly (benchmark configuration 0)."""
    rb = pkg.lib.row_bytes(kind, cols)
    w = np.zeros(rows * rb, dtype=np.uint8)
    pkg.lib.check(pkg.lib.synth().aotcu_synth_tensor(kind, rows, cols, 1e-3, 1e-2, seed, w.ctypes.data))
    return w


def time_product(pkg, ctx, kind: int, rows: int, cols: int, m: int, iters: int, host_w=None, repeats: int = 1, alone: int = 0):
    """Device time per launch of the (m x cols)·(rows x cols)^T product with the weights streamed
    from HBM: the launches rotate through enough copies of the matrix to exceed the L2 size.
    Returns (microseconds per launch, weight bytes, copies); with `repeats` > 1 the first item
    is the median of that many timed loops and a fourth item holds {min, max, all, and with
    `alone` > 0 the median time of that many launches each timed alone on a drained stream}."""
    w = host_w if host_w is not None else _synth_matrix(pkg, kind, rows, cols, 7)
    copies = max(1, -(-int(1.25 * L2_BYTES) // w.nbytes))
    stride = (w.nbytes + 255) & ~255
    dw = ctx.alloc(stride * copies)
    for i in range(copies):
        dw.upload(w, i * stride)
    x = np.random.default_rng(5).standard_normal(m * cols).astype(np.float32)
    dxf = ctx.to_device(x)
    if kind >= KINDS["q4_k"]:      # K-quants take Q8_K activation blocks (292 bytes per 256 values)
        dx = ctx.alloc(m * cols // 256 * 292)
        ctx.quantize_q8_k(dxf, m * cols, dx)
    elif kind >= KINDS["q4_0"]:    # Q4_0 / Q5_0 / Q8_0 take Q8_0 blocks (36 bytes per 32 values)
        dx = ctx.alloc(m * cols // 32 * 36)
        ctx.quantize_q8_0(dxf, m * cols, dx)
    else:                          # float kinds take f32
        dx = dxf
    dout = ctx.alloc(m * rows * 4)
    runs = [ctx.bench_matmul(kind, dout, dw, stride, copies, dx, m, rows, cols, iters) * 1e3 for _ in range(max(1, repeats))]
    lone = [ctx.bench_matmul(kind, dout, dw, stride, copies, dx, m, rows, cols, 1) * 1e3 for _ in range(alone)]
    dw.free(); dx.free(); dout.free()
    if dxf is not dx:
        dxf.free()
    us = float(np.median(runs))
    if repeats <= 1 and not alone:
        return us, w.nbytes, copies
    extra = {"repeats": len(runs), "min_us": min(runs), "max_us": max(runs), "all_us": runs}
    if lone:
        extra["alone_us_median"] = float(np.median(lone))
        extra["alone_launches"] = len(lone)
    return us, w.nbytes, copies, extra


def cpu_matvec_gbs(pkg, kind: int, rows: int, cols: int, threads: int, seconds: float = 2.0):
    """The oracle's matvec on the host cores (weights larger than the CPU caches are not
    arranged for: a 6.5 MB matrix is cache resident there, as it is in the reference's own
    micro-benchmarks)."""
    from oracle import binding as ob
    w = _synth_matrix(pkg, kind, rows, cols, 7)
    x = np.random.default_rng(5).standard_normal(cols).astype(np.float32)
    q = ob.quantize_act(kind, x)
    pool, tab = ob.Pool(threads), ob.detect_table()
    ob.matvec(pool, tab, kind, w, q, rows, cols)
    n, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        ob.matvec(pool, tab, kind, w, q, rows, cols)
        n += 1
    dt = time.perf_counter() - t0
    return w.nbytes * n / dt / 1e9, n


def profiled_traffic(name: str):
    """DRAM bytes (read + write) of one launch from the committed ncu summary `profiles/<name>`:
    the line `dram_bytes_per_launch = N`. None when the summary or the line is missing."""
    import re
    try:
        text = open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "profiles", name)).read()
    except OSError:
        return None
    m = re.search(r"^dram_bytes_per_launch\s*=\s*(\d+)", text, re.M)
    return int(m.group(1)) if m else None


def prompt_tokens_n(vocab: int, n: int):
    return np.random.default_rng(PROMPT_SEED + 1).integers(0, vocab, n).tolist()


def run_sweep(args):
    """Benchmark configuration 4: every quant type at four matrix shapes, M = 1 and M = 64."""
    pkg = graft.import_package()
    ctx = pkg.Context(0)
    peak, peak_src = measured_peak_gbs()
    shapes = [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)]
    if args.sweep_small:
        shapes = shapes[:2]
    if args.sweep_shapes:
        shapes = [tuple(int(v) for v in sh.split("x")) for sh in args.sweep_shapes.split(",")]
    names = ("q4_0", "q5_0", "q8_0", "q4_k", "q5_k", "q6_k", "f16", "bf16")
    if args.sweep_kinds:
        names = tuple(args.sweep_kinds.split(","))
    ms = tuple(int(v) for v in args.sweep_m.split(","))
    rows_out = []
    for name in names:
        kind = KINDS[name]
        for rows, cols in shapes:
            w = _synth_matrix(pkg, kind, rows, cols, 7)
            for m in ms:
                iters = 20 if m == 1 else 5
                us, nbytes, copies = time_product(pkg, ctx, kind, rows, cols, m, iters, host_w=w)
                rows_out.append({"kind": name, "rows": rows, "cols": cols, "m": m, "us_per_launch": round(us, 2),
                                 "weight_gbs": round(nbytes / us / 1e3, 1), "frac_of_hbm_peak": round(nbytes / us / 1e3 / peak, 4),
                                 "tera_ops": round(2.0 * rows * cols * m / us / 1e6, 2), "copies": copies})
            del w
    print(json.dumps({"metric": "quant_kernel_sweep", "unit": "GB/s of weight bytes per launch", "peak": peak,
                      "peak_source": peak_src, "l2_policy": "launches rotate through copies of the matrix that together exceed L2",
                      "rows": rows_out}))


def prompt_tokens(vocab: int):
    return np.random.default_rng(PROMPT_SEED).integers(0, vocab, PROMPT_LEN).tolist()


def cpu_decode(spec, steps: int, warmup: int, threads: int):
    """Times `steps` decode tokens of the oracle after the prompt and `warmup` tokens."""
    from oracle import binding as ob
    om = ob.model_from_spec(spec, PROMPT_LEN + warmup + steps + 2, 8, n_threads=threads)
    om.forward_batch(prompt_tokens(spec.head.dims.vocab), 0, True)
    tok, pos = ob.argmax(om.logits()), PROMPT_LEN
    for _ in range(warmup):
        om.forward(tok, pos, True)
        tok, pos = ob.argmax(om.logits()), pos + 1
    t0 = time.perf_counter()
    for _ in range(steps):
        om.forward(tok, pos, True)
        tok, pos = ob.argmax(om.logits()), pos + 1
    dt = time.perf_counter() - t0
    om.close()
    return steps / dt, dt


def workload_config(spec):
    d = spec.head.dims
    return {"workload": "configs[1]: TinyLlama-shaped Llama decode, Q4_K_M mix, random-init weights, 6-token prompt then greedy decode",
            "dim": d.dim, "hidden": d.hidden, "n_layer": d.n_layer, "n_head": d.n_head, "n_kv_head": d.n_kv_head,
            "head_dim": d.head_dim, "vocab": d.vocab, "context": N_CTX, "batch": 1,
            "weight_bytes_per_token": spec.weight_bytes_per_token(),
            "l2_policy": "inputs_larger_than_l2 (633 MB of weights streamed per step, L2 is 126 MB)"}


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    pkg = graft.import_package()
    spec = pkg.model.tinyllama()
    cores = os.cpu_count() or 1
    steps = max(1, min(args.steps, 64))
    warmup = max(1, min(args.warmup, 16))
    # The reference defaults to min(cores, 8) threads (crates/aot-kernels/src/app.rs:214-216)
    # and takes --threads; both settings are timed and the faster one is the line's value.
    tried = {}
    for threads in sorted({min(cores, 8), cores}):
        tried[threads] = cpu_decode(spec, steps, warmup, threads)[0]
    threads = max(tried, key=tried.get)
    tps = tried[threads]
    cfg = workload_config(spec)
    sample = f"{steps} decode steps after the {PROMPT_LEN}-token prompt and {warmup} warm-up tokens"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": 0, "steps": steps,
        "warmup": warmup, "ms_per_step": 1e3 / tps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 block dot products with f32 accumulation (Q8 activations x Q4_K/Q6_K weights)",
        "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                         "host_cores": cores, "tok_s_by_threads": {str(k): v for k, v in tried.items()},
                         "note": "C++ restatement of the reference's AVX2 kernel table and forward pass (oracle/); the Rust reference cannot be built here"},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args, rank: int, world: int, local_rank: int):
    pkg = graft.import_package()
    # N GPUs = N independent replicas of the decode path (no data-path collective); the
    # process group only brackets the timed regions and takes the slowest rank's time.
    ranks = pkg.ranks.Ranks(pkg.ranks.RankInfo(rank, world, local_rank), backend="nccl")
    barrier, max_over_ranks = ranks.barrier, ranks.max_over_ranks

    spec = pkg.model.tinyllama()
    d = spec.head.dims
    ctx = pkg.Context(local_rank)
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, N_CTX, 8)
    if args.pdl >= 0:
        g.set_option("pdl", args.pdl)   # default: the library's own default (on)
    prompt = prompt_tokens(d.vocab)
    steps, warmup = args.steps, max(args.warmup, 3)

    # ---- device-resident throughput -----------------------------------------------------
    g.forward_batch(prompt, 0, True)
    first = int(np.argmax(g.logits()))
    warm_ids, _ = g.generate(first, PROMPT_LEN, warmup)
    ctx.sync()
    barrier()
    launches0 = g.dispatches()
    with ClockSampler(local_rank) as clk:
        ids, ms = g.generate(int(warm_ids[-1]), PROMPT_LEN + warmup, steps)
        ctx.sync()
    barrier()
    launches = g.dispatches() - launches0
    ms = max_over_ranks(ms)
    tps = world * steps / (ms * 1e-3)

    # ---- end to end through the host-facing step call --------------------------------------
    e2e_steps = min(steps, 64)
    g.forward_batch(prompt, 0, True)
    tok, pos = int(np.argmax(g.logits())), PROMPT_LEN
    for _ in range(3):
        g.forward(tok, pos, True)
        tok, pos = int(np.argmax(g.logits())), pos + 1
    ctx.sync()
    barrier()
    ctx.timer_start()                      # CUDA events on the launching stream
    for _ in range(e2e_steps):
        g.forward(tok, pos, True)          # token id + position go host -> device
        tok, pos = int(np.argmax(g.logits())), pos + 1  # vocab floats come device -> host
    e2e_s = max_over_ranks(ctx.timer_stop() * 1e-3)
    barrier()
    e2e_tps = world * e2e_steps / e2e_s

    # ---- roofline of the dominant kernel --------------------------------------------------
    # The timed region is `steps` launches of decode_step_kernel (one per token, CUDA-graph
    # replays); its average launch duration is the device time of the loop over the steps.
    peak, peak_src = measured_peak_gbs()
    mid_pos = PROMPT_LEN + warmup + steps // 2
    step_bytes = spec.weight_bytes_per_token() + spec.kv_bytes_per_position() * (mid_pos + 1)
    step_gbs = step_bytes / (ms * 1e-3 / steps) / 1e9
    one_kernel = launches == steps
    # The single-row product kernel alone (operator API, models the one-kernel step does not cover):
    # every matrix product of one decode step, back to back.
    sweep_ms, sweep_launches, sweep_bytes = g.gemv_sweep(20)
    gemv_gbs = sweep_bytes / (sweep_ms * 1e-3) / 1e9

    # ---- configs[0]: one Q4_K matvec, 5632 x 2048, weights streamed from HBM ----------------
    mv_us, mv_bytes, mv_copies, mv_extra = time_product(pkg, ctx, KINDS["q4_k"], 5632, 2048, 1, 200, repeats=5, alone=20)

    # ---- configs[2]: a 512-token prompt in chunks of 64 --------------------------------------
    p_tokens = prompt_tokens_n(d.vocab, 512)
    gp = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 1024, 64)

    def prompt_pass():
        for c0 in range(0, 512, 64):
            gp.forward_batch(p_tokens[c0:c0 + 64], c0, c0 + 64 == 512)

    prompt_pass()
    ctx.sync()
    barrier()
    ctx.timer_start()
    prompt_pass()
    prompt_ms = max_over_ranks(ctx.timer_stop())
    barrier()
    gp.close()

    # ---- configs[3]: the 8B-shaped model, sharded over the ranks (one token stream) -----------
    tp = None
    if not args.no_tp:
        g.close()
        try:
            tp = measure_tp(args, pkg, ranks, ctx, local_rank, min(steps, 64), min(warmup, 4))
        except Exception as e:  # the replica line above stands on its own
            tp = {"error": f"{type(e).__name__}: {e}"[:400]} if rank == 0 else None

    if rank != 0:
        ranks.close()
        return

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        cpu_steps = 24
        tried = {}
        for threads in sorted({min(cores, 8), cores}):
            tried[threads] = cpu_decode(spec, cpu_steps, 2, threads)
        threads = max(tried, key=lambda k: tried[k][0])
        cpu_tps, cpu_dt = tried[threads]
        cpu = {"value": cpu_tps, "unit": UNIT, "cores": threads, "kind": "port", "host_cores": cores,
               "tok_s_by_threads": {str(k): v[0] for k, v in tried.items()},
               "sample": f"{cpu_steps} decode steps of the same model after the prompt and 2 warm-up tokens ({cpu_dt:.1f} s), best of the reference's default thread count and all host threads"}

    extra_cpu = {}
    if cpu:
        from oracle import binding as ob
        cpu_threads = cpu["cores"]
        gbs, n_calls = cpu_matvec_gbs(pkg, KINDS["q4_k"], 5632, 2048, cpu_threads)
        extra_cpu["matvec"] = {"value": gbs, "unit": "GB/s", "cores": cpu_threads, "kind": "port",
                               "sample": f"{n_calls} calls of the oracle's matvec_q4_k, 5632x2048 (cache resident on the host)"}
        om = ob.model_from_spec(spec, 1024, 64, n_threads=cpu_threads)
        om.forward_batch(p_tokens[:64], 0, False)
        t0 = time.perf_counter()
        om.forward_batch(p_tokens[64:128], 64, False)
        om.forward_batch(p_tokens[128:192], 128, True)
        dt = time.perf_counter() - t0
        om.close()
        extra_cpu["prompt"] = {"value": 128 / dt, "unit": "tok/s", "cores": cpu_threads, "kind": "port",
                               "sample": f"chunks 2 and 3 (128 tokens) of the same prompt ({dt:.1f} s)"}

    out = {
        "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 block dot products with f32 accumulation (Q8 activations x Q4_K/Q6_K weights)",
        "data": "synthetic", "config": workload_config(spec),
        "numerics": "exact (bit-identical to the CPU path; the reordering switches of the step kernel are off)",
        "clocks": clk.summary(),
        "e2e": {"value": e2e_tps, "unit": UNIT, "h2d_bytes_per_step": 16, "d2h_bytes_per_step": 4 * d.vocab,
                "steps": e2e_steps},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "kernel": "decode_step_kernel" if one_kernel else "per-operator kernels (whole step)",
                     "achieved": step_gbs, "peak": peak, "unit": "GB/s", "frac": step_gbs / peak,
                     "peak_source": peak_src, "traffic": profiled_traffic("decode_step_kernel_tinyllama_decode.md") if one_kernel else None,
                     "algorithmic_bytes_per_launch": int(step_bytes), "avg_launch_us": ms * 1e3 / steps,
                     "roofline_tok_s": peak * 1e9 / step_bytes,
                     "how": "weights + KV bytes of one token / (device time of the timed loop / steps), CUDA events on the launching stream; traffic = dram read+write of one launch from the ncu capture summarised in profiles/decode_step_kernel_tinyllama_decode.md (position 9; it grows by 90 KB of KV rows per position)"},
        "gemv_kernel_sweep": {"kernel": "gemv_stream_kernel", "achieved": gemv_gbs, "unit": "GB/s", "frac": gemv_gbs / peak,
                              "launches": int(sweep_launches), "algorithmic_bytes": int(sweep_bytes),
                              "avg_launch_us": sweep_ms * 1e3 / sweep_launches},
        "matvec_q4_k": {"workload": "configs[0]: Q4_K matvec, W 5632x2048, x f32 quantized to Q8_K", "value": mv_bytes / mv_us / 1e3,
                        "unit": "GB/s", "frac": mv_bytes / mv_us / 1e3 / peak, "us_per_launch": mv_us,
                        "weight_bytes": int(mv_bytes), "copies_rotated": int(mv_copies),
                        "how": "median of 5 loops of 200 back-to-back launches (dependent launches overlap: a launch streams its weights while its predecessor drains); alone_us_median = one launch on a drained stream",
                        **{k: v for k, v in mv_extra.items() if k != "all_us"},
                        "alone_gbs": mv_bytes / mv_extra["alone_us_median"] / 1e3,
                        "cpu_baseline": extra_cpu.get("matvec")},
        "prompt": {"workload": "configs[2]: 512-token prompt in chunks of 64 on the same model", "value": world * 512 / (prompt_ms * 1e-3),
                   "unit": "tok/s", "ms": prompt_ms, "cpu_baseline": extra_cpu.get("prompt")},
        "generated_head": [int(x) for x in ids[:8]],
    }
    if cpu:
        out["cpu_baseline"] = cpu
    if tp:
        for k in ("metric", "unit", "higher_is_better", "vs_baseline", "dtype", "data"):
            tp.pop(k, None)
        if "value" in tp:
            tp["tok_s"], tp["ms_per_token"] = tp.pop("value"), tp.pop("ms_per_step")
        out["tp"] = tp
    print(json.dumps(out))
    ranks.close()


def tp_parity(pkg, ranks, ctx, n_layer: int = 2, n_steps: int = 8):
    """The sharded path against the whole model on rank 0's GPU: a short 8B-shaped model, one
    prompt chunk and a few decode steps; every rank's gathered logits must agree with the
    single-device ones to f32 rounding (only the order of the additions over blocks differs)."""
    info = ranks.info
    full = pkg.model.qwen3_8b(n_layer=n_layer, seed=0x7A11)
    sh = pkg.tp.shard_spec(full, info.rank, info.world)
    g = pkg.Gpu(ctx, sh.head, sh.layers, sh.weights, 128, 64)
    pkg.tp.join(g, ranks, fused=True)
    one = pkg.Gpu(ctx, full.head, full.layers, full.weights, 128, 64) if ranks.is_root and info.world > 1 else None
    toks = prompt_tokens_n(full.head.dims.vocab, 48)
    worst, agree, total = 0.0, 0, 0

    def compare(lg):
        nonlocal worst, agree, total
        if one is None:
            return
        lf = one.logits()
        worst = max(worst, float(np.max(np.abs(lg - lf)) / np.max(np.abs(lf))))
        agree += int(np.argmax(lg) == np.argmax(lf))
        total += 1

    g.forward_batch(toks, 0, True)
    if one:
        one.forward_batch(toks, 0, True)
    lg = g.logits()
    compare(lg)
    tok, pos = int(np.argmax(lg)), len(toks)
    for _ in range(n_steps):
        g.forward(tok, pos, True)
        if one:
            one.forward(tok, pos, True)
        lg = g.logits()
        compare(lg)
        tok, pos = int(np.argmax(lg)), pos + 1
    ids, _ = g.generate(tok, pos, 8)         # in-kernel argmax exchange
    same = None
    if one:
        ids1, _ = one.generate(tok, pos, 8)
        same = [int(i) for i in ids] == [int(i) for i in ids1]
        one.close()
    ranks.barrier()
    g.close()
    return {"layers": n_layer, "worst_rel_logit_diff": worst, "same_greedy_choice": f"{agree}/{total}",
            "same_generated_ids": same, "tolerance": 1e-3}


def measure_tp(args, pkg, ranks, ctx, local_rank: int, steps: int, warmup: int):
    """Benchmark configuration 3: Qwen3-8B-shaped decode, row-sharded over the ranks, one token
    stream (strong scaling). Every rank builds the synthetic model from the same seed and
    keeps its shard. Returns the result on rank 0, None elsewhere."""
    rank, world = ranks.info.rank, ranks.info.world
    t_build = time.perf_counter()
    full = pkg.model.qwen3_8b(n_layer=args.tp_layers)
    full_bytes = full.weight_bytes_per_token()
    spec = pkg.tp.shard_spec(full, rank, world)
    del full
    t_build = time.perf_counter() - t_build
    d = spec.head.dims
    n_prompt = 512
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_prompt + warmup + steps + 8, 64)
    pkg.tp.join(g, ranks, fused=not args.tp_nccl)
    one_kernel = bool(g.set_option("mega_available", 0))
    toks = prompt_tokens_n(d.vocab, n_prompt)

    def prompt_pass():
        for c0 in range(0, n_prompt, 64):
            g.forward_batch(toks[c0:c0 + 64], c0, c0 + 64 == n_prompt)

    prompt_pass()
    ctx.sync()
    ranks.barrier()
    ctx.timer_start()
    prompt_pass()
    prompt_ms = ranks.max_over_ranks(ctx.timer_stop())
    first = int(np.argmax(g.logits()))
    warm_ids, _ = g.generate(first, n_prompt, warmup)
    ctx.sync()
    ranks.barrier()
    launches0 = g.dispatches()
    with ClockSampler(local_rank) as clk:
        ids, ms = g.generate(int(warm_ids[-1]), n_prompt + warmup, steps)
        ctx.sync()
    ranks.barrier()
    launches = g.dispatches() - launches0
    ms = ranks.max_over_ranks(ms)
    g.close()
    tps = steps / (ms * 1e-3)
    peak, peak_src = measured_peak_gbs()
    mid_pos = n_prompt + warmup + steps // 2
    step_bytes = spec.weight_bytes_per_token() + spec.kv_bytes_per_position() * (mid_pos + 1)
    gbs = step_bytes / (ms * 1e-3 / steps) / 1e9
    sharded_head = spec.head.output.rows != d.vocab
    rank_bytes = spec.weight_bytes_per_token()
    del spec
    parity = tp_parity(pkg, ranks, ctx) if world > 1 and not args.tp_nccl else None
    if rank != 0:
        return None
    return {
        "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 block dot products with f32 accumulation (Q8 activations x Q4_K/Q6_K weights)", "data": "synthetic",
        "config": {"workload": "configs[3]: Qwen3-8B-shaped decode, Q4_K_M mix, random-init weights, 512-token prompt then greedy decode; "
                               "query/KV heads, FFN rows and the output head's vocabulary rows sharded over the ranks; partial rows of "
                               "attn_output and ffn_down summed across ranks, best {logit, id} exchanged for the greedy choice",
                   "dim": d.dim, "hidden_per_rank": d.hidden, "n_layer": d.n_layer, "n_head_per_rank": d.n_head,
                   "n_kv_head_per_rank": d.n_kv_head, "head_dim": d.head_dim, "vocab": d.vocab, "parallelism": f"tp{world}",
                   "output_head": "vocabulary rows sharded" if sharded_head else "whole on every rank",
                   "exchange": ("tagged words over peer memory inside the one-kernel step" if one_kernel and world > 1 else
                                "none" if world == 1 else "NCCL all-reduce between per-operator kernels"),
                   "weight_bytes_per_token_whole_model": int(full_bytes),
                   "weight_bytes_per_token_per_rank": int(rank_bytes),
                   "l2_policy": "inputs_larger_than_l2"},
        "clocks": clk.summary(), "gpu_launches": int(launches),
        "prompt": {"value": n_prompt / (prompt_ms * 1e-3), "unit": "tok/s", "ms": prompt_ms},
        "roofline": {"bound": "hbm", "kernel": "decode_step_kernel of one rank" if one_kernel else "whole decode step of one rank",
                     "achieved": gbs, "peak": peak, "unit": "GB/s",
                     "frac": gbs / peak, "peak_source": peak_src, "traffic": None,
                     "algorithmic_bytes_per_launch": int(step_bytes), "roofline_tok_s": peak * 1e9 / step_bytes},
        "parity": parity,
        "host_build_s": t_build, "generated_head": [int(x) for x in ids[:8]],
    }


def run_tp(args, rank: int, world: int, local_rank: int):
    pkg = graft.import_package()
    ranks = pkg.ranks.Ranks(pkg.ranks.RankInfo(rank, world, local_rank), backend="nccl")
    ctx = pkg.Context(local_rank)
    out = measure_tp(args, pkg, ranks, ctx, local_rank, args.steps, max(args.warmup, 3))
    if out is not None:
        print(json.dumps(out))
    ranks.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--pdl", type=int, default=-1, help="programmatic dependent launch: 0 off, 1 on, -1 library default")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tp", action="store_true", help="configs[3]: Qwen3-8B-shaped decode sharded over the ranks")
    ap.add_argument("--tp-layers", type=int, default=36)
    ap.add_argument("--no-tp", action="store_true", help="skip the sharded 8B-shaped model (the line's \"tp\" key)")
    ap.add_argument("--tp-nccl", action="store_true", help="with --tp: exchange through NCCL all-reduces (per-operator path)")
    ap.add_argument("--sweep", action="store_true", help="quant-type kernel sweep (configs[4]) instead of the decode benchmark")
    ap.add_argument("--sweep-small", action="store_true", help="with --sweep: only the two smaller shapes")
    ap.add_argument("--sweep-kinds", default="", help="with --sweep: comma-separated kinds (default: all eight)")
    ap.add_argument("--sweep-shapes", default="", help="with --sweep: comma-separated ROWSxCOLS (default: the four of configs[4])")
    ap.add_argument("--sweep-m", default="1,64", help="with --sweep: comma-separated activation row counts")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference" and not (args.sweep or args.tp):
        graft.build_host_only()  # the CPU arm maps no product library
        run_reference(args, rank, world)
        return
    graft.build()
    if args.sweep:
        if rank == 0:
            run_sweep(args)
        return
    if args.tp:
        run_tp(args, rank, world, local_rank)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
