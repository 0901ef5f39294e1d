#!/usr/bin/env python3
"""Benchmark of the library on one B200: decode tokens per second of Hunyuan dense with random
weights, a prompt-sized prefill, the decode step's fraction of the measured HBM bandwidth, and
the dominant kernels alone with their own roofline fractions.  Prints ONE JSON line on standard output.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config 1p8b|4b|7b|tinyA|tinyB] [--batch B] [--prefill N] [--decode N] [--dtype bf16|fp32] [--reps R]
                    [--layers L] [--settle S] [--verify-split] [--profile] [--no-points] [--no-kernels] [--no-graph]

The default is the Hy-MT2 1.8B layer sizes in bfloat16: a batch of 8 sequences that each hold a 2,048-token
prompt, a 2,048-token prefill, decode at batch 1 and 64.  `--config 4b` and `--config 7b` run the two larger
families of sizes with their own workloads (16 prompts of 64 to 4,096 tokens and 256 decode steps; 64 prompts of
16 to 2,048 tokens and 512 steps).  A "step" is one decode step of the whole batch.  `value` is timed on the device
with CUDA events around K steps of the captured decode graph; `e2e` is the same batch through Engine.generate
(host token ids in and out every step), the host's clock read at the call's token callback.  Both time K steps that
come after `--settle` untimed steps (and the warm-up): the prompts of a batch run at the power cap, and for some tens
of milliseconds after them the clocks are still low (the first steps take 2.05 ms instead of 1.62).  `--verify-split` adds, under `verify`, the comparison of logits between
the ways of cutting the work, between the precisions and against the plain implementation of the tests
(src/HyMT2Sharp.Benchmark/Program.cs:124-177); `--profile` adds per-kernel times of a prefill and of
decode steps, kernel after kernel (:243-261).  The shape of the program follows src/HyMT2Sharp.Benchmark/Program.cs:179-241 (warm-up, timed
prefill repetitions reported one by one, timed decode including sampling).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import shutil
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

COMMON = dict(rope_theta=10000.0, rope_alpha=1000.0, rms_norm_eps=1e-5, use_qk_norm=True, head_dim=128,
              max_position_embeddings=8192)
CONFIGS = {
    # the Hy-MT2 1.8B layer sizes: the configuration that the published benchmark names
    "1p8b": dict(name="hunyuan-dense-1.8B-sizes", seed=2, layers=32,
                 sizes=dict(COMMON, hidden_size=2048, num_attention_heads=16, num_key_value_heads=4,
                            intermediate_size=6144, vocab_size=120818, tie_word_embeddings=True),
                 workload=dict(batch=8, prompt=(2048, 2048), steps=64)),
    "4b": dict(name="hunyuan-dense-4B-family-sizes", seed=3, layers=32,
               sizes=dict(COMMON, hidden_size=3072, num_attention_heads=32, num_key_value_heads=8,
                          intermediate_size=8192, vocab_size=120818, tie_word_embeddings=True),
               workload=dict(batch=16, prompt=(64, 4096), steps=256)),
    "7b": dict(name="hunyuan-dense-7B-family-sizes", seed=4, layers=32,
               sizes=dict(COMMON, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                          intermediate_size=14336, vocab_size=128167, tie_word_embeddings=False),
               workload=dict(batch=64, prompt=(16, 2048), steps=512)),
}
# the two tiny configurations of the tests' workloads (head sizes 16 and 32: every kernel is the general CUDA-core one)
CONFIGS["tinyA"] = dict(name="hunyuan-dense-tiny-A", seed=0, layers=2,
                        sizes=dict(hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=160,
                                   vocab_size=256, rope_theta=10000.0, rope_alpha=1.0, rms_norm_eps=1e-5, use_qk_norm=True,
                                   tie_word_embeddings=True, max_position_embeddings=8192),
                        workload=dict(batch=3, lengths=[5, 9, 1], steps=8))
CONFIGS["tinyB"] = dict(name="hunyuan-dense-tiny-B", seed=1, layers=3,
                        sizes=dict(hidden_size=96, num_attention_heads=6, num_key_value_heads=1, head_dim=32, intermediate_size=224,
                                   vocab_size=509, rope_theta=1e6, rope_alpha=1000.0, rms_norm_eps=1e-6, use_qk_norm=False,
                                   tie_word_embeddings=False, max_position_embeddings=8192),
                        workload=dict(batch=4, lengths=[17, 3, 11, 6], steps=12))
CONTEXT = 8192
PREFILL_GROUP_TOKENS = 16384   # prompts go in by groups of at most this many tokens: bounded activation memory
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            data = json.load(f)
        out = dict(FALLBACK_PEAKS)
        for k in out:
            if isinstance(data.get(k), (int, float)):
                out[k] = float(data[k])
        return out, "measured"
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi samples of the SM clock and the throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        os.remove(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w": statistics.median(power) if power else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def reference_arm() -> int:
    # sdcb/HyMT2Sharp is a C#/.NET 10 project (Directory.Build.props) with no Python packaging: pip has
    # nothing to install, and neither machine has a .NET SDK or runtime.
    print(json.dumps({"impl": "reference", "unavailable":
                      "sdcb/HyMT2Sharp is C#/.NET 10 with no Python package (pip install finds no setup.py or "
                      "pyproject.toml) and no dotnet runtime exists here or on the GPU box"}))
    return 0


def make_model(config: str, layers: int) -> str:
    """A model folder with random weights of the named sizes (N(0, 0.02), the configuration's seed), in a temporary folder."""
    from hymt2sharp_b200.config import HunyuanDenseConfig
    from hymt2sharp_b200.weights import write_random_model
    spec = CONFIGS[config]
    data = dict(spec["sizes"], num_hidden_layers=layers, architectures=["HunYuanDenseV1ForCausalLM"],
                rope_scaling={"type": "dynamic", "alpha": spec["sizes"]["rope_alpha"]})
    data.pop("rope_alpha")
    cfg = HunyuanDenseConfig.from_dict(data)
    folder = tempfile.mkdtemp(prefix="hymt2_bench_model_")
    write_random_model(folder, cfg, spec["seed"], 0.02)
    return folder


def step_flops(cfg, prompt_lens, wanted_rows: int) -> float:
    """Flops of a step that runs whole prompts of these lengths (products, causal attention, head on the wanted rows)."""
    per_layer = (cfg.q_size + 2 * cfg.kv_size) * cfg.hidden_size + cfg.hidden_size * cfg.q_size \
        + 3 * cfg.intermediate_size * cfg.hidden_size
    tokens = sum(prompt_lens)
    gemm = 2.0 * tokens * per_layer * cfg.num_hidden_layers
    attn = sum(4.0 * cfg.num_attention_heads * cfg.head_dim * (n * (n + 1) / 2) for n in prompt_lens) * cfg.num_hidden_layers
    head = 2.0 * wanted_rows * cfg.vocab_size * cfg.hidden_size
    return gemm + attn + head


def groups_under_budget(lengths, budget=PREFILL_GROUP_TOKENS):
    """Index ranges of consecutive prompts whose tokens stay under the budget (a prompt alone may exceed it)."""
    out, start, used = [], 0, 0
    for i, n in enumerate(lengths):
        if i > start and used + n > budget:
            out.append((start, i))
            start, used = i, 0
        used += n
    out.append((start, len(lengths)))
    return out


def kernel_fractions(cfg, batch: int, prefill_tokens: int, context: int, pk: dict) -> dict:
    """The dominant kernels alone (captured into a graph, operands rotating so that they come from memory):
    microseconds, the bytes or flops that the kernel has to move or do, and the fraction of the measured peak
    (memory bandwidth for the decode kernels, burst tensor throughput for the prompt kernels)."""
    from hymt2sharp_b200.kernels import microbench as mb
    H, F, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nh, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    big = 2 if V * H * 2 > (1 << 29) else 4
    runs = {
        "gate_up_decode": ("hbm", lambda: mb.measure_gemm(batch, F, H, "swiglu", copies=8)),
        "down_decode": ("hbm", lambda: mb.measure_gemm(batch, H, F, "accumulate", copies=8)),
        # q/k/v with rotation, per-head norm and cache append, the kernel the engine runs (heads of 128), else the plain product
        "qkv_decode": ("hbm", (lambda: mb.measure_qkv_rope(batch, nh, nkv, H, copies=16)) if d == 128 else
                       (lambda: mb.measure_gemm(batch, cfg.q_size + 2 * cfg.kv_size, H, "store", copies=16))),
        "o_proj_decode": ("hbm", lambda: mb.measure_gemm(batch, H, cfg.q_size, "accumulate", copies=16)),
        "lm_head_decode": ("hbm", lambda: mb.measure_gemm(batch, V, H, "store", float_out=True, copies=big, iters=8)),
        "attention_decode": ("hbm", lambda: mb.measure_attention_decode(batch, context, nh, nkv, d, copies=8)),
        "qkv_prefill": ("tensor", (lambda: mb.measure_qkv_rope(prefill_tokens, nh, nkv, H, copies=4)) if d == 128 else
                        (lambda: mb.measure_gemm(prefill_tokens, cfg.q_size + 2 * cfg.kv_size, H, "store", copies=4))),
        "o_proj_prefill": ("tensor", lambda: mb.measure_gemm(prefill_tokens, H, cfg.q_size, "accumulate", copies=4)),
        "gate_up_prefill": ("tensor", lambda: mb.measure_gemm(prefill_tokens, F, H, "swiglu", copies=4)),
        "down_prefill": ("tensor", lambda: mb.measure_gemm(prefill_tokens, H, F, "accumulate", copies=4)),
        "attention_prefill": ("tensor", lambda: mb.measure_attention_prefill(prefill_tokens, nh, nkv, d)),
    }
    out = {}
    for name, (bound, fn) in runs.items():
        m = fn()
        if bound == "hbm":
            achieved, peak, unit = m["bytes"] / m["us"] / 1e3, pk["hbm_gbs"], "GB/s"
        else:
            achieved, peak, unit = m["flops"] / m["us"] / 1e6, pk["bf16_tflops"], "TFLOP/s"
        out[name] = {"us": round(m["us"], 2), "bound": bound, "achieved": round(achieved, 1), "unit": unit,
                     "frac": round(achieved / peak, 3)}
    return out


def run_verify(config: str, layers: int) -> dict:
    """Logits compared between the cuts and the precisions at `layers` layers of the configuration's widths, and the
    32-bit engine against the plain implementation of the tests at 2 layers."""
    import numpy as np
    import torch
    from hymt2sharp_b200.engine.verify import verify_split
    vocab = CONFIGS[config]["sizes"]["vocab_size"]
    rng = np.random.default_rng(11)
    requests = [rng.integers(0, vocab, n).tolist() for n in (300, 70, 1100)]
    out = {}
    folder = make_model(config, layers)
    try:
        t0 = time.time()
        out[f"layers_{layers}"] = verify_split(folder, requests)
        out[f"layers_{layers}"]["seconds"] = round(time.time() - t0, 1)
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    folder = make_model(config, 2)
    try:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from plain.hunyuan_plain import PlainModel
        plain = PlainModel(folder)
        t0 = time.time()
        res = verify_split(folder, requests, reference=lambda toks: plain.logits(toks))
        res["seconds"] = round(time.time() - t0, 1)
        out["layers_2_against_plain"] = res
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    out["ok"] = all(v["ok"] for v in out.values())
    torch.cuda.empty_cache()
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed decode steps (default: 64; the workload's own for 4b and 7b)")
    ap.add_argument("--decode", type=int, default=None, help="the same as --steps (src/HyMT2Sharp.Benchmark --bench-decode)")
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--settle", type=int, default=48,
                    help="untimed decode steps between the prompts and the warm-up: the prompts of a batch run at the power cap and the "
                         "clocks need some tens of ms to come back")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="1p8b", choices=sorted(CONFIGS))
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--prefill", type=int, default=2048, help="tokens of the timed prefill (src/HyMT2Sharp.Benchmark --bench-prefill)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--reps", type=int, default=3, help="timed repetitions of the prefill")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has, only where memory or time needs it")
    ap.add_argument("--verify-split", action="store_true")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-kernels", action="store_true", help="skip the kernels timed alone")
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    spec = CONFIGS[args.config]
    work = spec["workload"]
    warmup = max(3, args.warmup)
    steps = max(1, args.decode or args.steps or (64 if args.config == "1p8b" else work["steps"]))
    settle = max(0, args.settle)
    batch = args.batch or work["batch"]
    layers = args.layers or spec["layers"]
    dtype = {"bf16": "bfloat16", "fp32": "float32"}[args.dtype]

    import numpy as np
    import torch
    import hymt2sharp_b200
    from hymt2sharp_b200.engine.decode_session import DecodeSession
    from hymt2sharp_b200.engine.engine import StepEntry
    from hymt2sharp_b200.kernels import ops
    from hymt2sharp_b200.sampling import BatchSampler, GREEDY

    pk, pk_source = peaks()
    verify = run_verify(args.config, layers) if args.verify_split else None

    rng = np.random.default_rng(1234)
    fixed = work.get("lengths")
    lo, hi = work["prompt"] if fixed is None else (min(fixed), max(fixed))
    uniform = lo == hi and fixed is None
    vocab = spec["sizes"]["vocab_size"]

    def prompt_lengths(n):
        if fixed is not None:
            return [fixed[i % len(fixed)] for i in range(n)]
        return [lo] * n if uniform else [int(x) for x in rng.integers(lo, hi + 1, n)]

    def prompts_of(lengths):
        return [rng.integers(0, vocab, n).tolist() for n in lengths]

    main_lengths = prompt_lengths(batch)
    point_batches = [] if (args.no_points or args.config != "1p8b") else [1, 64]
    reserve = lambda lengths: sum(-(-(n + settle + warmup + steps + 8) // 64) * 64 for n in lengths)
    capacity = max([reserve(main_lengths), args.prefill + 64] + [reserve([lo] * b) for b in point_batches]) + 4096
    folder = make_model(args.config, layers)
    try:
        engine = hymt2sharp_b200.load(folder, dtype=dtype, max_tokens=capacity, max_batch=max([batch] + point_batches),
                                      max_sequence_tokens=CONTEXT)
    finally:
        shutil.rmtree(folder, ignore_errors=True)   # the weights are on the device now; leave nothing in the temporary folder
    cfg = engine.config
    ev = lambda: torch.cuda.Event(enable_timing=True)

    # ---- prefill of --prefill tokens: warm-up, then the mean of the timed repetitions ----------------------
    prompt = prompts_of([args.prefill])[0]
    times = []
    for rep in range(3 + args.reps):
        slot = engine.alloc_slots(1)
        t0, t1 = ev(), ev()
        torch.cuda.synchronize()
        t0.record()
        engine.step([StepEntry(slot[0], prompt, [args.prefill - 1])])
        t1.record()
        torch.cuda.synchronize()
        engine.free_slots(slot)
        if rep >= 3:
            times.append(t0.elapsed_time(t1))
    pf_ms = sum(times) / len(times)
    pf_flops = step_flops(cfg, [args.prefill], 1)
    prefill = {"value": args.prefill / pf_ms * 1000.0, "tokens": args.prefill, "ms": pf_ms, "reps_ms": [round(t, 3) for t in times],
               "frac": pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12) if args.dtype == "bf16" else None,
               "peak": pk_source if args.dtype == "bf16" else "no measured 32-bit peak"}

    # ---- decode ----------------------------------------------------------------------------------
    def decode_run(lengths: list, k: int, w: int, sample_clocks: bool):
        n = len(lengths)
        slots = engine.alloc_slots(n)
        prompts = prompts_of(lengths)
        firsts = []
        t0, t1 = ev(), ev()
        t0.record()
        for g0, g1 in groups_under_budget(lengths):
            entries = [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots[g0:g1], prompts[g0:g1])]
            firsts.append(engine.step(entries))
        t1.record()
        torch.cuda.synchronize()
        batch_prefill_ms = t0.elapsed_time(t1)
        sampler = BatchSampler([GREEDY] * n, engine.device)
        first = sampler.sample(torch.cat(firsts), None)
        session = DecodeSession(engine, slots, sampler, first, max(lengths) + settle + w + k + 2, use_graph=not args.no_graph)
        for _ in range(settle + w):
            session.step()
        torch.cuda.synchronize()
        clocks = ClockSampler()
        if sample_clocks:
            clocks.start()
        launches0 = ops.launches
        t0, t1 = ev(), ev()
        t0.record()
        for _ in range(k):
            session.step()
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1)
        clk = clocks.stop() if sample_clocks else None
        launches = ops.launches - launches0
        mean_tokens = sum(lengths) + n * (settle + w + (k + 1) / 2.0)   # cached tokens that a timed step reads, on average
        engine.check()
        engine.free_slots(slots)
        return ms, launches, mean_tokens, clk, batch_prefill_ms

    ms, launches, mean_tokens, clocks, batch_prefill_ms = decode_run(main_lengths, steps, warmup, True)
    ms_per_step = ms / steps
    value = batch * steps / ms * 1000.0
    step_bytes = engine.model.streamed_weight_bytes() + mean_tokens * engine.cache.bytes_per_token() \
        + batch * cfg.hidden_size * 2
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "peak_source": pk_source, "bytes_per_step": int(step_bytes)}
    if not uniform:
        # the workload's own prefill: all prompts of the unequal batch, in groups under the token budget
        flops = step_flops(cfg, main_lengths, batch)
        prefill["batch"] = {"value": sum(main_lengths) / batch_prefill_ms * 1000.0, "tokens": sum(main_lengths),
                            "ms": batch_prefill_ms, "groups": len(groups_under_budget(main_lengths)),
                            "frac": flops / (batch_prefill_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12)
                            if args.dtype == "bf16" else None, "peak": "sustained"}

    points = {}
    for b in point_batches:
        k = max(8, min(steps, 32))
        pms, _, _, _, _ = decode_run([lo] * b, k, warmup, False)
        points[f"decode_b{b}"] = b * k / pms * 1000.0

    # ---- end to end: Engine.generate, host token ids in and out every step ------------------------
    prompts = prompts_of(main_lengths)
    # warm-up of the entry point with the same batch shape: the decode graph of that shape is captured here,
    # as it is once in a serving process, not in the timed run
    engine.generate(prompts, max_new_tokens=4, max_batch=batch)
    # One call of the entry point for settle + K + 1 tokens a request.  The host's clock is read whenever a step's tokens
    # have arrived on the host (the call's own token callback); the timed region is the last K steps of the call, each with
    # its copies in both directions.  The steps before them are the same settling as in the device-timed run.
    stamps, arrived = [], []

    def on_tokens(pairs):
        stamps.append(time.perf_counter())
        arrived.append(len(pairs))

    out = engine.generate(prompts, max_new_tokens=settle + steps + 1, max_batch=batch, on_tokens=on_tokens)
    k_e2e = min(steps, len(stamps) - 1)
    e2e_ms = (stamps[-1] - stamps[-1 - k_e2e]) * 1000.0
    e2e_tokens = sum(arrived[-k_e2e:])
    e2e = {"value": e2e_tokens / max(e2e_ms, 1e-9) * 1000.0, "unit": "tokens/s",
           # every step: which rows run (slot and row number of each, int32) from pinned memory; the sampled tokens back
           "h2d_bytes_per_step": 8 * batch, "d2h_bytes_per_step": 4 * batch,
           "steps": k_e2e, "ms": e2e_ms, "settle_steps": len(stamps) - 1 - k_e2e,
           "call": {"decode_tokens": out.stats.decode_tokens, "decode_ms": out.stats.decode_ms, "prefill_ms": out.stats.prefill_ms,
                    "tokens_per_s": out.stats.decode_tokens / max(out.stats.decode_ms, 1e-9) * 1000.0}}

    profile = None
    if args.profile:
        prof = engine.generate(prompts[:batch], max_new_tokens=min(steps, 16) + 1, max_batch=batch, profile=True)
        profile = {phase: {k: round(v, 3) for k, v in t.items()} for phase, t in prof.stats.profile.items()}
        for phase, t in prof.stats.profile.items():
            print(ops.profile_line(phase, t), file=sys.stderr)

    kernels = None
    if not args.no_kernels and args.dtype == "bf16" and not args.config.startswith("tiny"):
        del engine, out
        torch.cuda.empty_cache()
        mean_ctx = int(mean_tokens / batch)
        kernels = kernel_fractions(cfg, batch, args.prefill, mean_ctx, pk)
        kernels["peaks"] = {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk_source}

    lengths_text = f"{batch} x {lo}" if uniform else f"lengths {main_lengths}" if fixed is not None else \
        f"{batch} lengths uniform in [{lo},{hi}], seed 1234"
    line = {
        "metric": ("decode tok/s at batch 8 (1.8B bf16, 2,048-token prompts); prefill tok/s at 2,048 tokens"
                   if (args.config, args.dtype, batch, args.prefill) == ("1p8b", "bf16", 8, 2048) else
                   f"decode tok/s at batch {batch} ({spec['name']}, {args.dtype}, prompts {lengths_text}); "
                   f"prefill tok/s at {args.prefill} tokens"),
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": args.dtype,
        "data": f"synthetic: seeded uniform-random token ids, random-init weights N(0, 0.02) seed {spec['seed']}",
        "impl": "ours",
        "config": {"model": spec["name"], "global_batch": batch, "seq_len": int(sum(main_lengths) / batch),
                   "prompts": lengths_text, "context": CONTEXT, "parallelism": "single-gpu", "layers": layers,
                   "layers_full": spec["layers"], "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
                   "vocab": cfg.vocab_size, "rope_alpha": cfg.rope_alpha, "qk_norm": cfg.use_qk_norm,
                   "tied": cfg.tie_word_embeddings, "sampling": "greedy on the GPU", "settle_steps": settle,
                   "l2": "inputs larger than L2: every step streams all weights (GBs) once" if step_bytes > 2 * 126e6 else
                         "model smaller than L2, nothing flushed: a tiny configuration times launches, not memory"},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "prefill": prefill, "roofline": roofline,
        "points": points,
    }
    if kernels is not None:
        line["kernels"] = kernels
    if verify is not None:
        line["verify"] = verify
    if profile is not None:
        line["profile"] = profile
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
