#!/usr/bin/env python3
"""Benchmark of the library on one B200: decode tokens per second of Hunyuan dense at the
1.8B layer sizes with random weights (bfloat16), a batch of 8 sequences that each hold a
2,048-token prompt, plus a 2,048-token prefill, decode at batch 1 and 64, and the decode
step's fraction of the measured HBM bandwidth.  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  `value` is timed on the device with CUDA
events around K steps of the captured decode graph; `e2e` is the same batch through
Engine.generate (host token ids in and out every step).  The shape of the program follows
src/HyMT2Sharp.Benchmark/Program.cs:179-241 (warm-up, timed prefill repetitions, timed decode).
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

# the Hy-MT2 1.8B layer sizes, random weights: the configuration that the published benchmark names
SIZES = dict(num_hidden_layers=32, hidden_size=2048, num_attention_heads=16, num_key_value_heads=4, head_dim=128,
             intermediate_size=6144, vocab_size=120818, rope_theta=10000.0, rope_alpha=1000.0, rms_norm_eps=1e-5,
             use_qk_norm=True, tie_word_embeddings=True, max_position_embeddings=8192)
FULL_LAYERS = 32
PROMPT = 2048
CONTEXT = 8192
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


def make_model(layers: int, seed: int = 2) -> str:
    from hymt2sharp_b200.config import HunyuanDenseConfig
    from hymt2sharp_b200.weights import write_random_model
    data = dict(SIZES, num_hidden_layers=layers, architectures=["HunYuanDenseV1ForCausalLM"],
                rope_scaling={"type": "dynamic", "alpha": SIZES["rope_alpha"]})
    data.pop("rope_alpha")
    cfg = HunyuanDenseConfig.from_dict(data)
    folder = tempfile.mkdtemp(prefix="hymt2_bench_model_")
    write_random_model(folder, cfg, seed, 0.02)
    return folder


def prefill_flops(cfg, tokens: int, wanted_rows: int) -> float:
    per_layer = (cfg.q_size + 2 * cfg.kv_size) * cfg.hidden_size + cfg.hidden_size * cfg.q_size \
        + 3 * cfg.intermediate_size * cfg.hidden_size
    gemm = 2.0 * tokens * per_layer * cfg.num_hidden_layers
    attn = 4.0 * cfg.num_attention_heads * cfg.head_dim * (tokens * (tokens + 1) / 2) * cfg.num_hidden_layers
    head = 2.0 * wanted_rows * cfg.vocab_size * cfg.hidden_size
    return gemm + attn + head


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than 32 only where memory or time needs it")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    import torch
    import hymt2sharp_b200
    from hymt2sharp_b200.engine.decode_session import DecodeSession
    from hymt2sharp_b200.engine.engine import StepEntry
    from hymt2sharp_b200.kernels import ops
    from hymt2sharp_b200.sampling import BatchSampler, GREEDY

    pk, pk_source = peaks()
    folder = make_model(args.layers)
    point_batches = [] if args.no_points else [1, 64]
    biggest = max([args.batch] + point_batches)
    per_seq = -(-(PROMPT + warmup + steps + 8) // 64) * 64
    try:
        engine = hymt2sharp_b200.load(folder, dtype="bfloat16", max_tokens=biggest * per_seq + 4096, max_batch=biggest,
                                      max_sequence_tokens=CONTEXT)
    finally:
        shutil.rmtree(folder, ignore_errors=True)   # the weights are on the device now; leave nothing in the temporary folder
    cfg = engine.config
    gen = torch.Generator().manual_seed(1234)
    rand_prompt = lambda: torch.randint(0, cfg.vocab_size, (PROMPT,), generator=gen).tolist()
    ev = lambda: torch.cuda.Event(enable_timing=True)

    # ---- prefill of 2,048 tokens: warm-up, then the mean of 3 timed repetitions -----------------
    prompt = rand_prompt()
    times = []
    for rep in range(3 + 3):
        slot = engine.alloc_slots(1)
        t0, t1 = ev(), ev()
        torch.cuda.synchronize()
        t0.record()
        engine.step([StepEntry(slot[0], prompt, [PROMPT - 1])])
        t1.record()
        torch.cuda.synchronize()
        engine.free_slots(slot)
        if rep >= 3:
            times.append(t0.elapsed_time(t1))
    pf_ms = sum(times) / len(times)
    pf_flops = prefill_flops(cfg, PROMPT, 1)
    prefill = {"value": PROMPT / pf_ms * 1000.0, "tokens": PROMPT, "ms": pf_ms, "reps_ms": [round(t, 3) for t in times],
               "frac": pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), "peak": pk_source}

    # ---- decode ----------------------------------------------------------------------------------
    def decode_run(batch: int, k: int, w: int, sample_clocks: bool):
        slots = engine.alloc_slots(batch)
        prompts = [rand_prompt() for _ in range(batch)]
        firsts = []
        group = max(1, 16384 // PROMPT)  # prompts go in by groups: bounded activation memory
        for g0 in range(0, batch, group):
            entries = [StepEntry(s, p, [PROMPT - 1]) for s, p in zip(slots[g0:g0 + group], prompts[g0:g0 + group])]
            firsts.append(engine.step(entries))
        sampler = BatchSampler([GREEDY] * batch, engine.device)
        first = sampler.sample(torch.cat(firsts), None)
        session = DecodeSession(engine, slots, sampler, first, PROMPT + w + k + 2, use_graph=not args.no_graph)
        for _ in range(w):
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
        mean_ctx = PROMPT + w + (k + 1) / 2.0
        engine.check()
        engine.free_slots(slots)
        return ms, launches, mean_ctx, clk

    ms, launches, mean_ctx, clocks = decode_run(args.batch, steps, warmup, True)
    ms_per_step = ms / steps
    value = args.batch * steps / ms * 1000.0
    step_bytes = engine.model.streamed_weight_bytes() + args.batch * mean_ctx * engine.cache.bytes_per_token() \
        + args.batch * cfg.hidden_size * 2
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "peak_source": pk_source, "bytes_per_step": int(step_bytes)}

    points = {}
    for b in point_batches:
        k = max(8, min(steps, 32))
        pms, _, _, _ = decode_run(b, k, warmup, False)
        points[f"decode_b{b}"] = b * k / pms * 1000.0

    # ---- end to end: Engine.generate, host token ids in and out every step ------------------------
    prompts = [rand_prompt() for _ in range(args.batch)]
    # warm-up of the entry point with the same batch shape: the decode graph of that shape is captured here,
    # as it is once in a serving process, not in the timed run
    engine.generate(prompts, max_new_tokens=4, max_batch=args.batch)
    out = engine.generate(prompts, max_new_tokens=steps + 1, max_batch=args.batch)
    e2e_tokens = out.stats.decode_tokens
    e2e = {"value": e2e_tokens / max(out.stats.decode_ms, 1e-9) * 1000.0, "unit": "tokens/s",
           "h2d_bytes_per_step": 4 * args.batch, "d2h_bytes_per_step": 4 * args.batch,
           "decode_ms": out.stats.decode_ms, "prefill_ms": out.stats.prefill_ms}

    line = {
        "metric": "decode tok/s at batch 8 (1.8B bf16, 2,048-token prompts); prefill tok/s at 2,048 tokens",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random-init weights N(0, 0.02) seed 2",
        "impl": "ours",
        "config": {"model": "hunyuan-dense-1.8B-sizes", "global_batch": args.batch, "seq_len": PROMPT,
                   "context": CONTEXT, "parallelism": "single-gpu", "layers": args.layers, "layers_full": FULL_LAYERS,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "rope_alpha": cfg.rope_alpha, "qk_norm": cfg.use_qk_norm, "tied": cfg.tie_word_embeddings,
                   "cache_block_tokens": engine.cache.block_tokens, "sampling": "greedy on the GPU",
                   "l2": "inputs larger than L2: every step streams all weights (GBs) once"},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "prefill": prefill, "roofline": roofline,
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
