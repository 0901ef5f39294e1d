"""Shared pieces of the tests: the tiny configurations, model folders, replay of traces
through bin/trace_run, and the tolerances."""
from __future__ import annotations

import json
import os
import subprocess
import sys
import shutil
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ARCH = "HunYuanDenseV1ForCausalLM"

# Two tiny configurations that differ in every size and option, and a third with a window.
CONFIGS = {
    # 2 kv groups, q width == hidden, no NTK scaling, qk-norm, tied head, even vocabulary
    "A": dict(config=dict(architectures=[ARCH], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                          num_key_value_heads=2, head_dim=16, intermediate_size=160, vocab_size=256,
                          rope_theta=10000.0, rope_scaling={"type": "dynamic", "alpha": 1.0}, rms_norm_eps=1e-5,
                          use_qk_norm=True, tie_word_embeddings=True, max_position_embeddings=4096),
              seed=0, sigma=0.02, gain_dtype="bfloat16"),
    # one kv head for 6 heads, q width 192 != hidden 96, NTK alpha 1000, no qk-norm, own head, odd vocabulary,
    # norm gains stored in 32-bit
    "B": dict(config=dict(architectures=[ARCH], num_hidden_layers=3, hidden_size=96, num_attention_heads=6,
                          num_key_value_heads=1, head_dim=32, intermediate_size=224, vocab_size=509,
                          rope_theta=1e6, rope_scaling={"type": "dynamic", "alpha": 1000.0}, rms_norm_eps=1e-6,
                          use_qk_norm=False, tie_word_embeddings=False, max_position_embeddings=2048),
              seed=1, sigma=0.05, gain_dtype="float32"),
    # a window of 40 positions, partial rotation (rope_dim 16 of 48), 3 heads per kv head
    "W": dict(config=dict(architectures=[ARCH], num_hidden_layers=2, hidden_size=80, num_attention_heads=6,
                          num_key_value_heads=2, head_dim=48, intermediate_size=112, vocab_size=131,
                          rope_theta=5000.0, rope_dim=16, rms_norm_eps=1e-5, use_qk_norm=True,
                          tie_word_embeddings=True, sliding_window=40, max_position_embeddings=1024),
              seed=2, sigma=0.04, gain_dtype="bfloat16"),
    # head_dim 64 with 4 heads per kv head: the bfloat16 engine runs its tensor-core attention kernels
    # (prompt and decode) on this one; the sizes above stay with the general kernels
    "M": dict(config=dict(architectures=[ARCH], num_hidden_layers=2, hidden_size=192, num_attention_heads=8,
                          num_key_value_heads=2, head_dim=64, intermediate_size=328, vocab_size=1003,
                          rope_theta=10000.0, rope_scaling={"type": "dynamic", "alpha": 1000.0}, rms_norm_eps=1e-5,
                          use_qk_norm=True, tie_word_embeddings=True, max_position_embeddings=4096),
              seed=3, sigma=0.03, gain_dtype="bfloat16"),
    # head_dim 128, the head size of the full-size models, with 2 heads per kv head and a q width (512) wider than
    # the hidden size: the bfloat16 engine runs every tcgen05 kernel on this one (projection with rotation and
    # cache append in its epilogue, decode attention with keys on the 128-row side, prompt attention, split-K products)
    "H": dict(config=dict(architectures=[ARCH], num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
                          num_key_value_heads=2, head_dim=128, intermediate_size=392, vocab_size=777,
                          rope_theta=50000.0, rope_scaling={"type": "dynamic", "alpha": 4.0}, rms_norm_eps=1e-5,
                          use_qk_norm=True, tie_word_embeddings=False, max_position_embeddings=4096),
              seed=4, sigma=0.03, gain_dtype="bfloat16"),
    # H with a window of 100 positions: the cache hands blocks back while a sequence grows, so the tcgen05
    # attention kernels meet block tables with -1 entries below the oldest visible key
    "HW": dict(config=dict(architectures=[ARCH], num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=128, intermediate_size=392, vocab_size=777,
                           rope_theta=50000.0, rope_scaling={"type": "dynamic", "alpha": 4.0}, rms_norm_eps=1e-5,
                           use_qk_norm=True, tie_word_embeddings=False, sliding_window=100,
                           max_position_embeddings=4096),
               seed=5, sigma=0.03, gain_dtype="bfloat16"),
    # heads of 24: a multiple of 8 that is no multiple of 16, three heads on one kv head, odd sizes all round
    "S": dict(config=dict(architectures=[ARCH], num_hidden_layers=2, hidden_size=88, num_attention_heads=3,
                          num_key_value_heads=1, head_dim=24, intermediate_size=136, vocab_size=301,
                          rope_theta=20000.0, rms_norm_eps=1e-6, use_qk_norm=True,
                          tie_word_embeddings=True, max_position_embeddings=2048),
              seed=6, sigma=0.05, gain_dtype="float32"),
}

# Tolerances, fixed before the kernels were tuned.  32-bit: differences come from the order of
# float32 sums only.  bfloat16: activations, keys and values are rounded to 8 bits of mantissa
# (2^-9 relative) a few dozen times on the way to the logits.
TOL = {"float32": dict(max_rel=2e-5, rms_rel=5e-6), "bfloat16": dict(max_rel=4e-2, rms_rel=1.5e-2)}


def make_model_dir(folder: str, name: str) -> str:
    import torch
    from hymt2sharp_b200.config import HunyuanDenseConfig
    from hymt2sharp_b200.weights import write_random_model
    spec = CONFIGS[name]
    cfg = HunyuanDenseConfig.from_dict(spec["config"])
    write_random_model(folder, cfg, spec["seed"], spec["sigma"], gain_dtype=getattr(torch, spec["gain_dtype"]))
    return folder


def random_tokens(vocab: int, n: int, seed: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def assert_close(got: np.ndarray, ref: np.ndarray, dtype: str, what: str = "", factor: float = 1.0) -> None:
    tol = TOL[dtype]
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    scale = np.abs(ref).max()
    rms_ref = np.sqrt((ref ** 2).mean())
    err = np.abs(got - ref)
    worst = np.unravel_index(err.argmax(), err.shape)
    assert err.max() <= factor * tol["max_rel"] * scale, \
        f"{what}: max error {err.max():.3e} at {worst} exceeds {factor * tol['max_rel']:.1e} x {scale:.3f}"
    rms = np.sqrt((err ** 2).mean())
    assert rms <= factor * tol["rms_rel"] * rms_ref, f"{what}: rms error {rms:.3e} exceeds {factor * tol['rms_rel']:.1e} x {rms_ref:.3f}"


def run_trace(model_dir: str, dtype: str, steps: list, max_tokens: int, vocab: int, timeout: int = 600) -> dict:
    """Runs bin/trace_run on `steps` from another working folder; returns {step: logits [wanted, vocab]}."""
    out_dir = tempfile.mkdtemp(prefix="trace_out_")
    text = "".join(json.dumps(s) + "\n" for s in steps)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    try:
        r = subprocess.run(cmd, input=text, capture_output=True, text=True, cwd=tempfile.gettempdir(), timeout=timeout)
        assert r.returncode == 0, f"trace_run failed ({r.returncode}):\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
        done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
        assert [l.split()[1] for l in done] == [str(s["step"]) for s in steps], "a 'done <step>' line is missing"
        result = {}
        for s in steps:
            wanted = sum(len(e.get("want", [])) for e in s["entries"])
            path = os.path.join(out_dir, f"{s['step']}.f32")
            if wanted:
                result[s["step"]] = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
            else:
                assert not os.path.exists(path)
        return result
    finally:
        shutil.rmtree(out_dir, ignore_errors=True)


class TraceBuilder:
    """Builds replay steps and remembers which (request, position) each wanted row is."""

    def __init__(self):
        self.steps = []
        self.rows = {}  # step -> [(request key, position)]

    def add(self, entries: list, end: list, keys: dict | None = None) -> None:
        """entries: [(id, tokens, first position, want positions-in-entry)]"""
        step = len(self.steps)
        rows = []
        recs = []
        for rid, toks, pos0, want in entries:
            recs.append({"id": rid, "tokens": list(toks), "want": list(want)})
            rows += [((keys or {}).get(rid, rid), pos0 + w) for w in want]
        self.steps.append({"step": step, "entries": recs, "end": list(end)})
        self.rows[step] = rows

    def whole(self, rid: str, tokens: list, key=None) -> None:
        self.add([(rid, tokens, 0, range(len(tokens)))], [rid], {rid: key or rid})

    def tail_one_by_one(self, rid: str, tokens: list, tail: int = 32, key=None) -> None:
        n = len(tokens) - tail
        assert n >= 1
        keys = {rid: key or rid}
        self.add([(rid, tokens[:n], 0, range(n))], [], keys)
        for i in range(n, len(tokens)):
            self.add([(rid, [tokens[i]], i, [0])], [rid] if i == len(tokens) - 1 else [], keys)

    def batch(self, requests: list, keys: dict | None = None) -> None:
        """requests: [(id, tokens, decode count)]: the prompts (all but the last `decode count`
        tokens) start together in one step, then every request goes on by one token a step
        and ends when its tokens are used up."""
        first = [(rid, toks[:len(toks) - d], 0, range(len(toks) - d)) for rid, toks, d in requests]
        self.add(first, [rid for rid, toks, d in requests if d == 0], keys)
        for s in range(1, max(d for _, _, d in requests) + 1):
            entries, end = [], []
            for rid, toks, d in requests:
                if d >= s:
                    pos = len(toks) - d + s - 1
                    entries.append((rid, [toks[pos]], pos, [0]))
                    if d == s:
                        end.append(rid)
            self.add(entries, end, keys)

    def collect(self, outputs: dict) -> dict:
        """{request key: {position: logits row}} from run_trace's outputs."""
        got = {}
        for step, rows in self.rows.items():
            if not rows:
                continue
            arr = outputs[step]
            assert arr.shape[0] == len(rows)
            for (key, pos), row in zip(rows, arr):
                got.setdefault(key, {}).setdefault(pos, []).append(row)
        return got
