"""Checks that the logits of a position do not depend on how the work was cut, at any model size.

The same requests are run through the engine in the three ways of the trace replay: every
request alone and whole; with its last 32 tokens one by one; and as a batch of unequal lengths
whose shorter requests end earlier, followed by a second batch in the slots and blocks that the
first gave back.  The logits of every (request, position) are kept on the device and compared:
every way of cutting against "whole", the bfloat16 engine against the 32-bit engine, and the
32-bit engine against a reference implementation that the caller brings (a callable from token
ids to logits [tokens, vocab]).  The figures are those of sdcb/HyMT2Sharp's own checks
(src/HyMT2Sharp.Benchmark/Program.cs:124-145 `--verify-prefill`: largest difference, RMS and both
top-1; :147-177 `--verify-decode`: per-step difference and top-1 agreement).
"""
from __future__ import annotations

import torch

from .engine import Engine, StepEntry

# relative to the largest |logit| of the reference (max) and to its RMS (rms).  32-bit: only the order of float32
# sums differs.  bfloat16: activations, keys and values carry 8 bits of mantissa.
TOLERANCE = {"float32": dict(max_rel=2e-5, rms_rel=5e-6), "bfloat16": dict(max_rel=4e-2, rms_rel=1.5e-2)}
TAIL = 32


def compare(got: torch.Tensor, ref: torch.Tensor) -> dict:
    """Largest difference, RMS of the difference, the same two relative to the reference's largest value and RMS,
    and the share of rows whose largest logit sits at the same index."""
    got, ref = got.double(), ref.double().to(got.device)
    diff = (got - ref).abs()
    scale, rms_ref = float(ref.abs().max()), float(ref.pow(2).mean().sqrt())
    rms = float(diff.pow(2).mean().sqrt())
    return {"max_abs": float(diff.max()), "rms": rms, "max_rel": float(diff.max()) / max(scale, 1e-30),
            "rms_rel": rms / max(rms_ref, 1e-30), "top1": float((got.argmax(-1) == ref.argmax(-1)).double().mean()),
            "rows": int(got.shape[0]), "finite": bool(torch.isfinite(got).all())}


def within(stats: dict, dtype: str, factor: float = 1.0) -> bool:
    tol = TOLERANCE[dtype]
    return stats["finite"] and stats["max_rel"] <= factor * tol["max_rel"] and stats["rms_rel"] <= factor * tol["rms_rel"]


def run_cuts(engine: Engine, requests: list, decodes: list, second_decodes: list) -> dict:
    """{"whole" | "tail" | "batch" | "batch2": [logits [len, vocab] of every request]}.  `decodes[i]` tokens of
    request i are decoded one by one in the first batch, `second_decodes[i]` in the second (which takes the
    requests in reverse order)."""
    n = len(requests)
    out = {}
    # 1. alone and whole
    rows = []
    for toks in requests:
        slot = engine.alloc_slots(1)
        rows.append(engine.step([StepEntry(slot[0], toks, list(range(len(toks))))]))
        engine.free_slots(slot)
    out["whole"] = rows
    # 2. the last TAIL tokens one by one
    rows = []
    for toks in requests:
        slot = engine.alloc_slots(1)
        cut = max(1, len(toks) - TAIL)
        parts = [engine.step([StepEntry(slot[0], toks[:cut], list(range(cut)))])]
        parts += [engine.step([StepEntry(slot[0], [t], [0])]) for t in toks[cut:]]
        engine.free_slots(slot)
        rows.append(torch.cat(parts))
    out["tail"] = rows
    # 3. unequal batches: prompts together, then one token each; a request that has used up its tokens ends and
    #    gives its slot back while the others go on; the second batch starts in what the first gave back
    for name, order, dec in (("batch", list(range(n)), decodes), ("batch2", list(range(n - 1, -1, -1)), second_decodes)):
        slots = dict(zip(order, engine.alloc_slots(n)))
        cut = {i: len(requests[i]) - min(dec[i], len(requests[i]) - 1) for i in order}
        first = engine.step([StepEntry(slots[i], requests[i][:cut[i]], list(range(cut[i]))) for i in order])
        parts, o = {}, 0
        for i in order:
            parts[i] = [first[o:o + cut[i]]]
            o += cut[i]
        step = 0
        while True:
            live = [i for i in order if cut[i] + step < len(requests[i])]
            if not live:
                break
            lg = engine.step([StepEntry(slots[i], [requests[i][cut[i] + step]], [0]) for i in live])
            for r, i in enumerate(live):
                parts[i].append(lg[r:r + 1])
            step += 1
            ended = [i for i in live if cut[i] + step >= len(requests[i])]
            engine.free_slots([slots[i] for i in ended])
        never_decoded = [i for i in order if cut[i] >= len(requests[i])]
        engine.free_slots([slots[i] for i in never_decoded])
        out[name] = [torch.cat(parts[i]) for i in range(n)]
    engine.check()
    engine.cache.book.audit()
    return out


def verify_split(model_dir: str, requests: list, dtypes=("float32", "bfloat16"), reference=None,
                 decodes=None, second_decodes=None, device="cuda:0") -> dict:
    """Runs `requests` (lists of token ids) through an engine of every dtype in every cut and compares.
    Returns {"cuts": {dtype: {cut: stats vs whole}}, "bfloat16_vs_float32": {cut: stats},
    "float32_vs_reference": stats, "ok": bool}; `reference(tokens) -> [len, vocab]` is optional."""
    n = len(requests)
    decodes = decodes or [(40, 10, 25, 1, 33, 64)[i % 6] for i in range(n)]
    second_decodes = second_decodes or [(5, 30, 64, 12, 1, 40)[i % 6] for i in range(n)]
    # the cache is exactly as large as the largest batch needs: no spare block hides a leak
    capacity = sum(-(-len(r) // 64) * 64 for r in requests)
    result = {"cuts": {}, "ok": True, "requests": [len(r) for r in requests]}
    logits = {}
    for dtype in dtypes:
        engine = Engine(model_dir, dtype=dtype, max_tokens=capacity, max_batch=n, device=device)
        cuts = run_cuts(engine, requests, decodes, second_decodes)
        logits[dtype] = cuts
        whole = torch.cat(cuts["whole"])
        result["cuts"][dtype] = {}
        for name in ("tail", "batch", "batch2"):
            st = compare(torch.cat(cuts[name]), whole)
            st["within"] = within(st, dtype)
            result["cuts"][dtype][name] = st
            result["ok"] &= st["within"]
        del engine
        torch.cuda.empty_cache()
    if "float32" in logits and "bfloat16" in logits:
        result["bfloat16_vs_float32"] = {}
        for name in ("whole", "tail", "batch", "batch2"):
            st = compare(torch.cat(logits["bfloat16"][name]), torch.cat(logits["float32"][name]))
            st["within"] = within(st, "bfloat16")
            result["bfloat16_vs_float32"][name] = st
            result["ok"] &= st["within"]
    if reference is not None and "float32" in logits:
        ref = torch.cat([torch.as_tensor(reference(r)).to(torch.float32) for r in requests])
        st = compare(torch.cat(logits["float32"]["whole"]), ref)
        st["within"] = within(st, "float32")
        result["float32_vs_reference"] = st
        result["ok"] &= st["within"]
    return result
