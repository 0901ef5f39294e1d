"""Logits at the widths of the full-size model (hidden 2,048, heads of 128, intermediate 6,144, a
vocabulary of 120,818, NTK alpha 1,000, tied head) with two layers: the 32-bit engine against the
plain implementation, the bfloat16 engine against the 32-bit one, and every way of cutting the work
against the whole run.  The function is the one that `bench.py --verify-split` runs at 32 layers."""
import shutil

import pytest

pytestmark = pytest.mark.gpu


def test_logits_at_full_widths_in_every_cut_and_precision():
    import numpy as np
    import bench
    from hymt2sharp_b200.engine.verify import TOLERANCE, verify_split
    from plain.hunyuan_plain import PlainModel
    import helpers
    assert TOLERANCE == helpers.TOL            # the product's figures are judged by the tests' tolerances
    folder = bench.make_model("1p8b", 2)
    try:
        plain = PlainModel(folder)
        rng = np.random.default_rng(11)
        requests = [rng.integers(0, plain.cfg.vocab, n).tolist() for n in (300, 70, 520)]
        res = verify_split(folder, requests, reference=lambda toks: plain.logits(toks))
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    for dtype, cuts in res["cuts"].items():
        for cut, st in cuts.items():
            assert st["within"], f"{dtype} {cut} against whole: {st}"
    # (not bit for bit: past 256 keys a decode step cuts the keys into chunks and folds their partial sums, a prompt's
    # step walks them in one running sum; the difference is the order of float32 additions and nothing else)
    assert all(st["top1"] == 1.0 for st in res["cuts"]["float32"].values()), res["cuts"]["float32"]
    for cut, st in res["bfloat16_vs_float32"].items():
        assert st["within"], f"bfloat16 against 32-bit, {cut}: {st}"
    assert res["float32_vs_reference"]["within"], res["float32_vs_reference"]
    assert res["ok"]


def test_a_long_prompt_gives_the_same_bits_whatever_else_is_in_the_step():
    """bfloat16, the real widths, two layers: a prompt of more than 128 tokens alone and the same prompt in a step with two
    others.  The tile widths of the products differ between the two steps (they depend on the step's tokens), the sums
    that a logit is made of do not: equal bit for bit.  (A difference in the last bit of one sum of squares once
    spread, through the roundings to bfloat16 behind it, to every logit within two layers.)"""
    import numpy as np
    import torch
    import bench
    from hymt2sharp_b200.engine.engine import Engine, StepEntry
    folder = bench.make_model("1p8b", 2)
    try:
        rng = np.random.default_rng(5)
        lens = (300, 70, 1100)
        reqs = [rng.integers(0, 120818, n).tolist() for n in lens]
        engine = Engine(folder, dtype="bfloat16", max_tokens=sum(-(-n // 64) * 64 for n in lens) + 64, max_batch=3)
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    alone = []
    for toks in reqs:
        slot = engine.alloc_slots(1)
        alone.append(engine.step([StepEntry(slot[0], toks, list(range(len(toks))))]).clone())
        engine.free_slots(slot)
    slots = engine.alloc_slots(3)
    together = engine.step([StepEntry(s, toks, list(range(len(toks)))) for s, toks in zip(slots, reqs)])
    engine.free_slots(slots)
    engine.check()
    assert torch.equal(together[:300], alone[0])
    assert torch.equal(together[370:], alone[2])
    # the prompt of 70 tokens runs through the kernels for few tokens when it is alone (K cut into splits that are folded):
    # another order of float32 additions, and bfloat16 roundings behind it
    diff = (together[300:370].float() - alone[1].float()).abs()
    assert float(diff.max()) <= 4e-2 * float(alone[1].float().abs().max())
