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
