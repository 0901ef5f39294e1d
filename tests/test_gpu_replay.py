"""Trace replay through bin/trace_run against the plain implementation: every request
alone and whole; with its last 32 tokens one by one; and in batches of unequal lengths
whose shorter requests end earlier, one batch after another so that slots and blocks are
used again — in 32-bit and in bfloat16, for every tiny configuration."""
import numpy as np
import pytest

import helpers
from helpers import TraceBuilder

pytestmark = pytest.mark.gpu

# lengths around the cache's block size of 64 and around the 32-key tiles of attention
LENGTHS = [150, 70, 33, 64, 65, 129]
DECODES = [40, 10, 25, 1, 33, 64]   # tokens that each request decodes in the batch mode


def _requests(vocab):
    return [(f"r{i}", helpers.random_tokens(vocab, n, 100 + i)) for i, n in enumerate(LENGTHS)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W", "M", "H", "HW", "S"])
def test_replay_matches_plain(name, dtype, model_dirs, plain_models):
    plain = plain_models(name)
    vocab = plain.cfg.vocab
    reqs = _requests(vocab)
    ref = {rid: plain.logits(toks).numpy() for rid, toks in reqs}

    tb = TraceBuilder()
    for rid, toks in reqs:                       # 1. alone and whole
        tb.whole(rid + "/whole", toks, key=(rid, "whole"))
    for rid, toks in reqs:                       # 2. the last 32 tokens one by one
        tb.tail_one_by_one(rid + "/tail", toks, 32, key=(rid, "tail"))
    for lo in (0, 3):                            # 3. two batches of three, the second in the first's slots
        group = [(rid + "/batch", toks, DECODES[lo + i]) for i, (rid, toks) in enumerate(reqs[lo:lo + 3])]
        tb.batch(group, keys={rid + "/batch": (rid, "batch") for rid, _ in reqs})
    # the cache is just large enough for the largest batch: 192 + 128 + 64 tokens in blocks of 64
    out = tb.collect(helpers.run_trace(model_dirs(name), dtype, tb.steps, max_tokens=384, vocab=vocab))

    for rid, toks in reqs:
        by_mode = {}
        for mode in ("whole", "tail", "batch"):
            rows = out[(rid, mode)]
            assert sorted(rows) == list(range(len(toks))), f"{rid} {mode}: positions {sorted(rows)[:5]}..."
            got = np.stack([rows[p][0] for p in range(len(toks))])
            by_mode[mode] = got
            helpers.assert_close(got, ref[rid], dtype, f"{name} {dtype} {rid} {mode}")
        # the ways of cutting agree with each other at least as well as with the plain model
        helpers.assert_close(by_mode["tail"], by_mode["whole"], dtype, f"{name} {dtype} {rid} tail vs whole")
        helpers.assert_close(by_mode["batch"], by_mode["whole"], dtype, f"{name} {dtype} {rid} batch vs whole")


def test_replay_with_chunked_prompt_and_idle_steps(model_dirs, plain_models):
    """A prompt cut into uneven pieces, steps that want nothing, and an entry with an empty
    want list: the logits of a position do not depend on the cut."""
    plain = plain_models("B")
    toks = helpers.random_tokens(plain.cfg.vocab, 200, 9)
    ref = plain.logits(toks).numpy()
    tb = TraceBuilder()
    pos = 0
    for n, want in ((1, []), (62, [0, 61]), (2, [0, 1]), (100, list(range(100))), (35, [34])):
        tb.add([("x", toks[pos:pos + n], pos, want)], ["x"] if pos + n == 200 else [])
        pos += n
    outputs = helpers.run_trace(model_dirs("B"), "float32", tb.steps, max_tokens=256, vocab=plain.cfg.vocab)
    assert 0 not in outputs  # nothing wanted, no file
    got = tb.collect(outputs)["x"]
    for p, rows in got.items():
        helpers.assert_close(rows[0][None], ref[p][None], "float32", f"chunked position {p}")
    assert sorted(got) == [1, 62, 63, 64] + list(range(65, 165)) + [199]
