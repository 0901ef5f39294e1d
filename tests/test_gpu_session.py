"""The decode session (the path that generation and the benchmark run: a captured CUDA graph,
positions moved on the device, ended rows turned into padding) checked on LOGITS against the
plain model, and the engine's truncate.

Given tokens are fed through DecodeSession.step_host, and the logits that the captured step left
in its buffer are read after every step.  The schedule crosses what the eager replay tests do not:
a length bound of 2,048 positions over sequences that start at 20 tokens; the block tables growing
in mid-session (the graph is captured again); rows that end at step 5 and at step 600 and stay in the
batch as padding; a second session of the same shape in the freed slots on the kept graph; a third
after the slot tables grew.
"""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def _prefill(eng, slots, seqs, prompt_lens, plain, dtype, what):
    from hymt2sharp_b200.engine.engine import StepEntry
    out = eng.step([StepEntry(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, prompt_lens)]).cpu().numpy()
    o = 0
    for i, n in enumerate(prompt_lens):
        helpers.assert_close(out[o:o + n], plain.logits(seqs[i][:n]).numpy(), dtype, f"{what} prompt {i}")
        o += n


def _decode(eng, slots, seqs, prompt_lens, steps_of, max_total_len):
    """Feeds seqs[r][prompt_lens[r] + s] to row r at step s, for steps_of[r] steps; row r is dropped after its
    last step.  Returns ({row: [logits of each step]}, the session)."""
    from hymt2sharp_b200.engine.decode_session import DecodeSession
    from hymt2sharp_b200.sampling import BatchSampler, GREEDY
    rows = len(slots)
    sampler = BatchSampler([GREEDY] * rows, eng.device)
    first = torch.tensor([seqs[r][prompt_lens[r]] for r in range(rows)], dtype=torch.int32, device=eng.device)
    session = DecodeSession(eng, slots, sampler, first, max_total_len, use_graph=True)
    assert session.use_graph
    got = {r: [] for r in range(rows)}
    for s in range(max(steps_of)):
        live = [r for r in range(rows) if steps_of[r] > s]
        session.step_host({r: seqs[r][prompt_lens[r] + s] for r in live})
        logits = session.buf.logits.cpu().numpy()
        for r in live:
            got[r].append(logits[r])
        session.drop([r for r in live if steps_of[r] == s + 1])
    return got, session


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "H", "HW"])
def test_decode_session_logits_over_a_long_run_with_rows_that_end(name, dtype, model_dirs, plain_models):
    from hymt2sharp_b200.engine.engine import Engine
    plain = plain_models(name)
    vocab = plain.cfg.vocab
    eng = Engine(model_dirs(name), dtype=dtype, max_tokens=4096, max_batch=3)
    for s in eng.cache.storage:
        s.fill_(float("nan"))          # a row read before it was written shows

    # ---- first session: 1,110 steps; rows end at steps 5 and 600 ---------------------------------
    prompt_lens, steps_of = [20, 7, 33], [1110, 5, 600]
    seqs = [helpers.random_tokens(vocab, p + d, 300 + i) for i, (p, d) in enumerate(zip(prompt_lens, steps_of))]
    slots = eng.alloc_slots(3)
    _prefill(eng, slots, seqs, prompt_lens, plain, dtype, f"{name} {dtype} session 1")
    layout_before = eng.cache.layout_version
    got, session = _decode(eng, slots, seqs, prompt_lens, steps_of, 1140)
    eng.check()
    assert session.max_total_len == 2048                       # the bound that the captured kernels were given
    assert eng.cache.layout_version > layout_before           # the tables grew under the session: captured again
    for r in range(3):
        ref = plain.logits(seqs[r]).numpy()[prompt_lens[r]:]
        helpers.assert_close(np.stack(got[r]), ref, dtype, f"{name} {dtype} session 1 row {r}")
    eng.cache.book.audit()
    assert eng.cache.free_tokens() == eng.cache.num_blocks * 64      # every row gave its slot and blocks back
    first_graph = session.buf.graph

    # ---- second session, same shape, in the freed slots: the kept graph replays at once -----------
    prompt_lens, steps_of = [64, 1, 130], [40, 40, 3]
    seqs = [helpers.random_tokens(vocab, p + d, 400 + i) for i, (p, d) in enumerate(zip(prompt_lens, steps_of))]
    slots = eng.alloc_slots(3)
    assert sorted(slots) == [0, 1, 2]
    _prefill(eng, slots, seqs, prompt_lens, plain, dtype, f"{name} {dtype} session 2")
    got, session = _decode(eng, slots, seqs, prompt_lens, steps_of, 1140)
    eng.check()
    assert session.buf.graph is first_graph
    for r in range(3):
        ref = plain.logits(seqs[r]).numpy()[prompt_lens[r]:]
        helpers.assert_close(np.stack(got[r]), ref, dtype, f"{name} {dtype} session 2 row {r}")

    # ---- more slots than the engine was made for: the tables are replaced, the graph is captured again
    layout_before = eng.cache.layout_version
    extra = eng.alloc_slots(6)
    assert eng.cache.layout_version > layout_before
    eng.free_slots(extra)
    prompt_lens, steps_of = [3, 90, 65], [30, 2, 30]
    seqs = [helpers.random_tokens(vocab, p + d, 500 + i) for i, (p, d) in enumerate(zip(prompt_lens, steps_of))]
    slots = eng.alloc_slots(3)
    _prefill(eng, slots, seqs, prompt_lens, plain, dtype, f"{name} {dtype} session 3")
    got, session = _decode(eng, slots, seqs, prompt_lens, steps_of, 1140)
    eng.check()
    assert session.buf.graph_layout == eng.cache.layout_version
    for r in range(3):
        ref = plain.logits(seqs[r]).numpy()[prompt_lens[r]:]
        helpers.assert_close(np.stack(got[r]), ref, dtype, f"{name} {dtype} session 3 row {r}")
    eng.cache.book.audit()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "H"])
def test_truncate_then_another_continuation(name, dtype, model_dirs, plain_models):
    """200 tokens, back to 130, then other tokens from there (src/HyMT2Sharp/HunyuanDenseModel.cs:187-240):
    the logits are those of the sequence that was never longer, in 32-bit bit for bit."""
    from hymt2sharp_b200.engine.engine import Engine, StepEntry
    plain = plain_models(name)
    vocab = plain.cfg.vocab
    a = helpers.random_tokens(vocab, 200, 61)
    b = a[:130] + helpers.random_tokens(vocab, 75, 62)
    eng = Engine(model_dirs(name), dtype=dtype, max_tokens=512, max_batch=2)
    slot = eng.alloc_slots(1)[0]
    eng.step([StepEntry(slot, a, [199])])
    free_before = eng.cache.free_tokens()
    eng.truncate(slot, 130)
    assert eng.length(slot) == 130 and eng.cache.free_tokens() == free_before + 64    # the block of 192..255 came back
    got = [eng.step([StepEntry(slot, b[130:170], list(range(40)))])]
    got += [eng.step([StepEntry(slot, [t], [0])]) for t in b[170:]]                 # 35 tokens one by one
    got = torch.cat(got).cpu().numpy()
    eng.check()
    helpers.assert_close(got, plain.logits(b).numpy()[130:], dtype, f"{name} {dtype} after truncate")
    # a fresh run of the same cut: the cache rows that the longer sequence left behind change nothing
    other = eng.alloc_slots(1)[0]
    eng.step([StepEntry(other, b[:130], [])])
    fresh = [eng.step([StepEntry(other, b[130:170], list(range(40)))])]
    fresh += [eng.step([StepEntry(other, [t], [0])]) for t in b[170:]]
    fresh = torch.cat(fresh).cpu().numpy()
    if dtype == "float32":
        assert np.array_equal(got, fresh)
    else:
        helpers.assert_close(got, fresh, dtype, "truncated against fresh")
    eng.reset(slot)
    assert eng.length(slot) == 0
    again = eng.step([StepEntry(slot, b[:50], [49])]).cpu().numpy()
    helpers.assert_close(again, plain.logits(b[:50]).numpy()[49:], dtype, "after reset")
    eng.free_slots([slot, other])
    eng.cache.book.audit()


def test_truncate_below_what_a_window_group_still_holds_is_refused(model_dirs):
    from hymt2sharp_b200.cache import CacheError
    from hymt2sharp_b200.engine.engine import Engine, StepEntry
    eng = Engine(model_dirs("W"), dtype="float32", max_tokens=512, max_batch=2)
    slot = eng.alloc_slots(1)[0]
    eng.step([StepEntry(slot, helpers.random_tokens(131, 200, 3), [])])
    with pytest.raises(CacheError):
        eng.truncate(slot, 100)            # the window of 40 has let go of the block that position 61.. lies in
    assert eng.length(slot) == 200
    eng.truncate(slot, 190)                # within what is still held
    assert eng.length(slot) == 190
    eng.cache.book.audit()


def test_a_sequence_past_the_models_positions_is_refused(model_dirs):
    from hymt2sharp_b200.engine.engine import Engine, EngineError, StepEntry
    eng = Engine(model_dirs("W"), dtype="float32", max_tokens=2048, max_batch=2)   # max_position_embeddings 1024
    slot = eng.alloc_slots(1)[0]
    eng.step([StepEntry(slot, [1] * 1000, [])])
    with pytest.raises(EngineError, match="max_position_embeddings"):
        eng.step([StepEntry(slot, [1] * 25, [])])
    assert eng.length(slot) == 1000
    eng.step([StepEntry(slot, [1] * 24, [23])])
    with pytest.raises(ValueError, match="max_position_embeddings"):
        eng.generate([[1] * 1000], max_new_tokens=30)
