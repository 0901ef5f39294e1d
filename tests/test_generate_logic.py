"""The generation loop's decisions, without a GPU: a scripted stepper stands in for the device."""
import pytest

from hymt2sharp_b200.engine.generate import (BatchState, GenerationStats, plan_batches, run_batch)


class ScriptedStepper:
    """Gives every sequence its scripted tokens; records what the loop asks of the device."""

    def __init__(self, scripts):
        self.scripts = scripts
        self.cursor = [0] * len(scripts)
        self.calls = []
        self.released = []
        self.closed = False

    def _next(self, rows):
        out = []
        for r in rows:
            out.append(self.scripts[r][self.cursor[r]])
            self.cursor[r] += 1
        return out

    def prefill(self):
        self.calls.append(("prefill", list(range(len(self.scripts)))))
        return self._next(range(len(self.scripts)))

    def decode(self, rows, tokens):
        self.calls.append(("decode", list(rows), list(tokens)))
        return self._next(rows)

    def release(self, rows):
        self.released += list(rows)

    def close(self):
        self.closed = True


def test_stop_token_is_not_kept_and_others_go_on():
    scripts = [[5, 6, 99, 1, 1], [7, 99, 1, 1, 1], [8, 9, 10, 11, 12]]
    stepper = ScriptedStepper(scripts)
    state = BatchState(["a", "b", "c"], [3, 4, 5], max_new_tokens=4, stop_token_ids=[99])
    stats = GenerationStats()
    seen = []
    run_batch(stepper, state, stats, on_tokens=seen.extend, clock=lambda: 0.0)
    res = state.results()
    assert [r.tokens for r in res] == [[5, 6], [7], [8, 9, 10, 11]]
    assert [r.finish_reason for r in res] == ["stop", "stop", "length"]
    # the batch shrinks: b leaves after step 1, a after step 2; each step feeds the last kept tokens
    assert stepper.calls == [("prefill", [0, 1, 2]), ("decode", [0, 1, 2], [5, 7, 8]),
                             ("decode", [0, 2], [6, 9]), ("decode", [2], [10])]
    assert stepper.released == [1, 0, 2] and stepper.closed
    assert stats.prefill_tokens == 12 and stats.decode_steps == 3 and stats.decode_tokens == 6
    assert seen == [("a", 5), ("b", 7), ("c", 8), ("a", 6), ("c", 9), ("c", 10), ("c", 11)]


def test_first_token_can_stop_and_limits():
    stepper = ScriptedStepper([[99], [4, 5]])
    state = BatchState([0, 1], [2, 2], max_new_tokens=1, stop_token_ids={99})
    run_batch(stepper, state, GenerationStats())
    assert [r.tokens for r in state.results()] == [[], [4]]
    assert [r.finish_reason for r in state.results()] == ["stop", "length"]
    assert stepper.calls == [("prefill", [0, 1])]  # one token each needs no decode step
    zero = BatchState([0], [2], max_new_tokens=0, stop_token_ids=())
    s2 = ScriptedStepper([[1]])
    run_batch(s2, zero, GenerationStats())
    assert zero.results()[0].tokens == [] and s2.calls == [] and s2.closed


def test_stepper_is_closed_when_a_step_fails():
    class Failing(ScriptedStepper):
        def decode(self, rows, tokens):
            raise RuntimeError("device fault")
    stepper = Failing([[1, 2]])
    with pytest.raises(RuntimeError):
        run_batch(stepper, BatchState([0], [1], 5, ()), GenerationStats())
    assert stepper.closed


def test_accept_needs_one_token_per_live_row():
    state = BatchState([0, 1], [1, 1], 3, ())
    with pytest.raises(ValueError):
        state.accept([1])


def test_plan_batches():
    # 5 requests, batches of at most 2, enough cache: in order
    assert plan_batches([10, 20, 30, 40, 50], 16, 2, 64 * 100, 64) == [[0, 1], [2, 3], [4]]
    # the cache bounds a batch: 100+28 tokens = 2 blocks each, 5 blocks in all
    assert plan_batches([100, 100, 100], 29, 8, 64 * 5, 64) == [[0, 1], [2]]
    # a prompt that ends exactly at a block's end needs the next block only for its second token
    assert plan_batches([64, 64], 1, 8, 64 * 2, 64) == [[0, 1]]
    assert plan_batches([64, 64], 2, 8, 64 * 2, 64) == [[0], [1]]
    with pytest.raises(ValueError):
        plan_batches([1000], 100, 8, 64 * 4, 64)
    with pytest.raises(ValueError):
        plan_batches([0], 1, 8, 64 * 4, 64)
    assert plan_batches([], 5, 8, 640, 64) == []


class AheadStepper(ScriptedStepper):
    """A stepper that can run a step ahead of the host: launch() starts a step, collect() hands over the oldest one's tokens."""

    def __init__(self, scripts):
        super().__init__(scripts)
        self.flying = []
        self.most_in_flight = 0

    def launch(self, rows):
        self.calls.append(("launch", list(rows)))
        self.flying.append(self._next(rows))
        self.most_in_flight = max(self.most_in_flight, len(self.flying))

    def collect(self):
        self.calls.append(("collect",))
        return self.flying.pop(0)


def test_a_step_ahead_gives_the_same_tokens_and_reasons():
    """With a step in flight beyond the one the host looks at, a stop token is seen one launch late: the extra token is
    dropped, the row leaves with the next launch; a row at its limit leaves at once.  Results are those of the waiting loop."""
    scripts = [[5, 6, 99, 41, 42], [7, 99, 43, 44, 45], [8, 9, 10, 11, 12]]
    waiting, ahead = ScriptedStepper(scripts), AheadStepper(scripts)
    results, streams = [], []
    for stepper in (waiting, ahead):
        state = BatchState(["a", "b", "c"], [3, 4, 5], max_new_tokens=4, stop_token_ids=[99])
        stats = GenerationStats()
        seen = []
        run_batch(stepper, state, stats, on_tokens=seen.extend, clock=lambda: 0.0)
        results.append([(r.tokens, r.finish_reason) for r in state.results()])
        streams.append(seen)
        assert stats.decode_steps == 3 and stats.decode_tokens == 6 and stepper.closed
    assert results[0] == results[1] == [([5, 6], "stop"), ([7], "stop"), ([8, 9, 10, 11], "length")]
    assert streams[0] == streams[1]
    # b's stop (sampled by launch 1) is seen after launch 2, which therefore still has b; c reaches its limit with launch 3
    assert ahead.calls == [("prefill", [0, 1, 2]), ("launch", [0, 1, 2]), ("launch", [0, 1, 2]), ("collect",),
                           ("launch", [0, 2]), ("collect",), ("collect",)]
    assert ahead.most_in_flight == 2 and sorted(ahead.released) == [0, 1, 2]


def test_a_step_ahead_with_a_limit_of_two_and_an_immediate_stop():
    ahead = AheadStepper([[1, 2, 3], [99, 5, 6], [4, 99, 7]])
    state = BatchState([0, 1, 2], [1, 1, 1], max_new_tokens=2, stop_token_ids={99})
    run_batch(ahead, state, GenerationStats())
    assert [(r.tokens, r.finish_reason) for r in state.results()] == [([1, 2], "length"), ([], "stop"), ([4], "stop")]
    assert ahead.calls == [("prefill", [0, 1, 2]), ("launch", [0, 2]), ("collect",)]   # one launch: both rows are at their limit


def test_the_token_callback_comes_once_a_step_with_that_steps_tokens():
    """The callback is called once after the prompts and once for every decode step, each time with the tokens that the
    step gave to the rows still running, in both loops: the end-to-end figure of the benchmark reads the host's clock there
    and counts the tokens of the last K calls."""
    scripts = [[5, 6, 7, 8, 9, 10], [11, 12, 13, 14, 15, 16]]
    for stepper in (ScriptedStepper(scripts), AheadStepper(scripts)):
        state = BatchState(["a", "b"], [3, 9], max_new_tokens=6, stop_token_ids=[])
        calls = []
        run_batch(stepper, state, GenerationStats(), on_tokens=lambda pairs: calls.append(list(pairs)), clock=lambda: 0.0)
        assert len(calls) == 6                                   # the prompts' first tokens, then five steps
        assert all(len(c) == 2 for c in calls)
        assert [t for c in calls for rid, t in c if rid == "a"] == scripts[0]
        assert [t for c in calls for rid, t in c if rid == "b"] == scripts[1]
