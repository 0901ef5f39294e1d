"""What the step function works out on the host before anything is launched: the packed tokens, each token's
batch row and position, the rows' offsets, slots and lengths, the wanted rows; and what it refuses.  The cache
here is a stand-in that only knows lengths, so this runs without a GPU."""
import numpy as np
import pytest
import torch

from hymt2sharp_b200.engine.engine import EngineError, StepEntry, make_context


class LengthsOnly:
    def __init__(self, lengths):
        self.lengths, self.begun = dict(lengths), None

    def length(self, slot):
        return self.lengths[slot]

    def begin_step(self, plan):
        self.begun = list(plan)


def test_the_step_context_packs_unequal_entries():
    cache = LengthsOnly({3: 0, 0: 70, 5: 2})
    entries = [StepEntry(3, [5, 17, 3], [0, 2]), StepEntry(0, np.array([9]), []), StepEntry(5, (1, 2, 4, 8), [3])]
    ctx, want, num_want, plan = make_context(cache, entries, 20, torch.float32, "cpu", None)
    assert plan == [(3, 3), (0, 1), (5, 4)] and cache.begun == plan
    assert ctx.num_tokens == 8 and ctx.num_seqs == 3 and ctx.max_new_tokens == 4 and ctx.max_kv_len == 71
    assert ctx.tokens.tolist() == [5, 17, 3, 9, 1, 2, 4, 8]
    assert ctx.token_seq.tolist() == [0, 0, 0, 1, 2, 2, 2, 2]
    assert ctx.token_pos.tolist() == [0, 1, 2, 70, 2, 3, 4, 5]
    assert ctx.cu_seqlens.tolist() == [0, 3, 4, 8]
    assert ctx.slot_ids.tolist() == [3, 0, 5] and ctx.kv_lens.tolist() == [3, 71, 6]
    assert want.tolist() == [0, 2, 7] and num_want == 3
    assert ctx.host_slots == [3, 0, 5] and ctx.host_new_tokens == [3, 1, 4] and ctx.host_starts == [0, 70, 2]
    assert all(t.dtype == torch.int32 for t in (ctx.tokens, ctx.token_seq, ctx.token_pos, ctx.cu_seqlens, want))
    assert not ctx.decode


def test_nothing_wanted_and_one_token_each():
    cache = LengthsOnly({0: 4, 1: 9})
    ctx, want, num_want, _ = make_context(cache, [StepEntry(0, [1], []), StepEntry(1, [2], [])], 10, torch.float32, "cpu", None)
    assert want is None and num_want == 0 and ctx.decode
    assert ctx.token_pos.tolist() == [4, 9]


@pytest.mark.parametrize("tokens, want, words", [
    ([1, 20], [0], "token id 20"), ([3, -1, 2], [0], "token id -1"), ([1, 2], [2], "wanted place 2"),
    ([1, 2], [-1], "wanted place -1"), (["a"], [0], "not integer ids"), ([2 ** 70], [0], "not integer ids")])
def test_what_the_step_refuses_before_it_touches_the_cache(tokens, want, words):
    cache = LengthsOnly({0: 0})
    with pytest.raises(EngineError, match=words):
        make_context(cache, [StepEntry(0, tokens, want)], 20, torch.float32, "cpu", None)
    assert cache.begun is None   # nothing was reserved
