"""The plain implementation checked against itself and against the behaviours that
sdcb/HyMT2Sharp's own tests pin down (tests/HyMT2Sharp.Tests/SamplerTests.cs,
AttentionTests.cs).  No GPU."""
import math

import numpy as np
import torch

import helpers
from plain.hunyuan_plain import (PlainModel, PlainSampler, Xoshiro256StarStar, argmax_first, causal_attention,
                                 neox_rope, ntk_rope_base, plain_generate, rms_norm, rope_inverse_frequencies,
                                 swiglu)


def test_rms_norm_and_swiglu_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    y = rms_norm(x, torch.tensor([2.0, 0.5]), 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]]))
    g, u = torch.tensor([0.0, 2.0]), torch.tensor([5.0, 3.0])
    assert torch.allclose(swiglu(g, u), torch.tensor([0.0, 2 / (1 + math.exp(-2)) * 3]))


def test_rope_rotates_pairs_and_keeps_the_rest():
    inv = rope_inverse_frequencies(ntk_rope_base(10000.0, 0.0, 8), 4)
    assert inv[0] == 1.0 and abs(inv[1] - 0.01) < 1e-9
    x = torch.arange(16, dtype=torch.float32).reshape(2, 1, 8) + 1
    y = neox_rope(x, torch.tensor([0, 3]), 4, inv)
    assert torch.equal(y[0], x[0])  # position 0 rotates by nothing
    assert torch.equal(y[1, 0, 4:], x[1, 0, 4:])  # dims from rope_dim on stay
    c, s = math.cos(3.0), math.sin(3.0)
    assert abs(y[1, 0, 0] - (x[1, 0, 0] * c - x[1, 0, 2] * s)) < 1e-5  # pairs (i, i + half)
    assert abs(y[1, 0, 2] - (x[1, 0, 0] * s + x[1, 0, 2] * c)) < 1e-5
    assert abs(torch.linalg.norm(y[1, 0, :4]) - torch.linalg.norm(x[1, 0, :4])) < 1e-4


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    out = causal_attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0  # later keys must not reach earlier queries
    assert torch.equal(causal_attention(q, k2, v2)[:4], out[:4])
    assert torch.allclose(out[0], v[0].repeat_interleave(2, dim=0).reshape(-1))  # heads 0,1 -> kv head 0
    w = causal_attention(q, k, v, window=2)
    assert torch.allclose(w[:2], out[:2]) and not torch.allclose(w[5], out[5])
    one = causal_attention(q, k, v, window=1)
    assert torch.allclose(one, v.repeat_interleave(2, dim=1).reshape(6, -1))  # sees only itself


def test_model_prefix_property_and_float64(plain_models, model_dirs):
    for name in ("A", "B", "W"):
        m = plain_models(name)
        toks = helpers.random_tokens(m.cfg.vocab, 60, 1)
        full = m.logits(toks)
        assert torch.allclose(m.logits(toks[:25]), full[:25], atol=1e-5)
        m64 = PlainModel(model_dirs(name), dtype=torch.float64)
        ref = m64.logits(toks)
        assert (full.double() - ref).abs().max() < 2e-5 * ref.abs().max()


def test_xoshiro_matches_published_vectors():
    # SplitMix64 from seed 0 gives the well-known first outputs
    r = Xoshiro256StarStar(0)
    assert r.s[0] == 0xE220A8397B1DCDAF and r.s[1] == 0x6E789E6AA1B965F4
    u = [float(r.next_single()) for _ in range(1000)]
    assert all(0.0 <= x < 1.0 for x in u) and 0.4 < np.mean(u) < 0.6


def test_sampler_behaviours():
    rng = np.random.default_rng(0)
    logits = rng.normal(size=200).astype(np.float32)
    assert PlainSampler(temperature=0.0).sample(logits) == argmax_first(logits)
    assert PlainSampler(temperature=1.0, top_k=1, seed=3).sample(logits) == argmax_first(logits)
    tie = np.array([1.0, 5.0, 5.0, 2.0], dtype=np.float32)
    assert argmax_first(tie) == 1  # the first index of the maximum
    a = PlainSampler(temperature=0.8, seed=42)
    b = PlainSampler(temperature=0.8, seed=42)
    assert [a.sample(logits) for _ in range(32)] == [b.sample(logits) for _ in range(32)]
    order = np.argsort(-logits)
    s = PlainSampler(temperature=1.0, top_k=5, seed=1)
    assert all(s.sample(logits) in order[:5] for _ in range(100))
    peaked = np.full(50, -5.0, dtype=np.float32); peaked[7] = 5.0; peaked[9] = 4.0
    s = PlainSampler(temperature=1.0, top_p=0.5, seed=1)
    assert all(s.sample(peaked) == 7 for _ in range(50))
    s = PlainSampler(temperature=1.0, min_p=0.5, seed=1)
    assert all(s.sample(peaked) == 7 for _ in range(50))
    pen = PlainSampler(temperature=0.0, repeat_penalty=100.0)
    two = np.array([0.1, 3.0, 2.9], dtype=np.float32)
    assert pen.sample(two) == 1 and pen.sample(two) == 2  # the penalty flips the winner


def test_plain_generate_stops(plain_models):
    m = plain_models("A")
    prompt = helpers.random_tokens(m.cfg.vocab, 7, 3)
    out, reason = plain_generate(m, prompt, 6)
    assert len(out) == 6 and reason == "length"
    out2, reason2 = plain_generate(m, prompt, 6, stop_ids={out[2]})
    assert out2 == out[:out.index(out[2])] and reason2 == "stop"
