"""Generation through the Python entry point and the command line against the plain loop."""
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
from plain.hunyuan_plain import PlainSampler, plain_generate

pytestmark = pytest.mark.gpu

PROMPT_LENS = {"A": [5, 9, 1], "B": [17, 3, 11, 6], "H": [70, 2, 130]}   # the workloads of the tiny configurations


@pytest.fixture(scope="module")
def engines(model_dirs):
    import hymt2sharp_b200
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = hymt2sharp_b200.load(model_dirs(name), dtype=dtype, max_tokens=2048, max_batch=4)
        return made[(name, dtype)]
    return get


def _margin_ok(plain, seq, tok, floor):
    """True when the plain model's top two logits at the end of `seq` are further apart than `floor`."""
    l = plain.logits(seq)[-1].numpy()
    top = np.sort(l)[-2:]
    return top[1] - top[0] > floor


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "H"])
def test_greedy_generation_matches_plain(name, dtype, engines, plain_models):
    plain = plain_models(name)
    eng = engines(name, dtype)
    steps = 8 if name == "A" else 12
    prompts = [helpers.random_tokens(plain.cfg.vocab, n, 40 + i) for i, n in enumerate(PROMPT_LENS[name])]
    out = eng.generate(prompts, max_new_tokens=steps + 1)
    assert out.stats.batches == 1 and out.stats.prefill_tokens == sum(PROMPT_LENS[name])
    for p, r in zip(prompts, out.results):
        want, _ = plain_generate(plain, p, steps + 1)
        assert r.finish_reason == "length" and len(r.tokens) == steps + 1
        if dtype == "float32":
            assert r.tokens == want
        else:
            # bfloat16 may pick another token where the plain model's two best are within rounding
            # of each other; up to there the tokens are the same
            for i, (a, b) in enumerate(zip(r.tokens, want)):
                if a != b:
                    assert not _margin_ok(plain, p + want[:i], b, 0.02), f"token {i}: {a} vs {b} with a clear margin"
                    break
    eng.cache.book.audit()
    assert eng.cache.free_tokens() == eng.cache.num_blocks * 64  # every slot and block came back


def test_stop_tokens_early_ends_and_batches_one_after_another(engines, plain_models):
    plain = plain_models("A")
    eng = engines("A", "float32")
    prompts = [helpers.random_tokens(plain.cfg.vocab, n, 70 + i) for i, n in enumerate([4, 12, 7, 2, 9, 5, 3])]
    free_run = [plain_generate(plain, p, 10)[0] for p in prompts]
    stop = {free_run[0][3], free_run[2][0]}  # request 0 stops after 3 tokens, request 2 at once
    want = [plain_generate(plain, p, 10, stop_ids=stop) for p in prompts]
    seen = []
    out = eng.generate(prompts, max_new_tokens=10, stop_token_ids=stop, max_batch=3, on_tokens=seen.extend)
    assert out.stats.batches == 3  # 3 + 3 + 1 requests, the later batches in the earlier ones' slots
    for r, (toks, reason) in zip(out.results, want):
        assert r.tokens == toks and r.finish_reason == reason
    assert out.results[2].tokens == [] and out.results[2].finish_reason == "stop"
    assert sorted(seen) == sorted((i, t) for i, r in enumerate(out.results) for t in r.tokens)
    eng.cache.book.audit()


def test_temperature_sampling_follows_the_plain_sampler(engines, plain_models):
    """Same seed, same stream (src/HyMT2Sharp/Sampling.cs:375-409): every sampled token is the
    one whose interval of the plain sampler's cumulative sums holds r, up to rounding of the sums."""
    plain = plain_models("A")
    eng = engines("A", "float32")
    from hymt2sharp_b200 import SamplingParams
    prompts = [helpers.random_tokens(plain.cfg.vocab, n, 90 + i) for i, n in enumerate([5, 9, 1])]
    params = [SamplingParams(temperature=0.8, seed=11 + i) for i in range(3)]
    out = eng.generate(prompts, max_new_tokens=9, sampling=params)
    for p, sp, r in zip(prompts, params, out.results):
        sampler = PlainSampler(temperature=0.8, seed=sp.seed)
        seq = list(p)
        for tok in r.tokens:
            logits = plain.logits(seq)[-1].numpy()
            mine = sampler.sample(logits)
            rr, cdf, prob = sampler.last_cdf
            if mine != tok:  # allowed only when r sits within rounding of the boundary between them
                lo = cdf[tok - 1] if tok > 0 else 0.0
                assert lo - 1e-4 * cdf[-1] <= rr <= cdf[tok] + 1e-4 * cdf[-1], f"token {tok} vs {mine}"
            seq.append(tok)
    again = eng.generate(prompts, max_new_tokens=9, sampling=params)
    assert [r.tokens for r in again.results] == [r.tokens for r in out.results]  # seeded: repeatable
    alone = eng.generate([prompts[1]], max_new_tokens=9, sampling=params[1])
    assert alone.results[0].tokens == out.results[1].tokens  # and independent of the batch


def test_filters_on_the_gpu_match_the_plain_sampler(plain_models):
    """top-k, top-p, min-p and the repetition penalty (src/HyMT2Sharp/Sampling.cs:141-293)."""
    from hymt2sharp_b200.sampling import BatchSampler, SamplingParams
    rng = np.random.default_rng(5)
    vocab = 1000
    cases = [SamplingParams(temperature=0.7, top_k=5, seed=1), SamplingParams(temperature=1.3, top_p=0.6, seed=2),
             SamplingParams(temperature=1.0, min_p=0.2, seed=3),
             SamplingParams(temperature=0.9, top_k=40, top_p=0.8, min_p=0.05, seed=4),
             SamplingParams(temperature=0.0, repeat_penalty=1.5, penalty_window=64),
             SamplingParams(temperature=1.1, top_k=3, repeat_penalty=1.3, penalty_window=64, seed=6)]
    prompts = [rng.integers(0, vocab, 10).tolist() for _ in cases]
    gpu = BatchSampler(cases, "cuda:0", prompts)
    plains = []
    for sp, pr in zip(cases, prompts):
        s = PlainSampler(sp.temperature, sp.top_k, sp.top_p, sp.min_p, sp.repeat_penalty, sp.penalty_window, sp.seed or 0)
        s.feed_history(pr)
        plains.append(s)
    for step in range(30):
        logits = (rng.normal(size=(len(cases), vocab)) * 3).astype(np.float32)
        logits[:, 17] = logits[:, 400] = logits[:, 3] = 4.25   # ties inside the top-k cut
        dev = torch.from_numpy(logits).cuda()
        got = gpu.sample(dev, None).tolist()
        for i, s in enumerate(plains):
            want = s.sample(logits[i])
            if got[i] != want:
                rr, cdf, prob = s.last_cdf
                assert prob[got[i]] > 0, f"case {i} step {step}: token {got[i]} was filtered out in the plain sampler"
                lo = cdf[got[i] - 1] if got[i] > 0 else 0.0
                assert lo - 1e-4 * cdf[-1] <= rr <= cdf[got[i]] + 1e-4 * cdf[-1], f"case {i} step {step}"
                s.window[-1:] = [got[i]] if s.window else []
        survivors = torch.isfinite(dev).sum(dim=1).tolist()
        assert survivors[0] == 5 and survivors[5] == 3 and survivors[4] == vocab  # exact top-k count, greedy untouched


def test_command_line(model_dirs, plain_models):
    plain = plain_models("A")
    prompt = helpers.random_tokens(plain.cfg.vocab, 6, 77)
    want, _ = plain_generate(plain, prompt, 6)
    r = subprocess.run([sys.executable, "-m", "hymt2sharp_b200", "--model", model_dirs("A"), "--dtype", "float32",
                        "--prompt", ",".join(map(str, prompt)), "--max-tokens", "5"],
                       capture_output=True, text=True, cwd=helpers.ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    assert "Assistant: " + ",".join(map(str, want)) in r.stdout  # --max-tokens 5: the first token + 5 decode steps
    assert "prefill tokens=6" in r.stdout and "decode tokens=5" in r.stdout
    assert "arch=HunYuanDenseV1ForCausalLM layers=2 hidden=64 heads=4/2 vocab=256" in r.stdout


@pytest.mark.parametrize("name,dtype", [("H", "bfloat16"), ("A", "float32")])
def test_profiled_generation_books_every_kernel_and_changes_no_token(name, dtype, engines, plain_models):
    """The profiling switch: decode steps are replayed from a graph that holds an event behind every kernel; the tokens are
    those of an unprofiled run, both phases are booked by product and kernel, and unprofiled steps afterwards still work."""
    eng = engines(name, dtype)
    vocab = plain_models(name).cfg.vocab
    prompts = [helpers.random_tokens(vocab, n, 70 + i) for i, n in enumerate(PROMPT_LENS[name])]
    plain_run = eng.generate(prompts, max_new_tokens=9)
    timed = eng.generate(prompts, max_new_tokens=9, profile=True)
    assert [r.tokens for r in timed.results] == [r.tokens for r in plain_run.results]
    assert set(timed.stats.profile) == {"prefill", "decode"}
    for phase, times in timed.stats.profile.items():
        assert {"qkv", "o_proj", "gate_up", "down", "head"} <= set(times) or {"qkv+rope", "o_proj", "gate_up", "down", "head"} <= set(times), times
        assert any(k.startswith("attention") for k in times), times
        assert all(v > 0 for v in times.values()), times
    # a decode kernel of these sizes takes microseconds: eight steps of a few layers stay far below what a host-bound
    # measurement (tens of microseconds per launch) would book
    layers = eng.config.num_hidden_layers
    assert timed.stats.profile["decode"]["o_proj"] < 8 * layers * 0.030
    assert plain_run.stats.profile == {}
    again = eng.generate(prompts, max_new_tokens=9)
    assert [r.tokens for r in again.results] == [r.tokens for r in plain_run.results]
    eng.cache.book.audit()
