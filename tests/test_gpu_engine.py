"""The engine in-process: long decoding, the first tokens of a sequence, a poisoned cache,
crafted scores that make one far key or a window's edge decide the result, errors that
leave the engine usable."""
import math

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _engine(model_dirs, name, dtype, **kw):
    from hymt2sharp_b200.engine.engine import Engine
    return Engine(model_dirs(name), dtype=dtype, **{"max_tokens": 1024, **kw})


def _poison(eng):
    for s in eng.cache.storage:
        s.fill_(float("nan"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W", "M", "H", "HW", "S"])
def test_long_decoding_from_the_first_token(name, dtype, model_dirs, plain_models):
    """A one-token prompt, then 420 tokens one by one (across block ends and past the length at
    which decode attention starts to split its keys), in a cache whose unwritten rows are NaN."""
    from hymt2sharp_b200.engine.engine import StepEntry
    plain = plain_models(name)
    toks = helpers.random_tokens(plain.cfg.vocab, 421, 21)
    ref = plain.logits(toks).numpy()
    eng = _engine(model_dirs, name, dtype)
    _poison(eng)
    slot = eng.alloc_slots(1)[0]
    rows = [eng.step([StepEntry(slot, [t], [0])]) for t in toks]
    got = torch.cat(rows).cpu().numpy()
    eng.check()
    helpers.assert_close(got[:3], ref[:3], dtype, f"{name} {dtype} first tokens")
    helpers.assert_close(got, ref, dtype, f"{name} {dtype} long decode")
    assert eng.length(slot) == 421


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_in_a_poisoned_reused_cache(dtype, model_dirs, plain_models):
    """Three rounds of batches in the same slots; before each, everything that the cache holds is
    overwritten with NaN: a kernel that reads a row it has not written shows."""
    from hymt2sharp_b200.engine.engine import StepEntry
    plain = plain_models("B")
    eng = _engine(model_dirs, "B", dtype, max_tokens=512)
    for rnd, lens in enumerate([(100, 3, 64), (1, 65, 127), (33, 128, 2)]):
        _poison(eng)
        seqs = [helpers.random_tokens(plain.cfg.vocab, n + 5, 50 * rnd + i) for i, n in enumerate(lens)]
        slots = eng.alloc_slots(3)
        assert sorted(slots) == [0, 1, 2]
        out = eng.step([StepEntry(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, lens)]).cpu().numpy()
        got = [list(out[sum(lens[:i]):sum(lens[:i + 1])]) for i in range(3)]
        for step in range(5):  # the middle sequence leaves after 2 decoded tokens
            live = [i for i in range(3) if not (i == 1 and step >= 2)]
            o = eng.step([StepEntry(slots[i], [seqs[i][lens[i] + step]], [0]) for i in live]).cpu().numpy()
            for row, i in zip(o, live):
                got[i].append(row)
            if step == 1:
                eng.free_slots([slots[1]])
        eng.free_slots([slots[0], slots[2]])
        eng.check()
        for i in range(3):
            n = lens[i] + (2 if i == 1 else 5)
            helpers.assert_close(np.stack(got[i]), plain.logits(seqs[i][:n]).numpy(), dtype, f"round {rnd} sequence {i}")
    eng.cache.book.audit()


def _attention_case(dtype, L, new, nh, nkv, d, window, hot_key, hot_value=7.0):
    """Random keys, but every query matches key `hot_key` so strongly that the softmax puts all
    its weight there (when that key is visible): the output is that key's value row."""
    from test_gpu_kernels import _paged
    torch.manual_seed(L + new)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    k = torch.randn(L, nkv, d, device=DEV) * 0.1
    v = torch.randn(L, nkv, d, device=DEV) * 0.1
    direction = torch.randn(d, device=DEV)
    direction /= direction.norm()
    k[hot_key] = direction * 30.0
    v[hot_key] = hot_value
    q = (direction * 30.0).repeat(new, nh, 1) + torch.randn(new, nh, d, device=DEV) * 0.1
    kp, vp, table = _paged([k.to(tdt)], [v.to(tdt)], 64, tdt, shuffle_seed=L)
    return q.to(tdt).reshape(new, nh * d), kp, vp, table, tdt


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("L, new", [(900, 1), (900, 130), (300, 300)])
def test_one_far_key_among_hundreds_decides(dtype, L, new):
    """The hot key sits early in the sequence (position 5, in the first block): every later query
    must find it through the block table, in prefill tiles and in decode splits alike."""
    from hymt2sharp_b200.kernels import ops
    nh, nkv, d = 4, 2, 64
    q, kp, vp, table, tdt = _attention_case(dtype, L, new, nh, nkv, d, 0, hot_key=5)
    out = torch.zeros(new, nh * d, dtype=tdt, device=DEV)
    cu = torch.tensor([0, new], dtype=torch.int32, device=DEV)
    one = torch.zeros(1, dtype=torch.int32, device=DEV)
    kv = torch.tensor([L], dtype=torch.int32, device=DEV)
    split = dict(split_keys=256, max_splits=4, part_acc=torch.empty(new * nh * 4 * d, device=DEV),
                 part_ml=torch.empty(new * nh * 8, device=DEV)) if new == 1 else {}
    ops.attention_simt(out, q, kp, vp, table, cu, one, kv, 1, new, nh, nkv, d, 1 / math.sqrt(d), 0, **split)
    first = L - new  # position of the first query
    seen = out.float()[max(0, 5 - first):]  # queries at or after position 5 see the hot key
    assert (seen - 7.0).abs().max() < 0.05, "a query lost the far key"
    if first < 5:
        assert out.float()[:5 - first].abs().max() < 1.0  # earlier queries cannot see it


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("new", [1, 40])
def test_window_edge(dtype, new):
    """Window 100: for the query at position p the key p-99 is the oldest visible one and p-100 is
    outside.  A hot key exactly at the edge is seen by exactly the queries that should see it."""
    from hymt2sharp_b200.kernels import ops
    nh, nkv, d, L, window = 6, 3, 32, 400, 100
    last = L - 1
    for hot, visible_from_last in ((last - 99, True), (last - 100, False)):
        q, kp, vp, table, tdt = _attention_case(dtype, L, new, nh, nkv, d, window, hot_key=hot)
        out = torch.zeros(new, nh * d, dtype=tdt, device=DEV)
        cu = torch.tensor([0, new], dtype=torch.int32, device=DEV)
        one = torch.zeros(1, dtype=torch.int32, device=DEV)
        kv = torch.tensor([L], dtype=torch.int32, device=DEV)
        split = dict(split_keys=256, max_splits=2, part_acc=torch.empty(new * nh * 2 * d, device=DEV),
                     part_ml=torch.empty(new * nh * 4, device=DEV)) if new == 1 else {}
        ops.attention_simt(out, q, kp, vp, table, cu, one, kv, 1, new, nh, nkv, d, 1 / math.sqrt(d), window, **split)
        o = out.float().reshape(new, nh * d)
        for i in range(new):
            p = L - new + i
            sees = p - window + 1 <= hot <= p
            if sees:
                assert (o[i] - 7.0).abs().max() < 0.05, f"query at {p} should see key {hot}"
            else:
                assert o[i].abs().max() < 1.0, f"query at {p} must not see key {hot}"
        assert ((o[-1] - 7.0).abs().max() < 0.05) == visible_from_last


def _fast_attention(q, kp, vp, table, L, new, nh, nkv, d, window):
    """The attention of one sequence through the kernel that the bfloat16 engine picks for it."""
    from types import SimpleNamespace
    from hymt2sharp_b200.kernels import fast
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    ctx = SimpleNamespace(decode=new == 1, max_kv_len=L, num_tokens=new, num_seqs=1, max_new_tokens=new,
                          cu_seqlens=i32([0, new]), slot_ids=i32([0]), kv_lens=i32([L]))
    out = torch.zeros(new, nh * d, dtype=q.dtype, device=DEV)
    assert fast.try_attention(out, q, kp, vp, table, ctx, nh, nkv, d, 1 / math.sqrt(d), window), "no fast kernel took it"
    return out.float()


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("L, new", [(900, 1), (900, 130), (300, 300)])
def test_one_far_key_decides_in_the_tensor_core_kernels(d, L, new):
    """As above, through the kernels that a bfloat16 engine runs for heads of 64 and 128: the streaming decode
    kernel, the tcgen05 decode kernel and the tcgen05 prompt kernel."""
    nh, nkv = 4, 2
    q, kp, vp, table, _ = _attention_case("bfloat16", L, new, nh, nkv, d, 0, hot_key=5)
    out = _fast_attention(q, kp, vp, table, L, new, nh, nkv, d, 0)
    first = L - new
    assert (out[max(0, 5 - first):] - 7.0).abs().max() < 0.05, "a query lost the far key"
    if first < 5:
        assert out[:5 - first].abs().max() < 1.0


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("new", [1, 40, 200])
@pytest.mark.parametrize("L, window", [(448, 128), (512, 128), (449, 128), (400, 100), (641, 257)])
def test_window_edge_in_the_tensor_core_kernels(d, new, L, window):
    """The oldest visible key and the one just outside, with the window's lower end in the second cache block of a
    128-key chunk (L 448), at a chunk's first key (L 512), one past a 64-key tile's first key (L 449: the newest
    position opens a tile), and off every boundary."""
    nh, nkv = 4, 2
    last = L - 1
    for hot in (last - window + 1, last - window):
        q, kp, vp, table, _ = _attention_case("bfloat16", L, new, nh, nkv, d, window, hot_key=hot)
        # blocks that lie wholly below the oldest key of the FIRST query are handed back by a window cache
        first_lo = max(0, (L - new) - window + 1)
        table[0, : first_lo // 64] = -1
        out = _fast_attention(q, kp, vp, table, L, new, nh, nkv, d, window)
        for i in range(new):
            p = L - new + i
            if p - window + 1 <= hot <= p:
                assert (out[i] - 7.0).abs().max() < 0.05, f"query at {p} should see key {hot}"
            else:
                assert out[i].abs().max() < 1.0, f"query at {p} must not see key {hot}"


def test_errors_leave_the_engine_usable(model_dirs, plain_models):
    from hymt2sharp_b200.cache import CacheFull
    from hymt2sharp_b200.engine.engine import EngineError, StepEntry
    plain = plain_models("A")
    eng = _engine(model_dirs, "A", "float32", max_tokens=256)
    a, b = eng.alloc_slots(2)
    toks = helpers.random_tokens(256, 100, 1)
    first = eng.step([StepEntry(a, toks[:50], [49])]).cpu().numpy()
    with pytest.raises(EngineError):
        eng.step([StepEntry(a, [256], [0])])             # a token outside the vocabulary
    with pytest.raises(EngineError):
        eng.step([StepEntry(a, [1, 2], [2])])            # a wanted place outside the entry
    with pytest.raises(CacheFull):
        eng.step([StepEntry(a, toks[50:60], []), StepEntry(b, [1] * 200, [])])   # 4 blocks, 3 free
    assert eng.length(a) == 50 and eng.length(b) == 0     # nothing of the refused steps stayed
    rest = eng.step([StepEntry(a, toks[50:], list(range(50)))]).cpu().numpy()
    ref = plain.logits(toks).numpy()
    helpers.assert_close(np.concatenate([first, rest]), ref[49:], "float32", "after refused steps")
    eng.check()
    eng.free_slots([a, b])
    eng.cache.book.audit()


def test_no_device_means_a_loud_error(monkeypatch):
    from hymt2sharp_b200.engine import engine as e
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    with pytest.raises(e.EngineError) as err:
        e.require_gpu("cuda:0")
    assert "no CPU path" in str(err.value)


def test_the_fast_kernels_are_what_a_bfloat16_step_of_full_size_heads_runs(model_dirs):
    """With heads of 128 a bfloat16 decode step is, per layer: the projection that also rotates and appends to the
    cache, attention, the request for the next weights, output projection, gate/up, down; the norms are folded into
    the products around them, all but the very first.  A silent fall to the general kernels would show as more
    launches (a norm, a rotation kernel, a split attention with its merge)."""
    from hymt2sharp_b200.engine.engine import StepEntry
    from hymt2sharp_b200.kernels import ops
    eng = _engine(model_dirs, "H", "bfloat16")
    slot = eng.alloc_slots(1)[0]
    eng.step([StepEntry(slot, list(range(1, 301)), [299])])
    before = ops.launches
    eng.step([StepEntry(slot, [5], [0])])
    layers = eng.config.num_hidden_layers
    assert ops.launches - before == 1 + 1 + 6 * layers + 2   # embedding; the first norm; the layers; final norm and head
    q = torch.empty(1, 4 * 128, dtype=torch.bfloat16, device=DEV)
    assert ops.gemm_tc_rope_kv_supported(torch.empty(1, 256, dtype=torch.bfloat16, device=DEV),
                                         eng.model.blocks[0].mixer.qkv.weight, 4, 2, 128, q.dtype, 128)
    eng.check()


def test_a_bounded_wait_that_runs_out_is_reported_and_the_engine_goes_on(model_dirs, plain_models):
    """One tensor-core product is launched with a fault put in: the producer never copies one k block, so the MMA
    issuer's wait for it gives up after a few thousand tries.  The kernel must say so in the status word (102), let
    every role leave, free its tensor memory and return; Engine.check() raises and clears; the next step is right."""
    from hymt2sharp_b200.engine.engine import EngineError, StepEntry
    from hymt2sharp_b200.kernels import ops
    plain = plain_models("H")
    eng = _engine(model_dirs, "H", "bfloat16")
    slot = eng.alloc_slots(1)[0]
    toks = helpers.random_tokens(plain.cfg.vocab, 90, 31)
    first = eng.step([StepEntry(slot, toks[:60], [59])]).cpu().numpy()
    eng.check()

    a = torch.randn(8, 128, device=DEV).to(torch.bfloat16)
    w = torch.randn(256, 128, device=DEV).to(torch.bfloat16)
    out = torch.zeros(8, 256, device=DEV)
    plan = ops.gemm_tc_describe(8, 256, 128, ops.EPILOGUE_STORE)
    assert plan["swapped"] and plan["k_splits"] == 1 and plan["ctas"] == 2      # the smallest launch there is
    ops.gemm_tc_debug(out, a, w, ops.EPILOGUE_STORE, eng.status, wait_limit=4096, withhold_block=1)
    torch.cuda.synchronize()                                                    # the kernel came back
    assert int(eng.status[0].item()) == 102
    with pytest.raises(EngineError, match="102"):
        eng.check()
    assert int(eng.status[0].item()) == 0
    # the same product without the fault, then the engine's next steps
    ops.gemm_tc(out, a, w, ops.EPILOGUE_STORE, eng.status)
    assert torch.allclose(out.double(), a.double() @ w.double().T, rtol=2e-2, atol=2e-2)
    rest = torch.cat([eng.step([StepEntry(slot, toks[60:80], list(range(20)))])] +
                     [eng.step([StepEntry(slot, [t], [0])]) for t in toks[80:]]).cpu().numpy()
    eng.check()
    ref = plain.logits(toks).numpy()
    helpers.assert_close(np.concatenate([first, rest]), ref[59:], "bfloat16", "after a wait that ran out")
    with pytest.raises(ops.KernelError):        # a product whose K is cut over CTAs is not offered with a fault
        ops.gemm_tc_debug(torch.zeros(8, 2048, device=DEV), torch.zeros(8, 2048, device=DEV, dtype=torch.bfloat16),
                          torch.zeros(2048, 2048, device=DEV, dtype=torch.bfloat16), ops.EPILOGUE_STORE, eng.status, 4096, 1)
