"""Each part of a layer alone, built from its own parameters with weights of its own, against
the plain functions: norm, rotary encoding inside attention, attention, feed-forward, block;
and a layer order that names a layer twice and lets a layer read another layer's cache."""
import math

import numpy as np
import pytest
import torch

import helpers
from plain import hunyuan_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _context(cache, slot_tokens, dtype):
    from hymt2sharp_b200.engine.engine import StepEntry, make_context
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    entries = [StepEntry(s, [0] * n, []) for s, n in slot_tokens]
    ctx, _, _, plan = make_context(cache, entries, 10, dtype, DEV, status)
    return ctx, plan


def _cache_for(mixer, dtype, tokens=1024, slots=4):
    from hymt2sharp_b200.cache import GroupSpec, PagedCache
    need = mixer.cache_need()
    return PagedCache([GroupSpec(need.kind, need.kv_heads, need.head_dim, 1, need.window)], dtype, DEV, tokens,
                      max_slots=slots)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from hymt2sharp_b200.parts import PartSpec, build_part
    part = build_part("norm", PartSpec("rmsnorm", dict(dim=200, eps=1e-4, weight="n.w")))
    assert list(part.tensors()) == ["n.w"] and part.tensors()["n.w"].shape == (200,)
    gain = (1 + 0.1 * torch.randn(200)).to(torch.bfloat16)
    part.load({"n.w": gain}, DEV, dtype)
    x = torch.randn(13, 200, device=DEV)
    y = part.forward(x, None, dtype)
    ref = plain.rms_norm(x.cpu(), gain.float(), 1e-4)
    assert y.dtype == dtype and torch.allclose(y.float().cpu(), ref, atol=2e-2 if dtype == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, heads, kv, d, rope_dim, alpha, qk_norm, window",
                         [(72, 6, 2, 32, 32, 0.0, True, None), (100, 4, 4, 16, 8, 50.0, False, None),
                          (64, 8, 1, 64, 64, 1000.0, True, 50)])
def test_attention_part_prefill_then_decode(dtype, hidden, heads, kv, d, rope_dim, alpha, qk_norm, window):
    from hymt2sharp_b200.parts import MixerSlot, PartSpec, build_part
    torch.manual_seed(hidden)
    base = float(plain.ntk_rope_base(10000.0, alpha, d))
    spec = PartSpec("gqa_attention", dict(
        hidden=hidden, heads=heads, kv_heads=kv, head_dim=d, eps=1e-5, qk_norm=qk_norm, window=window,
        position=PartSpec("neox_rope", dict(head_dim=d, rope_dim=rope_dim, base=base)),
        q_proj="q", k_proj="k", v_proj="v", o_proj="o", q_norm="qn", k_norm="kn"))
    part = build_part("mixer", spec)
    shapes = part.tensors()
    assert shapes["q"].shape == (heads * d, hidden) and shapes["o"].shape == (hidden, heads * d)
    assert ("qn" in shapes) == qk_norm
    w = {n: (torch.randn(s.shape) * (0.1 if len(s.shape) == 2 else 0.05) + (0 if len(s.shape) == 2 else 1)).to(torch.bfloat16)
         for n, s in shapes.items()}
    part.load(w, DEV, dtype)
    cache = _cache_for(part, dtype)
    slots = cache.alloc_slots(2)
    L = [130, 70]
    xs = [torch.randn(n, hidden).to(torch.bfloat16).float() for n in L]

    def reference(x):
        T = x.shape[0]
        wf = {n: t.float() for n, t in w.items()}
        q = (x @ wf["q"].T).reshape(T, heads, d)
        k = (x @ wf["k"].T).reshape(T, kv, d)
        v = (x @ wf["v"].T).reshape(T, kv, d)
        inv = plain.rope_inverse_frequencies(np.float32(base), rope_dim)
        pos = torch.arange(T)
        q, k = plain.neox_rope(q, pos, rope_dim, inv), plain.neox_rope(k, pos, rope_dim, inv)
        if qk_norm:
            q, k = plain.rms_norm(q, wf["qn"], 1e-5), plain.rms_norm(k, wf["kn"], 1e-5)
        return plain.causal_attention(q, k, v, window or 0) @ wf["o"].T

    refs = [reference(x) for x in xs]
    slot = MixerSlot(group=0, plane=0)
    tol = dict(atol=3e-2, rtol=3e-2) if dtype == torch.bfloat16 else dict(atol=2e-5, rtol=2e-5)
    # both sequences: all but the last 3 tokens in one step, then three single-token steps
    pre = [n - 3 for n in L]
    ctx, plan = _context(cache, list(zip(slots, pre)), dtype)
    x = torch.cat([xs[i][:pre[i]] for i in range(2)]).to(DEV).to(dtype)
    residual = torch.ones(sum(pre), hidden, device=DEV)
    part.forward(x, residual, ctx, slot)
    cache.end_step(plan)
    got = residual.cpu() - 1
    assert torch.allclose(got, torch.cat([refs[i][:pre[i]] for i in range(2)]), **tol)
    for step in range(3):
        ctx, plan = _context(cache, [(s, 1) for s in slots], dtype)
        x = torch.stack([xs[i][pre[i] + step] for i in range(2)]).to(DEV).to(dtype)
        residual = torch.zeros(2, hidden, device=DEV)
        part.forward(x, residual, ctx, slot)
        cache.end_step(plan)
        assert torch.allclose(residual.cpu(), torch.stack([refs[i][pre[i] + step] for i in range(2)]), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from hymt2sharp_b200.parts import PartSpec, build_part
    part = build_part("feed_forward", PartSpec("swiglu", dict(hidden=72, intermediate=200, gate_proj="g",
                                                              up_proj="u", down_proj="d")))
    assert {n: s.shape for n, s in part.tensors().items()} == {"g": (200, 72), "u": (200, 72), "d": (72, 200)}
    w = {n: (torch.randn(s.shape) * 0.1).to(torch.bfloat16) for n, s in part.tensors().items()}
    part.load(w, DEV, dtype)
    x = torch.randn(21, 72).to(torch.bfloat16).float()
    residual = torch.full((21, 72), 2.0, device=DEV)
    part.forward(x.to(DEV).to(dtype), residual, None)
    ref = plain.swiglu(x @ w["g"].float().T, x @ w["u"].float().T) @ w["d"].float().T
    tol = dict(atol=3e-2, rtol=3e-2) if dtype == torch.bfloat16 else dict(atol=2e-5, rtol=2e-5)
    assert torch.allclose(residual.cpu() - 2.0, ref, **tol)


def test_block_part_equals_the_plain_layer(model_dirs, plain_models):
    """One pre-norm block, built from the architecture's spec of layer 1, run alone."""
    from hymt2sharp_b200.config import load_config
    from hymt2sharp_b200.parts import MixerSlot, build_part
    from hymt2sharp_b200.weights import load_checkpoint
    pm = plain_models("A")
    arch, cfg = load_config(model_dirs("A"))
    spec = arch.build_spec(cfg)
    block = build_part("block", spec.layers[1])
    weights = load_checkpoint(model_dirs("A"), arch.tensor_shapes(cfg))
    block.load(weights, DEV, torch.float32)
    cache = _cache_for(block.mixer, torch.float32)
    slot_id = cache.alloc_slots(1)[0]
    h = torch.randn(90, cfg.hidden_size)
    ref = pm.layer(h, 1, torch.arange(90))
    ctx, plan = _context(cache, [(slot_id, 90)], torch.float32)
    residual = h.clone().to(DEV)
    block.forward(residual, ctx, [MixerSlot(group=0, plane=0)])
    assert torch.allclose(residual.cpu(), ref, atol=1e-5, rtol=1e-5)


def test_order_names_a_layer_twice_and_shares_a_cache(model_dirs, plain_models, tmp_path):
    """The order of layers is data.  [0, 1, 1]: layer 1 runs twice with a cache plane for each run,
    which equals a three-layer model whose third layer has layer 1's weights.  [0, 1, 1 reading
    entry 1's cache]: the third run writes no keys and attends over the second run's."""
    import json, os
    from hymt2sharp_b200.engine.engine import Engine, StepEntry
    from hymt2sharp_b200.engine.spec import Run
    from hymt2sharp_b200.weights import SafetensorsFile, write_safetensors
    from plain.hunyuan_plain import PlainModel
    folder = model_dirs("A")
    src = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: src.tensor(n) for n in src.names()}
    for n in list(tensors):
        if n.startswith("model.layers.1."):
            tensors[n.replace("layers.1.", "layers.2.")] = tensors[n]
    cfg3 = json.load(open(os.path.join(folder, "config.json")))
    cfg3["num_hidden_layers"] = 3
    (tmp_path / "config.json").write_text(json.dumps(cfg3))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    ref = PlainModel(str(tmp_path))
    toks = helpers.random_tokens(256, 100, 4)

    def twice(cfg):
        from hymt2sharp_b200.engine.hunyuan_dense import build_spec
        spec = build_spec(cfg)
        spec.order = [Run(0), Run(1), Run(1)]
        return spec

    eng = Engine(folder, dtype="float32", max_tokens=256, spec_override=twice)
    assert eng.model.groups[0].planes == 3
    slot = eng.alloc_slots(1)[0]
    got = [eng.step([StepEntry(slot, toks[:70], list(range(70)))]).cpu()]
    got += [eng.step([StepEntry(slot, [t], [0])]).cpu() for t in toks[70:]]
    helpers.assert_close(torch.cat(got).numpy(), ref.logits(toks).numpy(), "float32", "order [0, 1, 1]")

    def shared(cfg):
        spec = twice(cfg)
        spec.order = [Run(0), Run(1), Run(1, cache_from=1)]
        return spec

    eng2 = Engine(folder, dtype="float32", max_tokens=256, spec_override=shared)
    assert eng2.model.groups[0].planes == 2 and not eng2.model.slots[2][0].writes
    slot = eng2.alloc_slots(1)[0]
    whole = eng2.step([StepEntry(slot, toks, list(range(100)))]).cpu().numpy()
    eng2.free_slots([slot])
    slot = eng2.alloc_slots(1)[0]
    cut = [eng2.step([StepEntry(slot, toks[:70], list(range(70)))]).cpu()]
    cut += [eng2.step([StepEntry(slot, [t], [0])]).cpu() for t in toks[70:]]
    helpers.assert_close(torch.cat(cut).numpy(), whole, "float32", "shared cache: cut vs whole")
    # the plain statement of the same thing: the third run's attention uses the second run's k, v
    pm = plain_models("A")
    h = pm.w["model.embed_tokens.weight"][torch.tensor(toks)]
    pos = torch.arange(100)
    h = pm.layer(h, 0, pos)
    c, w, p = pm.cfg, pm.w, "model.layers.1."
    n1 = plain.rms_norm(h, w[p + "input_layernorm.weight"], c.eps)
    k = plain.neox_rope((n1 @ w[p + "self_attn.k_proj.weight"].T).reshape(100, c.kv_heads, c.head_dim), pos, c.rope_dim, pm.inv_freq)
    k = plain.rms_norm(k, w[p + "self_attn.key_layernorm.weight"], c.eps)
    v = (n1 @ w[p + "self_attn.v_proj.weight"].T).reshape(100, c.kv_heads, c.head_dim)
    h = pm.layer(h, 1, pos)
    n1 = plain.rms_norm(h, w[p + "input_layernorm.weight"], c.eps)
    q = plain.neox_rope((n1 @ w[p + "self_attn.q_proj.weight"].T).reshape(100, c.heads, c.head_dim), pos, c.rope_dim, pm.inv_freq)
    q = plain.rms_norm(q, w[p + "self_attn.query_layernorm.weight"], c.eps)
    h = h + plain.causal_attention(q, k, v) @ w[p + "self_attn.o_proj.weight"].T
    n2 = plain.rms_norm(h, w[p + "post_attention_layernorm.weight"], c.eps)
    h = h + plain.swiglu(n2 @ w[p + "mlp.gate_proj.weight"].T, n2 @ w[p + "mlp.up_proj.weight"].T) @ w[p + "mlp.down_proj.weight"].T
    logits = plain.rms_norm(h, w["model.norm.weight"], c.eps) @ w["model.embed_tokens.weight"].T
    helpers.assert_close(whole, logits.numpy(), "float32", "shared cache vs plain")
