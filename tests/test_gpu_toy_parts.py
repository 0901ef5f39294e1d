"""More toy parts, defined here and registered without any change to the library: a
feed-forward with routing (every token goes to the one of a few small experts that a router
picks), another position encoding (neighbouring pairs are rotated, and with other
frequencies than the library's), and a block that holds TWO mixers side by side (attention
with its cache and a running sum with state of its own).  A model alternates them with the
library's own parts layer by layer; the engine's logits are compared with a plain
whole-sequence computation written here, for the whole prompt, token by token, and in a batch
of two.  Not a model of anyone's."""
import json
import math

import numpy as np
import pytest
import torch

import helpers
from plain.hunyuan_plain import causal_attention, rms_norm, swiglu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class RoutedExperts:
    """residual += gate_e(x) * (silu(x·A_e) · B_e), e = argmax(x·R) in float32, gate = softmax(x·R)[e]."""

    def __init__(self, hidden, width, experts, router, up, down):
        self.hidden, self.width, self.experts = hidden, width, experts
        self.names = dict(r=router, a=up, b=down)

    def tensors(self):
        from hymt2sharp_b200.weights import TensorSpec
        n, e, h, w = self.names, self.experts, self.hidden, self.width
        t = {n["r"]: TensorSpec((e, h))}   # stored in 32-bit, and a tensor stored in 32-bit stays so
        for i in range(e):
            t[f"{n['a']}.{i}"] = TensorSpec((w, h))
            t[f"{n['b']}.{i}"] = TensorSpec((h, w))
        return t

    def load(self, weights, device, dtype):
        n = self.names
        self.router = weights[n["r"]].to(device).float()
        self.a = torch.stack([weights[f"{n['a']}.{i}"] for i in range(self.experts)]).to(device).float()
        self.b = torch.stack([weights[f"{n['b']}.{i}"] for i in range(self.experts)]).to(device).float()

    def forward(self, x, residual, ctx):
        x = x.float()[:ctx.num_tokens]
        logits = x @ self.router.T                      # router logits in float32
        choice = logits.argmax(dim=-1)
        gate = torch.softmax(logits, dim=-1).gather(1, choice[:, None])
        hidden = torch.einsum("th,twh->tw", x, self.a[choice])
        hidden = hidden / (1 + torch.exp(-hidden))
        residual[:ctx.num_tokens] += gate * torch.einsum("tw,thw->th", hidden, self.b[choice])


class NeighbourPairRotary:
    """Rotates the pairs (2i, 2i+1) of q and k by position * base^(-i / (d/2)); in place, before the
    library's kernel appends k and v (which then gets no table and rotates nothing)."""

    def __init__(self, head_dim, base):
        self.head_dim, self.base = head_dim, float(base)

    def tensors(self):
        return {}

    def load(self, weights, device, dtype):
        half = self.head_dim // 2
        self.freq = (self.base ** (-torch.arange(half, dtype=torch.float64) / half)).float().to(device)

    def kernel_epilogue(self, ctx):
        return None   # no kernel rotates neighbouring pairs: `apply` does it

    def apply(self, qkv, ctx, heads, kv_heads, head_dim):
        T = ctx.num_tokens
        angle = ctx.token_pos[:T].float()[:, None] * self.freq[None, :]
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        rot = qkv[:T, :(heads + kv_heads) * head_dim].reshape(T, heads + kv_heads, head_dim // 2, 2).float()
        even, odd = rot[..., 0].clone(), rot[..., 1].clone()
        rot[..., 0] = even * cos - odd * sin
        rot[..., 1] = even * sin + odd * cos
        qkv[:T, :(heads + kv_heads) * head_dim] = rot.reshape(T, -1).to(qkv.dtype)


HIDDEN, HEADS, KV_HEADS, HEAD_DIM, VOCAB, LAYERS, EXPERTS, WIDTH, EPS = 40, 4, 2, 16, 83, 4, 3, 24, 1e-5


def build_spec(cfg=None):
    from hymt2sharp_b200.engine.spec import ModelSpec
    from hymt2sharp_b200.parts import PartSpec
    layers = []
    for l in range(LAYERS):
        p = f"l{l}."
        norm = lambda n: PartSpec("rmsnorm", dict(dim=HIDDEN, eps=EPS, weight=p + n))
        # odd layers rotate neighbouring pairs, even layers use no position encoding at all
        position = PartSpec("toy_pair_rope", dict(head_dim=HEAD_DIM, base=50.0)) if l % 2 else None
        mixer = PartSpec("gqa_attention", dict(hidden=HIDDEN, heads=HEADS, kv_heads=KV_HEADS, head_dim=HEAD_DIM, eps=EPS,
                                               qk_norm=False, position=position, q_proj=p + "q", k_proj=p + "k",
                                               v_proj=p + "v", o_proj=p + "o"))
        # layers 1 and 2 route, layers 0 and 3 are dense: feed-forwards are chosen layer by layer
        if l in (1, 2):
            ffn = PartSpec("toy_routed", dict(hidden=HIDDEN, width=WIDTH, experts=EXPERTS, router=p + "router",
                                              up=p + "expert_up", down=p + "expert_down"))
        else:
            ffn = PartSpec("swiglu", dict(hidden=HIDDEN, intermediate=64, gate_proj=p + "g", up_proj=p + "u", down_proj=p + "d"))
        layers.append(PartSpec("pre_norm", dict(norm1=norm("n1"), mixer=mixer, norm2=norm("n2"), feed_forward=ffn)))
    return ModelSpec(VOCAB, HIDDEN, "emb", layers, PartSpec("rmsnorm", dict(dim=HIDDEN, eps=EPS, weight="norm")), head=None)


def plain_logits(w, tokens):
    """The same model for one whole sequence, nothing cached (float32 on the CPU)."""
    T = len(tokens)
    h = w["emb"][torch.tensor(tokens)].clone()
    pos = torch.arange(T, dtype=torch.float32)
    for l in range(LAYERS):
        p = f"l{l}."
        x = rms_norm(h, w[p + "n1"], EPS)
        q = (x @ w[p + "q"].T).reshape(T, HEADS, HEAD_DIM)
        k = (x @ w[p + "k"].T).reshape(T, KV_HEADS, HEAD_DIM)
        v = (x @ w[p + "v"].T).reshape(T, KV_HEADS, HEAD_DIM)
        if l % 2:
            half = HEAD_DIM // 2
            freq = (50.0 ** (-torch.arange(half, dtype=torch.float64) / half)).float()
            angle = pos[:, None] * freq[None, :]
            cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]

            def rotate(t):
                pairs = t.reshape(T, -1, half, 2)
                return torch.stack([pairs[..., 0] * cos - pairs[..., 1] * sin, pairs[..., 0] * sin + pairs[..., 1] * cos],
                                   dim=-1).reshape(t.shape)
            q, k = rotate(q), rotate(k)
        h = h + causal_attention(q, k, v) @ w[p + "o"].T
        x = rms_norm(h, w[p + "n2"], EPS)
        if l in (1, 2):
            logits = x @ w[p + "router"].T
            out = torch.zeros_like(h)
            for t in range(T):
                e = int(logits[t].argmax())
                gate = torch.softmax(logits[t], dim=-1)[e]
                hid = x[t] @ w[f"{p}expert_up.{e}"].T
                out[t] = gate * ((hid / (1 + torch.exp(-hid))) @ w[f"{p}expert_down.{e}"].T)
            h = h + out
        else:
            h = h + swiglu(x @ w[p + "g"].T, x @ w[p + "u"].T) @ w[p + "d"].T
    return (rms_norm(h, w["norm"], EPS) @ w["emb"].T).numpy()


def test_routed_feed_forward_and_another_position_encoding(tmp_path):
    from hymt2sharp_b200.config import register_architecture
    from hymt2sharp_b200.engine.engine import Engine, StepEntry
    from hymt2sharp_b200.engine.model import DecoderModel
    from hymt2sharp_b200.parts import register_part
    from hymt2sharp_b200.weights import write_safetensors

    register_part("feed_forward", "toy_routed", RoutedExperts)
    register_part("position", "toy_pair_rope", NeighbourPairRotary)

    class ToyConfig:
        architecture = "ToyRoutedForCausalLM"

        @classmethod
        def from_dict(cls, data, source="config.json"):
            return cls()

    register_architecture("ToyRoutedForCausalLM", ToyConfig, build_spec, lambda cfg: DecoderModel(build_spec()).tensors())
    (tmp_path / "config.json").write_text(json.dumps(dict(architectures=["ToyRoutedForCausalLM"])))
    shapes = DecoderModel(build_spec()).tensors()
    gen = torch.Generator().manual_seed(5)
    tensors = {}
    for name, spec in shapes.items():
        t = torch.randn(spec.shape, generator=gen) * (1.0 if name.endswith("router") else 1.0 / math.sqrt(spec.shape[-1]))
        if spec.init == "gain":
            t = 1.0 + 0.1 * t
        # what the checkpoint stores is what both sides compute with: bfloat16 values, the router in float32
        tensors[name] = t.float() if name.endswith("router") else t.to(torch.bfloat16)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    w = {n: t.float() for n, t in tensors.items()}

    eng = Engine(str(tmp_path), dtype="float32", max_tokens=512)
    assert eng.model.blocks[1].feed_forward.router.dtype == torch.float32
    toks = [helpers.random_tokens(VOCAB, 37, 11), helpers.random_tokens(VOCAB, 12, 12)]
    want = [plain_logits(w, t) for t in toks]
    # every expert is used somewhere, or the routing would be tested on one expert only
    x_probe = torch.randn(200, HIDDEN, generator=gen)
    assert len(set((x_probe @ w["l1.router"].T).argmax(-1).tolist())) == EXPERTS

    def run(cuts):
        slots = eng.alloc_slots(2)
        rows, pos = [[], []], [0, 0]
        for step in cuts:
            entries = [StepEntry(slots[i], toks[i][pos[i]:pos[i] + n], list(range(n))) for i, n in enumerate(step) if n]
            out = eng.step(entries).cpu()
            o = 0
            for i, n in enumerate(step):
                rows[i].append(out[o:o + n]); o += n; pos[i] += n
        eng.free_slots(slots)
        return [torch.cat(r).numpy() for r in rows]

    whole = run([(37, 12)])
    for got, ref in zip(whole, want):
        helpers.assert_close(got, ref, "float32", "toy parts: engine vs plain")
    cut = run([(25, 7)] + [(1, 1)] * 5 + [(7, 0)])
    for got, ref in zip(cut, want):
        helpers.assert_close(got, ref, "float32", "toy parts: cut vs plain")
    # the position encoding matters: with another base the logits move
    eng.model.blocks[1].mixer.position.base = 9.0
    eng.model.blocks[1].mixer.position.load(None, DEV, torch.float32)
    moved = run([(37, 12)])
    assert np.abs(moved[0] - whole[0]).max() > 1e-3


class ParallelMixersBlock:
    """h += attention(norm1(h)) + decayed_sum(norm1(h)); h += feed_forward(norm2(h)): two mixers in one block, one
    with keys and values in the cache, one with a fixed-size state.  The model learns both needs from the block."""

    def __init__(self, norm1, attention, running, norm2, feed_forward):
        from hymt2sharp_b200.parts import build_part
        self.norm1, self.norm2 = build_part("norm", norm1), build_part("norm", norm2)
        self.attention, self.running = build_part("mixer", attention), build_part("mixer", running)
        self.feed_forward = build_part("feed_forward", feed_forward)
        self.graph_safe = False   # the running sum is plain torch on the host's lists

    def _parts(self):
        return (self.norm1, self.attention, self.running, self.norm2, self.feed_forward)

    def tensors(self):
        t = {}
        for p in self._parts():
            t.update(p.tensors())
        return t

    def load(self, weights, device, dtype):
        for p in self._parts():
            p.load(weights, device, dtype)

    def cache_needs(self):
        return [self.attention.cache_need(), self.running.cache_need()]

    def state_bytes(self):
        return [self.attention.state_bytes(), self.running.state_bytes()]

    def forward(self, residual, ctx, slots):
        x = self.norm1.forward(residual, ctx, ctx.dtype)   # both mixers read the same normed input
        self.attention.forward(x, residual, ctx, slots[0])
        self.running.forward(x, residual, ctx, slots[1])
        self.feed_forward.forward(self.norm2.forward(residual, ctx, ctx.dtype), residual, ctx)


def test_a_block_with_two_mixers(tmp_path):
    from hymt2sharp_b200.config import register_architecture
    from hymt2sharp_b200.engine.engine import Engine, StepEntry
    from hymt2sharp_b200.engine.model import DecoderModel
    from hymt2sharp_b200.engine.spec import ModelSpec
    from hymt2sharp_b200.parts import PartSpec, register_part
    from hymt2sharp_b200.weights import write_safetensors
    from test_gpu_toy_mixer import DecaySumMixer

    register_part("mixer", "toy_decay_sum", DecaySumMixer)
    register_part("block", "toy_parallel_mixers", ParallelMixersBlock)
    H, W, V, DECAY = 48, 12, 61, 0.8

    def spec(cfg=None):
        layers = []
        for l in range(3):
            p = f"l{l}."
            norm = lambda n: PartSpec("rmsnorm", dict(dim=H, eps=EPS, weight=p + n))
            attn = PartSpec("gqa_attention", dict(hidden=H, heads=2, kv_heads=1, head_dim=24, eps=EPS, qk_norm=False,
                                                  position=None, q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", o_proj=p + "o"))
            ffn = PartSpec("swiglu", dict(hidden=H, intermediate=56, gate_proj=p + "g", up_proj=p + "u", down_proj=p + "d"))
            if l == 1:   # the middle layer is one of the library's own blocks
                layers.append(PartSpec("pre_norm", dict(norm1=norm("n1"), mixer=attn, norm2=norm("n2"), feed_forward=ffn)))
            else:
                run = PartSpec("toy_decay_sum", dict(hidden=H, width=W, decay=DECAY, proj=p + "proj", out=p + "out"))
                layers.append(PartSpec("toy_parallel_mixers", dict(norm1=norm("n1"), attention=attn, running=run,
                                                                   norm2=norm("n2"), feed_forward=ffn)))
        # the embedding rows are scaled and so are the logits: both are plain numbers of the spec
        return ModelSpec(V, H, "emb", layers, PartSpec("rmsnorm", dict(dim=H, eps=EPS, weight="norm")), head=None,
                         embed_scale=3.0, logit_scale=0.25)

    class Cfg:
        architecture = "ToyTwoMixersForCausalLM"

        @classmethod
        def from_dict(cls, data, source="config.json"):
            return cls()

    register_architecture(Cfg.architecture, Cfg, spec, lambda cfg: DecoderModel(spec()).tensors())
    (tmp_path / "config.json").write_text(json.dumps(dict(architectures=[Cfg.architecture])))
    gen = torch.Generator().manual_seed(9)
    tensors = {}
    for name, ts in DecoderModel(spec()).tensors().items():
        t = torch.randn(ts.shape, generator=gen) / math.sqrt(ts.shape[-1])
        tensors[name] = ((1.0 + 0.1 * t) if ts.init == "gain" else t).to(torch.bfloat16)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    w = {n: t.float() for n, t in tensors.items()}

    eng = Engine(str(tmp_path), dtype="float32", max_tokens=512)
    m = eng.model
    assert not m.graph_safe and len(m.groups) == 1 and m.groups[0].planes == 3     # three attention mixers, one group
    assert [[s.state_bytes for s in row] for row in m.slots] == [[0, 4 * W], [0], [0, 4 * W]]
    assert m.state_bytes == 2 * 4 * W

    def plain(tokens):
        T = len(tokens)
        h = w["emb"][torch.tensor(tokens)] * 3.0
        for l in range(3):
            p = f"l{l}."
            x = rms_norm(h, w[p + "n1"], EPS)
            q, k, v = ((x @ w[p + n].T).reshape(T, -1, 24) for n in "qkv")
            add = causal_attention(q, k, v) @ w[p + "o"].T
            if l != 1:
                u, state = x @ w[p + "proj"].T, torch.zeros(W)
                for t in range(T):
                    state = DECAY * state + u[t]
                    add[t] += state @ w[p + "out"].T
            h = h + add
            x = rms_norm(h, w[p + "n2"], EPS)
            h = h + swiglu(x @ w[p + "g"].T, x @ w[p + "u"].T) @ w[p + "d"].T
        return (0.25 * rms_norm(h, w["norm"], EPS) @ w["emb"].T).numpy()

    toks = [helpers.random_tokens(V, 50, 1), helpers.random_tokens(V, 9, 2)]
    for cuts in ([(50, 9)], [(20, 3), (1, 1), (1, 1), (28, 4)]):
        slots = eng.alloc_slots(2)
        rows, pos = [[], []], [0, 0]
        for step in cuts:
            entries = [StepEntry(slots[i], toks[i][pos[i]:pos[i] + n], list(range(n))) for i, n in enumerate(step) if n]
            out = eng.step(entries).cpu()
            o = 0
            for i, n in enumerate(step):
                rows[i].append(out[o:o + n]); o += n; pos[i] += n
        eng.free_slots(slots)
        for i in range(2):
            helpers.assert_close(torch.cat(rows[i]).numpy(), plain(toks[i]), "float32", f"two mixers, cut {cuts[0]}, sequence {i}")
    # generation goes the eager way for a model that says it is not safe to capture
    out = eng.generate([toks[1]], max_new_tokens=4)
    assert len(out.results[0].tokens) == 4
    eng.check()
