"""A toy mixer with state of its own, defined here, is registered, built into a model and
stepped without any change to the library: a running, decayed sum of the inputs per
sequence, kept in the cache's fixed-size state area.  Not a model of anyone's."""
import json

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class DecaySumMixer:
    """state <- decay * state + x·W for every token in order; residual += state.
    State: one float32 vector of `width` per sequence."""

    def __init__(self, hidden, width, decay, proj, out):
        self.hidden, self.width, self.decay = hidden, width, float(decay)
        self.names = (proj, out)

    def tensors(self):
        from hymt2sharp_b200.weights import TensorSpec
        return {self.names[0]: TensorSpec((self.width, self.hidden)), self.names[1]: TensorSpec((self.hidden, self.width))}

    def cache_need(self):
        return None

    def state_bytes(self):
        return 4 * self.width

    def load(self, weights, device, dtype):
        self.w = weights[self.names[0]].to(device).float()
        self.o = weights[self.names[1]].to(device).float()

    def forward(self, x, residual, ctx, slot):
        state = ctx.state_view(slot, torch.float32, (self.width,))
        u = x.float() @ self.w.T
        t0 = 0
        for s, n in zip(ctx.host_slots, ctx.host_new_tokens):   # a toy: plain torch, token by token
            for t in range(t0, t0 + n):
                state[s] = self.decay * state[s] + u[t]
                residual[t] += state[s] @ self.o.T
            t0 += n


def test_toy_mixer_with_state(tmp_path):
    from hymt2sharp_b200.config import register_architecture
    from hymt2sharp_b200.config.base import ConfigReader
    from hymt2sharp_b200.engine.engine import Engine, StepEntry
    from hymt2sharp_b200.engine.model import DecoderModel
    from hymt2sharp_b200.engine.spec import ModelSpec
    from hymt2sharp_b200.parts import PartSpec, register_part
    from hymt2sharp_b200.weights import write_safetensors

    register_part("mixer", "toy_decay_sum", DecaySumMixer)

    class ToyConfig:
        architecture = "ToyDecayForCausalLM"

        def __init__(self, hidden, width, vocab, layers, decay):
            self.hidden, self.width, self.vocab, self.layers, self.decay = hidden, width, vocab, layers, decay

        @classmethod
        def from_dict(cls, data, source="config.json"):
            r = ConfigReader(data, source)
            return cls(r.integer("hidden_size"), r.integer("state_width"), r.integer("vocab_size"),
                       r.integer("num_hidden_layers"), r.number("decay"))

    def build_spec(cfg):
        layers = []
        for l in range(cfg.layers):
            p = f"l{l}."
            norm = lambda n: PartSpec("rmsnorm", dict(dim=cfg.hidden, eps=1e-5, weight=p + n))
            # layers alternate between the toy mixer and attention: mixers are chosen layer by layer
            if l % 2 == 0:
                mixer = PartSpec("toy_decay_sum", dict(hidden=cfg.hidden, width=cfg.width, decay=cfg.decay,
                                                       proj=p + "proj", out=p + "out"))
            else:
                mixer = PartSpec("gqa_attention", dict(hidden=cfg.hidden, heads=2, kv_heads=1, head_dim=16, eps=1e-5,
                                                       qk_norm=False, position=None, q_proj=p + "q", k_proj=p + "k",
                                                       v_proj=p + "v", o_proj=p + "o"))
            ffn = PartSpec("swiglu", dict(hidden=cfg.hidden, intermediate=2 * cfg.hidden, gate_proj=p + "g",
                                          up_proj=p + "u", down_proj=p + "d"))
            layers.append(PartSpec("pre_norm", dict(norm1=norm("n1"), mixer=mixer, norm2=norm("n2"), feed_forward=ffn)))
        return ModelSpec(cfg.vocab, cfg.hidden, "emb", layers,
                         PartSpec("rmsnorm", dict(dim=cfg.hidden, eps=1e-5, weight="norm")), head=None)

    register_architecture("ToyDecayForCausalLM", ToyConfig, build_spec,
                          lambda cfg: DecoderModel(build_spec(cfg)).tensors())

    cfg = dict(architectures=["ToyDecayForCausalLM"], hidden_size=48, state_width=20, vocab_size=97,
               num_hidden_layers=3, decay=0.9)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    shapes = DecoderModel(build_spec(ToyConfig.from_dict(cfg))).tensors()
    gen = torch.Generator().manual_seed(0)
    tensors = {n: ((torch.randn(s.shape, generator=gen) * 0.1) + (1.0 if s.init == "gain" else 0.0)).to(torch.bfloat16)
               for n, s in shapes.items()}
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)

    eng = Engine(str(tmp_path), dtype="float32", max_tokens=512)
    assert eng.model.state_bytes == 80 + 80 and len(eng.model.groups) == 1 and eng.model.groups[0].planes == 1
    assert [s[0].state_bytes for s in eng.model.slots] == [80, 0, 80]
    toks = [helpers.random_tokens(97, n, 3 + n) for n in (40, 9)]

    def run(cuts):
        slots = eng.alloc_slots(2)
        rows = [[], []]
        pos = [0, 0]
        for step in cuts:
            entries = []
            for i, n in enumerate(step):
                if n:
                    entries.append(StepEntry(slots[i], toks[i][pos[i]:pos[i] + n], list(range(n))))
            out = eng.step(entries).cpu()
            o = 0
            for i, n in enumerate(step):
                rows[i].append(out[o:o + n]); o += n; pos[i] += n
        eng.free_slots(slots)
        return [torch.cat(r).numpy() for r in rows]

    whole = run([(40, 9)])
    cut = run([(30, 5), (1, 1), (1, 1), (8, 2)])
    for a, b in zip(whole, cut):
        helpers.assert_close(b, a, "float32", "toy mixer: cut vs whole")
    # a slot that is used again starts from a zero state
    again = run([(40, 9)])
    for a, b in zip(whole, again):
        assert np.array_equal(a, b)
    # and the state matters: with another decay the logits move
    eng.model.blocks[0].mixer.decay = 0.5
    moved = run([(40, 9)])
    assert np.abs(moved[0] - whole[0]).max() > 1e-3
