"""Plain, slow Hunyuan-dense forward pass: whole sequences, no cache, CPU only.

This file rests on the formulas of sdcb/HyMT2Sharp alone: that project is C#
(.NET 10) and has no Python or C build that could be imported or compiled
here, and its model class only accepts quantized GGUF matrices, so no tiny
float model can be pushed through it.  Every function cites the file:line of
the formula it restates (paths inside the HyMT2Sharp project).

It shares no code with the product package: it reads config.json with json,
the weights with the `safetensors` library, and computes with torch on the
CPU in float32 (or float64 to size tolerances).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass

import numpy as np
import torch


@dataclass
class PlainConfig:
    layers: int
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    rope_theta: float
    rope_alpha: float
    rope_dim: int
    eps: float
    qk_norm: bool
    tied: bool
    window: int  # 0 = every earlier key is visible


def read_config(folder: str) -> PlainConfig:
    """config.json keys → the hyper-parameters of src/HyMT2Sharp/ModelConfig.cs:21-51."""
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    heads = c["num_attention_heads"]
    head_dim = c.get("head_dim", c.get("attention_head_dim"))
    if head_dim is None:
        head_dim = c["hidden_size"] // heads  # ModelConfig.cs:27-29
    scaling = c.get("rope_scaling") or {}
    return PlainConfig(
        layers=c["num_hidden_layers"],
        hidden=c["hidden_size"],
        heads=heads,
        kv_heads=c.get("num_key_value_heads", heads),  # ModelConfig.cs:26
        head_dim=head_dim,
        intermediate=c["intermediate_size"],
        vocab=c["vocab_size"],
        rope_theta=float(c.get("rope_theta", 10000.0)),  # ModelConfig.cs:31
        rope_alpha=float(scaling.get("alpha", 0.0)),  # ModelConfig.cs:32
        rope_dim=int(c.get("rope_dim", head_dim)),  # ModelConfig.cs:30
        eps=float(c.get("rms_norm_eps", 1e-5)),  # ModelConfig.cs:49
        qk_norm=bool(c.get("use_qk_norm", True)),
        tied=bool(c.get("tie_word_embeddings", True)),
        window=int(c.get("sliding_window") or 0),
    )


def read_weights(folder: str, dtype=torch.float32) -> dict:
    from safetensors.torch import load_file

    tensors = load_file(os.path.join(folder, "model.safetensors"))
    return {k: v.to(dtype) for k, v in tensors.items()}


def ntk_rope_base(theta: float, alpha: float, head_dim: int) -> np.float32:
    """base = theta * alpha^(d/(d-2)) in float32 when alpha > 0 and d > 2
    (src/HyMT2Sharp/ModelConfig.cs:31-34)."""
    base = np.float32(theta)
    if alpha > 0 and head_dim > 2:
        expo = np.float32(head_dim) / np.float32(head_dim - 2)
        base = np.float32(base * np.float32(math.pow(float(np.float32(alpha)), float(expo))))
    return base


def rope_inverse_frequencies(base: np.float32, rope_dim: int) -> np.ndarray:
    """f_i = 1 / base^(i/half), i in [0, half), float32 (src/HyMT2Sharp/Ops.cs:175-177)."""
    half = rope_dim // 2
    out = np.empty(half, dtype=np.float32)
    for i in range(half):
        expo = np.float32(i) / np.float32(half)
        out[i] = np.float32(1.0) / np.float32(math.pow(float(base), float(expo)))
    return out


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * (1/sqrt(sum(x^2)/dim + eps)) * gain (src/HyMT2Sharp/Ops.cs:29-89, scale at :62)."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    scale = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return x * scale * gain


def neox_rope(x: torch.Tensor, positions: torch.Tensor, rope_dim: int, inv_freq: np.ndarray) -> torch.Tensor:
    """Rotate-half rotary embedding on x[T, heads, d] (src/HyMT2Sharp/Ops.cs:98-195):
    angle = pos * f_i as a float32 product (:184), pairs (i, i+half) (:159-164),
    dims beyond rope_dim unchanged."""
    half = rope_dim // 2
    pos32 = positions.to(torch.float32)
    angle = pos32[:, None] * torch.from_numpy(inv_freq)[None, :]  # float32 product
    cos = torch.cos(angle).to(x.dtype)[:, None, :]
    sin = torch.sin(angle).to(x.dtype)[:, None, :]
    x0 = x[..., :half]
    x1 = x[..., half:rope_dim]
    out = x.clone()
    out[..., :half] = x0 * cos - x1 * sin
    out[..., half:rope_dim] = x0 * sin + x1 * cos
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0) -> torch.Tensor:
    """q[T, nh, d], k/v[T, nkv, d] → [T, nh*d].
    scores = (q·k)/sqrt(d) with kv head = h / (nh/nkv) (src/HyMT2Sharp/Ops.cs:359-455,
    group :374, kvh :381); softmax over keys j <= t (Ops.cs:198-325; the true row
    maximum is used, the reference's -80 floor only matters when every score is
    below -80); combine = sum_j p_j v_j (Ops.cs:535-595)."""
    T, nh, d = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    scale = 1.0 / math.sqrt(d)
    out = torch.empty(T, nh, d, dtype=q.dtype)
    idx = torch.arange(T)
    visible = idx[None, :] <= idx[:, None]
    if window > 0:
        visible &= idx[None, :] > idx[:, None] - window
    for h in range(nh):
        kvh = h // g
        s = (q[:, h, :] @ k[:, kvh, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, kvh, :]
    return out.reshape(T, nh * d)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """a = gate/(1+exp(-gate)) * up (src/HyMT2Sharp/Ops.cs:999-1055, scalar form :1053)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def round_bf16(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even to bfloat16 and back (src/HyMT2Sharp/Ops.cs:658-680)."""
    return x.to(torch.bfloat16).to(x.dtype)


class PlainModel:
    """Whole-sequence forward pass of Hunyuan dense (src/HyMT2Sharp/HunyuanDenseModel.cs:342-436,
    layer body src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:14-89)."""

    def __init__(self, folder: str, dtype=torch.float32, kv_bf16: bool = False):
        self.cfg = read_config(folder)
        self.w = read_weights(folder, dtype)
        self.dtype = dtype
        self.kv_bf16 = kv_bf16
        c = self.cfg
        self.inv_freq = rope_inverse_frequencies(ntk_rope_base(c.rope_theta, c.rope_alpha, c.head_dim), c.rope_dim)

    def layer(self, h: torch.Tensor, l: int, positions: torch.Tensor) -> torch.Tensor:
        c, w = self.cfg, self.w
        p = f"model.layers.{l}."
        T = h.shape[0]
        n1 = rms_norm(h, w[p + "input_layernorm.weight"], c.eps)  # Prefill.cs:20
        q = (n1 @ w[p + "self_attn.q_proj.weight"].T).reshape(T, c.heads, c.head_dim)  # Prefill.cs:49
        k = (n1 @ w[p + "self_attn.k_proj.weight"].T).reshape(T, c.kv_heads, c.head_dim)
        v = (n1 @ w[p + "self_attn.v_proj.weight"].T).reshape(T, c.kv_heads, c.head_dim)
        q = neox_rope(q, positions, c.rope_dim, self.inv_freq)  # Prefill.cs:53-54
        k = neox_rope(k, positions, c.rope_dim, self.inv_freq)
        if c.qk_norm:  # per-head norm after the rotation, Prefill.cs:57-58
            q = rms_norm(q, w[p + "self_attn.query_layernorm.weight"], c.eps)
            k = rms_norm(k, w[p + "self_attn.key_layernorm.weight"], c.eps)
        if self.kv_bf16:  # Prefill.cs:60-61
            k, v = round_bf16(k), round_bf16(v)
        ao = causal_attention(q, k, v, c.window)  # Prefill.cs:65-83
        h = h + ao @ w[p + "self_attn.o_proj.weight"].T  # Prefill.cs:88, :23
        n2 = rms_norm(h, w[p + "post_attention_layernorm.weight"], c.eps)  # Prefill.cs:27
        gate = n2 @ w[p + "mlp.gate_proj.weight"].T  # Prefill.cs:31
        up = n2 @ w[p + "mlp.up_proj.weight"].T
        h = h + swiglu(gate, up) @ w[p + "mlp.down_proj.weight"].T  # Prefill.cs:33-34
        return h

    def hidden(self, tokens) -> torch.Tensor:
        ids = torch.as_tensor(list(tokens), dtype=torch.long)
        h = self.w["model.embed_tokens.weight"][ids]  # HunyuanDenseModel.cs:390, 494-558
        positions = torch.arange(len(ids))
        for l in range(self.cfg.layers):
            h = self.layer(h, l, positions)
        return h

    def logits(self, tokens) -> torch.Tensor:
        """Logits at every position of one sequence, [T, vocab]
        (final norm HunyuanDenseModel.cs:411-413, head :416-419 with the tied fallback)."""
        h = self.hidden(tokens)
        n = rms_norm(h, self.w["model.norm.weight"], self.cfg.eps)
        head = self.w["model.embed_tokens.weight"] if self.cfg.tied else self.w["lm_head.weight"]
        return n @ head.T


# ---------------------------------------------------------------------------
# Sampling (src/HyMT2Sharp/Sampling.cs)
# ---------------------------------------------------------------------------

_MASK = (1 << 64) - 1


class Xoshiro256StarStar:
    """Sampling.cs:375-409: SplitMix64 seeding, xoshiro256** steps, u = (next >> 40) * 2^-24."""

    def __init__(self, seed: int):
        z = seed & _MASK
        s = []
        for _ in range(4):
            z = (z + 0x9E3779B97F4A7C15) & _MASK
            x = z
            x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
            x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
            s.append(x ^ (x >> 31))
        self.s = s

    @staticmethod
    def _rotl(x, k):
        return ((x << k) | (x >> (64 - k))) & _MASK

    def next(self) -> int:
        s0, s1, s2, s3 = self.s
        r = (self._rotl((s1 * 5) & _MASK, 7) * 9) & _MASK
        t = (s1 << 17) & _MASK
        s2 ^= s0
        s3 ^= s1
        s1 ^= s2
        s0 ^= s3
        s2 ^= t
        s3 = self._rotl(s3, 45)
        self.s = [s0, s1, s2, s3]
        return r

    def next_single(self) -> np.float32:
        return np.float32(self.next() >> 40) * np.float32(1.0 / 16777216.0)


def argmax_first(logits: np.ndarray) -> int:
    """First index holding the maximum (Sampling.cs:298-334)."""
    return int(np.argmax(logits))


class PlainSampler:
    """Sampler.Sample (Sampling.cs:76-92): penalty, then argmax when temperature <= 0,
    else scale, top-k, softmax numerators, top-p/min-p, inverse-CDF walk."""

    def __init__(self, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0,
                 penalty_window=64, seed=0):
        self.t = float(temperature)
        self.top_k, self.top_p, self.min_p = int(top_k), float(top_p), float(min_p)
        self.pen, self.win_cap = float(repeat_penalty), int(penalty_window)
        self.rng = Xoshiro256StarStar(seed)
        self.window: list[int] = []
        self.last_cdf = None  # (r, cumulative sums) of the last stochastic pick, for tolerance checks

    def feed_history(self, tokens):
        """Sampling.cs:67-74."""
        if self.pen != 1.0 and self.win_cap > 0:
            for t in list(tokens)[-self.win_cap:]:
                self._record(t)

    def _record(self, t):
        if self.pen != 1.0 and self.win_cap > 0:
            self.window.append(int(t))
            self.window = self.window[-self.win_cap:]

    def sample(self, logits: np.ndarray) -> int:
        x = np.array(logits, dtype=np.float32)
        if self.pen != 1.0:  # Sampling.cs:141-156: every window entry applies, repeats included
            for t in reversed(self.window):
                if 0 <= t < len(x):
                    x[t] = x[t] * np.float32(self.pen) if x[t] <= 0 else x[t] / np.float32(self.pen)
        tok = argmax_first(x) if self.t <= 0 else self._stochastic(x)
        self._record(tok)
        return tok

    def _stochastic(self, x: np.ndarray) -> int:
        n = len(x)
        inv_t = np.float32(1.0) / np.float32(self.t)
        if inv_t != 1.0:
            x = x * inv_t  # Sampling.cs:97-99
        if 0 < self.top_k < n:  # Sampling.cs:171-225: exactly k survive, ties kept in index order
            order = np.sort(x)[::-1]
            kth = order[self.top_k - 1]
            free = self.top_k - int((x > kth).sum())
            for i in range(n):
                if x[i] < kth:
                    x[i] = -np.inf
                elif x[i] == kth:
                    if free <= 0:
                        x[i] = -np.inf
                    free -= 1
        m = x.max()
        p = np.where(np.isneginf(x), np.float32(0), np.exp(x - m, dtype=np.float32)).astype(np.float32)
        total = np.float32(0)
        for v in p:  # serial float32 sum, Sampling.cs:105-113
            total = np.float32(total + v)
        if self.top_p < 1.0 or self.min_p > 0.0:  # Sampling.cs:229-293
            ids = [i for i in range(n) if p[i] > 0]
            ids.sort(key=lambda i: (-p[i], i))
            keep = len(ids)
            if self.min_p > 0.0:
                thr = p[ids[0]] * np.float32(self.min_p)
                j = 1
                while j < keep and p[ids[j]] >= thr:
                    j += 1
                keep = j
            if self.top_p < 1.0:
                limit = np.float32(self.top_p) * total
                cum = np.float32(0)
                j = 0
                while j < keep and cum < limit:
                    cum = np.float32(cum + p[ids[j]])
                    j += 1
                keep = j
            dropped = np.float32(0)
            for i in ids[keep:]:
                dropped = np.float32(dropped + p[i])
                p[i] = 0
            total = np.float32(total - dropped)
        r = self.rng.next_single() * total  # Sampling.cs:119
        cdf = np.cumsum(p.astype(np.float64))
        self.last_cdf = (float(r), cdf, p)
        acc = np.float32(0)
        for i in range(n):  # Sampling.cs:120-129
            if p[i] <= 0:
                continue
            acc = np.float32(acc + p[i])
            if acc >= r:
                return i
        nz = np.nonzero(p > 0)[0]  # Sampling.cs:131-138
        return int(nz[-1]) if len(nz) else argmax_first(p)


def plain_generate(model: PlainModel, prompt, max_new_tokens: int, stop_ids=(), sampler: PlainSampler | None = None):
    """The caller's loop of src/HyMT2Sharp.Cli/Program.cs:84-110: the first token comes from
    the prompt's last logits, a stop token ends the reply and is not kept, max_new_tokens
    bounds the tokens kept."""
    sampler = sampler or PlainSampler(temperature=0.0)
    seq = list(prompt)
    out = []
    while len(out) < max_new_tokens:
        logits = model.logits(seq)[-1].to(torch.float32).numpy()
        tok = sampler.sample(logits)
        if tok in stop_ids:
            return out, "stop"
        out.append(tok)
        seq.append(tok)
    return out, "length"
