"""Grouped-query causal attention over the paged cache, as a mixer part.

q, k, v = x·Wq^T, x·Wk^T, x·Wv^T (one fused product); position encoding on q
and k; optional per-head RMSNorm of q and k after it; k, v appended to the
cache; softmax((q·k)/sqrt(d)) over the visible keys; · v; output projection
added to the residual stream
(src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:38-89).  An optional window limits
the visible keys to the last `window` positions.
"""
from __future__ import annotations

import math

import torch

from ..cache.allocator import GroupSpec
from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import MixerSlot, PartSpec, Prenormed, RotaryEpilogue, build_part, register_part
from .linear import Linear, compute_form

SPLIT_KEYS = 256  # decode: keys per partial, a constant so that the cut depends on nothing else


class GQAAttention:
    graph_safe = True  # its forward only launches kernels on the current stream
    takes_prenormed = True  # x may be a parts.base.Prenormed: the projection applies the norm's row scale itself

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, eps: float, qk_norm: bool,
                 position: PartSpec | None, q_proj: str, k_proj: str, v_proj: str, o_proj: str,
                 q_norm: str | None = None, k_norm: str | None = None, window: int | None = None):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} kv heads")
        if head_dim % 8 or head_dim > 256:   # what the general kernels take; the tensor-core kernels take 64 and 128
            raise ValueError(f"head_dim {head_dim} must be a multiple of 8, at most 256")
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, head_dim
        self.eps, self.qk_norm, self.window = float(eps), bool(qk_norm), int(window or 0)
        self.names = dict(q=q_proj, k=k_proj, v=v_proj, o=o_proj, qn=q_norm, kn=k_norm)
        self.position = build_part("position", position) if position is not None else None
        self.scale = 1.0 / math.sqrt(head_dim)  # src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:64
        self.qkv = self.out = self.q_gain = self.k_gain = None

    # -- what it needs ----------------------------------------------------------
    def tensors(self):
        qd, kd, h, n = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.hidden, self.names
        t = {n["q"]: TensorSpec((qd, h)), n["k"]: TensorSpec((kd, h)), n["v"]: TensorSpec((kd, h)),
             n["o"]: TensorSpec((h, qd))}
        if self.qk_norm:
            t[n["qn"]] = TensorSpec((self.head_dim,), init="gain")
            t[n["kn"]] = TensorSpec((self.head_dim,), init="gain")
        if self.position is not None:
            t.update(self.position.tensors())
        return t

    def cache_need(self):
        kind = "window" if self.window > 0 else "full"
        return GroupSpec(kind, self.kv_heads, self.head_dim, planes=0, window=self.window)

    def state_bytes(self) -> int:
        return 0

    def load(self, weights, device, dtype):
        n = self.names
        fused = torch.cat([weights[n["q"]], weights[n["k"]], weights[n["v"]]], dim=0)
        self.qkv = Linear(compute_form(fused, device, dtype), role="qkv")
        self.out = Linear(compute_form(weights[n["o"]], device, dtype), ops.EPILOGUE_ACCUMULATE, role="o_proj")
        if self.qk_norm:
            self.q_gain = compute_form(weights[n["qn"]], device, dtype)
            self.k_gain = compute_form(weights[n["kn"]], device, dtype)
            if self.q_gain.dtype != self.k_gain.dtype:
                self.q_gain, self.k_gain = self.q_gain.float(), self.k_gain.float()
        if self.position is not None:
            self.position.load(weights, device, dtype)

    # -- the step ---------------------------------------------------------------
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, slot: MixerSlot) -> None:
        from ..kernels import fast
        T = ctx.num_tokens
        nh, nkv, d = self.heads, self.kv_heads, self.head_dim
        # the position encoding in the form that the appending kernels take, or None: it rotates q and k itself
        epilogue = self.position.kernel_epilogue(ctx) if self.position is not None else RotaryEpilogue.none()
        k_plane, v_plane = ctx.cache.plane(slot.group, slot.plane)
        block_table = ctx.cache.tables[slot.group]
        planes = (k_plane, v_plane) if slot.writes else (None, None)
        q = None
        pre = x if isinstance(x, Prenormed) else None
        if epilogue is not None and x.shape[0] == T:
            # projection, rotation, norm and cache append as one kernel, where the kernels have one for the shape
            q = fast.try_project_rope_kv(pre.normed if pre else x, self.qkv.weight, epilogue, ctx, planes, k_plane.dtype,
                                         block_table, self.q_gain, self.k_gain, self.eps, nh, nkv, d,
                                         row_scale=pre.row_scale() if pre else None)
        if q is None:
            qkv = self.qkv(x, ctx=ctx)
            if epilogue is None:
                self.position.apply(qkv, ctx, nh, nkv, d)
                epilogue = RotaryEpilogue.none()
            q = torch.empty((T, nh * d), dtype=qkv.dtype, device=qkv.device)
            ops.rope_kv(qkv, q, planes[0], planes[1], block_table, ctx.cache.block_tokens, ctx.token_seq, ctx.token_pos,
                        ctx.slot_ids, epilogue.inv_freq, epilogue.rope_dim, self.q_gain, self.k_gain, self.eps, nh, nkv, d)
        out = torch.empty((T, nh * d), dtype=q.dtype, device=q.device)
        self.attend(out, q, k_plane, v_plane, block_table, ctx)
        if ctx.decode and ctx.weights_ahead is not None:
            # the feed-forward's first weights come into L2 beside the output projection and the norm, which leave
            # the memory idle; the request starts once the attention is through (not earlier: its last loads and
            # the folding of its partials are sensitive to traffic)
            ops.prefetch_beside(ctx.weights_ahead)
        self.out.add_then_norm(out, residual, getattr(ctx, "norm_ahead", None), ctx)

    def attend(self, out, q, k_plane, v_plane, block_table, ctx) -> None:
        from ..kernels import fast
        nh, nkv, d = self.heads, self.kv_heads, self.head_dim
        if fast.try_attention(out, q, k_plane, v_plane, block_table, ctx, nh, nkv, d, self.scale, self.window):
            return
        split, max_splits, acc, ml = 0, 0, None, None
        if ctx.decode and ctx.max_kv_len > SPLIT_KEYS:
            split = SPLIT_KEYS
            max_splits = -(-ctx.max_kv_len // SPLIT_KEYS)
            na, nm = ops.attention_simt_scratch(ctx.num_tokens, nh, d, max_splits)
            acc = torch.empty(na, dtype=torch.float32, device=out.device)
            ml = torch.empty(nm, dtype=torch.float32, device=out.device)
        ops.attention_simt(out, q, k_plane, v_plane, block_table, ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens,
                           ctx.num_seqs, ctx.max_new_tokens, nh, nkv, d, self.scale, self.window, split,
                           max_splits, acc, ml)


register_part("mixer", "gqa_attention", GQAAttention)
