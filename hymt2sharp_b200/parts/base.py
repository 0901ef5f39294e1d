"""What the parts of a layer have in common.

A layer is put together from parts: a *mixer* (attention here), a
*feed-forward*, *norms*, a *position encoding*, and a *block* that arranges
them.  Every part gets its sizes and constants as parameters, names the
checkpoint tensors it reads, and computes on what a StepContext tells it
about the running step.  No part knows which model it is in.

Interfaces (duck-typed, see the classes in this package for examples):

  every part
      tensors() -> {checkpoint name: TensorSpec}
      load(weights: {name: CPU tensor}, device, dtype) -> None
  norm
      forward(x [rows, dim], ctx, out_dtype, rows_index=None) -> [rows, dim]
  position encoding
      kernel_epilogue(ctx) -> RotaryEpilogue or None
          what the kernels that append k and v can do on the way (rotate-half pairs by a table of
          frequencies); None: the encoding has no such form and rotates q and k itself in `apply`
      apply(qkv, ctx, heads, kv_heads, head_dim) -> None   (in place; used when kernel_epilogue() is None)
  mixer
      cache_need() -> GroupSpec or None      (planes is filled in by the model)
      state_bytes() -> int                   (fixed-size state per sequence)
      graph_safe: bool                       (its forward launches kernels on the current stream and nothing else)
      forward(x [T, hidden], residual float32 [T, hidden], ctx, slot: MixerSlot) -> None
          adds its output to `residual`
  feed-forward
      forward(x [T, hidden], residual float32 [T, hidden], ctx) -> None
  block  (it may hold any number of mixers, none included; the model asks the block, never its parts)
      cache_needs() -> [GroupSpec or None]   one entry per mixer it holds, in a fixed order
      state_bytes() -> [int]                 one entry per mixer, same order
      graph_safe: bool                       every part it holds is graph_safe
      forward(residual, ctx, slots: [MixerSlot]) -> None     slots[i] belongs to the i-th mixer

New kinds are added with `register_part(category, kind, factory)`; a model
spec names parts by (category, kind) and gives the factory's parameters.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

import torch

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block")
_REGISTRY: dict[tuple[str, str], Callable] = {}


def register_part(category: str, kind: str, factory: Callable) -> None:
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category '{category}' (known: {', '.join(CATEGORIES)})")
    _REGISTRY[(category, kind)] = factory


def build_part(category: str, spec: "PartSpec"):
    try:
        factory = _REGISTRY[(category, spec.kind)]
    except KeyError:
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise ValueError(f"unknown {category} kind '{spec.kind}' (known: {', '.join(known)})") from None
    return factory(**spec.params)


@dataclass
class PartSpec:
    kind: str
    params: dict = field(default_factory=dict)


@dataclass
class RotaryEpilogue:
    """A position encoding in the form that the kernels take which rotate q and k while they append k and v to the
    cache: dims i and i + rope_dim/2 are a pair, rotated by position * inv_freq[i]; dims from rope_dim on stay."""
    inv_freq: torch.Tensor | None     # float32 [rope_dim / 2] on the device; None with rope_dim 0
    rope_dim: int
    pairing: str = "half"             # the only pairing the kernels know; anything else is refused by them

    @staticmethod
    def none() -> "RotaryEpilogue":
        return RotaryEpilogue(None, 0)


@dataclass
class Prenormed:
    """An RMSNorm's output in two pieces, left behind by the product that last changed the residual rows: `normed` =
    bf16(x * gain) [T, dim] and `ss` = partial sums of squares of x's rows [T, tiles].  The product that consumes it applies
    the row scale 1 / sqrt(sum(ss) / dim + eps) to its own sums (kernels.ops.gemm_tc, `row_scale`), so the norm never runs
    as a kernel.  Only parts that say `takes_prenormed = True` are handed one; `materialize()` gives the plain tensor."""
    normed: torch.Tensor
    ss: torch.Tensor
    dim: int
    eps: float
    source: torch.Tensor          # the residual rows it was made from
    norm: object                  # the norm part it stands for

    @property
    def shape(self):
        return self.normed.shape

    @property
    def dtype(self):
        return self.normed.dtype

    @property
    def device(self):
        return self.normed.device

    def row_scale(self) -> tuple:
        return (self.ss, self.dim, self.eps)

    def materialize(self, ctx) -> torch.Tensor:
        return self.norm.forward(self.source, ctx, self.normed.dtype, fresh=True)


@dataclass
class MixerSlot:
    """Where one run of a mixer keeps what it remembers."""
    group: int | None = None      # cache group of its keys and values
    plane: int | None = None      # its plane inside the group
    writes: bool = True           # False: it reads the plane that another run wrote
    state_offset: int = 0         # byte offset of its fixed-size state in a sequence's state row
    state_bytes: int = 0


@dataclass
class StepContext:
    """One step as the parts see it.  All index tensors are int32 on the device.

    The step runs T new tokens of B sequences; sequence b contributes the tokens
    cu_seqlens[b]..cu_seqlens[b+1], sits in cache slot slot_ids[b] (or -1 for a
    padding row) and is kv_lens[b] tokens long once this step's tokens are in."""
    device: torch.device
    dtype: torch.dtype
    num_tokens: int
    num_seqs: int
    tokens: torch.Tensor
    token_seq: torch.Tensor
    token_pos: torch.Tensor
    cu_seqlens: torch.Tensor
    slot_ids: torch.Tensor
    kv_lens: torch.Tensor
    max_new_tokens: int          # the longest sequence's new tokens
    max_kv_len: int              # the longest sequence after the step (an upper bound is allowed)
    cache: object                # cache.PagedCache
    status: torch.Tensor         # int32 [4] device error word(s)
    host_slots: list = field(default_factory=list)       # the same facts on the host, for parts
    host_new_tokens: list = field(default_factory=list)  # that plan their work there
    host_starts: list = field(default_factory=list)
    # a hint from whoever arranges the parts: the weights that the next large kernel AFTER the running part will
    # stream (or None); a part that leaves the memory idle towards its end may ask for them ahead of time
    # (kernels.ops.prefetch_beside)
    weights_ahead: torch.Tensor | None = None
    # what parts worked out from the step's tokens and other parts of the same kind can use again, by key: the
    # angles of a rotary table, say, are the same in every layer that rotates by that table
    shared: dict = field(default_factory=dict)
    # An RMSNorm can be folded into the products around it (see Prenormed).  Whoever arranges the parts names the norm that
    # will be applied next to the residual rows (`norm_ahead`: set by a block around its mixer and its feed-forward; the
    # model names `next_first_norm`, the first norm of the block after this one); a part whose last product adds into the
    # residual may then leave a Prenormed in `prenormed`, and that norm hands it on instead of running.
    norm_ahead: object = None
    next_first_norm: object = None
    prenormed: object = None

    @property
    def decode(self) -> bool:
        return self.max_new_tokens == 1

    def state_view(self, slot: MixerSlot, dtype: torch.dtype, shape: tuple) -> torch.Tensor:
        """The state rows of all slots as [max_slots, *shape] of `dtype`."""
        raw = self.cache.state[:, slot.state_offset: slot.state_offset + slot.state_bytes]
        return raw.view(dtype).view(raw.shape[0], *shape)
