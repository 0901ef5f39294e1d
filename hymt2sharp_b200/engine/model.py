"""A decoder model put together from a ModelSpec: token embedding, the layers in
their order, the final norm and the output head.  It owns the weights and says
what cache and state it needs; the step function drives it."""
from __future__ import annotations

import torch

from ..cache.allocator import GroupSpec
from ..kernels import ops
from ..parts.base import MixerSlot, build_part
from ..parts.linear import Linear, compute_form
from ..weights.loader import TensorSpec
from .spec import ModelSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.blocks = [build_part("block", b) for b in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.embedding = None
        self.head = None
        self.groups: list[GroupSpec] = []
        self.slots: list[list[MixerSlot]] = []   # per entry of the order: one MixerSlot for each mixer of its block
        self.state_bytes = 0
        # a step can be captured into a CUDA graph only if every part launches kernels and nothing else
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.blocks)
        self._plan_memory()

    # -- what the checkpoint must hold -----------------------------------------
    def tensors(self) -> dict[str, TensorSpec]:
        s = self.spec
        t = {s.embedding: TensorSpec((s.vocab, s.hidden))}
        for b in self.blocks:
            t.update(b.tensors())
        t.update(self.final_norm.tensors())
        if s.head is not None:
            t[s.head] = TensorSpec((s.vocab, s.hidden))
        elif s.head_copy is not None:
            t[s.head_copy] = TensorSpec((s.vocab, s.hidden), optional=True, same_as=s.embedding)
        return t

    # -- cache planes and state offsets of every run ---------------------------
    def _plan_memory(self) -> None:
        """Walks the order: every mixer of every run gets its state bytes and, if it keeps keys and values, a
        plane in the group of its needs (or the plane of the run whose cache it reads).  The blocks answer;
        the model never looks inside one."""
        keys: list[tuple] = []
        planes: list[int] = []
        specs: list[GroupSpec] = []
        offset = 0
        for i, run in enumerate(self.spec.order):
            block = self.blocks[run.layer]
            needs, states = list(block.cache_needs()), list(block.state_bytes())
            if len(needs) != len(states):
                raise ValueError(f"layer {run.layer}: cache_needs() and state_bytes() must have one entry per mixer")
            row = []
            for j, (need, sb) in enumerate(zip(needs, states)):
                slot = MixerSlot()
                if sb:
                    offset = -(-offset // 16) * 16
                    slot.state_offset, slot.state_bytes = offset, int(sb)
                    offset += int(sb)
                if need is not None:
                    if run.cache_from is not None:
                        src_needs = list(self.blocks[self.spec.order[run.cache_from].layer].cache_needs())
                        if j >= len(src_needs) or src_needs[j] is None or src_needs[j].key() != need.key():
                            raise ValueError(f"order[{i}] cannot read the cache of entry {run.cache_from}: different needs")
                        src = self.slots[run.cache_from][j]
                        slot.group, slot.plane, slot.writes = src.group, src.plane, False
                    else:
                        if need.key() not in keys:
                            keys.append(need.key())
                            planes.append(0)
                            specs.append(need)
                        g = keys.index(need.key())
                        slot.group, slot.plane = g, planes[g]
                        planes[g] += 1
                row.append(slot)
            self.slots.append(row)
        self.groups = [GroupSpec(s.kind, s.kv_heads, s.head_dim, planes[g], s.window) for g, s in enumerate(specs)]
        self.state_bytes = offset

    # -- weights ------------------------------------------------------------------
    def load(self, weights: dict, device, dtype: torch.dtype) -> None:
        s = self.spec
        self.embedding = compute_form(weights[s.embedding], device, dtype)
        for b in self.blocks:
            b.load(weights, device, dtype)
        self.final_norm.load(weights, device, dtype)
        self.head = Linear(self.embedding if s.head is None else compute_form(weights[s.head], device, dtype), role="head")
        if dtype == torch.bfloat16:
            # a tensor stored in 32-bit stays so; for a MATRIX that means its product runs on the CUDA-core kernel,
            # many times slower than the tensor cores.  That is a property of the checkpoint worth saying aloud.
            wide = [name for name, spec in self.tensors().items()
                    if len(spec.shape) == 2 and name in weights and weights[name].dtype == torch.float32]
            if wide:
                import warnings
                warnings.warn(f"{len(wide)} matrices of the checkpoint are stored in 32-bit (first: {wide[0]}); the bfloat16 "
                              f"engine keeps them so and computes their products on CUDA cores, not on the tensor cores. "
                              f"Store them in bfloat16 for full speed.", RuntimeWarning, stacklevel=2)

    def streamed_weight_bytes(self) -> int:
        """Bytes of weights that a step reads whatever its tokens are: every layer that runs,
        the final norm and the output head (an embedding table that is not the head is only
        read row by row and is left out)."""
        seen: set[int] = set()
        total = 0

        def visit(obj, depth=0):
            nonlocal total
            if isinstance(obj, torch.Tensor):
                if obj.is_floating_point() and obj.data_ptr() not in seen:
                    seen.add(obj.data_ptr())
                    total += obj.numel() * obj.element_size()
            elif isinstance(obj, (list, tuple)):
                for v in obj:
                    visit(v, depth + 1)
            elif hasattr(obj, "__dict__") and depth < 6:
                for v in vars(obj).values():
                    visit(v, depth + 1)

        for layer in sorted({run.layer for run in self.spec.order}):
            visit(self.blocks[layer])
        visit(self.final_norm)
        visit(self.head)
        return total

    # -- one step -----------------------------------------------------------------
    def forward(self, ctx, want_rows: torch.Tensor | None, num_want: int) -> torch.Tensor:
        """Runs the step's tokens through all layers; returns float32 logits [num_want, vocab]
        of the token rows that `want_rows` names (int32, device)."""
        T = ctx.num_tokens
        residual = torch.empty((T, self.spec.hidden), dtype=torch.float32, device=ctx.device)
        ops.embed(residual, self.embedding, ctx.tokens, ctx.status, self.spec.embed_scale or 1.0)
        order = self.spec.order
        for i, (run, slots) in enumerate(zip(order, self.slots)):
            # the first norm of the block that runs next, for a block whose last product can prepare it (parts.base.Prenormed)
            nxt = self.blocks[order[i + 1].layer] if i + 1 < len(order) else None
            ctx.next_first_norm = getattr(nxt, "first_norm", lambda: None)() if nxt is not None else None
            self.blocks[run.layer].forward(residual, ctx, slots)
        ctx.next_first_norm = ctx.prenormed = None
        ops.join_beside(ctx.device)   # what parts asked into L2 on the side stream
        if num_want == 0:
            return torch.empty((0, self.spec.vocab), dtype=torch.float32, device=ctx.device)
        # a model that scales its logits gives the factor to the final norm: (s * norm(x)) W = s * (norm(x) W)
        scale = {} if self.spec.logit_scale is None else {"scale": float(self.spec.logit_scale)}
        normed = self.final_norm.forward(residual, ctx, ctx.dtype, rows_index=want_rows, rows=num_want, **scale)
        return self.head(normed, out_dtype=torch.float32)
