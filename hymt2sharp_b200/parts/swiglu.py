"""Dense SwiGLU feed-forward: residual += (silu(x·Wg^T) * (x·Wu^T)) · Wd^T
(src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:27-34, src/HyMT2Sharp/Ops.cs:1053).
Gate and up are one product over the stacked weight [2F, H] whose epilogue applies
the activation, so the [T, 2F] intermediate never reaches memory."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import register_part
from .linear import Linear, compute_form


class SwiGLU:
    graph_safe = True  # its forward only launches kernels on the current stream
    takes_prenormed = True  # x may be a parts.base.Prenormed: the gate/up product applies the norm's row scale itself

    def __init__(self, hidden: int, intermediate: int, gate_proj: str, up_proj: str, down_proj: str):
        self.hidden, self.intermediate = int(hidden), int(intermediate)
        self.names = dict(g=gate_proj, u=up_proj, d=down_proj)
        self.gate_up = self.down = None

    def tensors(self):
        h, f, n = self.hidden, self.intermediate, self.names
        return {n["g"]: TensorSpec((f, h)), n["u"]: TensorSpec((f, h)), n["d"]: TensorSpec((h, f))}

    def load(self, weights, device, dtype):
        n = self.names
        stacked = torch.cat([weights[n["g"]], weights[n["u"]]], dim=0)
        self.gate_up = Linear(compute_form(stacked, device, dtype), ops.EPILOGUE_SWIGLU, role="gate_up")
        self.down = Linear(compute_form(weights[n["d"]], device, dtype), ops.EPILOGUE_ACCUMULATE, role="down")

    def first_weights(self):
        """The weights that this part's first kernel streams."""
        return self.gate_up.weight if self.gate_up is not None else None

    def forward(self, x, residual: torch.Tensor, ctx) -> None:
        act = self.gate_up(x, ctx=ctx)
        self.down.add_then_norm(act, residual, getattr(ctx, "norm_ahead", None), ctx)


register_part("feed_forward", "swiglu", SwiGLU)
