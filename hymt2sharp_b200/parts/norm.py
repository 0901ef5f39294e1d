"""RMSNorm part: y = x / sqrt(mean(x^2) + eps) * gain
(src/HyMT2Sharp/Ops.cs:29-89)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import register_part
from .linear import compute_form


class RMSNorm:
    graph_safe = True  # its forward only launches kernels on the current stream
    foldable = True    # y = x * r * gain with a row scale r: the products around it can take it over (parts.base.Prenormed)

    def __init__(self, dim: int, eps: float, weight: str):
        self.dim, self.eps, self.weight_name = int(dim), float(eps), weight
        self.gain = None

    def tensors(self):
        return {self.weight_name: TensorSpec((self.dim,), init="gain")}

    def load(self, weights, device, dtype):
        self.gain = compute_form(weights[self.weight_name], device, dtype)

    def forward(self, x: torch.Tensor, ctx, out_dtype: torch.dtype, rows_index: torch.Tensor | None = None,
                rows: int | None = None, scale: float = 1.0, fresh: bool = False):
        """The normed rows; or, when the product that last changed `x` prepared this very norm, what it left behind
        (a Prenormed, for a consumer that takes one).  `fresh`: compute in any case."""
        pre = getattr(ctx, "prenormed", None)
        if pre is not None and not fresh:
            ctx.prenormed = None
            if pre.norm is self and pre.source is x and rows_index is None and scale == 1.0 and pre.normed.dtype == out_dtype:
                return pre
        n = rows if rows is not None else (rows_index.shape[0] if rows_index is not None else x.shape[0])
        out = torch.empty((n, self.dim), dtype=out_dtype, device=x.device)
        ops.rmsnorm(out, x, self.gain, self.eps, rows_index, scale)
        return out


register_part("norm", "rmsnorm", RMSNorm)
