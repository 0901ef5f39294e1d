"""A weight matrix [out, in] and the choice of the matrix-product kernel for it."""
from __future__ import annotations

import torch

from ..kernels import fast, ops
from .base import Prenormed


def compute_form(t: torch.Tensor, device, dtype: torch.dtype) -> torch.Tensor:
    """A stored tensor as the engine computes with it: the 32-bit path widens everything
    to float32; the bfloat16 path keeps each tensor as it is stored (bfloat16, or 32-bit
    where the checkpoint has 32-bit)."""
    t = t.to(device)
    if dtype == torch.float32 and t.is_floating_point():
        t = t.to(torch.float32)
    return t.contiguous()


# Whether products that add into the residual prepare the norm that follows them (parts.base.Prenormed).  A switch, so that
# the two ways can be timed and compared against each other; both give the same result to bfloat16 rounding.
fold_norms = True


class Linear:
    """y = epilogue(x @ W^T) with W [out, in]; for the SwiGLU epilogue W is [2*out, in]."""

    def __init__(self, weight: torch.Tensor, epilogue: int = ops.EPILOGUE_STORE, role: str | None = None):
        self.weight = weight
        self.epilogue = epilogue
        self.role = role   # what a profile books this product under
        rows = weight.shape[0]
        self.out_features = rows // 2 if epilogue == ops.EPILOGUE_SWIGLU else rows
        self.in_features = weight.shape[1]

    def __call__(self, x, out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None, ctx=None):
        """x: the activations, or a Prenormed (a norm's output in two pieces; `ctx` is then needed for the case that the
        kernel at hand cannot apply the row scale and the norm has to run after all)."""
        if out is None:
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype or x.dtype, device=x.device)
        ops.tag = self.role
        try:
            if isinstance(x, Prenormed):
                if self.epilogue != ops.EPILOGUE_ACCUMULATE and fast.try_matmul(out, x.normed, self.weight, self.epilogue, x.row_scale()):
                    return out
                x = x.materialize(ctx)
            matmul(out, x, self.weight, self.epilogue)
        finally:
            ops.tag = None
        return out

    def add_then_norm(self, x: torch.Tensor, residual: torch.Tensor, norm, ctx) -> None:
        """residual += x @ W^T.  `norm` (or None) is the norm that will be applied to the residual rows next: where the
        kernel can, it also leaves that norm's input behind (ctx.prenormed), and the norm will not run."""
        if fold_norms and ctx is not None and norm is not None and getattr(norm, "foldable", False) and getattr(norm, "gain", None) is not None \
                and norm.dim == residual.shape[1] and residual.shape[0] == x.shape[0]:
            ops.tag = self.role
            try:
                left = fast.try_matmul_then_norm(residual, x, self.weight, norm.gain)
            finally:
                ops.tag = None
            if left is not None:
                ctx.prenormed = Prenormed(left[0], left[1], norm.dim, norm.eps, residual, norm)
                return
        if ctx is not None:
            ctx.prenormed = None
        self(x, out=residual)


def matmul(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int) -> None:
    """Picks the kernel: tensor-core kernels where they take the shape and types, else CUDA cores."""
    if fast.try_matmul(out, x, w, epilogue):
        return
    ops.gemm_simt(out, x, w, epilogue)
