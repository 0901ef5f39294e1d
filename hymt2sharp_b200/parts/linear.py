"""A weight matrix [out, in] and the choice of the matrix-product kernel for it."""
from __future__ import annotations

import torch

from ..kernels import ops


def compute_form(t: torch.Tensor, device, dtype: torch.dtype) -> torch.Tensor:
    """A stored tensor as the engine computes with it: the 32-bit path widens everything
    to float32; the bfloat16 path keeps each tensor as it is stored (bfloat16, or 32-bit
    where the checkpoint has 32-bit)."""
    t = t.to(device)
    if dtype == torch.float32 and t.is_floating_point():
        t = t.to(torch.float32)
    return t.contiguous()


class Linear:
    """y = epilogue(x @ W^T) with W [out, in]; for the SwiGLU epilogue W is [2*out, in]."""

    def __init__(self, weight: torch.Tensor, epilogue: int = ops.EPILOGUE_STORE, role: str | None = None):
        self.weight = weight
        self.epilogue = epilogue
        self.role = role   # what a profile books this product under
        rows = weight.shape[0]
        self.out_features = rows // 2 if epilogue == ops.EPILOGUE_SWIGLU else rows
        self.in_features = weight.shape[1]

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None):
        if out is None:
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype or x.dtype, device=x.device)
        ops.tag = self.role
        try:
            matmul(out, x, self.weight, self.epilogue)
        finally:
            ops.tag = None
        return out


def matmul(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int) -> None:
    """Picks the kernel: tensor-core kernels where they take the shape and types, else CUDA cores."""
    from ..kernels import fast
    if fast.try_matmul(out, x, w, epilogue):
        return
    ops.gemm_simt(out, x, w, epilogue)
