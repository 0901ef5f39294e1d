"""Choice of the tensor-core kernels.  Each function answers whether it ran; a False
sends the caller to the general CUDA-core kernel.  A kernel that takes a shape must
give the right result for it; what it does not take it refuses here."""
from __future__ import annotations

import torch


def try_matmul(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int) -> bool:
    """bfloat16 operands with 16-byte aligned rows go to the tcgen05 kernel; anything else is refused."""
    from . import ops
    if not ops.gemm_tc_supported(out, x, w, epilogue):
        return False
    ops.gemm_tc(out, x, w, epilogue, ops.device_status(out.device))
    return True


def try_attention(out, q, k_plane, v_plane, block_table, ctx, nh, nkv, d, scale, window) -> bool:
    return False
