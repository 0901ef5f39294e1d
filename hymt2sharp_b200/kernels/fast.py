"""Choice of the tensor-core kernels.  Each function answers whether it ran; a False
sends the caller to the general CUDA-core kernel.  A kernel that takes a shape must
give the right result for it; what it does not take it refuses here."""
from __future__ import annotations

import torch

from . import ops


def try_matmul(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int, row_scale: tuple | None = None) -> bool:
    """bfloat16 operands with 16-byte aligned rows go to the tcgen05 kernel; anything else is refused.  `row_scale`: see
    ops.gemm_tc (the activations are a norm's input times its gain; the row scale is applied to the sums)."""
    if not ops.gemm_tc_supported(out, x, w, epilogue):
        return False
    ops.gemm_tc(out, x, w, epilogue, ops.device_status(out.device), row_scale=row_scale, checked=True)
    return True


def try_matmul_then_norm(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, gain: torch.Tensor):
    """out += x @ w^T on the tcgen05 kernel, which also leaves behind what the RMSNorm after it needs: returns
    (bf16(out_new * gain) [T, N], partial sums of squares [T, tiles]); or None (nothing ran) where the kernel or this
    shape's plan cannot do that."""
    T, N = out.shape
    if gain.dtype not in (torch.bfloat16, torch.float32) or out.dtype != torch.float32 or not out.is_contiguous() or N % 8:
        return None
    if not ops.gemm_tc_supported(out, x, w, ops.EPILOGUE_ACCUMULATE):
        return None
    tiles = ops.gemm_tc_norm_tiles(T, N, x.shape[1], ops.EPILOGUE_ACCUMULATE)
    if tiles == 0:
        return None
    normed = torch.empty((T, N), dtype=torch.bfloat16, device=out.device)
    ss = torch.empty((T, tiles), dtype=torch.float32, device=out.device)
    ops.gemm_tc(out, x, w, ops.EPILOGUE_ACCUMULATE, ops.device_status(out.device), norm_after=(normed, gain, ss), checked=True)
    return normed, ss


def try_project_rope_kv(x, weight, epilogue, ctx, planes, cache_dtype, block_table, q_gain, k_gain, eps, nh, nkv, d,
                        row_scale: tuple | None = None):
    """The fused q/k/v projection whose epilogue rotates, norms and appends to the cache (tcgen05, heads of 128,
    rotate-half pairs): returns q [T, nh * d], or None when that kernel does not take the operands and the caller
    goes the two-kernel way.  `planes` = (k_plane, v_plane), or (None, None) for a run that writes no keys."""
    if epilogue.pairing != "half" or x.dtype != torch.bfloat16:
        return None
    if not ops.gemm_tc_rope_kv_supported(x, weight, nh, nkv, d, cache_dtype, epilogue.rope_dim):
        return None
    T = x.shape[0]
    q = torch.empty((T, nh * d), dtype=x.dtype, device=x.device)
    angles = None
    if ops.gemm_tc_rope_kv_wants_angles(T, epilogue.rope_dim):
        # a prompt's worth of tokens: their angles once per step and table, not once per head and layer
        key = ("rotary angles", epilogue.inv_freq.data_ptr())
        angles = ctx.shared.get(key)
        if angles is None:
            angles = ctx.shared[key] = ops.rope_angles(ctx.token_pos[:T], epilogue.inv_freq)
    ops.tag = "qkv+rope"
    try:
        ops.gemm_tc_rope_kv(x, weight, q, planes[0], planes[1], block_table, ctx.cache.block_tokens, ctx.token_seq,
                            ctx.token_pos, ctx.slot_ids, epilogue.inv_freq, epilogue.rope_dim, q_gain, k_gain, eps, nh, nkv,
                            ops.device_status(x.device), angles=angles, row_scale=row_scale, checked=True)
    finally:
        ops.tag = None
    return q


DECODE_CHUNK_KEYS = 256     # keys per partial of the streaming decode kernel, a constant of the kernel
DECODE_TC_MAX_ROWS = 512       # sequences that one launch of the tcgen05 decode kernel takes
DECODE_TC_CHUNK_KEYS = 128  # keys per partial of the tensor-core decode kernel
DECODE_TC_MAX_CHUNKS = 2048  # chunks of one sequence that it takes


def try_attention(out, q, k_plane, v_plane, block_table, ctx, nh, nkv, d, scale, window) -> bool:
    """bfloat16 with head_dim 64 or 128: decode steps go to the streaming decode kernel, steps with
    longer pieces to the tcgen05 flash-attention kernel (cache blocks of 64 tokens)."""
    bt = k_plane.shape[2]
    if out.dtype != torch.bfloat16 or d not in (64, 128) or bt & (bt - 1):
        return False
    if (ctx.decode and d == 128 and bt == 64 and nh // nkv <= 16 and ctx.max_kv_len <= DECODE_TC_MAX_CHUNKS * DECODE_TC_CHUNK_KEYS
            and ctx.num_tokens <= DECODE_TC_MAX_ROWS):
        splits = max(1, -(-ctx.max_kv_len // DECODE_TC_CHUNK_KEYS))
        na, nm, nc = ops.attention_decode_tc_scratch(ctx.num_tokens, nh, nkv, d, splits)
        acc = torch.empty(na, dtype=torch.float32, device=out.device)
        ml = torch.empty(nm, dtype=torch.float32, device=out.device)
        ops.attention_decode_tc(out, q, k_plane, v_plane, block_table, ctx.slot_ids, ctx.kv_lens, nh, nkv, d, scale,
                                window, splits, acc, ml, ops.zeroed_counters(out.device, nc),
                                ops.device_status(out.device))
        return True
    if ctx.decode:
        splits = max(1, -(-ctx.max_kv_len // DECODE_CHUNK_KEYS))
        na, nm = ops.attention_simt_scratch(ctx.num_tokens, nh, d, splits)
        acc = torch.empty(na, dtype=torch.float32, device=out.device)
        ml = torch.empty(nm, dtype=torch.float32, device=out.device)
        ops.attention_decode(out, q, k_plane, v_plane, block_table, ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens,
                             nh, nkv, d, scale, window, splits, acc, ml, ops.zeroed_counters(out.device, ctx.num_tokens * nh))
        return True
    if bt == 64:
        ops.attention_prefill_tc(out, q, k_plane, v_plane, block_table, ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens,
                                 ctx.num_seqs, ctx.max_new_tokens, nh, nkv, d, scale, window,
                                 ops.device_status(out.device))
        return True
    return False
