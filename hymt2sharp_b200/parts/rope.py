"""Rotate-half (NeoX) rotary position encoding with an optional dynamic-NTK base.

frequencies f_i = 1 / base^(i / half), i in [0, half), half = rope_dim / 2
(src/HyMT2Sharp/Ops.cs:175-177); angle = position * f_i as a float32 product;
pairs (i, i + half); dims from rope_dim on are left as they are
(src/HyMT2Sharp/Ops.cs:159-164).  The base is theta, or theta * alpha^(d/(d-2))
for alpha > 0 (src/HyMT2Sharp/ModelConfig.cs:31-34), and arrives here already
computed.  The table of frequencies is built once on the host and handed to the
kernel that rotates q and k while it appends k and v to the cache.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import RotaryEpilogue, register_part


_TABLES: dict = {}   # (device, the frequencies' bytes) -> their tensor on the device


class NeoXRotary:
    def __init__(self, head_dim: int, rope_dim: int, base: float):
        if rope_dim % 2 or rope_dim > head_dim or rope_dim < 0:
            raise ValueError(f"rope_dim {rope_dim} must be even and at most head_dim {head_dim}")
        self.head_dim, self.rope_dim, self.base = int(head_dim), int(rope_dim), float(base)
        half = self.rope_dim // 2
        freq = np.empty(half, dtype=np.float32)
        base32 = np.float32(self.base)
        for i in range(half):
            expo = np.float32(i) / np.float32(half)
            freq[i] = np.float32(1.0) / np.float32(math.pow(float(base32), float(expo)))
        self._host = freq
        self.inv_freq = None

    def tensors(self):
        return {}

    def load(self, weights, device, dtype):
        # layers with the same frequencies share one tensor on the device: what a step works out from a table
        # (the angles of its tokens) then serves all of them
        key = (str(torch.device(device)), self._host.tobytes())
        if key not in _TABLES:
            _TABLES[key] = torch.from_numpy(self._host).to(device)
        self.inv_freq = _TABLES[key]

    def kernel_epilogue(self, ctx) -> RotaryEpilogue:
        """Rotate-half pairs by a table of frequencies: exactly what the appending kernels do on the way."""
        return RotaryEpilogue(self.inv_freq if self.rope_dim else None, self.rope_dim)

    def apply(self, qkv, ctx, heads, kv_heads, head_dim):
        raise NotImplementedError("NeoXRotary is applied by the fused rotation kernel")


register_part("position", "neox_rope", NeoXRotary)
