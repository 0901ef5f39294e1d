"""Random-weights mode: writes a model folder (config.json, model.safetensors)
from a configuration and a seed.

Matrices and embeddings are N(0, sigma); norm gains are 1 + N(0, sigma).  The
values are drawn tensor by tensor, in the order of the architecture's tensor
list, from one torch CPU generator seeded with `seed`, in float32, then stored
as bfloat16 (norm gains as float32 when `gain_dtype` says so).
"""
from __future__ import annotations

import json
import os

import torch

from .safetensors_io import write_safetensors


def write_random_model(folder: str, config, seed: int, sigma: float = 0.02,
                       gain_dtype: torch.dtype = torch.bfloat16, chunk_rows: int = 1 << 14) -> str:
    from ..config.registry import get_architecture

    arch = get_architecture(config.architecture)
    specs = arch.tensor_shapes(config)
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    tensors = {}
    for name, spec in specs.items():
        if spec.optional:
            continue
        if spec.kind != "float":
            raise ValueError(f"random weights: no rule for the integer tensor '{name}'")
        is_gain = spec.init == "gain"
        out = torch.empty(spec.shape, dtype=gain_dtype if is_gain else torch.bfloat16)
        rows = spec.shape[0]
        flat = out.reshape(rows, -1)
        for r0 in range(0, rows, chunk_rows):  # bounded float32 scratch for big tables
            r1 = min(rows, r0 + chunk_rows)
            x = torch.randn((r1 - r0, flat.shape[1]), generator=gen, dtype=torch.float32) * sigma
            if is_gain:
                x += 1.0
            flat[r0:r1] = x.to(out.dtype)
        tensors[name] = out
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed, "sigma": sigma})
    return folder
