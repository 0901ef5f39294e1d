"""Weights by tensor name from a model folder.

The architecture says which tensors it expects (name → shape and kind); the
loader reads them from model.safetensors (or the shards that
model.safetensors.index.json lists), checks all of them, and fails with ONE
error that lists every missing tensor, every unexpected tensor and every
wrong shape.  Nothing is half-loaded: either every tensor is returned or the
error is raised.

Stored types: bfloat16 stays bfloat16, a tensor stored in 32-bit float stays
32-bit, float16/float64 become bfloat16/float32, integer tables become int32.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


@dataclass(frozen=True)
class TensorSpec:
    shape: tuple
    kind: str = "float"  # "float" or "int"
    optional: bool = False
    init: str = "normal"  # random-weights rule: "normal" = N(0, sigma), "gain" = 1 + N(0, sigma)


class WeightError(ValueError):
    """The checkpoint does not match the architecture; lists all that is wrong."""

    def __init__(self, folder, missing=(), unexpected=(), wrong_shape=(), wrong_type=(), other=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_type = list(wrong_type)
        lines = [f"weights in '{folder}' do not match the architecture:"]
        lines += list(other)
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, want, got in self.wrong_type:
            lines.append(f"  wrong type: {name} is stored as {got}, expected a {want} tensor")
        super().__init__("\n".join(lines))


def _open_files(folder: str) -> dict[str, SafetensorsFile]:
    """tensor name → the opened file that holds it."""
    index = os.path.join(folder, "model.safetensors.index.json")
    single = os.path.join(folder, "model.safetensors")
    owners: dict[str, SafetensorsFile] = {}
    if os.path.exists(single):
        f = SafetensorsFile(single)
        for n in f.names():
            owners[n] = f
    elif os.path.exists(index):
        with open(index) as fh:
            weight_map = json.load(fh).get("weight_map", {})
        files: dict[str, SafetensorsFile] = {}
        for shard in sorted(set(weight_map.values())):
            files[shard] = SafetensorsFile(os.path.join(folder, shard))
        for f in files.values():
            for n in f.names():
                owners[n] = f
    else:
        raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json found")
    return owners


def _stored_form(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32, torch.int32):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    return t.to(torch.int32)


def load_checkpoint(folder: str, expected: dict[str, TensorSpec]) -> dict[str, torch.Tensor]:
    """All expected tensors, as CPU tensors that view the mapped file."""
    owners = _open_files(folder)
    missing = [n for n, s in expected.items() if n not in owners and not s.optional]
    unexpected = [n for n in owners if n not in expected]
    wrong_shape, wrong_type = [], []
    for name, spec in expected.items():
        if name not in owners:
            continue
        e = owners[name].entries[name]
        if tuple(e["shape"]) != tuple(spec.shape):
            wrong_shape.append((name, tuple(spec.shape), tuple(e["shape"])))
        is_float = e["dtype"] in ("BF16", "F16", "F32", "F64")
        if (spec.kind == "float") != is_float or e["dtype"] == "BOOL":
            wrong_type.append((name, spec.kind, e["dtype"]))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(folder, sorted(missing), sorted(unexpected), wrong_shape, wrong_type)
    return {name: _stored_form(owners[name].tensor(name)) for name in expected if name in owners}
