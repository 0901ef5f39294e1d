"""Weights by tensor name from a model folder.

The architecture says which tensors it expects (name → shape and kind); the
loader reads them from model.safetensors (or the shards that
model.safetensors.index.json lists), checks all of them, and fails with ONE
error that lists every missing tensor, every unexpected tensor and every
wrong shape.  Nothing is half-loaded: either every tensor is returned or the
error is raised.  Two kinds of extra tensors are not errors, because folders
that sdcb/HyMT2Sharp would run hold them (it looks its tensors up by name and
never asks what else a file has, src/HyMT2Sharp/HunyuanDenseModel.cs:438-443):
names that the architecture declares ignorable (buffers that are recomputed,
such as a rotary table), and a copy of another tensor under a second name
(`same_as`: an output head stored beside the embedding it is tied to), which
must then hold the same bytes.  Both are reported as warnings.

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
    same_as: str | None = None  # an optional tensor that, when present, must equal this other tensor; it is not loaded


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


def _open_files(folder: str, problems: list | None = None) -> dict[str, SafetensorsFile]:
    """tensor name → the opened file that holds it.  What the index says and the shards do not hold goes to
    `problems` as text."""
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
        for name, shard in sorted(weight_map.items()):
            if name not in files[shard].entries and problems is not None:
                where = next((s for s, f in files.items() if name in f.entries), None)
                problems.append(f"  the index places {name} in {shard}, which does not hold it" +
                                (f" ({where} does)" if where else ""))
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


def load_checkpoint(folder: str, expected: dict[str, TensorSpec], ignorable=()) -> dict[str, torch.Tensor]:
    """All expected tensors, as CPU tensors that view the mapped file.  `ignorable`: regular expressions of tensor
    names that the checkpoint may hold and the model does not read."""
    import re
    import warnings
    other: list = []
    owners = _open_files(folder, other)
    missing = [n for n, s in expected.items() if n not in owners and not s.optional]
    patterns = [re.compile(p) for p in ignorable]
    extra = [n for n in owners if n not in expected]
    ignored = [n for n in extra if any(p.fullmatch(n) for p in patterns)]
    unexpected = [n for n in extra if n not in ignored]
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
    bad = {w[0] for w in wrong_shape} | {w[0] for w in wrong_type}
    copies = [n for n, s in expected.items() if s.same_as is not None and n in owners]
    for name in copies:
        twin = expected[name].same_as
        if name in bad or twin in bad or twin not in owners:
            continue
        a, b = owners[name].tensor(name), owners[twin].tensor(twin)
        if a.dtype != b.dtype or not torch.equal(a, b):
            other.append(f"  {name} is stored beside {twin}, which the configuration ties it to, but holds other values")
    if missing or unexpected or wrong_shape or wrong_type or other:
        raise WeightError(folder, sorted(missing), sorted(unexpected), wrong_shape, wrong_type, other)
    if ignored or copies:
        warnings.warn(f"'{folder}': not read: " + ", ".join(sorted(ignored) + [f"{n} (a copy of {expected[n].same_as})" for n in copies]),
                      RuntimeWarning, stacklevel=2)
    return {name: _stored_form(owners[name].tensor(name)) for name in expected if name in owners and expected[name].same_as is None}
