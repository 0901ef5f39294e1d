"""The description of a model that the engine builds from: which parts make up
each layer, in which order the layers run, and where the embedding, the final
norm and the output head come from.  An architecture's builder turns its
configuration into this; nothing below it knows the architecture."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..parts.base import PartSpec


@dataclass
class Run:
    """One entry of the order in which layers run.  A layer may be named by several
    entries (it then runs several times with the same weights, each run with a cache
    plane of its own), and an entry may read the cache plane that an earlier entry
    wrote (`cache_from` = that entry's index in the order) instead of writing one."""
    layer: int
    cache_from: int | None = None


@dataclass
class ModelSpec:
    vocab: int
    hidden: int
    embedding: str                    # checkpoint name of the [vocab, hidden] table
    layers: list[PartSpec]            # block specs (category "block")
    final_norm: PartSpec
    head: str | None                  # checkpoint name of the [vocab, hidden] head; None = the embedding table
    order: list[Run] = field(default_factory=list)
    max_positions: int | None = None  # the longest sequence the model takes (None: whatever the cache holds)
    embed_scale: float | None = None  # the embedding rows are multiplied by this (None: as they are)
    logit_scale: float | None = None  # the logits are multiplied by this (None: as they are)
    # regular expressions of tensor names that checkpoints of this architecture may hold and the model does not read
    ignorable_tensors: list[str] = field(default_factory=list)
    head_copy: str | None = None      # with a tied head: the name under which a checkpoint may store the head once more

    def __post_init__(self):
        if not self.order:
            self.order = [Run(i) for i in range(len(self.layers))]
        for i, run in enumerate(self.order):
            if not (0 <= run.layer < len(self.layers)):
                raise ValueError(f"order[{i}] names layer {run.layer}, the model has {len(self.layers)}")
            if run.cache_from is not None:
                if not (0 <= run.cache_from < i):
                    raise ValueError(f"order[{i}] reads the cache of entry {run.cache_from}, which does not run before it")
                if self.order[run.cache_from].cache_from is not None:
                    raise ValueError(f"order[{i}] reads the cache of entry {run.cache_from}, which has none of its own")
