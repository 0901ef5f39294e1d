"""The engine: a loaded model, its cache, and the one step function.

`Engine.step` runs a batch of sequences: each entry brings the next tokens of one
sequence (a whole prompt, a part of it, or one decoded token) and names the places
among them whose logits are wanted.  The step runs exactly the tokens it is given,
as one batch, on top of what earlier steps left in the cache, and returns the
float32 logits of the wanted places.  Padding changes no result: kernels see the
packed tokens and each sequence's own length.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import PagedCache
from ..config.registry import load_config
from ..kernels import build as kernel_build, ops
from ..parts.base import StepContext
from ..weights.loader import load_checkpoint
from .model import DecoderModel

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class EngineError(RuntimeError):
    pass


@dataclass
class StepEntry:
    slot: int
    tokens: list
    want: list = field(default_factory=list)  # indices into `tokens`


def require_gpu(device) -> torch.device:
    if not torch.cuda.is_available():
        raise EngineError("hymt2sharp_b200 needs a CUDA device (sm_100a); none is visible, and there is no CPU path")
    device = torch.device(device)
    major, minor = torch.cuda.get_device_capability(device)
    if major != 10:
        raise EngineError(f"the kernels are built for sm_100a; device {device} is sm_{major}{minor}")
    return device


def make_context(cache, entries: list, vocab: int, dtype, device, status, meta_buffer=None,
                 max_positions: int | None = None):
    """Checks the entries, takes the cache blocks that their tokens need (all or nothing) and
    builds the StepContext: packed tokens, each token's batch row and position, the rows'
    offsets, slots and lengths.  Returns (context, wanted rows or None, their count, plan);
    `plan` goes to cache.end_step once the step has been launched.  `max_positions`: the longest
    sequence that the model's position encoding was made for (config.json's
    max_position_embeddings); a step that would go past it is refused before anything changed."""
    # whole arrays at a time: a prompt of thousands of tokens costs the host microseconds, not one Python step a token
    tokens, token_seq, token_pos, cu, slots, kv_lens, want = [], [], [], [0], [], [], []
    starts, news = [], []
    for b, e in enumerate(entries):
        try:
            ids = np.asarray(e.tokens, dtype=np.int64).reshape(-1)
        except (OverflowError, TypeError, ValueError) as err:
            raise EngineError(f"the tokens of an entry are not integer ids: {err}") from None
        n = int(ids.shape[0])
        start = cache.length(e.slot)
        if n and (int(ids.min()) < 0 or int(ids.max()) >= vocab):
            bad = ids[(ids < 0) | (ids >= vocab)][0]
            raise EngineError(f"token id {int(bad)} is outside the vocabulary of {vocab}")
        if max_positions is not None and start + n > max_positions:
            raise EngineError(f"slot {e.slot} would hold {start + n} tokens; the model's max_position_embeddings is "
                              f"{max_positions}")
        for w in e.want:
            if not (0 <= int(w) < n):
                raise EngineError(f"wanted place {w} is outside the {n} tokens of the entry")
            want.append(cu[-1] + int(w))
        tokens.append(ids.astype(np.int32))
        token_seq.append(np.full(n, b, dtype=np.int32))
        token_pos.append(np.arange(start, start + n, dtype=np.int32))
        cu.append(cu[-1] + n)
        slots.append(e.slot)
        kv_lens.append(start + n)
        starts.append(start)
        news.append(n)
    num_tokens = cu[-1]
    tokens, token_seq, token_pos = (np.concatenate(a) for a in (tokens, token_seq, token_pos))
    plan = list(zip(slots, news))
    cache.begin_step(plan)  # raises CacheFull before anything changed
    arrays = [np.asarray(a, dtype=np.int32) for a in (tokens, token_seq, token_pos, cu, slots, kv_lens, want)]
    sizes = [len(a) for a in arrays]
    total = sum(sizes)
    meta = meta_buffer(total) if meta_buffer is not None else torch.empty(total, dtype=torch.int32, device=device)
    meta[:total].copy_(torch.from_numpy(np.concatenate(arrays)))
    v, o = [], 0
    for n in sizes:
        v.append(meta[o:o + n])
        o += n
    ctx = StepContext(device=torch.device(device), dtype=dtype, num_tokens=num_tokens, num_seqs=len(entries),
                      tokens=v[0], token_seq=v[1], token_pos=v[2], cu_seqlens=v[3], slot_ids=v[4], kv_lens=v[5],
                      max_new_tokens=max(news), max_kv_len=max(kv_lens), cache=cache, status=status,
                      host_slots=slots, host_new_tokens=news, host_starts=starts)
    return ctx, (v[6] if want else None), len(want), plan


class Engine:
    def __init__(self, model_dir: str, dtype="bfloat16", max_tokens: int = 8192, max_batch: int = 8,
                 block_tokens: int = 64, device="cuda:0", max_sequence_tokens: int | None = None,
                 spec_override=None):
        if dtype not in DTYPES:
            raise EngineError(f"dtype must be 'bfloat16' or 'float32', got {dtype!r}")
        self.dtype = DTYPES[dtype]
        self.device = require_gpu(device)
        kernel_build.load_library()  # fails loudly when the CUDA library cannot be built or loaded
        self.architecture, self.config = load_config(model_dir)
        spec = self.architecture.build_spec(self.config) if spec_override is None else spec_override(self.config)
        self.model = DecoderModel(spec)
        weights = load_checkpoint(model_dir, self.model.tensors(), spec.ignorable_tensors)
        with torch.cuda.device(self.device):
            self.model.load(weights, self.device, self.dtype)
            self.cache = PagedCache(self.model.groups, self.dtype, self.device, capacity_tokens=max_tokens,
                                    block_tokens=block_tokens, max_slots=max_batch,
                                    state_bytes=self.model.state_bytes, max_sequence_tokens=max_sequence_tokens)
            self.status = ops.device_status(self.device)
            self._meta = torch.zeros(4096, dtype=torch.int32, device=self.device)
        self.vocab = spec.vocab
        self.max_positions = spec.max_positions
        self.steps_run = 0

    # -- slots ------------------------------------------------------------------
    def alloc_slots(self, n: int) -> list[int]:
        with torch.cuda.device(self.device):
            return self.cache.alloc_slots(n)

    def free_slots(self, slots) -> None:
        self.cache.free_slots(list(slots))

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def truncate(self, slot: int, length: int) -> None:
        """Forgets the sequence in `slot` from position `length` on; the next step of that slot goes on from
        there (src/HyMT2Sharp/HunyuanDenseModel.cs:187-240, TruncateCache).  Whole blocks behind the new end go
        back to the pool.  A layer group with a window may already have handed back blocks that the shorter
        sequence would need again: that is refused (CacheError), nothing changes."""
        with torch.cuda.device(self.device):
            self.cache.truncate(slot, int(length))

    def reset(self, slot: int) -> None:
        """The slot keeps its place in the batch and starts over as an empty sequence (ResetCache)."""
        self.truncate(slot, 0)

    # -- the step ---------------------------------------------------------------
    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        """Runs one step; returns float32 logits [wanted places, vocab] on the device, in the
        order of the entries and of each entry's `want`."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            ctx, want, num_want, plan = make_context(self.cache, entries, self.vocab, self.dtype, self.device,
                                                     self.status, self._meta_buffer, self.max_positions)
            logits = self.model.forward(ctx, want, num_want)
            self.cache.end_step(plan)
        self.steps_run += 1
        return logits

    def _meta_buffer(self, n: int) -> torch.Tensor:
        if n > self._meta.numel():
            self._meta = torch.zeros(max(n, 2 * self._meta.numel()), dtype=torch.int32, device=self.device)
        return self._meta

    def check(self) -> None:
        """Waits for the device and raises if a kernel flagged a fault (a token id outside the
        embedding table, a bounded wait that gave up).  The engine stays usable: the status word is
        cleared, and so are the arrival counters that kernels share between launches (a kernel that
        gave up may have left them half counted, and every kernel relies on finding them at zero);
        what the faulted step computed is not to be trusted, the cache keeps the tokens it was given."""
        code = int(self.status[0].item())
        if code != 0:
            with torch.cuda.device(self.device):
                self.status.zero_()
                ops.reset_counters(self.device)
            raise EngineError(f"a kernel reported device status {code}")

    # -- convenience --------------------------------------------------------------
    def generate(self, prompts, **kwargs):
        from .generate import generate
        return generate(self, prompts, **kwargs)
