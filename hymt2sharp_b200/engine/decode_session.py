"""Decoding of a running batch without a host round trip per token.

After the prompts' step a DecodeSession owns the batch: its token ids, positions and
lengths live in device buffers that the decode step reads and that the step itself
moves on (the sampler writes the next tokens into the token buffer, a small kernel
adds one to positions and lengths).  The host only reserves cache blocks ahead and,
when asked, reads the sampled tokens.  The whole step (all layers, head, sampler,
advance) is captured once per batch shape into a CUDA graph and replayed; the idea of
recording the decode step once and patching a small parameter buffer is the one of
src/HyMT2Sharp/Backends/Vulkan/VulkanBackend.cs:400-568,1091-1102.  The graph and
the buffers it points to belong to the engine (a DecodeSlot per batch size, length
bound and kind of sampling), so the next batch of the same shape replays at once.

Rows of finished sequences are marked with slot -1 ("padding"): kernels skip them, so
the batch keeps its shape and the graph stays valid while sequences end early.
"""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from ..parts.base import StepContext

LENGTH_BUCKET = 1024   # the length bound of a captured step is rounded up to this: fewer captures


class DecodeSlot:
    """The fixed buffers of a decode step of `rows` sequences, and the graph captured on them."""

    def __init__(self, engine, rows: int, max_total_len: int):
        dev = engine.device
        B = rows
        self.rows, self.max_total_len = rows, max_total_len
        # one buffer, fixed offsets: tokens | token_seq | token_pos | cu_seqlens | slot_ids | row_map | kv_lens | want
        # (slot_ids and row_map lie side by side: together they say which rows run, and go to the device in one copy)
        self.meta = torch.zeros(8 * B + 1, dtype=torch.int32, device=dev)
        o = [0, B, 2 * B, 3 * B, 4 * B + 1, 5 * B + 1, 6 * B + 1, 7 * B + 1, 8 * B + 1]
        v = [self.meta[o[i]:o[i + 1]] for i in range(8)]
        self.tokens, self.token_seq, self.token_pos, self.cu, self.slot_ids, self.row_map, self.kv_lens, self.want = v
        self.rows_running = self.meta[o[4]:o[6]]
        self.host_in = torch.zeros(B, dtype=torch.int32).pin_memory()
        self.host_out = torch.zeros(B, dtype=torch.int32).pin_memory()
        # for steps that are launched ahead of the host: two sets of pinned buffers and events that take turns
        self.host_running = [torch.zeros(2 * B, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.host_tokens = [torch.zeros(B, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.copied = [torch.cuda.Event() for _ in range(2)]
        self.sampler_tensors = None
        self.argmax_scratch = None
        self.graph = None
        self.graph_layout = None
        self.logits = None
        self.kernels_per_step = 0


def decode_slot(engine, rows: int, max_total_len: int, sampler) -> DecodeSlot:
    bound = -(-max_total_len // LENGTH_BUCKET) * LENGTH_BUCKET
    key = (rows, bound, sampler.signature())
    slots = engine.__dict__.setdefault("_decode_slots", {})
    if key not in slots:
        slots[key] = DecodeSlot(engine, rows, bound)
    return slots[key]


class DecodeSession:
    def __init__(self, engine, slots: list, sampler, first_tokens: torch.Tensor, max_total_len: int,
                 use_graph: bool = True, live_rows=None):
        self.engine = engine
        self.cache = engine.cache
        self.sampler = sampler
        self.slots = list(slots)
        self.rows = len(slots)
        self.live = [live_rows is None or r in live_rows for r in range(self.rows)]
        self.use_graph = use_graph and engine.model.graph_safe
        self._timed_graph, self._timed_events, self._timed_layout = None, [], None
        B = self.rows
        lens = [self.cache.length(s) if alive else 0 for s, alive in zip(slots, self.live)]
        dev_slots = [s if alive else -1 for s, alive in zip(slots, self.live)]
        self.lengths = list(lens)
        with torch.cuda.device(engine.device):
            self.buf = decode_slot(engine, B, max_total_len, sampler)
            self.max_total_len = self.buf.max_total_len
            row_map = [r if alive else -1 for r, alive in enumerate(self.live)]
            host = np.concatenate([np.zeros(B), np.arange(B), np.asarray(lens), np.arange(B + 1), np.asarray(dev_slots),
                                   np.asarray(row_map), np.asarray(lens) + 1, np.arange(B)]).astype(np.int32)
            self.buf.meta.copy_(torch.from_numpy(host))
            self.buf.tokens.copy_(first_tokens.to(torch.int32))
            if self.buf.sampler_tensors is None:   # the first batch of this shape lends its tensors to the slot
                self.buf.sampler_tensors = sampler.tensors()
                self.buf.argmax_scratch = sampler.ensure_argmax_scratch(B, engine.vocab)
            else:
                sampler.adopt(self.buf.sampler_tensors, self.buf.argmax_scratch)
        self.steps = 0
        self._reserved = False   # whether the blocks of the coming step are already taken

    # -- what the step reads --------------------------------------------------------
    @property
    def tokens(self) -> torch.Tensor:
        return self.buf.tokens

    @property
    def kernels_per_step(self) -> int:
        return self.buf.kernels_per_step

    # -- host bookkeeping ---------------------------------------------------------
    def _plan(self) -> list:
        return [(s, 1) for s, alive in zip(self.slots, self.live) if alive]

    def _reserve(self) -> None:
        self.cache.begin_step(self._plan())
        self._reserved = True

    def _reserve_ahead(self) -> None:
        """Blocks for the step after this one, taken while this one runs on the device.  A row that ends
        meanwhile gives them back with its slot; a cache too full for it is asked again when the step comes."""
        from ..cache.allocator import CacheFull
        if self.max_total_len < max((l for l, a in zip(self.lengths, self.live) if a), default=0) + 1:
            return
        try:
            self._reserve()
        except CacheFull:
            self._reserved = False

    def _commit(self) -> None:
        self.cache.end_step(self._plan())
        self._reserved = False
        for i, alive in enumerate(self.live):
            if alive:
                self.lengths[i] += 1

    def drop(self, rows: list) -> None:
        """Sequences that ended: their rows become padding and their slots go back."""
        rows = [r for r in rows if self.live[r]]
        if not rows:
            return
        for r in rows:
            self.live[r] = False
        idx = torch.tensor(rows, dtype=torch.int64, device=self.engine.device)
        self.buf.slot_ids.index_fill_(0, idx, -1)
        self.buf.row_map.index_fill_(0, idx, -1)
        self.engine.free_slots([self.slots[r] for r in rows])

    # -- the step -----------------------------------------------------------------
    def _context(self) -> StepContext:
        b = self.buf
        return StepContext(device=self.engine.device, dtype=self.engine.dtype, num_tokens=self.rows,
                           num_seqs=self.rows, tokens=b.tokens, token_seq=b.token_seq, token_pos=b.token_pos,
                           cu_seqlens=b.cu, slot_ids=b.slot_ids, kv_lens=b.kv_lens, max_new_tokens=1,
                           max_kv_len=self.max_total_len, cache=self.cache, status=self.engine.status,
                           host_slots=self.slots, host_new_tokens=[1] * self.rows, host_starts=self.lengths)

    def _launch(self) -> None:
        b = self.buf
        b.logits = self.engine.model.forward(self._context(), b.want, self.rows)
        self.sampler.sample(b.logits, b.row_map, out=b.tokens)
        ops.advance_decode(b.token_pos, b.kv_lens, b.slot_ids)

    def step(self) -> torch.Tensor:
        """One token for every live row; returns the device buffer [rows] that now holds the
        sampled tokens (also the next step's input).  Asynchronous."""
        if self.max_total_len < max((l for l, a in zip(self.lengths, self.live) if a), default=0) + 1:
            raise RuntimeError("the session was opened for shorter sequences")
        with torch.cuda.device(self.engine.device):
            if not self._reserved:
                self._reserve()
            if not self.use_graph:
                self._launch()
            elif ops.profile_active():
                self._step_profiled()
            elif self.buf.graph is None or self.buf.graph_layout != self.cache.layout_version:
                self._capture()
            else:
                self.buf.graph.replay()
                ops.launches += self.buf.kernels_per_step
            self._commit()
            self._reserve_ahead()
        self.steps += 1
        return self.buf.tokens

    def step_host(self, tokens_by_row: dict | None = None) -> list:
        """The step for a caller on the host: sends the given last tokens {row: token id} from
        pinned memory, runs the step, reads the sampled tokens back and waits for them."""
        b = self.buf
        if tokens_by_row:
            staged = b.host_out.numpy().copy()
            for r, t in tokens_by_row.items():
                staged[r] = t
            b.host_in.numpy()[:] = staged
            b.tokens.copy_(b.host_in, non_blocking=True)
        self.step()
        b.host_out.copy_(b.tokens, non_blocking=True)
        torch.cuda.current_stream(self.engine.device).synchronize()
        return b.host_out.tolist()

    def step_async(self) -> int:
        """The step for a caller that does not want to wait for it: which rows still run goes to the device from pinned
        memory, the step runs on the tokens that the step before left on the device, and the sampled tokens start their
        way to pinned host memory.  Returns a ticket for wait().  At most two steps may be in flight."""
        b = self.buf
        k = self.steps & 1
        running = b.host_running[k].numpy()
        for r, alive in enumerate(self.live):
            running[r] = self.slots[r] if alive else -1
            running[self.rows + r] = r if alive else -1
        with torch.cuda.device(self.engine.device):
            b.rows_running.copy_(b.host_running[k], non_blocking=True)
            self.step()
            b.host_tokens[k].copy_(b.tokens, non_blocking=True)
            b.copied[k].record()
        return k

    def wait(self, ticket: int) -> list:
        """The tokens that the step of this ticket sampled, one for every row of the batch (rows that do not run keep
        what they held)."""
        self.buf.copied[ticket].synchronize()
        return self.buf.host_tokens[ticket].tolist()

    def _step_profiled(self) -> None:
        """The step while kernels are being timed: a graph of this session's own, captured with a clock stamp behind every
        kernel, replayed and read.  The graph that unprofiled steps share is left alone."""
        if self._timed_graph is None or self._timed_layout != self.cache.layout_version:
            self._timed_graph, self._timed_events = self._capture_graph(timed=True)
            self._timed_layout = self.cache.layout_version
        self._timed_graph.replay()
        ops.launches += self.buf.kernels_per_step
        ops.book_captured(self._timed_events)

    def _capture(self) -> None:
        b = self.buf
        b.graph, _ = self._capture_graph(timed=False)
        b.graph_layout = self.cache.layout_version
        b.graph.replay()

    def _capture_graph(self, timed: bool):
        # one eager step first (it also sets up what kernels set up at their first launch), then
        # the capture, which runs nothing: the state that the eager step changed is put back
        b = self.buf
        saved = b.meta.clone()
        rng = self.sampler.snapshot()
        stream = torch.cuda.Stream(device=self.engine.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream), ops.profile_suspended():
            self._launch()
        torch.cuda.current_stream().wait_stream(stream)
        b.meta.copy_(saved)
        self.sampler.restore(rng)
        before = ops.launches
        graph, events = torch.cuda.CUDAGraph(), []
        with torch.cuda.graph(graph, stream=stream):
            if timed:
                ops.capture_begin(self.engine.device)
            try:
                self._launch()
            finally:
                events = ops.capture_end() if timed else []
        b.kernels_per_step = ops.launches - before
        return graph, events
