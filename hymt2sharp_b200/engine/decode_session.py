"""Decoding of a running batch without a host round trip per token.

After the prompts' step a DecodeSession owns the batch: its token ids, positions and
lengths live in device buffers that the decode step reads and that the step itself
moves on (the sampler writes the next tokens into the token buffer, a small kernel
adds one to positions and lengths).  The host only reserves cache blocks ahead and,
when asked, reads the sampled tokens.  The whole step (all layers, head, sampler,
advance) is captured once per batch size into a CUDA graph and replayed; the idea of
recording the decode step once and patching a small parameter buffer is the one of
src/HyMT2Sharp/Backends/Vulkan/VulkanBackend.cs:400-568,1091-1102.

Rows of finished sequences are marked with slot -1 ("padding"): kernels skip them, so
the batch keeps its shape and the graph stays valid while sequences end early.
"""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from ..parts.base import StepContext


class DecodeSession:
    def __init__(self, engine, slots: list, sampler, first_tokens: torch.Tensor, max_total_len: int,
                 use_graph: bool = True, live_rows=None):
        self.engine = engine
        self.cache = engine.cache
        self.sampler = sampler
        self.slots = list(slots)
        self.rows = len(slots)
        self.live = [live_rows is None or r in live_rows for r in range(self.rows)]
        self.use_graph = use_graph
        dev = engine.device
        B = self.rows
        lens = [self.cache.length(s) if alive else 0 for s, alive in zip(slots, self.live)]
        slots = [s if alive else -1 for s, alive in zip(slots, self.live)]
        self.lengths = list(lens)
        # one buffer, fixed offsets: tokens | token_seq | token_pos | cu_seqlens | slot_ids | kv_lens | want
        host = np.concatenate([np.zeros(B), np.arange(B), np.asarray(lens), np.arange(B + 1), np.asarray(slots),
                               np.asarray(lens) + 1, np.arange(B)]).astype(np.int32)
        self.meta = torch.from_numpy(host).to(dev)
        o = [0, B, 2 * B, 3 * B, 4 * B + 1, 5 * B + 1, 6 * B + 1, 7 * B + 1]
        v = [self.meta[o[i]:o[i + 1]] for i in range(7)]
        self.tokens, self.token_seq, self.token_pos, self.cu, self.slot_ids, self.kv_lens, self.want = v
        self.tokens.copy_(first_tokens.to(torch.int32))
        self.row_map = torch.tensor([r if alive else -1 for r, alive in enumerate(self.live)], dtype=torch.int32,
                                    device=dev)
        self.max_total_len = int(max_total_len)
        self.graph = None
        self.graph_layout = None
        self.logits = None
        self.kernels_per_step = 0
        self.steps = 0
        # pinned staging for callers that feed and read token ids on the host every step
        self._host_in = torch.zeros(B, dtype=torch.int32).pin_memory()
        self._host_out = torch.zeros(B, dtype=torch.int32).pin_memory()

    # -- host bookkeeping ---------------------------------------------------------
    def _reserve(self) -> None:
        plan = [(s, 1) for s, alive in zip(self.slots, self.live) if alive]
        self.cache.begin_step(plan)
        self._plan = plan

    def _commit(self) -> None:
        self.cache.end_step(self._plan)
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
        self.slot_ids.index_fill_(0, idx, -1)
        self.row_map.index_fill_(0, idx, -1)
        self.engine.free_slots([self.slots[r] for r in rows])

    # -- the step -----------------------------------------------------------------
    def _context(self) -> StepContext:
        return StepContext(device=self.engine.device, dtype=self.engine.dtype, num_tokens=self.rows,
                           num_seqs=self.rows, tokens=self.tokens, token_seq=self.token_seq,
                           token_pos=self.token_pos, cu_seqlens=self.cu, slot_ids=self.slot_ids, kv_lens=self.kv_lens,
                           max_new_tokens=1, max_kv_len=self.max_total_len, cache=self.cache,
                           status=self.engine.status, host_slots=self.slots, host_new_tokens=[1] * self.rows,
                           host_starts=self.lengths)

    def _launch(self) -> None:
        self.logits = self.engine.model.forward(self._context(), self.want, self.rows)
        self.sampler.sample(self.logits, self.row_map, out=self.tokens)
        ops.advance_decode(self.token_pos, self.kv_lens, self.slot_ids)

    def step(self) -> torch.Tensor:
        """One token for every live row; returns the device buffer [rows] that now holds the
        sampled tokens (also the next step's input).  Asynchronous."""
        if self.max_total_len < max(l for l, a in zip(self.lengths, self.live) if a) + 1:
            raise RuntimeError("the session was opened for shorter sequences")
        with torch.cuda.device(self.engine.device):
            self._reserve()
            if not self.use_graph or not self.engine.model.graph_safe:
                self._launch()
            else:
                if self.graph is None or self.graph_layout != self.cache.layout_version:
                    self._capture()
                else:
                    self.graph.replay()
                    ops.launches += self.kernels_per_step
            self._commit()
        self.steps += 1
        return self.tokens

    def step_host(self, tokens_by_row: dict | None = None) -> list:
        """The step for a caller on the host: sends the given last tokens {row: token id} from
        pinned memory, runs the step, reads the sampled tokens back and waits for them."""
        if tokens_by_row:
            self._host_in.copy_(self._host_out)
            for r, t in tokens_by_row.items():
                self._host_in[r] = int(t)
            self.tokens.copy_(self._host_in, non_blocking=True)
        self.step()
        self._host_out.copy_(self.tokens, non_blocking=True)
        torch.cuda.current_stream(self.engine.device).synchronize()
        return self._host_out.tolist()

    def _capture(self) -> None:
        # one eager step first (it also sets up what kernels set up at their first launch), then
        # the capture, which runs nothing: the state that the eager step changed is put back
        saved = self.meta.clone()
        rng = self.sampler.snapshot()
        stream = torch.cuda.Stream(device=self.engine.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            self._launch()
        torch.cuda.current_stream().wait_stream(stream)
        self.meta.copy_(saved)
        self.sampler.restore(rng)
        before = ops.launches
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=stream):
            self._launch()
        self.kernels_per_step = ops.launches - before
        self.graph_layout = self.cache.layout_version
        self.graph.replay()
