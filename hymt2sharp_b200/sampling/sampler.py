"""Sampling of a batch on the GPU.

A BatchSampler holds, for the sequences of one batch, what sdcb/HyMT2Sharp's Sampler
holds for one (src/HyMT2Sharp/Sampling.cs:41-66): the options, the xoshiro256**
stream and the ring of recent tokens for the repetition penalty — as device
arrays with one row per sequence.  `sample` turns the logits of the sequences that
are still running into one token each without leaving the device.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams


class BatchSampler:
    def __init__(self, params: list[SamplingParams], device, prompts: list | None = None):
        for p in params:
            p.validate()
        self.params = list(params)
        self.device = torch.device(device)
        n = len(params)
        self._argmax_scratch = None
        self.all_greedy = all(p.greedy for p in params)
        self.any_filter = any(p.needs_filter for p in params)
        f32 = lambda vals: torch.tensor(vals, dtype=torch.float32, device=self.device)
        # 0 marks a greedy row for the kernels
        self.inv_temperature = f32([0.0 if p.greedy else float(np.float32(1.0) / np.float32(p.temperature))
                                    for p in params])
        if not self.all_greedy:
            seeds = [p.seed if p.seed is not None else int.from_bytes(os.urandom(8), "little") for p in params]
            seeds = np.array([s & ((1 << 64) - 1) for s in seeds], dtype=np.uint64).view(np.int64)
            self.rng = torch.zeros((n, 4), dtype=torch.int64, device=self.device)
            ops.seed_rng(self.rng, torch.arange(n, dtype=torch.int32, device=self.device),
                         torch.from_numpy(seeds).to(self.device))
        if self.any_filter:
            self.top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32, device=self.device)
            self.top_p = f32([p.top_p for p in params])
            self.min_p = f32([p.min_p for p in params])
            self.penalty = f32([p.repeat_penalty if p.penalty_window > 0 else 1.0 for p in params])
            width = max([p.penalty_window for p in params if p.repeat_penalty != 1.0] or [0])
            self.history = None
            if width > 0:
                # rows with a shorter window than `width` keep their own ring inside the first entries
                host = np.full((n, width), -1, dtype=np.int32)
                counts = np.zeros(n, dtype=np.int32)
                self.windows = [p.penalty_window if p.repeat_penalty != 1.0 else 0 for p in params]
                if len(set(w for w in self.windows if w > 0)) > 1:
                    raise ValueError("sequences of one batch must share one penalty_window")
                if prompts is not None:  # Sampling.cs:67-74: the prompt's tail is history too
                    for i, (p, prompt) in enumerate(zip(params, prompts)):
                        if self.windows[i] > 0:
                            tail = list(prompt)[-self.windows[i]:]
                            host[i, :len(tail)] = tail
                            counts[i] = len(tail)
                self.history = torch.from_numpy(host).to(self.device)
                self.counts = torch.from_numpy(counts).to(self.device)

    def sample(self, logits: torch.Tensor, row_map: torch.Tensor | None, out: torch.Tensor | None = None) -> torch.Tensor:
        """One token per row of `logits`; row_map[r] names the sequence (row of this sampler)
        that logits row r belongs to, None = row r is sequence r.  Changes `logits` in place
        when filters are on."""
        rows = logits.shape[0]
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if self.any_filter:
            ops.filter_logits(logits, self.inv_temperature, self.top_k, self.top_p, self.min_p, self.penalty,
                              self.history, row_map)
        ops.argmax(out, logits, row_map, self.ensure_argmax_scratch(rows, logits.shape[1]))
        if not self.all_greedy:
            ops.sample(out, logits, self.inv_temperature, self.rng, row_map)
        if self.any_filter and self.history is not None:
            ops.record_history(self.history, self.counts, out, row_map, rows)
        return out

    # -- fixed buffers for captured graphs -----------------------------------------------------------
    _TENSORS = ("inv_temperature", "rng", "top_k", "top_p", "min_p", "penalty", "history", "counts")

    def signature(self) -> tuple:
        """Two samplers with the same signature launch the same kernels on tensors of the same shapes."""
        width = self.history.shape[1] if self.any_filter and self.history is not None else 0
        return (len(self.params), self.all_greedy, self.any_filter, width)

    def tensors(self) -> dict:
        """The device tensors that sampling reads and writes, by name."""
        return {n: getattr(self, n) for n in self._TENSORS if isinstance(getattr(self, n, None), torch.Tensor)}

    def adopt(self, tensors: dict, argmax_scratch=None) -> None:
        """Moves this sampler's state into the given tensors (same names and shapes, e.g. the ones a
        captured graph points to) and uses them from now on."""
        for name, t in tensors.items():
            t.copy_(getattr(self, name))
            setattr(self, name, t)
        if argmax_scratch is not None:
            self._argmax_scratch = argmax_scratch

    def ensure_argmax_scratch(self, rows: int, vocab: int):
        need = rows * (-(-vocab // ops.ARGMAX_PIECE))
        if self._argmax_scratch is None or self._argmax_scratch[0].numel() < need:
            self._argmax_scratch = (torch.empty(need, dtype=torch.float32, device=self.device),
                                    torch.empty(need, dtype=torch.int32, device=self.device))
        return self._argmax_scratch

    def snapshot(self):
        """The state that sampling changes (random streams, penalty rings), to put back later."""
        rng = self.rng.clone() if not self.all_greedy else None
        hist = (self.history.clone(), self.counts.clone()) if self.any_filter and self.history is not None else None
        return rng, hist

    def restore(self, snap) -> None:
        rng, hist = snap
        if rng is not None:
            self.rng.copy_(rng)
        if hist is not None:
            self.history.copy_(hist[0])
            self.counts.copy_(hist[1])
