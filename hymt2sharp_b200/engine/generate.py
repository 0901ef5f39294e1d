"""The generation loop: batches of unequal prompts, stop tokens, sequences that end
earlier than others, and as many batches one after another as there are requests.

The loop is the one that sdcb/HyMT2Sharp's callers write around Forward
(src/HyMT2Sharp.Cli/Program.cs:84-110): the prompt's last logits give the first
token; a stop token ends the reply and is not kept; the token limit ends it with
"length".  Here it runs for a whole batch: all prompts in one step, then one token
for every sequence that is still running.  The loop's decisions are plain Python
over token ids (`BatchState`, `plan_batches`); the device work sits behind a
stepper object, so the decisions can be tested without a GPU.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

from ..sampling.params import GREEDY, SamplingParams


@dataclass
class GenerationResult:
    tokens: list
    finish_reason: str          # "stop" or "length"
    prompt_tokens: int


@dataclass
class GenerationStats:
    batches: int = 0
    prefill_tokens: int = 0
    prefill_ms: float = 0.0
    decode_tokens: int = 0      # tokens produced by decode steps
    decode_steps: int = 0
    decode_ms: float = 0.0
    profile: dict = field(default_factory=dict)   # with profiling on: {"prefill" | "decode": {kernel or product: ms}}

    def line(self) -> str:
        """The timing line of src/HyMT2Sharp.Cli/Program.cs:121-126."""
        pre = f"prefill tokens={self.prefill_tokens}  {self.prefill_ms:.1f} ms  " \
              f"{self.prefill_tokens / max(self.prefill_ms, 1e-9) * 1000.0:.2f} tok/s"
        if self.decode_tokens > 0:
            return pre + f"  |  decode tokens={self.decode_tokens}  {self.decode_ms:.1f} ms  " \
                         f"{self.decode_tokens / max(self.decode_ms, 1e-9) * 1000.0:.2f} tok/s"
        return pre + "  |  decode tokens=0"


@dataclass
class GenerationOutput:
    results: list
    stats: GenerationStats

    def __iter__(self):
        return iter(self.results)

    def __getitem__(self, i):
        return self.results[i]

    def __len__(self):
        return len(self.results)


def plan_batches(prompt_lens: list, max_new_tokens: int, max_batch: int, capacity_tokens: int,
                 block_tokens: int) -> list:
    """Cuts the requests, in their order, into batches: at most `max_batch` sequences each, and
    the blocks that a batch can come to hold (prompt + max_new_tokens - 1 cached tokens per
    sequence, rounded up to whole blocks) fit the cache."""
    if max_batch <= 0:
        raise ValueError("max_batch must be positive")
    capacity_blocks = capacity_tokens // block_tokens
    batches, current, used = [], [], 0
    for i, n in enumerate(prompt_lens):
        if n <= 0:
            raise ValueError(f"request {i} has an empty prompt")
        need = -(-(n + max(0, max_new_tokens - 1)) // block_tokens)
        if need > capacity_blocks:
            raise ValueError(f"request {i} ({n} prompt tokens + {max_new_tokens} new) needs {need} cache blocks of "
                             f"{block_tokens} tokens; the cache has {capacity_blocks}")
        if current and (len(current) >= max_batch or used + need > capacity_blocks):
            batches.append(current)
            current, used = [], 0
        current.append(i)
        used += need
    if current:
        batches.append(current)
    return batches


class BatchState:
    """What the loop knows about one running batch: each sequence's kept tokens, and which
    sequences still run."""

    def __init__(self, request_ids: list, prompt_lens: list, max_new_tokens: int, stop_token_ids):
        self.request_ids = list(request_ids)
        self.max_new_tokens = int(max_new_tokens)
        self.stop = frozenset(int(t) for t in stop_token_ids)
        self.outputs = [[] for _ in request_ids]
        self.reasons = [None] * len(request_ids)
        self.prompt_lens = list(prompt_lens)
        self.live = list(range(len(request_ids)))  # rows of the batch that still run
        if self.max_new_tokens <= 0:
            for r in self.live:
                self.reasons[r] = "length"
            self.live = []

    def accept(self, tokens: list) -> tuple:
        """Takes one sampled token for every live row (in the order of `live`).  Returns
        (rows that go on, rows that ended now)."""
        if len(tokens) != len(self.live):
            raise ValueError("one token for every live sequence is needed")
        go_on, ended = [], []
        for row, tok in zip(self.live, tokens):
            tok = int(tok)
            if tok in self.stop:
                self.reasons[row] = "stop"       # a stop token is not kept
                ended.append(row)
                continue
            self.outputs[row].append(tok)
            if len(self.outputs[row]) >= self.max_new_tokens:
                self.reasons[row] = "length"
                ended.append(row)
            else:
                go_on.append(row)
        self.live = go_on
        return go_on, ended

    def last_tokens(self) -> list:
        return [self.outputs[r][-1] for r in self.live]

    def results(self) -> list:
        return [GenerationResult(self.outputs[r], self.reasons[r] or "length", self.prompt_lens[r])
                for r in range(len(self.request_ids))]


class EngineStepper:
    """The device side of the loop for one batch: slots, the prompts' step, then a
    DecodeSession that keeps tokens, positions and lengths on the device."""

    def __init__(self, engine, params: list, prompts: list, max_new_tokens: int, use_graph: bool = True):
        from ..sampling.sampler import BatchSampler
        from .engine import StepEntry
        self._StepEntry = StepEntry
        self.engine = engine
        self.prompts = prompts
        self.max_new_tokens = max_new_tokens
        self.use_graph = use_graph
        self.slots = engine.alloc_slots(len(prompts))
        self.sampler = BatchSampler(params, engine.device, prompts)
        self.held = set(range(len(prompts)))
        self.session = None
        self._first = None

    def prefill(self) -> list:
        entries = [self._StepEntry(s, p, [len(p) - 1]) for s, p in zip(self.slots, self.prompts)]
        logits = self.engine.step(entries)
        self._first = self.sampler.sample(logits, None)
        return self._first.tolist()

    def decode(self, rows: list, tokens: list) -> list:
        """One more token for the batch rows `rows` (the rows that still run), whose last tokens
        are `tokens`: they go to the device from pinned memory, the sampled ones come back."""
        if self.session is None:
            from .decode_session import DecodeSession
            longest = max(len(p) for p in self.prompts) + self.max_new_tokens
            self.session = DecodeSession(self.engine, self.slots, self.sampler, self._first, longest, self.use_graph,
                                         live_rows=set(self.held))
        out = self.session.step_host(dict(zip(rows, tokens)))
        return [out[r] for r in rows]

    # -- the same without a wait in every step: launch(rows) starts a step and the copy of its tokens to the host,
    #    collect() waits for the OLDEST step that was launched and not yet collected -------------------------------
    def launch(self, rows: list) -> None:
        """One more token for the batch rows `rows`, whose last tokens are already on the device (the step before left
        them there).  What goes to the device from pinned host memory is which rows still run; nothing is waited for."""
        if self.session is None:
            from .decode_session import DecodeSession
            longest = max(len(p) for p in self.prompts) + self.max_new_tokens
            self.session = DecodeSession(self.engine, self.slots, self.sampler, self._first, longest, self.use_graph,
                                         live_rows=set(self.held))
        self._flying = getattr(self, "_flying", [])
        self._flying.append((list(rows), self.session.step_async()))

    def collect(self) -> list:
        rows, ticket = self._flying.pop(0)
        out = self.session.wait(ticket)
        return [out[r] for r in rows]

    def release(self, rows: list) -> None:
        rows = [r for r in rows if r in self.held]
        self.held.difference_update(rows)
        if self.session is not None:
            self.session.drop(rows)
        else:
            self.engine.free_slots([self.slots[r] for r in rows])

    def close(self) -> None:
        self.release(list(self.held))


def _book(stats: GenerationStats, phase: str, times: dict) -> None:
    into = stats.profile.setdefault(phase, {})
    for k, v in times.items():
        into[k] = into.get(k, 0.0) + v


def run_batch(stepper, state: BatchState, stats: GenerationStats, on_tokens=None, clock=time.perf_counter,
              profiler=None) -> None:
    """Drives one batch to its end through `stepper` (prefill(), decode(rows, tokens),
    release(rows), close()).  `profiler`: an object with profile_begin() and profile_end() -> {name: ms}
    (kernels.ops); what it measured is booked under "prefill" and "decode" in stats.profile."""
    try:
        if not state.live:
            return
        t0 = clock()
        if profiler:
            profiler.profile_begin()
        tokens = stepper.prefill()
        if profiler:
            _book(stats, "prefill", profiler.profile_end())
        stats.prefill_ms += (clock() - t0) * 1000.0
        stats.prefill_tokens += sum(state.prompt_lens)
        rows_before = list(state.live)
        go_on, ended = state.accept(tokens)
        if on_tokens:
            on_tokens([(state.request_ids[r], t) for r, t in zip(rows_before, tokens) if state.reasons[r] != "stop"])
        stepper.release(ended)
        t0 = clock()
        if profiler and state.live:
            profiler.profile_begin()
        profiling = bool(profiler and state.live)
        if hasattr(stepper, "launch") and not profiling:
            _decode_ahead(stepper, state, stats, on_tokens)
        while state.live:
            rows_before = list(state.live)
            tokens = stepper.decode(rows_before, state.last_tokens())
            stats.decode_steps += 1
            stats.decode_tokens += len(tokens)
            go_on, ended = state.accept(tokens)
            if on_tokens:
                on_tokens([(state.request_ids[r], t) for r, t in zip(rows_before, tokens)
                           if state.reasons[r] != "stop"])
            stepper.release(ended)
        if profiling:
            _book(stats, "decode", profiler.profile_end())
        stats.decode_ms += (clock() - t0) * 1000.0
    finally:
        stepper.close()


def _decode_ahead(stepper, state: BatchState, stats: GenerationStats, on_tokens) -> None:
    """The decode loop with one step in flight beyond the one whose tokens the host is looking at: step n + 1 is
    launched before step n's tokens are waited for, so the device never idles while the host decides.  The price: a
    sequence that sampled a stop token in step n has already run in step n + 1; that extra token is dropped here, and
    the row leaves with the launch after.  A sequence that reaches its token limit leaves without that lag (the limit
    needs no token to be seen).  The tokens and reasons are those of the loop that waits every step."""
    produced = {r: len(state.outputs[r]) for r in state.live}     # tokens launched so far for each row, the prompt's first included
    running = list(state.live)                                     # rows that the next launch takes
    flying: list = []                                              # rows of the launches that are not collected yet, oldest first
    gone: set = set()                                              # rows that were released already
    while running or flying:
        if running:
            stepper.launch(running)
            flying.append(list(running))
            for r in running:
                produced[r] += 1
            at_limit = [r for r in running if produced[r] >= state.max_new_tokens]
            running = [r for r in running if produced[r] < state.max_new_tokens]
            stepper.release(at_limit)           # their last token is on its way; they take no further step
            gone.update(at_limit)
        if len(flying) > 1 or not running:
            rows, tokens = flying.pop(0), stepper.collect()
            by_row = dict(zip(rows, tokens))
            live_before = list(state.live)      # rows that had not ended by the tokens of the steps before
            go_on, ended = state.accept([by_row[r] for r in live_before])
            stats.decode_steps += 1
            stats.decode_tokens += len(live_before)
            if on_tokens:
                on_tokens([(state.request_ids[r], by_row[r]) for r in live_before if state.reasons[r] != "stop"])
            stopped = [r for r in ended if r in running]
            running = [r for r in running if r not in stopped]
            stepper.release([r for r in ended if r not in gone])
            gone.update(ended)


def generate(engine, prompts, max_new_tokens: int = 256, sampling=None, stop_token_ids=(),
             max_batch: int | None = None, on_tokens=None, stepper_factory=None, profile: bool = False) -> GenerationOutput:
    """Generates for every prompt (a list of token ids).  `sampling` is one SamplingParams for
    all requests or a list with one per request; the default is greedy.  Returns the kept
    tokens and the finish reason of every request, in the order of `prompts`.  `profile`: every
    kernel is timed by a pair of CUDA events and booked by name in stats.profile (the counterpart of
    HunyuanDenseModel.ProfileEnabled, src/HyMT2Sharp/HunyuanDenseModel.cs:48-78); kernels then run
    one after the other and the host waits for every decode step (whose graph holds the events), so the
    total is slower than an unprofiled run."""
    prompts = [list(map(int, p)) for p in prompts]
    if sampling is None:
        sampling = GREEDY
    params = [sampling] * len(prompts) if isinstance(sampling, SamplingParams) else list(sampling)
    if len(params) != len(prompts):
        raise ValueError("one SamplingParams for every prompt is needed")
    limit = getattr(engine, "max_positions", None)
    if limit is not None:
        # checked before anything runs, as the reference's callers refuse a prompt that does not fit the context
        # (src/HyMT2Sharp.Server/ChatCompletionService.cs:123-124); the last sampled token is never fed back
        for i, p in enumerate(prompts):
            if len(p) + max(0, max_new_tokens - 1) > limit:
                raise ValueError(f"request {i}: {len(p)} prompt tokens + {max_new_tokens} new ones go past the model's "
                                 f"max_position_embeddings of {limit}")
    max_batch = max_batch or engine.cache.max_slots
    capacity = engine.cache.free_tokens()
    batches = plan_batches([len(p) for p in prompts], max_new_tokens, max_batch, capacity, engine.cache.block_tokens)
    factory = stepper_factory or EngineStepper
    profiler = None
    if profile:
        from ..kernels import ops as profiler
    stats = GenerationStats()
    results = [None] * len(prompts)
    for ids in batches:
        state = BatchState(ids, [len(prompts[i]) for i in ids], max_new_tokens, stop_token_ids)
        stepper = factory(engine, [params[i] for i in ids], [prompts[i] for i in ids], max_new_tokens)
        run_batch(stepper, state, stats, on_tokens, profiler=profiler)
        stats.batches += 1
        for i, res in zip(ids, state.results()):
            results[i] = res
    engine.check()
    return GenerationOutput(results, stats)
