"""The Python entry point: requests in (token ids), tokens out.

It follows AIR's InferenceService (include/air/serving.hpp:237-286; src/runtime/serving.cpp:
1494-2010) in names and meanings: `SchedulerConfig`, `GenerationConfig`, `generate`,
`generate_cohort`, `snapshot`; a bounded queue; admission of the queue's head only, by
worst-case reservation; cycles of decode-first micro-batches under a token budget; the first
token comes from the last prompt portion; a finished request gives its pages back before the
next admission.  Differences: there is no worker thread (the caller's thread runs the cycles),
no tokenizer (prompts are token ids), and every cycle is ONE engine step that holds the
cycle's prompt portions and decoded tokens together.

Decoding one step ahead.  While every active request is decoding and its tokens are chosen on the
device, a cycle launches the next step BEFORE it reads the tokens of the step in flight: the
device feeds each request's last choice back by itself (`LAST_SAMPLED`), so the host's reading,
bookkeeping and scheduling run while the device computes, instead of between its steps.  A request
that ends by its token count is known beforehand and left out; one that ends by an end-of-sequence
token has one more token computed, which is dropped.  Tokens reach the caller one cycle later.
`SchedulerConfig.decode_ahead = False` gives the strictly alternating loop.

When pages run out.  With `reserve_worst_case` (the default, AIR's policy) an admitted request
has its worst case reserved, so a step can never run out of pages.  Without it, requests are
admitted while their next portion fits, and a step may find the pool empty: the engine then
reports OutOfPages with nothing changed, and the scheduler takes the youngest active request
out of the batch, gives its pages back and puts it at the head of the queue, to be computed
again from its prompt and the tokens it has produced (its sampler keeps its state, so the
continuation is the same); it retries the step with the rest.  A request that does not fit the
empty pool fails with "insufficient KV pages for one sequence".
"""
from __future__ import annotations

import collections
import time
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..cache.manager import OutOfPages
from ..sampling.sampler import GenerationConfig, HostSampler, SamplingConfig
from .batch import LAST_SAMPLED, Entry
from .scheduler import Runnable, StepScheduler


@dataclass
class SchedulerConfig:
    """AIR's names (include/air/serving.hpp:46-62).  The defaults are sized for a B200 rather
    than for AIR's laptop GPU: AIR has 8 / 256 / 256 / 32 / 16.  A prompt portion may take the whole
    budget of a cycle: the products of a 2,048-token portion run at 1.4 PFLOP/s, those of a 512-token
    one at 0.9-1.2."""
    max_active_requests: int = 64
    max_queued_requests: int = 256
    token_budget_per_cycle: int = 2048
    prefill_quantum_tokens: int = 2048
    kv_page_tokens: int = 64
    reserve_worst_case: bool = True
    decode_ahead: bool = True      # (not in AIR) launch a decode step before the one in flight is read
    sample_cuts_on_device: bool = True   # (not in AIR) top-k / top-p draws on the device too: AIR's distribution,
                                         # but not the token that AIR's walk gives for a seed (False: host sampler)


@dataclass
class RequestMetrics:
    """include/air/serving.hpp:75-104."""
    prompt_tokens: int = 0
    generated_tokens: int = 0
    queue_ms: float = 0.0
    prefill_ms: float = 0.0
    ttft_ms: float = 0.0
    decode_ms: float = 0.0
    total_ms: float = 0.0
    preemptions: int = 0


@dataclass
class InferenceResponse:
    request_id: int
    tokens: List[int]
    hit_eos: bool = False
    error: Optional[str] = None
    metrics: RequestMetrics = field(default_factory=RequestMetrics)


class QueueFull(RuntimeError):
    pass


class CancellationToken:
    """include/air/serving.hpp:212-224: what a request carries; true once its source was cancelled."""

    def __init__(self, state=None):
        self._state = state

    def is_cancelled(self) -> bool:
        return bool(self._state and self._state[0])

    def __bool__(self) -> bool:
        return self._state is not None


class CancellationSource:
    """include/air/serving.hpp:226-235: `token()` goes with the request, `cancel()` ends it: a queued request
    at the next admission ("request cancelled while queued"), an active one before the next step
    ("request cancelled while active"); its pages go back like those of a finished request."""

    def __init__(self):
        self._state = [False]

    def token(self) -> CancellationToken:
        return CancellationToken(self._state)

    def cancel(self) -> None:
        self._state[0] = True

    def is_cancelled(self) -> bool:
        return self._state[0]


@dataclass
class _WorkItem:
    request_id: int
    prompt: List[int]               # what has to be in the cache before decoding goes on
    prompt_tokens: int              # length of the prompt as submitted
    generation: GenerationConfig
    sampler: HostSampler
    generated: List[int] = field(default_factory=list)
    prompt_position: int = 0
    reservation_pages: int = 0
    done: bool = False
    hit_eos: bool = False
    error: Optional[str] = None
    submitted: float = 0.0
    admitted: float = 0.0
    first_token: float = 0.0
    metrics: RequestMetrics = field(default_factory=RequestMetrics)
    cancellation: CancellationToken = field(default_factory=CancellationToken)

    @property
    def decoding(self) -> bool:
        return self.prompt_position >= len(self.prompt)


@dataclass
class _InFlight:
    """A decode step that has been launched and whose tokens are on their way to the host."""
    items: List[_WorkItem]          # in the order of the rows
    tokens: object                  # pinned int32 tensor [rows + 1]: the chosen tokens, then the device's status word
    event: object                   # recorded after the copy


class InferenceService:
    def __init__(self, engine, scheduler: Optional[SchedulerConfig] = None):
        self.engine = engine
        self.config = scheduler or SchedulerConfig()
        for name in ("max_active_requests", "max_queued_requests", "token_budget_per_cycle",
                     "prefill_quantum_tokens"):
            if getattr(self.config, name) <= 0:
                raise ValueError(f"scheduler {name} must be greater than zero")
        self.scheduler = StepScheduler(
            self.config.max_active_requests, self.config.token_budget_per_cycle, self.config.prefill_quantum_tokens,
            engine.cache.page_tokens, graph_sizes=getattr(engine, "graph_sizes", ()))
        self.queued: Deque[_WorkItem] = collections.deque()
        self.active: List[_WorkItem] = []
        self.finished: Dict[int, InferenceResponse] = {}
        self._next_id = 0
        self.cycles = 0
        self.preemptions = 0
        self.cancelled_requests = 0
        self.last_plan = None
        self.failed_steps = 0
        self._inflight: Optional[_InFlight] = None
        self._pinned = {}

    # ------------------------------------------------------------------ construction
    @classmethod
    def create(cls, model: str, dtype="bfloat16", scheduler: Optional[SchedulerConfig] = None,
               max_tokens: Optional[int] = None, device: str = "cuda:0") -> "InferenceService":
        """Loads the model folder and makes its cache for `max_tokens` tokens; None takes the device memory
        that is left once the weights are resident (EngineConfig.memory_fraction of it)."""
        from .engine import Engine, EngineConfig, parse_dtype
        scheduler = scheduler or SchedulerConfig()
        engine = Engine.from_folder(model, EngineConfig(
            dtype=parse_dtype(dtype), page_tokens=scheduler.kv_page_tokens, max_tokens=max_tokens,
            max_requests=scheduler.max_active_requests, device=device))
        return cls(engine, scheduler)

    # ------------------------------------------------------------------ requests
    def submit(self, prompt_tokens: Sequence[int], generation: Optional[GenerationConfig] = None,
               cancellation: Optional[CancellationToken] = None) -> int:
        generation = generation or GenerationConfig()
        generation.sampling.validate()
        spec = self.engine.model.spec
        prompt = [int(t) for t in prompt_tokens]
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        if any(not (0 <= t < spec.vocab_size) for t in prompt):
            raise ValueError("input token is outside model vocabulary")
        if len(prompt) + generation.max_new_tokens > spec.max_positions:
            raise ValueError("prompt plus max_new_tokens exceeds the model context length")
        if len(self.queued) >= self.config.max_queued_requests:
            raise QueueFull("inference submission queue is full")
        item = _WorkItem(self._next_id, prompt, len(prompt), generation, HostSampler(generation.sampling),
                         submitted=time.perf_counter(), cancellation=cancellation or CancellationToken())
        self._next_id += 1
        self.queued.append(item)
        return item.request_id

    def restore(self, request: Hashable, last_token: int, generation: Optional[GenerationConfig] = None) -> int:
        """Takes over a request that the engine already holds (its tokens are in the cache) as an
        active, decoding request whose next input is `last_token`
        (AIR: PreparedModel::restore_sequence, src/runtime/backend.hpp:97-145)."""
        generation = generation or GenerationConfig()
        length = self.engine.cache.length(request)
        item = _WorkItem(request, [0] * length, length, generation, HostSampler(generation.sampling),
                         submitted=time.perf_counter())
        item.prompt_position = length
        item.generated = [int(last_token)]
        item.generation = GenerationConfig(generation.max_new_tokens + 1, generation.sampling,
                                           generation.stop_on_eos)
        item.admitted = item.first_token = item.submitted
        item.reservation_pages = self.engine.cache.pages_needed(length + generation.max_new_tokens)
        self.active.append(item)
        return item.request_id

    def generate(self, prompt_tokens: Sequence[int], generation: Optional[GenerationConfig] = None,
                 cancellation: Optional[CancellationToken] = None) -> InferenceResponse:
        request = self.submit(prompt_tokens, generation, cancellation)
        while request not in self.finished:
            if not self.run_cycle() and not self.active and not self.queued:
                break
        return self.finished.pop(request)

    def generate_cohort(self, requests) -> List[InferenceResponse]:
        """Submits the requests together and runs cycles until all of them are finished."""
        ids = []
        for r in requests:
            prompt, generation = r if isinstance(r, tuple) else (r, None)
            ids.append(self.submit(prompt, generation))
        while any(i not in self.finished for i in ids):
            if not self.run_cycle() and not self.active and not self.queued:
                break
        return [self.finished.pop(i) for i in ids]

    # ------------------------------------------------------------------ one cycle
    def _cancellations(self) -> None:
        """src/runtime/serving.cpp:1522-1530, 1761-1766: cancelled requests leave before admission and
        before the cycle's batch is made."""
        for item in [i for i in self.queued if i.cancellation.is_cancelled()]:
            self.queued.remove(item)
            self.cancelled_requests += 1
            self._finish(item, error="request cancelled while queued")
        hit = False
        for item in self.active:
            if not item.done and item.cancellation.is_cancelled():
                item.done, item.error = True, "request cancelled while active"
                self.cancelled_requests += 1
                hit = True
        if hit and self._inflight is None:
            self._retire()      # (with a step in flight they leave when it has been read)

    def _admit(self) -> None:
        cache = self.engine.cache
        self._cancellations()
        while self.queued:
            item = self.queued[0]
            worst = len(item.prompt) + max(0, item.generation.max_new_tokens - len(item.generated))
            if self.config.reserve_worst_case:
                reserved = sum(i.reservation_pages for i in self.active)
                decision = self.scheduler.admit(len(self.active), reserved, cache.num_pages, worst)
            else:
                first = min(len(item.prompt), self.config.prefill_quantum_tokens)
                decision = self.scheduler.admit(len(self.active), cache.num_pages - cache.free_pages(),
                                                cache.num_pages, first)
                if decision.admit and cache.pages_needed(worst) > cache.num_pages:
                    decision.admit, decision.reason = False, "device-capacity"
            if not decision.admit:
                never = decision.reason == "device-capacity" and (
                    not self.active or cache.pages_needed(worst) > cache.num_pages)
                if never:
                    self.queued.popleft()
                    self._finish(item, error="insufficient KV pages for one sequence")
                    continue
                break
            self.queued.popleft()
            item.reservation_pages = decision.pages if self.config.reserve_worst_case else 0
            item.admitted = time.perf_counter()
            self.active.append(item)

    def run_cycle(self) -> bool:
        """Admission, one micro-batch, one engine step, sampling, finishing.  Returns False when
        there was nothing to run."""
        self._admit()
        if self._inflight is not None:
            done = self._inflight
            self._inflight = self._launch_ahead(done)
            self._complete(done)
            return True
        if not self.active:
            return False
        plan = self.scheduler.plan([
            Runnable(i.request_id, i.prompt, i.prompt_position, i.generated[-1] if i.generated else None,
                     wants_token=len(i.generated) < i.generation.max_new_tokens) for i in self.active])
        if not plan.entries:
            return False
        entries = plan.entries
        while True:
            try:
                logits = self.engine.step(entries)
                break
            except OutOfPages:
                victim = self._preempt_youngest()
                entries = [e for e in entries if e.request != victim]
                if not entries:
                    return True
        self.last_plan = plan
        self.cycles += 1
        if self._may_decode_ahead(entries):
            items = self._items(entries)
            self._inflight = self._read_later(items, self._choose_on_device(items, logits))
            return True
        self._accept(entries, logits)
        self._retire()
        return True

    # ------------------------------------------------------------------ decoding one step ahead
    def _items(self, entries: Sequence[Entry]) -> List[_WorkItem]:
        by_id = {i.request_id: i for i in self.active}
        return [by_id[e.request] for e in entries]

    def _may_decode_ahead(self, entries: Sequence[Entry]) -> bool:
        """The step that has just run is a plain decode step of every active request, with tokens
        chosen on the device, on an engine that feeds them back by itself."""
        if not (self.config.decode_ahead and getattr(self.engine, "feeds_back_tokens", False)):
            return False
        if len(entries) != len(self.active):
            return False
        return all(i.decoding and self._on_device(i) for i in self.active) and \
            all(len(e.tokens) == 1 and len(e.want) == 1 for e in entries)

    def _on_device(self, item: _WorkItem) -> bool:
        s = item.generation.sampling
        return s.on_device or (self.config.sample_cuts_on_device and getattr(self.engine, "feeds_back_tokens", False))

    def _choose_on_device(self, items: Sequence[_WorkItem], logits):
        temps = [float(i.generation.sampling.temperature) for i in items]
        if any(t > 0.0 for t in temps):
            uniforms = [i.sampler.next_uniform() if t > 0.0 else 0.0 for i, t in zip(items, temps)]
            cuts = [i.generation.sampling for i in items]
            if any(c.top_k != 0 or c.top_p < 1.0 for c in cuts):
                return self.engine.sample(logits, temps, uniforms, [int(c.top_k) for c in cuts],
                                          [float(c.top_p) for c in cuts])
            return self.engine.sample(logits, temps, uniforms)
        return self.engine.sample(logits)

    def _read_later(self, items: List[_WorkItem], ids) -> _InFlight:
        """Starts the copy of the chosen tokens, and of the device's status word behind them, into pinned
        memory; the step's tokens and its faults arrive together, with one wait."""
        import torch
        n = len(items)
        ring = self._pinned.get(n)
        if ring is None:
            ring = self._pinned[n] = [[torch.empty(n + 1, dtype=torch.int32).pin_memory(), torch.cuda.Event()]
                                      for _ in range(2)]
        ring.append(ring.pop(0))
        host, event = ring[0]
        host[:n].copy_(ids, non_blocking=True)
        host[n:].copy_(self.engine.status, non_blocking=True)
        event.record()
        return _InFlight(list(items), host, event)

    def _fault(self, code: int, items: Sequence[_WorkItem]) -> None:
        """The device reported a fault during a step (a bounded wait that ran out, a page that the request
        does not hold, logits that are not finite): its word is cleared, and the step's requests fail with the
        engine's message for it, as AIR fails the item whose logits are not finite
        (src/runtime/serving.cpp:1037-1040)."""
        message = self.engine.clear_status(code)
        self.failed_steps += 1
        for item in items:
            if not item.done:
                item.done, item.error = True, message

    def _launch_ahead(self, flying: _InFlight) -> Optional[_InFlight]:
        """The step after the one in flight, for the requests that go on whatever it brings; None
        when that step needs what the one in flight will tell (a new request, pages running out)."""
        if len(self.active) != len(flying.items) or any(i.done for i in flying.items):
            return None
        items = [i for i in flying.items if len(i.generated) + 1 < i.generation.max_new_tokens]
        if not items or len(items) > self.config.token_budget_per_cycle:
            return None
        entries = [Entry(i.request_id, [LAST_SAMPLED], [0]) for i in items]
        try:
            logits = self.engine.step(entries)
        except OutOfPages:
            return None
        self.cycles += 1
        return self._read_later(items, self._choose_on_device(items, logits))

    def _complete(self, flying: _InFlight) -> None:
        """Reads the tokens of a launched step and accepts them.  (A request that ended meanwhile, by
        an end-of-sequence token of the step before, had one token too many computed: dropped.)"""
        flying.event.synchronize()
        *chosen, status = flying.tokens.tolist()
        if status:
            self._fault(status, flying.items)
        now = time.perf_counter()
        for item, token in zip(flying.items, chosen):
            if not item.done:
                self._accept_token(item, int(token), now)
        self._retire()

    def _retire(self) -> None:
        for item in [i for i in self.active if i.done]:
            self.active.remove(item)
            if item.request_id in self.engine.cache.sequences:
                self.engine.finish(item.request_id)
            self._finish(item, error=item.error)

    def _preempt_youngest(self) -> int:
        """Takes the active request that was admitted last out of the engine and puts it back
        at the head of the queue; it will be computed again from its prompt and its tokens."""
        if len(self.active) <= 1:
            item = self.active.pop()
            if item.request_id in self.engine.cache.sequences:
                self.engine.finish(item.request_id)
            self._finish(item, error="insufficient KV pages for one sequence")
            return item.request_id
        item = max(self.active, key=lambda i: i.admitted)
        self.active.remove(item)
        if item.request_id in self.engine.cache.sequences:
            self.engine.finish(item.request_id)
        item.prompt = item.prompt[:item.prompt_tokens] + item.generated
        item.prompt_position = 0
        item.metrics.preemptions += 1
        self.preemptions += 1
        self.queued.appendleft(item)
        return item.request_id

    def _accept(self, entries: Sequence[Entry], logits) -> None:
        by_id = {i.request_id: i for i in self.active}
        rows = [by_id[e.request] for e in entries if e.want]
        chosen: List[Optional[int]] = [None] * len(rows)
        if rows:
            if all(self._on_device(i) for i in rows):
                chosen = [int(t) for t in self._choose_on_device(rows, logits).tolist()]
            else:
                host = logits.float().cpu().numpy()
                chosen = [i.sampler.sample(host[r]) for r, i in enumerate(rows)]
        status = self.engine.read_status() if hasattr(self.engine, "read_status") else 0
        if status:      # (the tokens were read above, so the step has ended and the word is final)
            self._fault(status, [by_id[e.request] for e in entries])
            return
        now = time.perf_counter()
        r = 0
        for e in entries:
            item = by_id[e.request]
            if not item.decoding:
                item.prompt_position += len(e.tokens)
            if e.want:
                self._accept_token(item, chosen[r], now)
                r += 1
            elif item.decoding and len(item.generated) >= item.generation.max_new_tokens:
                item.done = True  # max_new_tokens == 0, or a recomputed request that had finished

    def _accept_token(self, item: _WorkItem, token: int, now: float) -> None:
        """src/runtime/serving.cpp:687-700."""
        if not item.generated:
            item.first_token = now
        item.generated.append(token)
        eos = self.engine.model.spec.eos_token_id
        if item.generation.stop_on_eos and eos is not None and token == eos:
            item.hit_eos = True
            item.done = True
        if len(item.generated) >= item.generation.max_new_tokens:
            item.done = True

    def _finish(self, item: _WorkItem, error: Optional[str] = None) -> None:
        now = time.perf_counter()
        m = item.metrics
        m.prompt_tokens, m.generated_tokens = item.prompt_tokens, len(item.generated)
        if item.admitted:
            m.queue_ms = (item.admitted - item.submitted) * 1e3
        if item.first_token:
            m.ttft_ms = (item.first_token - item.submitted) * 1e3
            m.prefill_ms = (item.first_token - item.admitted) * 1e3
            m.decode_ms = (now - item.first_token) * 1e3
        m.total_ms = (now - item.submitted) * 1e3
        self.finished[item.request_id] = InferenceResponse(item.request_id, list(item.generated), item.hit_eos,
                                                           error, m)

    # ------------------------------------------------------------------ figures
    def snapshot(self) -> dict:
        """A few of the gauges of AIR's ServiceSnapshot (include/air/serving.hpp:131-208)."""
        cache = self.engine.cache
        return {"queued_requests": len(self.queued), "active_requests": len(self.active),
                "reserved_pages": sum(i.reservation_pages for i in self.active),
                "kv_pages_total": cache.num_pages, "kv_pages_free": cache.free_pages(),
                "cycles": self.cycles, "preemptions": self.preemptions,
                "cancelled_requests": self.cancelled_requests, "failed_steps": self.failed_steps}
