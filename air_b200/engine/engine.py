"""The step function and what it stands on: a loaded model, its cache manager and the
device context.  `Engine.step` is the only way tokens reach the model: generation, the
scheduler and trace replay all call it.
"""
from __future__ import annotations

import gc
import os
from dataclasses import dataclass
from typing import Hashable, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager, OutOfPages
from ..config import ConfigError, load_config
from ..parts import registry
from ..parts.base import Runtime
from ..weights.loader import LoadReport, load_tensors, random_tensors, write_model_folder
from ..csrc import ops
from .batch import Entry, StepContext, build_context, LAST_SAMPLED
from .model import Model

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(name) -> torch.dtype:
    try:
        return _DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype {name!r}: the engine computes in bfloat16 or float32") from None


class StepError(RuntimeError):
    """A step failed; no request's length has advanced."""


@dataclass
class EngineConfig:
    """page_tokens: tokens per cache page.  max_tokens: how many tokens the cache pool holds
    over all live requests (each request's count rounded up to whole pages); None sizes the pool
    from the device memory that is free once the weights are resident, of which it takes the share
    `memory_fraction` (AIR admits against free device memory plus pool bytes,
    src/runtime/backend.cpp:538-556).  max_requests: live requests (state slots).  AIR:
    KvPolicy.page_tokens (include/air/execution.hpp:103-105) and SchedulerConfig.max_active_requests
    (include/air/serving.hpp:46-62).  keep_float32: matrices that the checkpoint stores in 32 bits stay
    so in a bfloat16 engine (and run the CUDA-core product) instead of being rounded to bfloat16."""
    dtype: torch.dtype = torch.bfloat16
    page_tokens: int = 64
    max_tokens: Optional[int] = 8192
    max_requests: int = 8
    device: str = "cuda:0"
    cuda_graphs: bool = True      # decode-only steps replay a captured graph
    memory_fraction: float = 0.9
    keep_float32: bool = False


_BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)


class DecodeGraph:
    """A decode step (every request brings one token) captured as a CUDA graph for a fixed
    number of tokens.  The batch lives in static device buffers; a step copies 4 ints per token
    from pinned host memory and replays the graph.  Fewer requests than the graph's size are
    padded with slot -1, which every kernel skips."""
    RING = 8

    def __init__(self, engine: "Engine", size: int):
        dev = engine.rt.device
        self.size, self.engine = size, engine
        self.ints = torch.zeros(4 * size, dtype=torch.int32, device=dev)
        self.ints[2 * size:3 * size] = -1
        self.fixed = torch.arange(size + 1, dtype=torch.int32, device=dev)
        self.host = [torch.zeros(4 * size, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.turn = 0
        ids, pos, slot, kvl = (self.ints[i * size:(i + 1) * size] for i in range(4))
        self.ctx = StepContext(
            num_tokens=size, num_seqs=size, token_ids=ids, positions=pos, token_seq=slot, q_start=self.fixed,
            kv_len=kvl, slots=slot, logit_rows=self.fixed[:size], row_slots=slot,
            block_tables=list(engine.cache.tables), status=engine.status, max_q_len=1, all_decode=True,
            last_token=engine.last_token)
        # once eagerly on padding (so that every lazy set-up is done), then captured
        engine.model.forward(self.ctx, engine.cache)
        torch.cuda.synchronize()
        before = ops.launches
        self.graph = torch.cuda.CUDAGraph()
        # No garbage collection while the stream is capturing: freeing another engine's graphs, events or
        # pinned memory then is a CUDA call that is not permitted during capture and would spoil it.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph):
                self.logits = engine.model.forward(self.ctx, engine.cache)
        finally:
            if collecting:
                gc.enable()
        self.kernels = ops.launches - before

    def run(self, ids, positions, slots) -> torch.Tensor:
        n, size = len(ids), self.size
        i = self.turn = (self.turn + 1) % self.RING
        if self.events[i] is not None:
            self.events[i].synchronize()
        pad = size - n
        self.host[i].copy_(torch.tensor(ids + [0] * pad + positions + [0] * pad + slots + [-1] * pad +
                                        [p + 1 for p in positions] + [0] * pad, dtype=torch.int32))
        self.ints.copy_(self.host[i], non_blocking=True)
        ev = self.events[i] = self.events[i] or torch.cuda.Event()
        ev.record()
        self.graph.replay()
        self.engine.graph_kernel_launches += self.kernels
        return self.logits[:n]


class Engine:
    feeds_back_tokens = True     # Entry(request, [LAST_SAMPLED]) takes the device's last choice for the request
    graph_sizes = _BUCKETS       # decode-only steps of up to so many requests replay a graph of the next size

    def __init__(self, model: Model, config: EngineConfig, model_config=None):
        self.model, self.config, self.model_config = model, config, model_config
        self.rt = model.rt
        self.load_report = None
        if config.page_tokens <= 0 or config.page_tokens % 16:
            raise ConfigError("unsupported", f"page size {config.page_tokens}: the cache takes positive multiples of 16")
        max_blocks = -(-model.spec.max_positions // config.page_tokens)
        if config.max_tokens is None:
            num_pages = self._pages_that_fit(model, config)
        else:
            num_pages = max(1, -(-config.max_tokens // config.page_tokens))
        self.cache = CacheManager(model.cache_needs(), config.page_tokens, num_pages, config.max_requests,
                                  dtype=self.rt.dtype, device=self.rt.device, max_blocks=max_blocks)
        self.status = self.rt.status if self.rt.status is not None else \
            torch.zeros(1, dtype=torch.int32, device=self.rt.device)
        self.last_token = torch.zeros(config.max_requests, dtype=torch.int32, device=self.rt.device)
        self.last_context: Optional[StepContext] = None
        self.steps = 0
        self.graph_kernel_launches = 0
        self.graphs = {}
        self.use_graphs = config.cuda_graphs and model.graph_safe

    @staticmethod
    def _pages_that_fit(model: Model, config: EngineConfig) -> int:
        """The pool's size from the memory that is left: free bytes (with the allocator's unused blocks given
        back first) times memory_fraction, over what a page number costs in all runs; at most what
        max_requests requests of the longest context could hold."""
        torch.cuda.empty_cache()
        free, _ = torch.cuda.mem_get_info(model.rt.device)
        per_page = CacheManager.bytes_per_page(model.cache_needs(), config.page_tokens, model.rt.dtype)
        if per_page == 0:
            return 1
        pages = int(free * config.memory_fraction) // per_page
        most = config.max_requests * -(-model.spec.max_positions // config.page_tokens)
        if pages < 1:
            raise RuntimeError(f"air_b200: {free >> 20} MiB of device memory are free after the weights, "
                               f"a cache page takes {per_page >> 10} KiB")
        return min(pages, most)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder: str, config: Optional[EngineConfig] = None) -> "Engine":
        config = config or EngineConfig()
        model_config = load_config(folder)
        arch = registry.architecture(model_config.architecture)
        model = Model(arch.build_spec(model_config))
        device = _device(config.device)
        rt = Runtime(device=device, dtype=parse_dtype(config.dtype), page_tokens=config.page_tokens,
                     status=torch.zeros(1, dtype=torch.int32, device=device))
        report = LoadReport()
        tensors = load_tensors(folder, model.tensor_specs(), rt.dtype, device, keep_float32=config.keep_float32,
                               report=report)
        model.load(tensors, rt)
        del tensors
        engine = cls(model, config, model_config)
        engine.load_report = report
        return engine

    @classmethod
    def from_random(cls, model_config, seed: int = 0, config: Optional[EngineConfig] = None) -> "Engine":
        """A model with seeded random weights drawn on the device, without files."""
        config = config or EngineConfig()
        if isinstance(model_config, dict):
            model_config = load_config(model_config)
        arch = registry.architecture(model_config.architecture)
        model = Model(arch.build_spec(model_config))
        device = _device(config.device)
        rt = Runtime(device=device, dtype=parse_dtype(config.dtype), page_tokens=config.page_tokens,
                     status=torch.zeros(1, dtype=torch.int32, device=device))
        model.load(random_tensors(model.tensor_specs(), seed, rt.dtype, device=device), rt)
        return cls(model, config, model_config)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[Entry]) -> torch.Tensor:
        """Runs one batch: for each entry the request's next tokens (a portion of its prompt or
        one decoded token, any mix).  Returns float32 logits [wanted places, vocab] on the
        device, in the order of the entries and of their `want`.  A request is opened at its
        first tokens.  On failure (OutOfPages, a token outside the vocabulary) nothing is
        committed and pages taken for the step are given back.  The returned logits may live in
        a buffer that the next step overwrites: use them (or copy them) before stepping again."""
        entries = [e if isinstance(e, Entry) else Entry(*e) for e in entries]
        vocab, limit = self.model.spec.vocab_size, self.model.spec.max_positions
        seen = set()
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.request!r} brings no tokens")
            if len(e.tokens) == 1 and int(e.tokens[0]) == LAST_SAMPLED and e.request in self.cache.sequences:
                continue
            for t in e.tokens:
                if not (0 <= int(t) < vocab):
                    raise StepError("input token is outside model vocabulary")
        opened = []
        try:
            for e in entries:
                if e.request not in self.cache.sequences:
                    self.cache.open(e.request)
                    opened.append(e.request)
                if self.cache.length(e.request) + len(e.tokens) > limit:
                    raise StepError("model context length exceeded")
            self.cache.reserve([(e.request, len(e.tokens)) for e in entries])
        except Exception:
            for r in opened:
                self.cache.close(r)
            raise
        try:
            if self.use_graphs and all(len(e.tokens) == 1 and tuple(e.want) == (0,) for e in entries) \
                    and len(entries) <= _BUCKETS[-1]:
                logits, ctx = self._decode_step(entries)
            else:
                ctx = build_context(entries, self.cache, self.rt.device, status=self.status,
                                    planners=self.model.planners())
                ctx.last_token = self.last_token
                logits = self.model.forward(ctx, self.cache)
        except Exception:
            for e in entries:
                if e.request in opened:
                    self.cache.close(e.request)
                else:
                    self.cache.trim(e.request)
            raise
        for e in entries:
            self.cache.commit(e.request, len(e.tokens))
        self.steps += 1
        self.last_context = ctx
        return logits

    def _decode_step(self, entries):
        seqs = [self.cache.sequences[e.request] for e in entries]
        size = next(b for b in _BUCKETS if b >= len(entries))
        graph = self.graphs.get(size)
        if graph is None:
            graph = self.graphs[size] = DecodeGraph(self, size)
        self.cache.flush_tables()
        ids = [int(e.tokens[0]) if int(e.tokens[0]) >= 0 else -(s.slot + 1) for e, s in zip(entries, seqs)]
        logits = graph.run(ids, [s.length for s in seqs], [s.slot for s in seqs])
        n = len(entries)
        c = graph.ctx
        ctx = StepContext(
            num_tokens=n, num_seqs=n, token_ids=c.token_ids[:n], positions=c.positions[:n], token_seq=c.token_seq[:n],
            q_start=c.q_start[:n + 1], kv_len=c.kv_len[:n], slots=c.slots[:n], logit_rows=c.logit_rows[:n],
            row_slots=c.row_slots[:n], block_tables=c.block_tables, status=self.status,
            q_start_host=list(range(n + 1)), kv_len_host=[s.length + 1 for s in seqs],
            slots_host=[s.slot for s in seqs], max_q_len=1, max_kv_len=max(s.length + 1 for s in seqs),
            all_decode=True, last_token=self.last_token)
        return logits, ctx

    def sample(self, logits: torch.Tensor, temperature=None, uniform=None, top_k=None, top_p=None) -> torch.Tensor:
        """Chooses a token for every row of the last step's logits on the device: the lowest
        index of the maximum where temperature[r] <= 0 (or temperature is None), else a draw from
        softmax(logits / temperature) with the uniform number uniform[r], cut to the top_k[r] largest logits
        (0: all) and the share top_p[r] of the weight (1: all) where given.  Returns int32 [rows] on
        the device; each choice is also remembered for its request, so that the next step can
        take it as Entry(request, [LAST_SAMPLED]) without a copy to the host."""
        ctx = self.last_context
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        if logits.shape[0] == 0:
            return out
        if ctx is None or ctx.row_slots.shape[0] != logits.shape[0]:
            raise StepError("sample() takes the logits of the step that has just run")

        def dev(x, dtype=torch.float32):
            if x is None or isinstance(x, torch.Tensor):
                return x
            return torch.tensor(x, dtype=dtype).to(logits.device, non_blocking=True)

        ops.sample(logits, dev(temperature), dev(uniform), out, status=self.status, slots=ctx.row_slots,
                   last_token=self.last_token, top_k=dev(top_k, torch.int32), top_p=dev(top_p))
        return out

    def kernel_launches(self) -> int:
        """Kernels of this package launched so far, those replayed inside CUDA graphs included."""
        return ops.launches + self.graph_kernel_launches

    def finish(self, request: Hashable) -> None:
        """The request is over: its pages and its slot are free for others."""
        self.cache.close(request)

    STATUS_TEXT = {1: "a token outside the vocabulary reached the embedding kernel",
                   2: "a token was to be written to a page that its request does not hold",
                   3: "non-finite logits",
                   4: "a wait inside the matrix-product kernel ran out",
                   5: "a wait inside the decode attention kernel ran out",
                   6: "a wait inside the prefill attention kernel ran out",
                   7: "a wait inside the tcgen05 prefill attention kernel ran out",
                   8: "the tile list of the tcgen05 prefill attention kernel is not in pairs of one request"}

    def read_status(self) -> int:
        """The device's error word (a synchronisation): 0, or the code of what a kernel could not do."""
        return int(self.status.item())

    def clear_status(self, code: int) -> str:
        """Zeroes the word after `code` was read from it; returns the message for that code."""
        self.status.zero_()
        return self.STATUS_TEXT.get(code, f"device status {code}")

    def check_status(self) -> None:
        """Reads the device's error word (a synchronisation) and raises StepError if it is set."""
        code = self.read_status()
        if code:
            raise StepError(self.clear_status(code))


def _device(name) -> torch.device:
    device = torch.device(name)
    if device.type != "cuda":
        raise RuntimeError("air_b200 computes on a CUDA device only; there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("air_b200: no CUDA device is available")
    torch.cuda.set_device(device)
    return device


def write_random_model(folder: str, model_config, seed: int = 0, dtype="bfloat16") -> None:
    """Random-weights mode: writes config.json and model.safetensors for a configuration and a
    seed.  Weights and biases are N(0, 0.02), norm weights 1 + N(0, 0.02), drawn on the CPU
    per tensor from (seed, tensor name) and rounded to `dtype`."""
    if isinstance(model_config, dict):
        model_config = load_config(model_config)
    arch = registry.architecture(model_config.architecture)
    model = Model(arch.build_spec(model_config))
    tensors = random_tensors(model.tensor_specs(), seed, parse_dtype(dtype), device="cpu")
    cfg = model_config.to_dict()
    cfg["torch_dtype"] = "bfloat16" if parse_dtype(dtype) == torch.bfloat16 else "float32"
    write_model_folder(folder, cfg, tensors)
