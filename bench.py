#!/usr/bin/env python3
"""Benchmark of the decode step, a 2,048-token prefill and a mixed step at the shapes of Qwen2.5-7B, 14B
and 32B with random bfloat16 weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--shape 7b|14b|32b|config.json] [--batch 8]
                    [--context N] [--layers L] [--repeats R] [--mixed D,P] [--output FILE]

With no flags it runs the 7B shape (28 layers, batch 8, 8,192 tokens of context).  A "step" is one decode
step of the whole batch.  It prints ONE JSON line:
  value      decoded tokens per second: the median of R repeats, each timed on the device with CUDA events
             over exactly K steps after W warm-up steps; every request holds `context` tokens in the cache at
             the end of a repeat and feeds its last sampled token back on the device (no host round trip);
             `repeat_ms_per_step` lists all repeats
  e2e        the same through the Python entry point (InferenceService.run_cycle): every step copies the
             step's token ids from pinned host memory and reads the sampled ids and the status word back
  prefill    one step of 2,048 prompt tokens of one request, the median of R timed steps, each after a pause
             of 0.2 s (a prompt is a burst, not a sustained load); frac = flops / time / bf16 peak
  roofline   bytes the decode step has to read (every weight once, the live requests' cache) / its time,
             against the measured copy bandwidth
  points     decode tokens per second at batch 1 and 64 (points_roofline_frac: their share of the copy
             bandwidth, counted as for roofline)
  mixed      with --mixed D,P: ONE Engine.step of D decoding requests at the context beside one P-token
             portion of a prompt that has (context - P) / 2 tokens in the cache: device_ms (CUDA events around
             the step), host_ms (the host's clock from the call of Engine.step to its return, i.e. packing and
             launching, nothing waited for), the shares of the copy bandwidth and of the bf16 peak, and frac =
             roofline_ms / device_ms, where roofline_ms adds what the step's phases need one after the other: the
             decoding requests' cache at the copy bandwidth, the products at the bf16 peak (or their weights at the
             copy bandwidth, if that is longer), the portion's attention at the bf16 peak
The pool of cache pages is sized from the device memory that is free once the weights are resident.  The cache
of the decoding requests is filled with random keys and values instead of running 64 prompts (data: synthetic);
timing does not depend on the values.  Between timed steps nothing is flushed: a step reads its weights (over
14 GB at 28 layers), far more than the 126 MB of L2.
--impl reference runs EmersonDowell/AIR's own CUDA executor, built from its unmodified sources (baseline/),
on the same shape, batch and context, and prints the same line with "impl": "reference".
For --gpus N > 1 it prints one line that says so and exits with 2: this engine runs on one GPU.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

_QWEN = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": 152064,
         "max_position_embeddings": 32768, "rope_theta": 1000000.0, "tie_word_embeddings": False,
         "sliding_window": 131072, "use_sliding_window": False, "hidden_act": "silu"}
SHAPES = {
    "7b": dict(_QWEN, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
               intermediate_size=18944, rms_norm_eps=1e-6, max_window_layers=28),
    "14b": dict(_QWEN, num_hidden_layers=48, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                intermediate_size=13824, rms_norm_eps=1e-5, max_window_layers=48),
    "32b": dict(_QWEN, num_hidden_layers=64, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                intermediate_size=27648, rms_norm_eps=1e-5, max_window_layers=64),
}
CONTEXTS = {"7b": 8192, "14b": 8192, "32b": 4096}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            found = {"hbm_gbs": _figure(d, "hbm_gbs"), "bf16_tflops": _figure(d, "bf16_tflops"), "source": "measured"}
            try:
                found["bf16_tflops_sustained"] = _figure(d, "bf16_tflops_sustained")
            except (ValueError, KeyError, TypeError):
                pass
            return found
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


def _figure(record, key):
    """A peak from the record: a number, or an object that holds it under 'value' (or the key's own name); the
    key may also lie one level down (under 'peaks', say)."""
    if key not in record:
        for inner in record.values():
            if isinstance(inner, dict) and key in inner:
                record = inner
                break
    v = record[key]
    if isinstance(v, dict):
        v = v["value"] if "value" in v else v[key]
    v = float(v)
    if not v > 0:
        raise ValueError(key)
    return v


class ClockSampler:
    """nvidia-smi in the background during the timed region (reading only)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.proc, self.lines = None, []
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def randomize_cache(engine, torch):
    """Random keys and values in every page of every run (once: pages keep them when they change hands)."""
    g = torch.Generator(device=engine.rt.device)
    g.manual_seed(1234)
    seen = set()
    for run in range(len(engine.model.spec.order)):
        for view in engine.cache.views(run):
            kv = getattr(view, "kv", None)
            if kv is not None and kv.data_ptr() not in seen:
                seen.add(kv.data_ptr())
                kv.normal_(0.0, 0.5, generator=g)


def open_requests(engine, requests, tokens):
    """Opens the requests with `tokens` tokens each (whatever lies in their pages)."""
    for r in requests:
        engine.cache.open(r)
        engine.cache.reserve([(r, tokens)])
        engine.cache.commit(r, tokens)


def release(engine, requests):
    for r in requests:
        if r in engine.cache.sequences:
            engine.finish(r)


def decode_device(engine, requests, context, steps, warmup, repeats, torch, Entry, LAST):
    """R repeats of K decode steps timed with CUDA events; tokens are fed back on the device.  Every repeat
    starts from the same length, so that its last step runs at `context` tokens."""
    times, clocks, launches = [], None, 0
    start_len = context - (steps + warmup + 2)
    for rep in range(repeats):
        open_requests(engine, requests, start_len)
        first = [Entry(r, [17 + i], [0]) for i, r in enumerate(requests)]
        engine.sample(engine.step(first))
        again = [Entry(r, [LAST], [0]) for r in requests]
        for _ in range(warmup):
            engine.sample(engine.step(again))
        torch.cuda.synchronize()
        launches0 = engine.kernel_launches()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler() if rep == 0 else None
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            engine.sample(engine.step(again))
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / steps)
        if sampler is not None:
            clocks = sampler.stop()
            launches = engine.kernel_launches() - launches0
        release(engine, requests)
    return times, clocks, launches


def decode_timeline(engine, requests, context, torch, Entry, LAST):
    """Spans of the kernels of one decode step as they run inside the CUDA graph (from the moment a
    kernel has passed the wait on its predecessor to the moment the next one has), by kernel."""
    import collections
    from air_b200.csrc import ops
    open_requests(engine, requests, context - 8)
    engine.sample(engine.step([Entry(r, [17 + i], [0]) for i, r in enumerate(requests)]))
    again = [Entry(r, [LAST], [0]) for r in requests]
    buf = torch.zeros(1 + 2 * 16384, dtype=torch.int64, device=engine.rt.device)
    ops.set_trace(buf)
    for _ in range(3):
        engine.sample(engine.step(again))
    torch.cuda.synchronize()
    ops.set_trace(None)
    release(engine, requests)
    b = buf.cpu().tolist()
    events = sorted((b[2 + 2 * i], b[1 + 2 * i]) for i in range(min(b[0], 16384)) if b[1 + 2 * i] < 100)
    start = [i for i, e in enumerate(events) if e[1] == 1][-1]           # the last step's embedding
    step = events[start:]
    spans = collections.defaultdict(lambda: [0, 0.0])
    for (t0, k), (t1, _) in zip(step, step[1:]):
        spans[ops.TRACE_NAMES[k]][0] += 1
        spans[ops.TRACE_NAMES[k]][1] += (t1 - t0) / 1e3
    total = (step[-1][0] - step[0][0]) / 1e3
    print(f"decode step inside the graph: {total:.1f} us from embedding to sampling, {len(step)} kernels")
    for name, (n, us) in sorted(spans.items(), key=lambda x: -x[1][1]):
        print(f"  {name:18s} {n:4d} launches {us:9.1f} us  {100 * us / total:5.1f} %  {us / n:7.1f} us each")
    # one layer from the middle of the step, kernel by kernel (from one attention kernel to the next)
    names = [ops.TRACE_NAMES[k] for _, k in step]
    marks = [i for i in range(len(step) // 2, len(step) - 1) if names[i] == "decode_attention"]
    if len(marks) >= 2:
        i, j = marks[0], marks[1]
        print("  one layer (us): " + " | ".join(f"{names[q]} {(step[q + 1][0] - step[q][0]) / 1e3:.1f}"
                                               for q in range(i, j)))


def prefill_timeline(engine, prompt, torch, Entry):
    """Spans between the starts of this package's kernels in one prefill step.  A library product has
    no trace point: its time is part of the span of the kernel before it."""
    import collections
    from air_b200.csrc import ops
    buf = torch.zeros(1 + 2 * 16384, dtype=torch.int64, device=engine.rt.device)
    ops.set_trace(buf)
    engine.step([Entry("p", prompt, [len(prompt) - 1])])
    torch.cuda.synchronize()
    ops.set_trace(None)
    engine.finish("p")
    b = buf.cpu().tolist()
    events = sorted((b[2 + 2 * i], b[1 + 2 * i]) for i in range(min(b[0], 16384)) if b[1 + 2 * i] < 100)
    spans = collections.defaultdict(lambda: [0, 0.0])
    order = []
    for (t0, k), (t1, k1) in zip(events, events[1:]):
        key = f"{ops.TRACE_NAMES[k]} -> {ops.TRACE_NAMES[k1]}"
        if key not in spans:
            order.append(key)
        spans[key][0] += 1
        spans[key][1] += (t1 - t0) / 1e3
    total = (events[-1][0] - events[0][0]) / 1e3
    print(f"prefill step of {len(prompt)} tokens: {total:.1f} us from embedding to sampling, {len(events)} traced kernels")
    for key in order:
        n, us = spans[key]
        print(f"  {key:42s} {n:4d} times {us:9.1f} us  {100 * us / total:5.1f} %  {us / n:7.1f} us each")


def decode_e2e(engine, requests, context, steps, warmup, torch):
    """The same through InferenceService.run_cycle, host tokens in and out every step."""
    from air_b200.engine.service import InferenceService, SchedulerConfig
    from air_b200.sampling.sampler import GenerationConfig
    open_requests(engine, requests, context - (steps + warmup + 2))
    service = InferenceService(engine, SchedulerConfig(max_active_requests=max(len(requests), 1),
                                                       token_budget_per_cycle=max(len(requests), 1)))
    for i, r in enumerate(requests):
        service.restore(r, 23 + i, GenerationConfig(max_new_tokens=steps + warmup + 1, stop_on_eos=False))
    for _ in range(warmup):
        service.run_cycle()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        service.run_cycle()
    torch.cuda.synchronize()
    sec = time.perf_counter() - t0
    release(engine, requests)
    # per step: 4 ints per token of the decode graph's batch from pinned memory; sampled ids and the status word back
    sizes = [g.size for g in engine.graphs.values() if g.size >= len(requests)]
    h2d = 16 * (min(sizes) if sizes else len(requests))
    return sec / steps, h2d, 4 * (len(requests) + 1)


def mixed_step(engine, decoders, portion, context, repeats, torch, Entry):
    """One Engine.step that holds `decoders` single next tokens of requests with `context` tokens and one portion of
    `portion` prompt tokens of a request that has (context - portion) / 2 tokens in the cache."""
    requests = [f"m{i}" for i in range(decoders)]
    prior = max(0, (context - portion) // 2 // 64 * 64)
    vocab = engine.model.spec.vocab_size
    g = torch.Generator().manual_seed(11)
    tokens = torch.randint(0, vocab, (portion,), generator=g).tolist()
    device_ms, host_ms = [], []
    for rep in range(repeats + 2):                 # the first two are warm-up
        open_requests(engine, requests, context - 1)
        open_requests(engine, ["portion"], prior)
        entries = [Entry(r, [5 + i], [0]) for i, r in enumerate(requests)] + [Entry("portion", tokens, [])]
        # (the pages of requests that earlier steps brought to their lengths are in the device's tables already:
        # without this the timed step would send the thousands of entries that opening the requests here made)
        engine.cache.flush_tables()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        t0 = time.perf_counter()
        logits = engine.step(entries)
        engine.sample(logits)
        t1 = time.perf_counter()
        end.record()
        torch.cuda.synchronize()
        if rep >= 2:
            device_ms.append(start.elapsed_time(end))
            host_ms.append((t1 - t0) * 1e3)
        release(engine, requests + ["portion"])
    return statistics.median(device_ms), statistics.median(host_ms), prior


def kernel_prefill_attention(cfg):
    """The tcgen05 attention kernel alone at the shape's heads: launches replayed as a CUDA graph of ten (a launch
    from the host costs more than the kernel takes), timed with CUDA events, median of five replays.  First one
    block per SM with streams of 4 to 128 key tiles (what a block costs beside its key tiles), then whole prompts
    and portions on top of long prefixes, with whole streams per block and with the planner's cut (if it cuts)."""
    import math
    import statistics
    import numpy as np
    import torch
    from air_b200.csrc import ops
    from air_b200.parts.attention import plan_segments
    d = cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    heads, kv_heads, P = cfg["num_attention_heads"], cfg["num_key_value_heads"], 64

    def case(H, K, prior, portion):
        """One request, or several (lists): `portion` new tokens each behind `prior` tokens."""
        priors, portions = (prior, portion) if isinstance(prior, (list, tuple)) else ([prior], [portion])
        most = max(-(-(a + b) // P) for a, b in zip(priors, portions))
        cache = (torch.randn(most * len(priors) + 1, 2, K, P, d, device="cuda") * 0.5).to(torch.bfloat16)
        table = torch.arange(most * len(priors), dtype=torch.int32, device="cuda").view(len(priors), most).contiguous()
        q = (torch.randn(sum(portions), H, d, device="cuda") * 0.5).to(torch.bfloat16)
        tiles, streams, row = [], [], 0
        for slot, (a, n) in enumerate(zip(priors, portions)):
            tiles += [[slot, row + i, a + i, min(16, n - i)] for i in range(0, n, 16)]
            tiles += [[slot, 0, 0, 0]] * (-len(tiles) % 16)
            streams += [(a + min(n, g + 256) - 1) // 64 + 1 for g in range(0, n, 256)]
            row += n
        return q, cache, table, torch.tensor(tiles, dtype=torch.int32, device="cuda"), streams

    def timed(q, cache, table, tiles, cut=None):
        out = torch.empty_like(q)
        more = {}
        if cut is not None:
            more = dict(segments=torch.from_numpy(cut[0]).cuda(), items=torch.from_numpy(cut[1]).cuda(), slots=cut[2])
        call = lambda: ops.prefill_attention_tc(q, cache, table, tiles, out, 0, 1 / math.sqrt(d), **more)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(10):
                call()
        graph.replay()
        torch.cuda.synchronize()
        us = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            us.append(a.elapsed_time(b) * 100.0)
        return statistics.median(us)

    print(f"prefill_attention_tc_kernel<{d}>: one block per SM (148 heads, 256 query rows), us per launch")
    for prior in (0, 256, 768, 1792, 3840, 7936):
        q, cache, table, tiles, streams = case(148, 4, prior, 256)
        print(f"  stream of {streams[0]:4d} key tiles: {timed(q, cache, table, tiles):7.1f}")
    print(f"{heads} query heads, {kv_heads} kv heads: whole streams per block | the planner's cut")
    for prior, portion in ((0, 1024), (0, 2048), (0, 8192), (2048, 2048), (3840, 512), (32768, 128), (32768, 512),
                           ([0, 0, 0, 0], [512, 2048, 256, 1024]), ([0, 1024, 8192, 0], [1024, 512, 128, 512])):
        q, cache, table, tiles, streams = case(heads, kv_heads, prior, portion)
        several = isinstance(prior, list)
        flops = sum(4.0 * d * heads * sum(a + i + 1 for i in range(n))
                    for a, n in (zip(prior, portion) if several else [(prior, portion)]))
        whole = timed(q, cache, table, tiles)
        cut = plan_segments(streams, heads)
        name = f"{portion} behind {prior}" if several else f"{portion:5d} tokens behind {prior:5d}"
        line = f"  {name}: {whole:8.1f} us ({flops / whole / 1e6:6.0f} TFLOP/s)"
        if cut is not None:
            t = timed(q, cache, table, tiles, cut)
            line += f" | {t:8.1f} us ({flops / t / 1e6:6.0f} TFLOP/s; {len(cut[0])} blocks, {cut[2]} partial results merged)"
        else:
            line += " | as it is"
        print(line)
    return 0


def kernel_prompt_elementwise(cfg, rows):
    """The memory-bound kernels of a prompt step alone at the shape's widths, each beside a plain copy of the same
    bytes: ten launches replayed as a CUDA graph (data in L2), and the same with a 512 MB buffer written before
    each launch (data from memory; the time of the writes alone is subtracted)."""
    import statistics
    import torch
    from air_b200.csrc import ops
    E, H, K = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d, I, P, T = cfg.get("head_dim", E // H), cfg["intermediate_size"], 64, rows
    big = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")

    def graph_time(calls, reps=10):
        for c in calls:
            c()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                for c in calls:
                    c()
        graph.replay()
        torch.cuda.synchronize()
        us = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            us.append(a.elapsed_time(b) * 1e3 / reps)
        return statistics.median(us)

    flush = lambda: big.zero_()
    t_flush = graph_time([flush])

    def report(name, f, nbytes):
        warm, cold = graph_time([f]), graph_time([flush, f]) - t_flush
        print(f"  {name:44s} {nbytes / 1e6:7.1f} MB  in L2 {warm:6.1f} us ({nbytes / warm / 1e6:5.2f} TB/s)  "
              f"from memory {cold:6.1f} us ({nbytes / cold / 1e6:5.2f} TB/s)", flush=True)
    print(f"{T} rows: hidden {E}, {H}/{K} heads of {d}, intermediate {I}")
    h = torch.randn(T, E, device="cuda")
    w = torch.ones(E, dtype=torch.bfloat16, device="cuda")
    x = torch.empty(T, E, dtype=torch.bfloat16, device="cuda")
    report("copy float32 -> bfloat16 [rows, hidden]", lambda: x.copy_(h), T * E * 6)
    report("add_rmsnorm, nothing to add", lambda: ops.add_rmsnorm(h, None, w, 1e-6, x), T * E * 6)
    delta = torch.randn(T, E, device="cuda")
    report("add_rmsnorm, a float32 delta", lambda: ops.add_rmsnorm(h, delta, w, 1e-6, x), T * E * 14)
    W = (H + 2 * K) * d
    qkv, bias = torch.randn(T, W, device="cuda"), torch.randn(W, device="cuda")
    table = torch.randn(T + 8, d, device="cuda")
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    seq = torch.zeros(T, dtype=torch.int32, device="cuda")
    pages = -(-T // P)
    bt = torch.arange(pages, dtype=torch.int32, device="cuda")[None, :].contiguous()
    q = torch.empty(T, H, d, dtype=torch.bfloat16, device="cuda")
    cache = torch.zeros(pages, 2, K, P, d, dtype=torch.bfloat16, device="cuda")
    report("bias + rotation + cache write", lambda: ops.qkv_rope_store(qkv, bias, table, positions, seq, bt, q, cache, H, K, d),
           T * W * 6)
    y = torch.empty(T, W, dtype=torch.bfloat16, device="cuda")
    report("copy float32 -> bfloat16 [rows, (H + 2K) d]", lambda: y.copy_(qkv), T * W * 6)
    gu = torch.randn(T, 2 * I, device="cuda").to(torch.bfloat16)
    act = torch.empty(T, I, dtype=torch.bfloat16, device="cuda")
    report("silu(gate) * up, blocks of 128", lambda: ops.silu_mul(gu, act, block=128), T * I * 6)
    z = torch.empty(T, 2 * I, dtype=torch.bfloat16, device="cuda")
    report("copy bfloat16 [rows, 2 x intermediate]", lambda: z.copy_(gu), T * I * 8)
    return 0


def reference_arm(args, cfg, context):
    """EmersonDowell/AIR's CUDA executor on the same shape: its own prefill and step_greedy_batch."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ref
    try:
        if args.batch > 8:
            raise ref.Unavailable("AIR decodes at most 8 sequences together (kMaxNativeDecodeBatch)")
        ref.build()
        clocks = ClockSampler()
        r = ref.bench(layers=args.layers or cfg["num_hidden_layers"], hidden=cfg["hidden_size"],
                      ffn=cfg["intermediate_size"], heads=cfg["num_attention_heads"],
                      kv_heads=cfg["num_key_value_heads"], vocab=cfg["vocab_size"],
                      max_positions=cfg["max_position_embeddings"], theta=cfg["rope_theta"], eps=cfg["rms_norm_eps"],
                      batch=args.batch, context=context, prefill=args.prefill_tokens, steps=args.steps,
                      warmup=args.warmup, fill="fork")
        clocks = clocks.stop()
    except ref.Unavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return 0
    ms = r["decode_ms_per_step"]
    value = args.batch / (ms / 1e3)
    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen2.5-{args.shape.upper()} shape, bf16 weights, random weights)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "reference",
        "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": args.layers or cfg["num_hidden_layers"],
                   "layers_of_model": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
                   "seq_len": context, "context": context, "page_tokens": 16, "prefill_tokens": args.prefill_tokens,
                   "parallelism": "single GPU",
                   "same_config": "same shape, batch, context and bf16 weights; AIR keeps activations and cache in "
                                  "float32 and runs its own scalar kernels; the context is one computed prompt, "
                                  "forked (CudaKvCache::fork) for the other sequences",
                   "timing": "host clock around AIR's blocking calls (step_greedy_batch, prefill_greedy)"},
        # AIR's call takes host tokens and returns host tokens: it is end to end by construction
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 4 * args.batch,
                "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": None, "clocks": clocks,
        "prefill": {"value": r["prefill_tokens"] / (r["prefill_ms"] / 1e3) if r["prefill_ms"] > 0 else None,
                    "tokens": r["prefill_tokens"], "ms": r["prefill_ms"]},
        "reference_record": r,
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--shape", default="7b", help="7b, 14b, 32b, or a config.json of the architecture")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=0, help="tokens per request (default: 8192; 4096 at 32b)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (for profiling)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--repeats", type=int, default=5, help="timed repeats of K decode steps and of the prefill step")
    ap.add_argument("--prefill-pause-ms", type=float, default=200.0, help="idle time before every prefill repeat")
    ap.add_argument("--mixed", default="", help="D,P: also time one step of D decoding requests beside a P-token portion")
    ap.add_argument("--max-tokens", type=int, default=0, help="tokens in the cache pool (default: what device memory is left)")
    ap.add_argument("--output", default="", help="also write the JSON line to this file")
    ap.add_argument("--no-points", action="store_true", help="skip decoding at batch 1 and 64")
    ap.add_argument("--skip-prefill", action="store_true", help="for profiling the decode step alone")
    ap.add_argument("--skip-e2e", action="store_true", help="for profiling the decode step alone")
    ap.add_argument("--skip-decode", action="store_true", help="for profiling the prefill step alone")
    ap.add_argument("--no-graphs", action="store_true", help="launch the decode step's kernels one by one (for ncu)")
    ap.add_argument("--kernel", default="", help="prefill_attention, or prompt_elementwise (at --prefill-tokens rows): time those kernels alone and exit")
    ap.add_argument("--timeline", action="store_true", help="also print the kernels' spans inside the decode graph and in the prefill step")
    args = ap.parse_args()
    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not supported",
                          "n_gpus": args.gpus}))
        return 2
    args.warmup = max(args.warmup, 3)
    if args.shape in SHAPES:
        cfg, context = dict(SHAPES[args.shape]), args.context or CONTEXTS[args.shape]
    else:
        with open(args.shape) as f:
            cfg = json.load(f)
        context = args.context or 8192
        args.shape = os.path.splitext(os.path.basename(args.shape))[0]
    if args.impl == "reference":
        return reference_arm(args, cfg, context)
    if args.kernel:
        if args.kernel == "prompt_elementwise":
            return kernel_prompt_elementwise(cfg, args.prefill_tokens)
        if args.kernel != "prefill_attention":
            print(json.dumps({"error": f"--kernel {args.kernel}: prefill_attention and prompt_elementwise are timed alone"}))
            return 2
        return kernel_prefill_attention(cfg)
    layers_of_model = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
        if "max_window_layers" in cfg:
            cfg["max_window_layers"] = args.layers

    import torch
    from air_b200.engine.batch import Entry, LAST_SAMPLED
    from air_b200.engine.engine import Engine, EngineConfig
    pk = peaks()
    mixed = tuple(int(x) for x in args.mixed.split(",")) if args.mixed else None
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    most = max(batches + ([mixed[0] + 1] if mixed else []))
    page = 64
    engine = Engine.from_random(cfg, seed=0, config=EngineConfig(
        dtype=torch.bfloat16, page_tokens=page, max_tokens=args.max_tokens or None, max_requests=most + 1,
        cuda_graphs=not args.no_graphs))
    mc = engine.model_config
    pool_tokens = engine.cache.num_pages * page
    per_request = -(-(context + 8) // page) * page
    batches = [b for b in batches if b * per_request <= pool_tokens] or [1]
    if args.batch not in batches:
        print(json.dumps({"error": f"the cache pool holds {pool_tokens} tokens: too few for batch {args.batch} at "
                                   f"{context} tokens"}))
        return 1
    weight_bytes = engine.model.weight_bytes()
    kv_bytes_per_token = engine.cache.bytes_per_page(engine.model.cache_needs(), page, torch.bfloat16) // page
    randomize_cache(engine, torch)

    results = {}
    if args.skip_decode:
        batches, args.skip_e2e = [], True
        results[args.batch] = {"times": [float("nan")], "ms": float("nan"), "clocks": None, "launches": 0}
    for b in batches:
        requests = [f"r{i}" for i in range(b)]
        times, clocks, launches = decode_device(engine, requests, context, args.steps, args.warmup,
                                                args.repeats if b == args.batch else max(1, min(3, args.repeats)),
                                                torch, Entry, LAST_SAMPLED)
        results[b] = {"times": times, "ms": statistics.median(times), "clocks": clocks, "launches": launches}
        if args.timeline and b == args.batch:
            decode_timeline(engine, requests, context, torch, Entry, LAST_SAMPLED)
        if b == args.batch and not args.skip_e2e:
            sec, h2d, d2h = decode_e2e(engine, requests, context, args.steps, args.warmup, torch)
            results[b]["e2e"] = {"value": b / sec, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                                 "d2h_bytes_per_step": d2h}

    # prefill of one request, one step
    T = args.prefill_tokens
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, mc.vocab_size, (T,), generator=g).tolist()
    times = []
    for i in range(0 if args.skip_prefill else 2 + max(1, args.repeats)):
        torch.cuda.synchronize()
        # A prompt's prefill is a burst of some tens of milliseconds, not a sustained load: every repeat starts
        # after a pause, so that it is not timed at the clocks that the repeats before it left (seven steps back
        # to back run into the power limit: 23.4, 23.4, 24.3, 25.0, 24.6 ms were measured so).
        time.sleep(args.prefill_pause_ms / 1e3)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        engine.step([Entry("p", prompt, [T - 1])])
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
        engine.finish("p")
    pre_ms = statistics.median(times[2:]) if times else float("nan")       # (the first two steps are warm-up)
    if args.timeline and not args.skip_prefill:
        prefill_timeline(engine, prompt, torch, Entry)
    L, E, I, V = len(engine.model.spec.order), mc.hidden_size, mc.intermediate_size, mc.vocab_size
    H, K, d = mc.num_attention_heads, mc.num_key_value_heads, mc.head_dim
    gemm_params = L * (E * (H + 2 * K) * d + H * d * E + 3 * E * I)
    flops = 2 * T * gemm_params + L * 4 * H * d * (T * (T + 1) // 2) + 2 * E * V
    prefill = {"value": T / (pre_ms / 1e3), "tokens": T, "ms": pre_ms, "repeat_ms": times[2:],
               "pause_ms": args.prefill_pause_ms,
               "frac": flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12)}
    if "bf16_tflops_sustained" in pk:      # the step is tens of milliseconds long: also against the figure under the power cap
        prefill["frac_sustained"] = flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12)

    mixed_record = None
    if mixed:
        D, P = mixed
        dev_ms, host_ms, prior = mixed_step(engine, D, P, context, max(5, args.repeats), torch, Entry)
        live = (D * context + prior + P) * kv_bytes_per_token
        step_flops = 2 * (D + P) * gemm_params + L * 4 * H * d * (P * prior + P * (P + 1) // 2) + 2 * E * V * D
        # The step's kernels run one after the other: the decode attention is bound by the cache it reads, the
        # products and the portion's attention by their flops (or by the weights, if those take longer to read).
        cache_ms = D * context * kv_bytes_per_token / (pk["hbm_gbs"] * 1e9) * 1e3
        product_ms = max(2 * (D + P) * gemm_params / (pk["bf16_tflops"] * 1e12), weight_bytes / (pk["hbm_gbs"] * 1e9)) * 1e3
        attention_ms = L * 4 * H * d * (P * prior + P * (P + 1) // 2) / (pk["bf16_tflops"] * 1e12) * 1e3
        mixed_record = {"decode": D, "portion": P, "portion_prior_tokens": prior, "device_ms": dev_ms,
                        "host_ms": host_ms, "tokens_per_s": (D + P) / (dev_ms / 1e3),
                        "bytes_frac": (weight_bytes + live) / (dev_ms / 1e3) / 1e9 / pk["hbm_gbs"],
                        "flops_frac": step_flops / (dev_ms / 1e3) / (pk["bf16_tflops"] * 1e12),
                        "roofline_ms": cache_ms + product_ms + attention_ms,
                        "frac": (cache_ms + product_ms + attention_ms) / dev_ms}

    main_r = results[args.batch]
    ms = main_r["ms"]

    def bytes_a_second(batch):        # what a decode step at this batch has to read, over its time (GB/s)
        live = batch * (context - (args.steps + 2) // 2) * kv_bytes_per_token
        return (weight_bytes + live) / (results[batch]["ms"] / 1e3) / 1e9
    achieved = bytes_a_second(args.batch)
    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen2.5-{args.shape.upper()} shape, bf16, random weights)",
        "value": args.batch / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": L, "layers_of_model": layers_of_model,
                   "hidden": E, "heads": H, "kv_heads": K, "head_dim": d, "intermediate": I, "vocab": V,
                   "global_batch": args.batch, "seq_len": context, "context": context,
                   "page_tokens": page, "pool_tokens": pool_tokens, "prefill_tokens": T, "repeats": args.repeats,
                   "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights read every step)", "peaks": pk["source"]},
        "repeat_ms_per_step": main_r["times"],
        "e2e": main_r.get("e2e"),
        "gpu_launches": main_r["launches"],
        "clocks": main_r["clocks"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": {f"decode_b{b}": b / (results[b]["ms"] / 1e3) for b in batches if b != args.batch},
        "points_roofline_frac": {f"decode_b{b}": bytes_a_second(b) / pk["hbm_gbs"] for b in batches if b != args.batch},
    }
    if mixed_record:
        line["mixed"] = mixed_record
    text = json.dumps(line)
    print(text)
    if args.output:
        with open(args.output, "w") as f:
            f.write(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
