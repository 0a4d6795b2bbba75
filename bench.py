#!/usr/bin/env python3
"""Benchmark of the decode step (and of a 2,048-token prefill) at the Qwen2.5-7B shape with
random bfloat16 weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 8192] [--layers L]

A "step" is one decode step of the whole batch.  It prints ONE JSON line:
  value      decoded tokens per second, timed on the device with CUDA events over exactly K
             steps after W warm-up steps; every request holds `context` tokens in the cache and
             feeds its last sampled token back on the device (no host round trip)
  e2e        the same through the Python entry point (InferenceService.run_cycle): every step
             copies the step's token ids and tables from pinned host memory and reads the
             sampled ids back
  prefill    one step of 2,048 prompt tokens of one request; frac = flops / time / bf16 peak
  roofline   bytes the decode step has to read (every weight once, the live requests' cache)
             / its time, against the measured copy bandwidth
  points     decode tokens per second at batch 1 and 64 (points_roofline_frac: their share of the
             copy bandwidth, counted as for roofline)
The cache of the decoding requests is filled with random keys and values instead of running
64 prompts of 8,192 tokens (data: synthetic); timing does not depend on the values.  Between
timed steps nothing is flushed: a step reads its weights (over 14 GB at 28 layers), far more
than the 126 MB of L2.
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

QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 28, "hidden_size": 3584,
    "num_attention_heads": 28, "num_key_value_heads": 4, "intermediate_size": 18944, "vocab_size": 152064,
    "max_position_embeddings": 32768, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "sliding_window": 131072, "use_sliding_window": False, "max_window_layers": 28, "hidden_act": "silu",
}
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


def fill_cache(engine, requests, context, torch):
    """Opens the requests with `context` tokens each and random keys and values in the pages."""
    for r in requests:
        engine.cache.open(r)
        engine.cache.reserve([(r, context)])
        engine.cache.commit(r, context)
    g = torch.Generator(device=engine.rt.device)
    g.manual_seed(1234)
    seen = set()
    for run in range(len(engine.model.spec.order)):
        for view in engine.cache.views(run):
            kv = getattr(view, "kv", None)
            if kv is not None and kv.data_ptr() not in seen:
                seen.add(kv.data_ptr())
                kv.normal_(0.0, 0.5, generator=g)


def decode_device(engine, requests, steps, warmup, torch, Entry, LAST):
    """K decode steps timed with CUDA events; tokens are fed back on the device."""
    first = [Entry(r, [17 + i], [0]) for i, r in enumerate(requests)]
    engine.sample(engine.step(first))
    again = [Entry(r, [LAST], [0]) for r in requests]
    for _ in range(warmup):
        engine.sample(engine.step(again))
    torch.cuda.synchronize()
    launches0 = engine.kernel_launches()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks = ClockSampler()
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        engine.sample(engine.step(again))
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    return ms / steps, clocks.stop(), engine.kernel_launches() - launches0


def decode_timeline(engine, requests, torch, Entry, LAST):
    """Spans of the kernels of one decode step as they run inside the CUDA graph (from the moment a
    kernel has passed the wait on its predecessor to the moment the next one has), by kernel."""
    import collections
    from air_b200.csrc import ops
    again = [Entry(r, [LAST], [0]) for r in requests]
    buf = torch.zeros(1 + 2 * 16384, dtype=torch.int64, device=engine.rt.device)
    ops.set_trace(buf)
    for _ in range(3):
        engine.sample(engine.step(again))
    torch.cuda.synchronize()
    ops.set_trace(None)
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
    # one layer from the middle of the step, kernel by kernel
    names = [ops.TRACE_NAMES[k] for _, k in step]
    for i in range(len(step) // 2, len(step) - 10):
        if names[i:i + 2] == ["add_rmsnorm", "gemm_tc"] and names[i + 2] in ("qkv_rope_store", "decode_attention"):
            j = next((j for j in range(i + 3, len(step) - 1) if names[j:j + 3] == names[i:i + 3]), None)
            if j is not None:
                print("  one layer (us): " + " | ".join(f"{names[q]} {(step[q + 1][0] - step[q][0]) / 1e3:.1f}"
                                                       for q in range(i, j)))
            break


def prefill_timeline(engine, prompt, torch, Entry):
    """Spans between the starts of this package's kernels in one prefill step.  A library product has
    no trace point: its time is part of the span of the kernel before it (add_rmsnorm before the QKV
    and gate/up products, prefill_attention before the output product, and so on)."""
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


def decode_e2e(engine, requests, steps, warmup, torch):
    """The same through InferenceService.run_cycle, host tokens in and out every step."""
    from air_b200.engine.service import InferenceService, SchedulerConfig
    from air_b200.sampling.sampler import GenerationConfig
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
    ctx = engine.last_context
    # per step: 4 ints per token of the decode graph's batch from pinned memory; sampled ids back
    size = next(iter(engine.graphs.values())).size if engine.graphs else len(requests)
    sizes = [g.size for g in engine.graphs.values() if g.size >= len(requests)]
    h2d = 16 * (min(sizes) if sizes else len(requests))
    return sec / steps, h2d, 4 * len(requests)


def release(engine, requests):
    for r in requests:
        if r in engine.cache.sequences:
            engine.finish(r)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=QWEN25_7B["num_hidden_layers"])
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip decoding at batch 1 and 64")
    ap.add_argument("--skip-prefill", action="store_true", help="for profiling the decode step alone")
    ap.add_argument("--skip-e2e", action="store_true", help="for profiling the decode step alone")
    ap.add_argument("--skip-decode", action="store_true", help="for profiling the prefill step alone")
    ap.add_argument("--no-graphs", action="store_true", help="launch the decode step's kernels one by one (for ncu)")
    ap.add_argument("--timeline", action="store_true", help="also print the kernels' spans inside the decode graph and in the prefill step")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "EmersonDowell/AIR is a CMake C++ project without setup.py or pyproject.toml (pip cannot "
                          "install it), reads GGUF files only and ships no sm_100 code path"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not supported",
                          "n_gpus": args.gpus}))
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    from air_b200.engine.batch import Entry, LAST_SAMPLED
    from air_b200.engine.engine import Engine, EngineConfig
    pk = peaks()
    cfg = dict(QWEN25_7B, num_hidden_layers=args.layers)
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    page = 64
    per_request = -(-(args.context + 8) // page) * page
    max_tokens = max(batches) * per_request + 4096
    engine = Engine.from_random(cfg, seed=0, config=EngineConfig(
        dtype=torch.bfloat16, page_tokens=page, max_tokens=max_tokens, max_requests=max(batches) + 1,
        cuda_graphs=not args.no_graphs))
    mc = engine.model_config
    weight_bytes = engine.model.weight_bytes()
    kv_bytes_per_token = 2 * mc.num_key_value_heads * mc.head_dim * 2 * len(engine.model.spec.order)

    results = {}
    if args.skip_decode:
        batches, args.skip_e2e = [], True
        results[args.batch] = {"ms": float("nan"), "clocks": None, "launches": 0}
    for b in batches:
        requests = [f"r{i}" for i in range(b)]
        start_len = args.context - (args.steps + args.warmup + 2)
        fill_cache(engine, requests, start_len, torch)
        ms, clocks, launches = decode_device(engine, requests, args.steps, args.warmup, torch, Entry, LAST_SAMPLED)
        results[b] = {"ms": ms, "clocks": clocks, "launches": launches}
        if args.timeline and b == args.batch:
            decode_timeline(engine, requests, torch, Entry, LAST_SAMPLED)
        release(engine, requests)
        if b == args.batch and not args.skip_e2e:
            fill_cache(engine, requests, start_len, torch)
            sec, h2d, d2h = decode_e2e(engine, requests, args.steps, args.warmup, torch)
            results[b]["e2e"] = {"value": b / sec, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                                 "d2h_bytes_per_step": d2h}
            release(engine, requests)

    # prefill of one request, one step
    T = args.prefill_tokens
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, mc.vocab_size, (T,), generator=g).tolist()
    times = []
    for i in range(0 if args.skip_prefill else 3):
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        engine.step([Entry("p", prompt, [T - 1])])
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
        engine.finish("p")
    pre_ms = min(times[1:]) if times else float("nan")
    if args.timeline and not args.skip_prefill:
        prefill_timeline(engine, prompt, torch, Entry)
    L, E, I, V = len(engine.model.spec.order), mc.hidden_size, mc.intermediate_size, mc.vocab_size
    H, K, d = mc.num_attention_heads, mc.num_key_value_heads, mc.head_dim
    gemm_params = L * (E * (H + 2 * K) * d + H * d * E + 3 * E * I)
    flops = 2 * T * gemm_params + L * 4 * H * d * (T * (T + 1) // 2) + 2 * E * V
    prefill = {"value": T / (pre_ms / 1e3), "tokens": T, "ms": pre_ms,
               "frac": flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12)}
    if "bf16_tflops_sustained" in pk:      # the step is tens of milliseconds long: also against the figure under the power cap
        prefill["frac_sustained"] = flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12)

    main_r = results[args.batch]
    ms = main_r["ms"]
    def bytes_a_second(batch):        # what a decode step at this batch has to read, over its time (GB/s)
        live = batch * (args.context - (args.steps + args.warmup + 2) // 2) * kv_bytes_per_token
        return (weight_bytes + live) / (results[batch]["ms"] / 1e3) / 1e9
    achieved = bytes_a_second(args.batch)
    line = {
        "metric": "decode tok/s at batch 8 (Qwen2.5-7B shape, bf16, random weights)",
        "value": args.batch / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": "Qwen2.5-7B shape", "layers": L, "layers_of_model": QWEN25_7B["num_hidden_layers"],
                   "hidden": E, "heads": H, "kv_heads": K, "head_dim": d, "intermediate": I, "vocab": V,
                   "global_batch": args.batch, "seq_len": args.context, "context": args.context,
                   "page_tokens": page, "prefill_tokens": T, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights read every step)", "peaks": pk["source"]},
        "e2e": main_r.get("e2e"),
        "gpu_launches": main_r["launches"],
        "clocks": main_r["clocks"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": {f"decode_b{b}": b / (results[b]["ms"] / 1e3) for b in batches if b != args.batch},
        "points_roofline_frac": {f"decode_b{b}": bytes_a_second(b) / pk["hbm_gbs"] for b in batches if b != args.batch},
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
