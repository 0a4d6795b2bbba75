"""Helpers of the tests: the tiny configurations, model folders in temporary places, traces
and their replay, and the comparison with the plain implementation."""
import functools
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

BASE = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu"}

# Two tiny configurations that differ in every size and option, and a third with a window.  A and B are the
# two tiny configurations that this engine's target names (2 layers / 64 / 4 heads of 16 in 2 groups / 128 / 256,
# tied; 3 layers / 128 / 4 heads of 32 in 1 group / 352 / 384, separate output matrix), but for A's
# max_position_embeddings, which is 512 here instead of 128 because the replay tests run longer requests.
TINY_A = dict(BASE, num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
              intermediate_size=128, vocab_size=256, max_position_embeddings=512, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, use_sliding_window=False)
TINY_B = dict(BASE, num_hidden_layers=3, hidden_size=128, num_attention_heads=4, num_key_value_heads=1,
              intermediate_size=352, vocab_size=384, max_position_embeddings=256, rope_theta=1e6,
              rms_norm_eps=1e-5, tie_word_embeddings=False, use_sliding_window=False, sliding_window=4096)
TINY_W = dict(BASE, num_hidden_layers=3, hidden_size=96, num_attention_heads=3, num_key_value_heads=3,
              intermediate_size=208, vocab_size=301, max_position_embeddings=512, rope_theta=50000.0,
              rms_norm_eps=3e-6, tie_word_embeddings=False, use_sliding_window=True, sliding_window=40,
              max_window_layers=1)
# Two more with the head sizes that the tensor-core attention kernels take (64 and 128; the three above
# have 16 and 32 and run the 32-bit attention kernel in both precisions), one of them with a window.
TINY_K = dict(BASE, num_hidden_layers=2, hidden_size=128, num_attention_heads=2, num_key_value_heads=1,
              intermediate_size=160, vocab_size=199, max_position_embeddings=512, rope_theta=30000.0,
              rms_norm_eps=2e-6, tie_word_embeddings=True, use_sliding_window=False)
TINY_L = dict(BASE, num_hidden_layers=2, hidden_size=384, num_attention_heads=3, num_key_value_heads=3,
              intermediate_size=256, vocab_size=230, max_position_embeddings=512, rope_theta=1e5,
              rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=True, sliding_window=70,
              max_window_layers=1)
TINY_M = dict(BASE, num_hidden_layers=2, hidden_size=512, num_attention_heads=2, num_key_value_heads=1,
              intermediate_size=192, vocab_size=150, max_position_embeddings=512, rope_theta=20000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, use_sliding_window=False)      # heads of 256
CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "W": (TINY_W, 2), "K": (TINY_K, 3), "L": (TINY_L, 4),
           "M": (TINY_M, 5)}

_folders = {}
_tmp = []


SCORE_STD = 2.5     # standard deviation of the attention scores that the test models are drawn for


def sharpen_attention(folder, cfg):
    """Rewrites a random model's q and k projections so that attention is far from uniform.

    Drawn at N(0, 0.02) like every other matrix, q and k give attention scores with a standard deviation of
    0.02 to 0.15: softmax is then all but flat, and a model without any position encoding, with a window that
    is one key too wide or with two swapped keys computes the same logits within bfloat16's tolerance.  Here q and
    k weights are scaled so that scores have a standard deviation of SCORE_STD (the largest probability among
    150 keys is then 10 to 40 times the uniform one), and their biases to N(0, 0.3).  tests/test_plain.py
    checks that this is so, for every configuration.  The numbers stay values that bfloat16 holds."""
    import torch
    from air_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    weight = (SCORE_STD ** 0.5) / (0.02 * cfg["hidden_size"] ** 0.5)
    for n, t in tensors.items():
        if n.endswith(("q_proj.weight", "k_proj.weight")):
            tensors[n] = (t.float() * weight).to(t.dtype)
        elif n.endswith(("q_proj.bias", "k_proj.bias")):
            tensors[n] = (t.float() * 15.0).to(t.dtype)
    del f
    write_safetensors(path, tensors, metadata={"format": "pt"})


def model_folder(name, dtype="bfloat16"):
    """A folder with config.json and model.safetensors for a tiny configuration, made once per
    session in a temporary place.  Weights are stored as bfloat16 values (also for the float32
    tests, so that both precisions and the plain implementation read the same numbers); q and k are
    scaled so that attention has something to look at (sharpen_attention)."""
    key = (name, dtype)
    if key not in _folders:
        from air_b200.engine.engine import write_random_model
        cfg, seed = CONFIGS[name]
        d = tempfile.TemporaryDirectory(prefix=f"air_b200_{name}_")
        _tmp.append(d)
        write_random_model(d.name, cfg, seed, dtype)
        sharpen_attention(d.name, cfg)
        _folders[key] = d.name
    return _folders[key]


@functools.lru_cache(maxsize=None)
def plain_model(folder):
    from plain import qwen2_plain as plain
    return plain.read_model(folder)


_plain_cache = {}


def plain_logits(folder, tokens):
    """Logits [len(tokens), vocab] of the plain implementation (cached per token list)."""
    from plain import qwen2_plain as plain
    key = (folder, tuple(tokens))
    if key not in _plain_cache:
        cfg, tensors = plain_model(folder)
        _plain_cache[key] = plain.forward(cfg, tensors, list(tokens))
    return _plain_cache[key]


def tokens_for(name, n, seed):
    cfg, _ = CONFIGS[name]
    return np.random.default_rng(1000 + seed).integers(0, cfg["vocab_size"], size=n).tolist()


# ------------------------------------------------------------------ traces
def step_line(step, entries, end=()):
    return {"step": step, "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries],
            "end": list(end)}


def trace_whole(streams):
    """Each request alone and whole, all logits wanted."""
    return [step_line(n, [(rid, toks, range(len(toks)))], end=[rid]) for n, (rid, toks) in enumerate(streams.items())]


def trace_bulk_tail(streams, tail=32):
    steps, n = [], 0
    for rid, toks in streams.items():
        cut = max(1, len(toks) - tail)
        steps.append(step_line(n, [(rid, toks[:cut], range(cut))]))
        n += 1
        for i in range(cut, len(toks)):
            steps.append(step_line(n, [(rid, [toks[i]], [0])], end=[rid] if i == len(toks) - 1 else []))
            n += 1
        if cut == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(streams, sizes=(33, 2, 17, 5, 2, 64, 3, 2, 31, 16, 1, 47, 2)):
    steps, n = [], 0
    for rid, toks in streams.items():
        i, k = 0, 0
        while i < len(toks):
            m = min(sizes[k % len(sizes)], len(toks) - i)
            steps.append(step_line(n, [(rid, toks[i:i + m], range(m))], end=[rid] if i + m == len(toks) else []))
            i += m
            k += 1
            n += 1
    return steps


def trace_mixed(streams, seed=0, live=4, tail=12, portions=(2, 5, 9, 16, 23, 31, 40)):
    """Up to `live` requests at a time: each is fed in portions of changing size, then its last
    `tail` tokens one by one, beside whatever the others are doing; a request that ends makes
    room for the next one, so pages are used again.  All logits are wanted."""
    rng = np.random.default_rng(seed)
    waiting = list(streams.items())
    active = {}
    steps, n = [], 0
    while waiting or active:
        while waiting and len(active) < live:
            rid, toks = waiting.pop(0)
            active[rid] = [toks, 0]
        entries, end = [], []
        for rid in list(active):
            toks, pos = active[rid]
            if rng.random() < 0.2 and len(active) > 1:
                continue  # left out of this step, goes on later
            rest = len(toks) - pos
            m = 1 if rest <= tail else min(int(rng.choice(portions)), rest - tail)
            entries.append((rid, toks[pos:pos + m], range(m)))
            active[rid][1] = pos + m
            if pos + m == len(toks):
                end.append(rid)
                del active[rid]
        if entries:
            steps.append(step_line(n, entries, end))
            n += 1
    return steps


def peak_tokens(steps, page=64):
    """The most tokens live requests hold at any time, each rounded up to whole pages."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-v // page) * page for v in held.values()))
        for r in s["end"]:
            held.pop(r, None)
    return peak


def replay(folder, dtype, steps, max_tokens, page_tokens=16, max_requests=8):
    """Runs the steps through Engine.step (in process) and returns {(request, position): logits}."""
    import torch
    from air_b200.engine.engine import Engine, EngineConfig
    from air_b200.engine.replay import run_trace
    engine = Engine.from_folder(folder, EngineConfig(dtype=dtype, page_tokens=page_tokens, max_tokens=max_tokens,
                                                     max_requests=max_requests))
    with tempfile.TemporaryDirectory() as out:
        run_trace(engine, [json.dumps(s) for s in steps], out)
        engine.cache.check()
        assert not engine.cache.sequences, "every request of the trace was ended"
        assert engine.cache.free_pages() == engine.cache.num_pages
        return collect(steps, out, engine.model.spec.vocab_size), engine


def collect(steps, out_dir, vocab):
    got, pos = {}, {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if wanted == 0:
            assert not os.path.exists(path)
        else:
            data = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        r = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = data[r]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            pos.pop(rid, None)
    return got


def run_trace_program(folder, dtype, steps, max_tokens, out_dir, extra=()):
    """Runs bin/trace_run as a program; checks the `done` lines."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)] + list(extra)
    p = subprocess.run(cmd, input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                       timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    return p


# ------------------------------------------------------------------ comparison
# Tolerances are set once, from the arithmetic: float32 differs from the 64-bit-accumulating
# plain implementation by a few units of 1e-7 per operation; bfloat16 rounds activations to 8
# bits of mantissa (2^-9 relative per rounding) at each of a few dozen places.  With the sharpened
# attention of these models (scores of a standard deviation of 2.5, so a rounding of q and k moves a
# score by up to 0.02 and a probability by 2 %), 60 configurations drawn at random gave, relative to the
# largest |logit|: the largest difference 0.011 in the median and 0.036 at most, the worst row's mean
# difference 0.0026 in the median and 0.0075 at most; 1,000 such configurations later, 33 lay above 0.006 in the
# worst row's mean, 0.0105 at most, and none failed in float32.  The tolerances stand where they stood for the
# unsharpened models; every model of the suite is inside them (another draw of the same configuration may lie in
# that tail of one in thirty), and tests/test_plain.py checks that a missing rotation or a window off by one is at
# least three times outside.
FP32_TOL = 2e-5     # of the largest |logit|
BF16_MAX_TOL = 4e-2
BF16_MEAN_TOL = 6e-3


def check_against_plain(got, folder, streams, dtype):
    worst = 0.0
    for rid, toks in streams.items():
        ref = plain_logits(folder, toks)
        scale = max(1.0, float(np.abs(ref).max()))
        rows = sorted(p for (r, p) in got if r == rid)
        assert rows, f"no logits for request {rid}"
        for p in rows:
            out = got[(rid, p)]
            assert np.isfinite(out).all()
            diff = np.abs(out - ref[p])
            if dtype == "float32":
                assert diff.max() <= FP32_TOL * scale, (rid, p, float(diff.max()))
                assert out.argmax() == ref[p].argmax() or np.sort(ref[p])[-1] - np.sort(ref[p])[-2] < 2 * FP32_TOL * scale
            else:
                assert diff.max() <= BF16_MAX_TOL * scale, (rid, p, float(diff.max()))
                assert diff.mean() <= BF16_MEAN_TOL * scale, (rid, p, float(diff.mean()))
                top2 = np.sort(ref[p])[-2:]
                if top2[1] - top2[0] > 2 * BF16_MAX_TOL * scale:
                    assert out.argmax() == ref[p].argmax()
            worst = max(worst, float(diff.max()) / scale)
    return worst
