"""Plain, slow implementation of the Qwen2 dense decoder, written from the formulas
of EmersonDowell/AIR's CPU reference executor.  It is the oracle of the tests.

It shares no code with ``air_b200``: it has its own reader for safetensors files, runs
whole sequences without any cache, on the CPU, and has one function for each part.
Storage is 32-bit; dot products, the mean of squares, rotation angles and the softmax are
accumulated in 64-bit and rounded to 32-bit at the places where AIR's reference executor
rounds (src/reference/reference_executor.cpp, src/reference/tensor_reader.cpp:369-394).

tests/golden/ holds logits of AIR's own compiled reference executor for a tiny random
model; tests/test_plain.py compares this file with them.
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np

F32 = np.float32
F64 = np.float64


# ----------------------------------------------------------------------------- files
def read_safetensors(path):
    """name -> float32 (or int) numpy array.  Format: 8-byte little-endian header
    length, a JSON header {name: {dtype, shape, data_offsets}}, then raw data."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    data = memoryview(raw)[8 + hlen:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = data[lo:hi]
        dt = info["dtype"]
        if dt == "F32":
            arr = np.frombuffer(buf, dtype="<f4").astype(F32)
        elif dt == "BF16":
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(F32)
        elif dt == "F16":
            arr = np.frombuffer(buf, dtype="<f2").astype(F32)
        elif dt == "I32":
            arr = np.frombuffer(buf, dtype="<i4")
        elif dt == "I64":
            arr = np.frombuffer(buf, dtype="<i8")
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = arr.reshape(info["shape"]).copy()
    return out


def read_model(folder):
    """(config dict, tensors) of a folder with config.json and model.safetensors."""
    with open(f"{folder}/config.json") as f:
        config = json.load(f)
    return config, read_safetensors(f"{folder}/model.safetensors")


def round_bf16(a):
    """Round a float32 array to the nearest bfloat16 (ties to even), as float32."""
    u = np.ascontiguousarray(a, dtype=F32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(F32).reshape(np.shape(a))


# ----------------------------------------------------------------------------- parts
def embed(table, tokens):
    """Row gather, no scaling (reference_executor.cpp:328-339)."""
    tokens = np.asarray(tokens)
    if tokens.min() < 0 or tokens.max() >= table.shape[0]:
        raise ValueError("input token is outside model vocabulary")
    return table[tokens].astype(F32)


def rms_norm(x, weight, eps):
    """x * (1/sqrt(mean(x^2)+eps)) * w; the sum in 64-bit, the scale rounded to 32-bit,
    the products in 32-bit in the order x*scale*w (reference_executor.cpp:17-27)."""
    x = x.astype(F32)
    mean = (x.astype(F64) ** 2).sum(axis=-1, keepdims=True) / x.shape[-1]
    scale = (1.0 / np.sqrt(mean + float(eps))).astype(F32)
    return ((x * scale).astype(F32) * weight.astype(F32)).astype(F32)


def linear(x, weight, bias=None):
    """y = W x with W [out, in]; the dot product in 64-bit, rounded to 32-bit
    (tensor_reader.cpp:369-394); the bias is added afterwards in 32-bit
    (reference_executor.cpp:315-323, 349-360)."""
    y = (x.astype(F64) @ weight.astype(F64).T).astype(F32)
    if bias is not None:
        y = (y + bias.astype(F32)).astype(F32)
    return y


def rope(x, positions, theta):
    """Half-split rotation of x [T, heads, d]: pairs (i, i+d/2), angle p / theta^(2i/d)
    in 64-bit, cos and sin rounded to 32-bit, rotation in 32-bit
    (reference_executor.cpp:37-72)."""
    t, heads, d = x.shape
    half = d // 2
    i = np.arange(half, dtype=F64)
    inv_freq = 1.0 / np.power(float(theta), (2.0 * i) / float(d))
    angle = np.asarray(positions, dtype=F64)[:, None] * inv_freq[None, :]
    c = np.cos(angle).astype(F32)[:, None, :]
    s = np.sin(angle).astype(F32)[:, None, :]
    first = x[..., :half].astype(F32)
    second = x[..., half:].astype(F32)
    out = np.empty_like(x, dtype=F32)
    out[..., :half] = first * c - second * s
    out[..., half:] = first * s + second * c
    return out


def attention(q, k, v, window=None):
    """Causal grouped-query attention over a whole sequence.
    q [T, H, d], k and v [T, K, d]; q head h reads kv head floor(h*K/H); scores
    (q.k)/sqrt(d), maximum, exp and sum in 64-bit, the probability rounded to 32-bit,
    the value mix accumulated in 32-bit (reference_executor.cpp:74-138).  Query i sees
    keys 0..i; with a window w only keys j with i - j < w (AIR itself rejects windows,
    src/model/qwen2_contract.cpp:62-64; the formula is the causal one with a lower bound).
    """
    t, h, d = q.shape
    kv = k.shape[1]
    out = np.zeros((t, h, d), dtype=F32)
    scale = 1.0 / math.sqrt(float(d))
    idx = np.arange(t)
    visible = idx[None, :] <= idx[:, None]
    if window is not None:
        visible &= (idx[:, None] - idx[None, :]) < int(window)
    for head in range(h):
        g = (head * kv) // h
        scores = (q[:, head, :].astype(F64) @ k[:, g, :].astype(F64).T) * scale
        scores = np.where(visible, scores, -np.inf)
        m = scores.max(axis=-1, keepdims=True)
        e = np.exp(scores - m)
        z = e.sum(axis=-1, keepdims=True)
        if not np.all(np.isfinite(z)) or np.any(z <= 0):
            raise FloatingPointError("attention softmax produced a non-finite denominator")
        p = (e / z).astype(F32)
        out[:, head, :] = (p @ v[:, g, :].astype(F32)).astype(F32)
    return out


def silu(x):
    """x / (1 + exp(-x)) in 32-bit (reference_executor.cpp:33-35)."""
    x = x.astype(F32)
    return (x / (F32(1.0) + np.exp(-x).astype(F32))).astype(F32)


def swiglu(x, w_gate, w_up, w_down):
    """down(silu(gate(x)) * up(x)), no biases (reference_executor.cpp:394-408)."""
    g = linear(x, w_gate)
    u = linear(x, w_up)
    a = (silu(g) * u).astype(F32)
    return linear(a, w_down)


# ----------------------------------------------------------------------------- model
def _layer_windows(config):
    """Which layers see a window: config.json's use_sliding_window, sliding_window and
    max_window_layers (layers from max_window_layers on are windowed)."""
    n = config["num_hidden_layers"]
    if not config.get("use_sliding_window", False) or config.get("sliding_window") is None:
        return [None] * n
    first = config.get("max_window_layers", n)
    return [int(config["sliding_window"]) if i >= first else None for i in range(n)]


def decoder_layer(h, positions, tensors, config, layer, window=None, shared_kv=None):
    """One pre-norm block: norm, q/k/v with bias, rope, attention, o-projection,
    residual; norm, SwiGLU, residual (reference_executor.cpp:343-413).
    Returns (h, (k, v)); with shared_kv the layer reads those keys and values instead
    of its own."""
    p = f"model.layers.{layer}."
    heads = config["num_attention_heads"]
    kv_heads = config.get("num_key_value_heads", heads)
    d = config["hidden_size"] // heads
    eps = config["rms_norm_eps"]
    t = h.shape[0]

    n = rms_norm(h, tensors[p + "input_layernorm.weight"], eps)
    q = linear(n, tensors[p + "self_attn.q_proj.weight"], tensors.get(p + "self_attn.q_proj.bias"))
    q = rope(q.reshape(t, heads, d), positions, config["rope_theta"])
    if shared_kv is None:
        k = linear(n, tensors[p + "self_attn.k_proj.weight"], tensors.get(p + "self_attn.k_proj.bias"))
        v = linear(n, tensors[p + "self_attn.v_proj.weight"], tensors.get(p + "self_attn.v_proj.bias"))
        k = rope(k.reshape(t, kv_heads, d), positions, config["rope_theta"])
        v = v.reshape(t, kv_heads, d)
    else:
        k, v = shared_kv
    a = attention(q, k, v, window=window).reshape(t, heads * d)
    h = (h + linear(a, tensors[p + "self_attn.o_proj.weight"])).astype(F32)

    n = rms_norm(h, tensors[p + "post_attention_layernorm.weight"], eps)
    f = swiglu(n, tensors[p + "mlp.gate_proj.weight"], tensors[p + "mlp.up_proj.weight"],
               tensors[p + "mlp.down_proj.weight"])
    h = (h + f).astype(F32)
    return h, (k, v)


def forward(config, tensors, tokens, order=None, kv_round=None):
    """Logits [T, V] (float32) of a whole sequence.

    order: the runs of layers, a list of (layer, source) where source is None or the
    index of an earlier run whose keys and values this run reads; default is every
    layer once (reference_executor.cpp:343-413).
    kv_round: an optional function applied to keys and values before attention, to
    imitate a cache of lower precision.
    """
    tokens = np.asarray(tokens, dtype=np.int64)
    positions = np.arange(len(tokens))
    n_layers = config["num_hidden_layers"]
    windows = _layer_windows(config)
    if order is None:
        order = [(i, None) for i in range(n_layers)]
    h = embed(tensors["model.embed_tokens.weight"], tokens)
    kept = []
    for layer, source in order:
        shared = kept[source] if source is not None else None
        h, kv = decoder_layer(h, positions, tensors, config, layer, window=windows[layer],
                              shared_kv=shared)
        if kv_round is not None and shared is None:
            kv = (kv_round(kv[0]), kv_round(kv[1]))
        kept.append(kv)
    y = rms_norm(h, tensors["model.norm.weight"], config["rms_norm_eps"])
    if config.get("tie_word_embeddings", False) or "lm_head.weight" not in tensors:
        w_out = tensors["model.embed_tokens.weight"]
    else:
        w_out = tensors["lm_head.weight"]
    return linear(y, w_out)


def greedy_generate(config, tensors, prompt, max_new_tokens, eos=None):
    """Greedy continuation: the lowest index of the maximum (src/runtime/sampling.cpp:13-16),
    stopping after max_new_tokens or at eos (src/runtime/generation.cpp:26-80)."""
    tokens = list(prompt)
    new = []
    for _ in range(max_new_tokens):
        logits = forward(config, tensors, tokens)[-1]
        nxt = int(np.argmax(logits))
        new.append(nxt)
        tokens.append(nxt)
        if eos is not None and nxt == eos:
            break
    return new


# ----------------------------------------------------------------------------- sampling
class MT19937_64:
    """The 64-bit Mersenne twister of the C++ standard library, which AIR's Sampler
    seeds with SamplingConfig.seed (src/runtime/sampling.cpp:9)."""
    NN, MM = 312, 156
    MATRIX_A, UM, LM = 0xB5026F5AA96619E9, 0xFFFFFFFF80000000, 0x7FFFFFFF
    MASK = (1 << 64) - 1

    def __init__(self, seed):
        mt = [0] * self.NN
        mt[0] = seed & self.MASK
        for i in range(1, self.NN):
            mt[i] = (6364136223846793005 * (mt[i - 1] ^ (mt[i - 1] >> 62)) + i) & self.MASK
        self.mt, self.mti = mt, self.NN

    def next(self):
        mt = self.mt
        if self.mti >= self.NN:
            for i in range(self.NN):
                x = (mt[i] & self.UM) | (mt[(i + 1) % self.NN] & self.LM)
                mt[i] = mt[(i + self.MM) % self.NN] ^ (x >> 1) ^ (self.MATRIX_A if x & 1 else 0)
            self.mti = 0
        x = mt[self.mti]
        self.mti += 1
        x ^= (x >> 29) & 0x5555555555555555
        x ^= (x << 17) & 0x71D67FFFEDA60000
        x ^= (x << 37) & 0xFFF7EEE000000000
        x ^= x >> 43
        return x & self.MASK

    def uniform(self, low, high):
        """One draw of std::uniform_real_distribution<double>(low, high)."""
        r = float(self.next()) / 18446744073709551616.0
        if r >= 1.0:
            r = math.nextafter(1.0, 0.0)
        return r * (high - low) + low


class PlainSampler:
    """AIR's Sampler (src/runtime/sampling.cpp:9-63): greedy for temperature <= 0, else
    weights exp((logit - max)/temperature) in 64-bit, sorted descending, cut to top_k,
    cut to the shortest prefix whose share reaches top_p, one uniform draw over the
    total, and a walk over the cumulative weights."""

    def __init__(self, temperature=0.0, top_k=0, top_p=1.0, seed=0):
        self.temperature, self.top_k, self.top_p = temperature, top_k, top_p
        self.random = MT19937_64(seed)

    def sample(self, logits):
        logits = np.asarray(logits, dtype=F32)
        if logits.size == 0:
            raise ValueError("cannot sample empty logits")
        if self.temperature <= 0.0:
            return int(np.argmax(logits))
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        w = np.exp((logits.astype(F64) - F64(logits.max())) * (1.0 / self.temperature))
        order = np.argsort(-w, kind="stable")
        if self.top_k and self.top_k < order.size:
            order = order[: self.top_k]
        weights = [float(w[i]) for i in order]
        total = 0.0
        for x in weights:
            total += x
        if not (total > 0.0) or not math.isfinite(total):
            raise FloatingPointError("sampling distribution is non-finite")
        if self.top_p < 1.0:
            cumulative, keep = 0.0, 0
            while keep < len(weights):
                cumulative += weights[keep] / total
                keep += 1
                if cumulative >= self.top_p:
                    break
            keep = max(1, keep)
            weights, order = weights[:keep], order[:keep]
            total = 0.0
            for x in weights:
                total += x
        selected = self.random.uniform(0.0, total)
        cumulative = 0.0
        for x, i in zip(weights, order):
            cumulative += x
            if selected <= cumulative:
                return int(i)
        return int(order[-1])
