#!/usr/bin/env python3
"""Makes tests/golden/air_reference_*.npz: logits of EmersonDowell/AIR's own compiled
CPU reference executor for tiny random Qwen2 models.

    python tests/golden/make_golden.py --reference /path/to/AIR [--config tiny|a|b]

`tiny` (air_reference_tiny.npz) has a head size of 12, which the engine's kernels refuse: it anchors
the plain implementation alone.  `a` and `b` (air_reference_tiny_a.npz, ..._b.npz) are the two tiny
configurations that the engine's tests use (head sizes 16 and 32; tied and separate output matrix):
the GPU tests compare the engine's own float32 logits with AIR's on them.

It draws the weights (numpy, seed 0, rounded to values that bfloat16 holds, so that the
file stores them as 16-bit words), writes them in the raw form that air_driver.cpp reads,
compiles air_driver.cpp with g++ -std=c++20 against AIR's unmodified sources
(src/model/{model,storage,qwen2_contract}.cpp, src/reference/{tensor_reader,
reference_executor}.cpp, src/runtime/{sampling,generation,verification}.cpp), runs it on
a fixed token sequence and stores weights, tokens and logits.  tests/test_plain.py
compares tests/plain/qwen2_plain.py with these logits.
"""
import argparse
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 48, "num_attention_heads": 4,
    "num_key_value_heads": 2, "intermediate_size": 80, "vocab_size": 96,
    "max_position_embeddings": 64, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "hidden_act": "silu", "use_sliding_window": False,
}
TOKENS = [5, 17, 3, 95, 0, 42, 42, 7, 61, 88, 13, 2, 30, 77, 9, 54, 21, 66, 1, 90, 33, 12, 48, 6]
BASE = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", "use_sliding_window": False}
CONFIG_A = dict(BASE, num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                intermediate_size=128, vocab_size=256, max_position_embeddings=128, rope_theta=10000.0,
                rms_norm_eps=1e-6, tie_word_embeddings=True)
CONFIG_B = dict(BASE, num_hidden_layers=3, hidden_size=128, num_attention_heads=4, num_key_value_heads=1,
                intermediate_size=352, vocab_size=384, max_position_embeddings=256, rope_theta=1e6,
                rms_norm_eps=1e-5, tie_word_embeddings=False)
CONFIGS = {"tiny": (CONFIG, 0, "air_reference_tiny.npz"), "a": (CONFIG_A, 1, "air_reference_tiny_a.npz"),
           "b": (CONFIG_B, 2, "air_reference_tiny_b.npz")}

AIR_SOURCES = [
    "src/model/model.cpp", "src/model/storage.cpp", "src/model/qwen2_contract.cpp",
    "src/reference/tensor_reader.cpp", "src/reference/reference_executor.cpp",
    "src/runtime/sampling.cpp", "src/runtime/generation.cpp", "src/runtime/verification.cpp",
]


def to_bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def draw_weights(config, seed):
    """Checkpoint-named float32 tensors [out, in]; weights and biases N(0, 0.02)
    (scaled up so that attention is not uniform), norm weights 1 + N(0, 0.02)."""
    rng = np.random.default_rng(seed)
    e, h, k = config["hidden_size"], config["num_attention_heads"], config["num_key_value_heads"]
    d, i, v = e // h, config["intermediate_size"], config["vocab_size"]

    def w(*shape, std=0.02):
        return from_bf16_bits(to_bf16_bits(rng.standard_normal(shape) * std)).reshape(shape)

    t = {"model.embed_tokens.weight": w(v, e, std=1.0), "model.norm.weight": 1 + w(e),
         "lm_head.weight": w(v, e, std=0.1)}
    if config.get("tie_word_embeddings"):
        del t["lm_head.weight"]        # AIR ties the output matrix when output.weight is absent
    t["model.norm.weight"] = from_bf16_bits(to_bf16_bits(t["model.norm.weight"]))
    for l in range(config["num_hidden_layers"]):
        p = f"model.layers.{l}."
        t[p + "input_layernorm.weight"] = from_bf16_bits(to_bf16_bits(1 + w(e)))
        t[p + "post_attention_layernorm.weight"] = from_bf16_bits(to_bf16_bits(1 + w(e)))
        t[p + "self_attn.q_proj.weight"] = w(h * d, e, std=0.3)
        t[p + "self_attn.k_proj.weight"] = w(k * d, e, std=0.3)
        t[p + "self_attn.v_proj.weight"] = w(k * d, e, std=0.1)
        t[p + "self_attn.q_proj.bias"] = w(h * d, std=0.2)
        t[p + "self_attn.k_proj.bias"] = w(k * d, std=0.2)
        t[p + "self_attn.v_proj.bias"] = w(k * d, std=0.1)
        t[p + "self_attn.o_proj.weight"] = w(e, h * d, std=0.1)
        t[p + "mlp.gate_proj.weight"] = w(i, e, std=0.2)
        t[p + "mlp.up_proj.weight"] = w(i, e, std=0.1)
        t[p + "mlp.down_proj.weight"] = w(e, i, std=0.1)
    return t


def air_name(name):
    """Checkpoint name -> AIR's tensor name (src/model/qwen2_contract.cpp:69-139)."""
    table = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
             "lm_head.weight": "output.weight"}
    if name in table:
        return table[name]
    parts = name.split(".")
    layer, rest = parts[2], ".".join(parts[3:])
    sub = {"input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
           "self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight",
           "self_attn.v_proj.weight": "attn_v.weight", "self_attn.q_proj.bias": "attn_q.bias",
           "self_attn.k_proj.bias": "attn_k.bias", "self_attn.v_proj.bias": "attn_v.bias",
           "self_attn.o_proj.weight": "attn_output.weight", "mlp.gate_proj.weight": "ffn_gate.weight",
           "mlp.up_proj.weight": "ffn_up.weight", "mlp.down_proj.weight": "ffn_down.weight"}[rest]
    return f"blk.{layer}.{sub}"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("AIR_REFERENCE_DIR"), required="AIR_REFERENCE_DIR" not in os.environ,
                    help="a checkout of EmersonDowell/AIR (or set AIR_REFERENCE_DIR)")
    ap.add_argument("--config", default="tiny", choices=sorted(CONFIGS))
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    ref = args.reference
    c, seed, file_name = CONFIGS[args.config]
    args.out = args.out or os.path.join(HERE, file_name)
    tensors = draw_weights(c, seed)
    tokens = TOKENS if args.config == "tiny" else \
        [int(t) for t in np.random.default_rng(100 + seed).integers(0, c["vocab_size"], size=40)]
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "air_driver")
        cmd = ["g++", "-std=c++20", "-O2", "-I", os.path.join(ref, "include"), "-I", os.path.join(ref, "src"),
               "-DAIR_VERSION_MAJOR=0", "-DAIR_VERSION_MINOR=0", "-DAIR_VERSION_PATCH=0",
               os.path.join(HERE, "air_driver.cpp")] + [os.path.join(ref, s) for s in AIR_SOURCES] + ["-o", exe]
        print(" ".join(cmd))
        subprocess.check_call(cmd)
        lines = ["%d %d %d %d %d %d %d %.17g %.17g" % (
            c["num_hidden_layers"], c["hidden_size"], c["intermediate_size"], c["num_attention_heads"],
            c["num_key_value_heads"], c["max_position_embeddings"], c["vocab_size"], c["rope_theta"],
            c["rms_norm_eps"])]
        offset = 0
        with open(os.path.join(tmp, "data.bin"), "wb") as f:
            for name, a in tensors.items():
                raw = np.ascontiguousarray(a, dtype="<f4").tobytes()
                dims = list(reversed(a.shape))  # AIR lists {in, out}
                lines.append(f"{air_name(name)} {len(dims)} {' '.join(map(str, dims))} {offset} {len(raw)}")
                f.write(raw)
                offset += len(raw)
        with open(os.path.join(tmp, "manifest.txt"), "w") as f:
            f.write("\n".join(lines) + "\n")
        out_bin = os.path.join(tmp, "logits.bin")
        subprocess.check_call([exe, os.path.join(tmp, "manifest.txt"), os.path.join(tmp, "data.bin"), out_bin]
                              + [str(t) for t in tokens])
        logits = np.fromfile(out_bin, dtype="<f4").reshape(len(tokens), c["vocab_size"])
    names = sorted(tensors)
    np.savez_compressed(
        args.out, logits=logits, tokens=np.array(tokens, dtype=np.int32), names=np.array(names),
        **{f"w{n}": to_bf16_bits(tensors[name]) for n, name in enumerate(names)},
        **{f"s{n}": np.array(tensors[name].shape) for n, name in enumerate(names)})
    print("wrote", args.out, logits.shape, "max |logit|", float(np.abs(logits).max()))


if __name__ == "__main__":
    sys.exit(main())
