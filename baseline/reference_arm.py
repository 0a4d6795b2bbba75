#!/usr/bin/env python3
"""The reference arm: EmersonDowell/AIR's own CUDA executor, built from its unmodified sources.

AIR is a CMake C++ project (no setup.py or pyproject.toml, so pip cannot install it), and its
stock build wants Boost and PCRE2 for the server and the tokenizer.  Its executor does not:
src/cuda/cuda_backend.cu with six sources of its core (model, storage, architecture contract,
sampling, generation, verification) links against cudart and cuBLAS alone.  This script

  * copies AIR's `include/` and `src/` into baseline/_ref/ (git-ignored) when they are not there,
    from --reference, $AIR_REFERENCE_DIR or a folder `reference` beside this repository,
  * compiles them with nvcc for sm_100 together with baseline/air_cuda_driver.cpp (this
    repository's driver, which only calls AIR's public classes),
  * `check`: runs the golden tiny model of tests/golden/ through AIR's CUDA executor on the GPU and
    compares its logits with those of AIR's CPU executor stored there,
  * `bench`: runs the driver's bench mode and returns its record.

    python baseline/reference_arm.py build [--reference DIR]
    python baseline/reference_arm.py check
    python baseline/reference_arm.py bench layers=28 hidden=3584 ...
"""
import json
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
BUILD = os.path.join(REF, "_build")
DRIVER = os.path.join(BUILD, "air_cuda_driver")
CORE_SOURCES = ["src/model/model.cpp", "src/model/storage.cpp", "src/model/qwen2_contract.cpp",
                "src/runtime/sampling.cpp", "src/runtime/generation.cpp", "src/runtime/verification.cpp"]
DEFINES = ["-DAIR_HAS_CUDA=1", "-DAIR_HAS_NVTX=0", "-DAIR_VERSION_MAJOR=0", "-DAIR_VERSION_MINOR=0",
           "-DAIR_VERSION_PATCH=0"]


class Unavailable(RuntimeError):
    pass


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise Unavailable("nvcc was not found")


def fetch(reference=None):
    """AIR's sources in baseline/_ref/, copied unmodified."""
    if os.path.exists(os.path.join(REF, "src", "cuda", "cuda_backend.cu")):
        return
    beside = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")      # a checkout next to this repository
    reference = next((r for r in (reference, os.environ.get("AIR_REFERENCE_DIR"), beside)
                      if r and os.path.exists(os.path.join(r, "src", "cuda", "cuda_backend.cu"))), None)
    if reference is None:
        raise Unavailable("AIR's sources are not in baseline/_ref and no checkout was given "
                          "(--reference DIR, AIR_REFERENCE_DIR, or a folder `reference` beside the repository)")
    os.makedirs(REF, exist_ok=True)
    for sub in ("include", "src"):
        shutil.copytree(os.path.join(reference, sub), os.path.join(REF, sub), dirs_exist_ok=True)
    for f in ("LICENSE", "CMakeLists.txt"):
        if os.path.exists(os.path.join(reference, f)):
            shutil.copy(os.path.join(reference, f), os.path.join(REF, f))


def build(reference=None, force=False):
    """Compiles AIR's executor and the driver; returns the driver's path."""
    fetch(reference)
    newest = max(os.path.getmtime(p) for p in
                 [os.path.join(HERE, "air_cuda_driver.cpp"), os.path.join(REF, "src", "cuda", "cuda_backend.cu")])
    if not force and os.path.exists(DRIVER) and os.path.getmtime(DRIVER) >= newest:
        return DRIVER
    nvcc = _nvcc()
    os.makedirs(BUILD, exist_ok=True)
    common = [nvcc, "-std=c++20", "-O2", "-gencode", "arch=compute_100,code=sm_100", "--expt-relaxed-constexpr",
              "-w"] + DEFINES + ["-I", os.path.join(REF, "include"), "-I", os.path.join(REF, "src")]
    obj = os.path.join(BUILD, "cuda_backend.o")
    for cmd in (common + ["-rdc=true", "-c", os.path.join(REF, "src", "cuda", "cuda_backend.cu"), "-o", obj],
                common + [os.path.join(HERE, "air_cuda_driver.cpp"), obj] +
                [os.path.join(REF, s) for s in CORE_SOURCES] + ["-lcublas", "-lcudart", "-o", DRIVER]):
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            first = next((l for l in p.stdout.splitlines() if "error" in l), p.stdout.strip().splitlines()[:1])
            raise Unavailable(f"AIR's CUDA executor does not build here: {first}")
    return DRIVER


def check():
    """The golden tiny model through AIR's CUDA executor; returns the largest differences from AIR's
    CPU executor (token by token, and the whole-prompt prefill's last row)."""
    import numpy as np
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "tests", "golden"))
    import make_golden as mg
    driver = build()
    z = np.load(os.path.join(os.path.dirname(HERE), "tests", "golden", "air_reference_tiny.npz"))
    names = [str(n) for n in z["names"]]
    c = mg.CONFIG
    with tempfile.TemporaryDirectory() as tmp:
        lines = ["%d %d %d %d %d %d %d %.17g %.17g" % (
            c["num_hidden_layers"], c["hidden_size"], c["intermediate_size"], c["num_attention_heads"],
            c["num_key_value_heads"], c["max_position_embeddings"], c["vocab_size"], c["rope_theta"],
            c["rms_norm_eps"])]
        offset = 0
        with open(os.path.join(tmp, "data.bin"), "wb") as f:
            for n, name in enumerate(names):
                a = mg.from_bf16_bits(z[f"w{n}"]).reshape(tuple(z[f"s{n}"]))
                raw = np.ascontiguousarray(a, dtype="<f4").tobytes()
                dims = list(reversed(a.shape))
                lines.append(f"{mg.air_name(name)} {len(dims)} {' '.join(map(str, dims))} {offset} {len(raw)}")
                f.write(raw)
                offset += len(raw)
        with open(os.path.join(tmp, "manifest.txt"), "w") as f:
            f.write("\n".join(lines) + "\n")
        out = os.path.join(tmp, "logits.bin")
        tokens = [int(t) for t in z["tokens"]]
        p = subprocess.run([driver, "check", os.path.join(tmp, "manifest.txt"), os.path.join(tmp, "data.bin"), out]
                           + [str(t) for t in tokens], capture_output=True, text=True, timeout=600)
        if p.returncode != 0:
            raise Unavailable(f"AIR's CUDA executor failed on the golden model: {p.stderr.strip()[:300]}")
        got = np.fromfile(out, dtype="<f4").reshape(len(tokens) + 1, c["vocab_size"])
    want = z["logits"]
    greedy = [int(x) for x in p.stdout.split()[1:3]]
    return {"step_max_abs": float(np.abs(got[:-1] - want).max()), "prefill_max_abs": float(np.abs(got[-1] - want[-1]).max()),
            "logit_max_abs": float(np.abs(want).max()), "greedy_batch": greedy, "argmax": int(want[-1].argmax())}


def bench(**sizes):
    """Runs the driver's bench mode; returns its record (a dict)."""
    driver = build()
    cmd = [driver, "bench"] + [f"{k}={v}" for k, v in sizes.items()]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=int(os.environ.get("AIR_REFERENCE_TIMEOUT", "1500")))
    if p.returncode != 0:
        raise Unavailable(f"AIR's CUDA executor failed (exit {p.returncode}): {p.stderr.strip()[:300]}")
    return json.loads(p.stdout.strip().splitlines()[-1])


def main(argv):
    if not argv:
        print(__doc__)
        return 2
    try:
        if argv[0] == "build":
            reference = argv[argv.index("--reference") + 1] if "--reference" in argv else None
            print(build(reference, force="--force" in argv))
        elif argv[0] == "check":
            print(json.dumps(check()))
        elif argv[0] == "bench":
            print(json.dumps(bench(**dict(a.split("=", 1) for a in argv[1:]))))
        else:
            print(__doc__)
            return 2
    except Unavailable as e:
        print(json.dumps({"unavailable": str(e)}))
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
