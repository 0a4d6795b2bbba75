"""Command line in the manner of air-cli (src/cli/main.cpp:21-33, 439-582), with token ids in
place of text since the engine has no tokenizer:

  air-b200 inspect <model-dir> [--tensors]
  air-b200 cuda-info
  air-b200 cuda <model-dir> <ids,comma,separated> [--tokens N] [--device N] [--dtype bfloat16|float32]
                [--temperature T] [--top-k K] [--top-p P] [--seed S] [--no-stop-on-eos] [--keep-float32]
  air-b200 cuda-compare <model-dir> <ids> [--device N] [--atol X]
  air-b200 random <config.json> <out-dir> [--seed S] [--dtype bfloat16|float32]

`--tokens N` is the number of tokens to generate, as in air-cli.  `cuda-compare` runs the
prompt through the float32 path whole and token by token and through the bfloat16 path, and
reports the largest differences of the logits (air-cli compares its CPU and CUDA executors).
Exit codes as air-cli: 2 usage, 3 load, 6 executor, 7 run, 9 mismatch.
"""
from __future__ import annotations

import json
import sys

USAGE = __doc__.split("\n\n")[1]


def _ids(text):
    return [int(t) for t in text.replace(" ", "").split(",") if t]


def _options(args, spec):
    out = {k: v[1] for k, v in spec.items()}
    rest = []
    i = 0
    while i < len(args):
        a = args[i]
        if a in spec:
            typ = spec[a][0]
            if typ is bool:
                out[a] = True
            else:
                if i + 1 >= len(args):
                    raise SystemExit(2)
                out[a] = typ(args[i + 1])
                i += 1
        elif a.startswith("--"):
            print(f"unknown option {a}\n{USAGE}", file=sys.stderr)
            raise SystemExit(2)
        else:
            rest.append(a)
        i += 1
    return out, rest


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(USAGE)
        return 0 if argv else 2
    if argv[0] == "--version":
        from . import __version__
        print(__version__)
        return 0
    cmd, args = argv[0], argv[1:]
    try:
        if cmd == "inspect":
            return _inspect(args)
        if cmd == "cuda-info":
            return _cuda_info()
        if cmd == "cuda":
            return _cuda(args)
        if cmd == "cuda-compare":
            return _compare(args)
        if cmd == "random":
            return _random(args)
    except SystemExit as e:
        return int(e.code or 0)
    print(f"unknown command {cmd}\n{USAGE}", file=sys.stderr)
    return 2


def _inspect(args) -> int:
    from .config import load_config, ConfigError
    from .parts import registry
    from .engine.model import Model
    opts, rest = _options(args, {"--tensors": (bool, False)})
    if len(rest) != 1:
        return 2
    try:
        cfg = load_config(rest[0])
        model = Model(registry.architecture(cfg.architecture).build_spec(cfg))
    except ValueError as e:       # ConfigError: a data error, or a size that the engine does not take
        print(e, file=sys.stderr)
        return 3
    specs = model.tensor_specs()
    params = sum(int(__import__("math").prod(s.shape)) for s in specs)
    print(json.dumps({"architecture": cfg.architecture, "config": cfg.to_dict(), "tensors": len(specs),
                      "parameters": params}, indent=2))
    if opts["--tensors"]:
        for s in specs:
            print(f"{s.name}\t{list(s.shape)}{'  (optional)' if s.optional else ''}")
    return 0


def _cuda_info() -> int:
    import torch
    if not torch.cuda.is_available():
        print("no CUDA device", file=sys.stderr)
        return 6
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        print(json.dumps({"device": i, "name": p.name, "compute_capability": f"{p.major}.{p.minor}",
                          "multiprocessors": p.multi_processor_count, "memory_bytes": p.total_memory}))
    return 0


def _load(folder, dtype, device, max_tokens, keep_float32=False):
    from .config import ConfigError
    from .engine.engine import Engine, EngineConfig, parse_dtype
    from .weights.loader import WeightError
    from .weights.safetensors_io import SafetensorsError
    try:
        engine = Engine.from_folder(folder, EngineConfig(dtype=parse_dtype(dtype), max_tokens=max_tokens,
                                                         device=f"cuda:{device}", keep_float32=keep_float32))
        if engine.load_report is not None and engine.load_report.summary():
            print("note: " + engine.load_report.summary(), file=sys.stderr)
        return engine
    except (ConfigError, WeightError, SafetensorsError, ValueError) as e:
        # a model that cannot be loaded: bad or missing geometry, tensors that do not fit, or sizes that
        # the kernels do not take ("unsupported"), as air-cli's exit code 3
        print(e, file=sys.stderr)
        raise SystemExit(3)
    except RuntimeError as e:
        print(e, file=sys.stderr)
        raise SystemExit(6)


def _cuda(args) -> int:
    from .engine.service import InferenceService, SchedulerConfig
    from .sampling.sampler import GenerationConfig, SamplingConfig
    opts, rest = _options(args, {"--tokens": (int, 32), "--device": (int, 0), "--dtype": (str, "bfloat16"),
                                 "--temperature": (float, 0.0), "--top-k": (int, 0), "--top-p": (float, 1.0),
                                 "--seed": (int, 0), "--no-stop-on-eos": (bool, False),
                                 "--keep-float32": (bool, False)})
    if len(rest) != 2:
        print(USAGE, file=sys.stderr)
        return 2
    prompt = _ids(rest[1])
    engine = _load(rest[0], opts["--dtype"], opts["--device"], len(prompt) + opts["--tokens"] + 64,
                   opts["--keep-float32"])
    service = InferenceService(engine, SchedulerConfig(max_active_requests=engine.config.max_requests))
    try:
        response = service.generate(prompt, GenerationConfig(
            max_new_tokens=opts["--tokens"], stop_on_eos=not opts["--no-stop-on-eos"],
            sampling=SamplingConfig(opts["--temperature"], opts["--top-k"], opts["--top-p"], opts["--seed"])))
    except (ValueError, RuntimeError) as e:
        print(e, file=sys.stderr)
        return 7
    if response.error:
        print(response.error, file=sys.stderr)
        return 7
    try:
        engine.check_status()       # once more before anything is printed: the last step's word
    except RuntimeError as e:
        print(e, file=sys.stderr)
        return 7
    print(",".join(str(t) for t in response.tokens))
    m = response.metrics
    print(f"prompt {m.prompt_tokens} tokens, generated {m.generated_tokens}, ttft {m.ttft_ms:.2f} ms, "
          f"decode {m.decode_ms:.2f} ms", file=sys.stderr)
    return 0


def _compare(args) -> int:
    from .engine.batch import Entry
    opts, rest = _options(args, {"--device": (int, 0), "--atol": (float, 1e-3)})
    if len(rest) != 2:
        print(USAGE, file=sys.stderr)
        return 2
    prompt = _ids(rest[1])
    n = len(prompt)
    fp32 = _load(rest[0], "float32", opts["--device"], 2 * n + 128)
    whole = fp32.step([Entry("whole", prompt, list(range(n)))]).cpu()
    single = [fp32.step([Entry("single", [t], [0])]).cpu() for t in prompt]
    import torch
    single = torch.cat(single)
    bf16 = _load(rest[0], "bfloat16", opts["--device"], n + 64)
    half = bf16.step([Entry("whole", prompt, list(range(n)))]).cpu()
    d_step = float((whole - single).abs().max())
    d_half = float((whole - half).abs().max())
    top1 = bool((whole.argmax(-1) == single.argmax(-1)).all())
    print(json.dumps({"tokens": n, "float32_whole_vs_token_by_token_max_abs": d_step,
                      "float32_vs_bfloat16_max_abs": d_half, "top1_parity": top1,
                      "finite": bool(torch.isfinite(whole).all()), "atol": opts["--atol"]}))
    return 0 if (d_step <= opts["--atol"] and top1) else 9


def _random(args) -> int:
    from .config import ConfigError
    from .engine.engine import write_random_model
    opts, rest = _options(args, {"--seed": (int, 0), "--dtype": (str, "bfloat16")})
    if len(rest) != 2:
        print(USAGE, file=sys.stderr)
        return 2
    try:
        with open(rest[0]) as f:
            cfg = json.load(f)
        write_random_model(rest[1], cfg, opts["--seed"], opts["--dtype"])
    except (OSError, ValueError, ConfigError) as e:
        print(e, file=sys.stderr)
        return 3
    print(rest[1])
    return 0


if __name__ == "__main__":
    sys.exit(main())
