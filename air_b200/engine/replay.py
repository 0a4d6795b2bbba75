"""Trace replay: feeds given token ids through a model step by step and writes logits.
It samples nothing, and has no forward pass, cache or loader of its own: it calls
Engine.step, the function that generation calls.

AIR's nearest tool is air-verify (src/verification/main.cpp:247-503): exact token ids in, a
whole-prompt prefill, then teacher-forced decisions one by one, full logits compared.  A trace
here may cut the tokens anywhere and mix requests.

Input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step that wants something, <out>/<step>.f32 holds the logits at the wanted places as
little-endian float32 [wanted, vocab], in the order of the entries and of `want`.  After every
step a line "done <step>" is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from .batch import Entry
from .engine import Engine, EngineConfig, parse_dtype


def run_trace(engine: Engine, lines, out_dir: str, done=None) -> int:
    os.makedirs(out_dir, exist_ok=True)
    steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries = [Entry(e["id"], e["tokens"], e.get("want", ())) for e in rec.get("entries", ())]
        if entries:
            logits = engine.step(entries)
            data = logits.to("cpu").contiguous().numpy().astype("<f4", copy=False) if logits.shape[0] else None
            engine.check_status()       # before anything is written: a step that faulted leaves no file
            if data is not None:
                data.tofile(os.path.join(out_dir, f"{rec['step']}.f32"))
        for r in rec.get("end", ()):
            engine.finish(r)
        steps += 1
        if done is not None:
            done(rec["step"])
    return steps


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (whole pages per request)")
    ap.add_argument("--page-tokens", type=int, default=64, help="tokens per cache page (a divisor of 64)")
    ap.add_argument("--max-requests", type=int, default=8)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    engine = Engine.from_folder(args.model, EngineConfig(
        dtype=parse_dtype(args.dtype), page_tokens=args.page_tokens, max_tokens=args.max_tokens,
        max_requests=args.max_requests, device=args.device))

    def done(step):
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()

    run_trace(engine, sys.stdin, args.out, done)
    return 0
