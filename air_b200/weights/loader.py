"""Weights by tensor name.

A model that has been built from its description lists the tensors it needs
(``TensorSpec``: name, shape, whether it may be absent, how to draw it at random); this
module finds them in a folder's safetensors file(s), checks them all, and raises ONE error
that lists every missing tensor, every unexpected one and every wrong shape, in the manner
of AIR's messages (src/model/qwen2_contract.cpp:14-29).

Precision.  In a float32 engine every floating tensor becomes float32 (exact for bfloat16
and float16).  In a bfloat16 engine a tensor stored in 16 bits is kept as bfloat16 (float16 is
rounded to it), integer tables become int32, and a tensor stored in 32 bits stays in 32 bits
where its part computes with it in 32 bits (``TensorSpec.wide``: norm weights, biases, router
weights).  A matrix that feeds the tensor cores is another matter: kept in 32 bits it would run
the CUDA-core product at a few percent of the speed, so a float32-stored operand of a matrix
product is rounded to bfloat16 (to nearest even), as AIR executes float32, float16 and bfloat16
checkpoints through one path (src/reference/tensor_reader.cpp:251-255), unless the caller asks
for ``keep_float32``.  Either way the load says what it did: ``LoadReport`` lists the rounded and
the kept tensors, and the engine keeps it (``Engine.load_report``).
"""
from __future__ import annotations

import json
import os
import zlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsFile, SafetensorsError, write_safetensors


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    optional: bool = False
    init: str = "normal"        # "normal": N(0, std);  "one_plus_normal": 1 + N(0, std);  "zeros"
    std: float = 0.02
    integer: bool = False
    wide: bool = False          # the part computes with this tensor in 32 bits: stored in 32 bits it stays so


class WeightError(ValueError):
    """Raised once per load, with everything that is wrong."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 other: Sequence[str] = ()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.other = list(wrong_shape), list(other)
        lines = [f"weights in {where} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n}: file has {list(got)}, model needs {list(want)}" for n, got, want in self.wrong_shape))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


def _open_files(folder: str) -> Dict[str, SafetensorsFile]:
    """name -> file that holds it; one model.safetensors, or the shards that
    model.safetensors.index.json names."""
    index = os.path.join(folder, "model.safetensors.index.json")
    single = os.path.join(folder, "model.safetensors")
    files: Dict[str, SafetensorsFile] = {}
    if os.path.exists(single):
        f = SafetensorsFile(single)
        return {n: f for n in f.names()}
    if os.path.exists(index):
        try:
            with open(index) as fh:
                weight_map = json.load(fh).get("weight_map")
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{index} is not valid JSON: {e}") from None
        if not isinstance(weight_map, dict) or not weight_map:
            raise SafetensorsError(f"{index} has no 'weight_map'")
        opened: Dict[str, SafetensorsFile] = {}
        for name, shard in weight_map.items():
            if shard not in opened:
                path = os.path.join(folder, shard)
                if not os.path.exists(path):
                    raise SafetensorsError(f"{index} names the shard {shard}, which is not in {folder}")
                opened[shard] = SafetensorsFile(path)
            if name not in opened[shard]._entries:
                where = [s for s, f in opened.items() if name in f._entries]
                raise SafetensorsError(f"{index}: '{name}' is not in {shard}" +
                                       (f" (it is in {where[0]})" if where else ""))
            files[name] = opened[shard]
        # a tensor that lies in a shard but that the index does not name is reported as unexpected by the load
        for shard, f in opened.items():
            for name in f.names():
                files.setdefault(name, f)
        return files
    raise SafetensorsError(f"no model.safetensors in {folder}")


@dataclass
class LoadReport:
    """What a load did to precisions in a bfloat16 engine."""
    rounded: List[str] = field(default_factory=list)     # stored in 32 bits (or float16), now bfloat16
    kept_float32: List[str] = field(default_factory=list)

    def summary(self) -> str:
        out = []
        if self.rounded:
            out.append(f"{len(self.rounded)} tensors stored in float32 or float16 were rounded to bfloat16 "
                       f"(first: {self.rounded[0]}); keep_float32 keeps float32 ones, at the CUDA-core product's speed")
        if self.kept_float32:
            out.append(f"{len(self.kept_float32)} tensors stay in float32 (first: {self.kept_float32[0]})")
        return "; ".join(out)


def stored_dtype_for(engine_dtype: torch.dtype, file_dtype: torch.dtype, wide: bool = False,
                     keep_float32: bool = False) -> torch.dtype:
    if not file_dtype.is_floating_point:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if file_dtype in (torch.float32, torch.float64) and (wide or keep_float32):
        return torch.float32
    return torch.bfloat16


def load_tensors(folder: str, specs: Sequence[TensorSpec], engine_dtype: torch.dtype,
                 device, keep_float32: bool = False, report: Optional[LoadReport] = None) -> Dict[str, torch.Tensor]:
    files = _open_files(folder)
    missing, wrong, found = [], [], {}
    wanted = set()
    for s in specs:
        wanted.add(s.name)
        f = files.get(s.name)
        if f is None:
            if not s.optional:
                missing.append(s.name)
            continue
        dt, shape = f.info(s.name)
        if tuple(shape) != tuple(s.shape):
            wrong.append((s.name, tuple(shape), tuple(s.shape)))
            continue
        found[s.name] = (f, dt, s)
    unexpected = sorted(n for n in files if n not in wanted)
    if missing or wrong or unexpected:
        raise WeightError(folder, missing, unexpected, wrong)
    out = {}
    for name, (f, dt, spec) in found.items():
        t = f.tensor(name)
        target = stored_dtype_for(engine_dtype, dt, spec.wide, keep_float32)
        if report is not None and engine_dtype != torch.float32 and dt.is_floating_point and dt != torch.bfloat16:
            (report.rounded if target == torch.bfloat16 else report.kept_float32).append(name)
        out[name] = t.to(device=device, dtype=target).contiguous()
    return out


def _seed_for(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B97F4A7C15 + zlib.crc32(name.encode("utf-8"))) & 0x7FFFFFFFFFFFFFFF


def random_tensors(specs: Sequence[TensorSpec], seed: int, dtype: torch.dtype, device="cpu",
                   include_optional: bool = True) -> Dict[str, torch.Tensor]:
    """Seeded random tensors: every tensor has a generator of its own, keyed by the seed
    and its name, so the values do not depend on the order or on which others are drawn.
    Drawn in float32 on ``device``, then rounded to ``dtype``."""
    out = {}
    for s in specs:
        if s.optional and not include_optional:
            continue
        g = torch.Generator(device=device)
        g.manual_seed(_seed_for(seed, s.name))
        if s.integer:
            out[s.name] = torch.zeros(s.shape, dtype=torch.int32, device=device)
            continue
        if s.init == "zeros":
            t = torch.zeros(s.shape, dtype=torch.float32, device=device)
        else:
            t = torch.empty(s.shape, dtype=torch.float32, device=device).normal_(0.0, s.std, generator=g)
            if s.init == "one_plus_normal":
                t += 1.0
        out[s.name] = t.to(dtype)
    return out


def write_model_folder(folder: str, config: dict, tensors: Dict[str, torch.Tensor], metadata=None) -> None:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f, indent=2)
        f.write("\n")
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata=metadata or {"format": "pt"})
