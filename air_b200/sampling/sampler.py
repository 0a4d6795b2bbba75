"""Choosing the next token.

`SamplingConfig` and `GenerationConfig` carry AIR's names, meanings and defaults
(include/air/generation.hpp:16-27).  `HostSampler` reproduces AIR's Sampler
(src/runtime/sampling.cpp:9-63) on the host, number for number: greedy for temperature <= 0
(the lowest index of the maximum), else weights exp((logit - max) / temperature) in 64-bit,
sorted descending, cut to top_k, cut to the shortest prefix whose share reaches top_p, and one
draw of std::uniform_real_distribution<double>(0, total) from std::mt19937_64(seed).

On the device (air_b200/csrc/sampling.cu) the engine samples without bringing logits to the
host: the request's generator supplies the uniform number, the kernel cuts to top_k and top_p
as AIR does and draws.  Without a cut it walks the weights in index order instead of sorted
order, and its weights are 32-bit, so the distribution is AIR's but the token for a given seed
need not be.  With `SchedulerConfig.sample_cuts_on_device = False` requests with top_k or top_p
are sampled by `HostSampler` from logits copied to the host, which gives AIR's token per seed.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import numpy as np


@dataclass
class SamplingConfig:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    def validate(self) -> None:
        if self.temperature > 0.0 and not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")

    @property
    def on_device(self) -> bool:
        return self.temperature <= 0.0 or (self.top_k == 0 and self.top_p >= 1.0)


@dataclass
class GenerationConfig:
    max_new_tokens: int = 32
    sampling: SamplingConfig = field(default_factory=SamplingConfig)
    stop_on_eos: bool = True


class Mt19937_64:
    """std::mt19937_64."""
    _N, _M = 312, 156
    _A, _UPPER, _LOWER, _MASK = 0xB5026F5AA96619E9, 0xFFFFFFFF80000000, 0x7FFFFFFF, 0xFFFFFFFFFFFFFFFF

    def __init__(self, seed: int):
        s = [seed & self._MASK]
        for i in range(1, self._N):
            s.append((6364136223846793005 * (s[-1] ^ (s[-1] >> 62)) + i) & self._MASK)
        self._s, self._i = s, self._N

    def _twist(self) -> None:
        s, n, m = self._s, self._N, self._M
        for i in range(n):
            x = (s[i] & self._UPPER) | (s[(i + 1) % n] & self._LOWER)
            v = s[(i + m) % n] ^ (x >> 1)
            if x & 1:
                v ^= self._A
            s[i] = v
        self._i = 0

    def __call__(self) -> int:
        if self._i >= self._N:
            self._twist()
        x = self._s[self._i]
        self._i += 1
        x ^= (x >> 29) & 0x5555555555555555
        x ^= (x << 17) & 0x71D67FFFEDA60000
        x ^= (x << 37) & 0xFFF7EEE000000000
        x ^= x >> 43
        return x & self._MASK

    def canonical(self) -> float:
        """std::generate_canonical<double, 53>: one draw, in [0, 1)."""
        r = float(self()) / 18446744073709551616.0
        return r if r < 1.0 else math.nextafter(1.0, 0.0)


class HostSampler:
    def __init__(self, config: Optional[SamplingConfig] = None):
        self.config = config or SamplingConfig()
        self.random = Mt19937_64(self.config.seed)

    def next_uniform(self) -> float:
        """The next number in [0, 1) of this request's generator (for the device sampler)."""
        return self.random.canonical()

    def sample(self, logits) -> int:
        c = self.config
        logits = np.asarray(logits, dtype=np.float32)
        if logits.size == 0:
            raise ValueError("cannot sample empty logits")
        if c.temperature <= 0.0:
            return int(np.argmax(logits))
        if not (0.0 < c.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        weights = np.exp((logits.astype(np.float64) - np.float64(logits.max())) * (1.0 / c.temperature))
        order = np.argsort(-weights, kind="stable")
        if c.top_k != 0 and c.top_k < order.size:
            order = order[: c.top_k]
        kept = weights[order].tolist()
        total = sum(kept, 0.0)
        if not (total > 0.0) or not math.isfinite(total):
            raise FloatingPointError("sampling distribution is non-finite")
        if c.top_p < 1.0:
            cumulative, keep = 0.0, 0
            for w in kept:
                cumulative += w / total
                keep += 1
                if cumulative >= c.top_p:
                    break
            keep = max(1, keep)
            kept, order = kept[:keep], order[:keep]
            total = sum(kept, 0.0)
        selected = self.random.canonical() * total
        cumulative = 0.0
        for w, i in zip(kept, order):
            cumulative += w
            if selected <= cumulative:
                return int(i)
        return int(order[-1])
