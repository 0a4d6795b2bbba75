"""The scheduler's decisions, as pure logic without a device.

Two small classes carry AIR's two decisions (src/runtime/scheduler.{hpp,cpp}):

* `CapacityScheduler.evaluate`: may the request at the head of the queue become active?  It is
  refused while as many requests are active as allowed, and while its worst case (prompt plus
  max_new_tokens, in whole pages) does not fit beside what the active requests have reserved.
  AIR reserves bytes (scheduler.cpp:8-41); here the unit is the cache page.
* `MicrobatchScheduler.schedule`: which tokens run in this cycle?  Decoding requests first, one
  token each, then prompt portions, each at most its own limit and what is left of the cycle's
  token budget; within each phase a cursor rotates the order from cycle to cycle, so that a small
  budget does not always serve the same request (scheduler.cpp:62-139).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Hashable, List, Sequence


class WorkPhase(enum.Enum):
    prefill = 0
    decode = 1


@dataclass
class SchedulableSequence:
    slot: Hashable
    phase: WorkPhase = WorkPhase.prefill
    max_tokens: int = 1     # decode: 1; prefill: min(rest of the prompt, quantum)


@dataclass
class ScheduledSlice:
    slot: Hashable
    phase: WorkPhase
    token_count: int


@dataclass
class ScheduledBatch:
    slices: List[ScheduledSlice] = field(default_factory=list)
    token_count: int = 0
    decode_tokens: int = 0
    prefill_tokens: int = 0
    prefill_sequences: int = 0


@dataclass
class CapacityDecision:
    admit: bool
    reservation_pages: int
    reason: str


class CapacityScheduler:
    def __init__(self, max_active_requests: int):
        self.max_active_requests = max_active_requests

    def evaluate(self, active_requests: int, active_reserved_pages: int, capacity_pages: int,
                 page_tokens: int, requested_tokens: int) -> CapacityDecision:
        if active_requests >= self.max_active_requests:
            return CapacityDecision(False, 0, "max-active-requests")
        reservation = -(-requested_tokens // page_tokens)
        if reservation > capacity_pages or active_reserved_pages > capacity_pages - reservation:
            return CapacityDecision(False, reservation, "device-capacity")
        return CapacityDecision(True, reservation, "admitted")


class MicrobatchScheduler:
    def __init__(self):
        self._decode_cursor = 0
        self._prefill_cursor = 0

    def order(self, candidates: Sequence[SchedulableSequence]) -> List[SchedulableSequence]:
        decode = [c for c in candidates if c.phase == WorkPhase.decode]
        prefill = [c for c in candidates if c.phase != WorkPhase.decode]

        def rotate(phase, cursor):
            if not phase:
                return phase, 0
            cursor %= len(phase)
            return phase[cursor:] + phase[:cursor], (cursor + 1) % len(phase)

        decode, self._decode_cursor = rotate(decode, self._decode_cursor)
        prefill, self._prefill_cursor = rotate(prefill, self._prefill_cursor)
        return decode + prefill

    def schedule(self, candidates: Sequence[SchedulableSequence], token_budget: int) -> ScheduledBatch:
        batch = ScheduledBatch()
        if token_budget <= 0 or not candidates:
            return batch
        remaining = token_budget
        for c in self.order(candidates):
            if remaining == 0:
                break
            if c.max_tokens <= 0:
                continue
            tokens = 1 if c.phase == WorkPhase.decode else min(c.max_tokens, remaining)
            if tokens <= 0 or tokens > remaining:
                continue
            batch.slices.append(ScheduledSlice(c.slot, c.phase, tokens))
            batch.token_count += tokens
            remaining -= tokens
            if c.phase == WorkPhase.decode:
                batch.decode_tokens += 1
            else:
                batch.prefill_tokens += tokens
                batch.prefill_sequences += 1
        return batch
