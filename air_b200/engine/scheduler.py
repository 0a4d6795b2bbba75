"""What the next step holds, and who may join: decisions without a device.

The policy is AIR's (src/runtime/scheduler.cpp, src/runtime/serving.cpp:1684-1700, 1796-1810):
a request becomes active only if its worst case (prompt plus max_new_tokens) fits beside what the
active requests have reserved, and while fewer than `max_active` are active; in a step every decoding
request comes first with its one token, then prompt portions, each at most `portion_limit` tokens and
what is left of the step's token budget; where the budget does not reach everybody, the start of each
walk moves on from step to step so that nobody starves.

The form is this engine's.  A cycle here is ONE step of one flat batch, so the plan is the batch itself: a
list of `Entry` that `Engine.step` takes as it is.  Reservations are counted in cache pages.  A portion
that the budget or the limit cuts (not the prompt's end) is shortened so that the step's rows, decoding
requests included, fill whole row tiles of the matrix products (`row_tile` rows; nine tenths of a prompt
step's time are products, and 416 rows cost them what 512 do), or else so that the request's next portion
starts on a page of the cache.  A step that only decodes says which captured graph it will replay
(`StepPlan.graph_size`; a step of 65 tokens runs the graph made for 96).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence, Tuple

from .batch import Entry


@dataclass
class Admission:
    admit: bool
    pages: int          # the worst case of the request, in pages
    reason: str         # "admitted", "max-active-requests", "device-capacity"


@dataclass
class Runnable:
    """An active request as the planner sees it.  `done` tokens of `prompt` are in the cache; when all
    are, the request decodes: its next input is `last_token`.  `wants_token`: the prompt's last portion
    asks for logits (the first generated token comes from them)."""
    request: Hashable
    prompt: Sequence[int]
    done: int
    last_token: Optional[int] = None
    wants_token: bool = True

    @property
    def decoding(self) -> bool:
        return self.done >= len(self.prompt)


@dataclass
class StepPlan:
    entries: List[Entry] = field(default_factory=list)
    decode_tokens: int = 0
    prompt_tokens: int = 0
    portions: List[Tuple[Hashable, int]] = field(default_factory=list)    # (request, tokens of its prompt)
    graph_size: Optional[int] = None      # decode-only steps: the size of the captured graph that runs

    @property
    def tokens(self) -> int:
        return self.decode_tokens + self.prompt_tokens


class StepScheduler:
    def __init__(self, max_active: int, token_budget: int, portion_limit: int, page_tokens: int,
                 row_tile: int = 128, graph_sizes: Sequence[int] = ()):
        if min(max_active, token_budget, portion_limit, page_tokens) <= 0:
            raise ValueError("the scheduler's limits must be greater than zero")
        self.max_active, self.token_budget, self.portion_limit = max_active, token_budget, portion_limit
        self.page_tokens, self.row_tile = page_tokens, row_tile
        self.graph_sizes = tuple(sorted(graph_sizes))
        self._decode_turn = 0      # where the walk over the decoding requests starts
        self._prompt_turn = 0

    # ------------------------------------------------------------------ who may join
    def pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_tokens)

    def admit(self, active: int, reserved_pages: int, pool_pages: int, worst_case_tokens: int) -> Admission:
        pages = self.pages_for(worst_case_tokens)
        if active >= self.max_active:
            return Admission(False, 0, "max-active-requests")
        if pages + reserved_pages > pool_pages:
            return Admission(False, pages, "device-capacity")
        return Admission(True, pages, "admitted")

    # ------------------------------------------------------------------ what runs
    def _cut(self, position: int, count: int, rows_before: int) -> int:
        """A portion of `count` tokens from `position` that does not end its prompt, in a step that holds
        `rows_before` tokens already.  The matrix products work on tiles of `row_tile` rows of the whole step, so
        the portion is shortened to make the step's rows a multiple of that (a budget that is one needs no
        shortening), unless that would take more than half of it; else it ends on a page of its request, where
        that leaves it any tokens."""
        total = rows_before + count
        fitting = total - total % self.row_tile - rows_before
        if fitting > 0 and 2 * fitting >= count:
            return fitting
        end = position + count
        aligned = end - end % self.page_tokens
        return aligned - position if aligned > position else count

    def plan(self, runnable: Sequence[Runnable]) -> StepPlan:
        plan = StepPlan()
        left = self.token_budget
        decoding = [r for r in runnable if r.decoding]
        prompts = [r for r in runnable if not r.decoding]
        if decoding and left > 0:
            start = self._decode_turn % len(decoding)
            served = (decoding[start:] + decoding[:start])[:left]
            for r in served:
                plan.entries.append(Entry(r.request, [r.last_token], [0]))
            plan.decode_tokens = len(served)
            left -= len(served)
            self._decode_turn = (start + len(served)) % len(decoding)
        if prompts and left > 0:
            start = self._prompt_turn % len(prompts)
            self._prompt_turn = (start + 1) % len(prompts)
            for r in prompts[start:] + prompts[:start]:
                if left <= 0:
                    break
                rest = len(r.prompt) - r.done
                count = min(rest, self.portion_limit, left)
                if count < rest:
                    count = self._cut(r.done, count, self.token_budget - left)
                last = count == rest
                plan.entries.append(Entry(r.request, r.prompt[r.done:r.done + count],
                                          [count - 1] if last and r.wants_token else []))
                plan.portions.append((r.request, count))
                plan.prompt_tokens += count
                left -= count
        if plan.entries and not plan.portions:
            plan.graph_size = next((g for g in self.graph_sizes if g >= plan.decode_tokens), None)
        return plan
