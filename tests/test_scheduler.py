"""The scheduler's decisions (no GPU): admission by reservation, decode first, the token budget,
rotation, finishing, and what happens when pages run out.  The engine is a fake that keeps the
real cache manager's books and returns logits that make the next token predictable."""
import numpy as np
import pytest
import torch

from air_b200.cache.manager import CacheManager, OutOfPages
from air_b200.engine.scheduler import Runnable, StepScheduler
from air_b200.engine.service import InferenceService, QueueFull, SchedulerConfig
from air_b200.parts.base import PagedKV
from air_b200.sampling.sampler import GenerationConfig, SamplingConfig


def prompt(request, tokens, done=0):
    return Runnable(request, list(range(tokens)), done)


def decoding(request, last=7):
    return Runnable(request, [1, 2], 2, last_token=last)


def shape(plan):
    return [(e.request, len(e.tokens), list(e.want)) for e in plan.entries]


def test_admission_arithmetic():
    s = StepScheduler(max_active=2, token_budget=64, portion_limit=64, page_tokens=16)
    assert s.admit(0, 0, 10, 160).admit                                   # exact fit
    assert s.admit(0, 0, 10, 161).reason == "device-capacity"
    assert s.admit(1, 6, 10, 64).admit and not s.admit(1, 7, 10, 64).admit
    assert s.admit(2, 0, 10, 1).reason == "max-active-requests"
    assert s.admit(0, 0, 10, 17).pages == 2
    with pytest.raises(ValueError):
        StepScheduler(0, 1, 1, 16)


def test_decode_first_then_prompts_under_the_budget():
    s = StepScheduler(8, token_budget=5, portion_limit=4, page_tokens=16)
    plan = s.plan([prompt("p1", 4), decoding("d1", 30), prompt("p2", 4), decoding("d2", 31)])
    assert shape(plan) == [("d1", 1, [0]), ("d2", 1, [0]), ("p1", 3, [])]
    assert plan.entries[0].tokens == [30] and plan.entries[2].tokens == [0, 1, 2]
    assert (plan.tokens, plan.decode_tokens, plan.prompt_tokens, plan.portions) == (5, 2, 3, [("p1", 3)])
    assert plan.graph_size is None                       # a step with a prompt portion replays no graph


def test_portion_limits_last_portions_and_empty_plans():
    s = StepScheduler(8, token_budget=9, portion_limit=4, page_tokens=16)
    plan = s.plan([prompt("a", 4), prompt("b", 9), prompt("c", 4)])
    # a's portion ends its prompt and wants its logits; b is cut by the limit; c by what is left of the budget
    assert shape(plan) == [("a", 4, [3]), ("b", 4, []), ("c", 1, [])]
    assert s.plan([]).entries == []
    no_token = Runnable("z", [5, 6], 0, wants_token=False)        # max_new_tokens == 0: nothing is asked for
    assert shape(StepScheduler(8, 9, 4, 16).plan([no_token])) == [("z", 2, [])]


def test_rotation_when_the_budget_does_not_reach_everybody():
    s = StepScheduler(8, token_budget=1, portion_limit=8, page_tokens=16)
    cands = [decoding("a"), decoding("b"), decoding("c")]
    assert [s.plan(cands).entries[0].request for _ in range(6)] == ["a", "b", "c", "a", "b", "c"]
    s = StepScheduler(8, token_budget=2, portion_limit=8, page_tokens=16)
    served = [tuple(e.request for e in s.plan(cands).entries) for _ in range(3)]
    assert served == [("a", "b"), ("c", "a"), ("b", "c")]         # everybody twice in three steps
    s = StepScheduler(8, token_budget=8, portion_limit=8, page_tokens=16)
    cands = [prompt("x", 100), prompt("y", 100)]
    assert [s.plan(cands).entries[0].request for _ in range(4)] == ["x", "y", "x", "y"]


def test_cut_portions_fill_the_step_s_row_tiles_or_end_on_a_page():
    s = StepScheduler(8, token_budget=300, portion_limit=300, page_tokens=16, row_tile=128)
    # 300 rows are 2.3 tiles of the products: shortened to 256
    assert s.plan([prompt("a", 1000, done=40)]).portions == [("a", 256)]
    # a portion that ends its prompt is not shortened
    assert s.plan([prompt("a", 340, done=40)]).portions == [("a", 300)]
    # decoding requests count: 3 single tokens and 253 of the prompt are 256 rows; a budget that is a multiple of
    # the tile is used whole
    assert s.plan([decoding("d0"), decoding("d1"), decoding("d2"), prompt("a", 1000, done=7)]).portions == [("a", 253)]
    s = StepScheduler(8, token_budget=512, portion_limit=2048, page_tokens=64, row_tile=128)
    assert s.plan([decoding(f"d{i}") for i in range(32)] + [prompt("a", 9000, done=3840)]).portions == [("a", 480)]
    # with two prompts in a step each portion leaves the step on a tile's edge
    s = StepScheduler(8, token_budget=512, portion_limit=200, page_tokens=64, row_tile=128)
    assert s.plan([prompt("a", 9000), prompt("b", 9000)]).portions == [("a", 128), ("b", 128)]
    # less than half a tile within reach: the portion ends on a page of its request, or stays as it is
    s = StepScheduler(8, token_budget=50, portion_limit=50, page_tokens=16, row_tile=128)
    assert s.plan([prompt("a", 1000, done=100)]).portions == [("a", 44)]      # ends at 144
    assert s.plan([prompt("a", 1000, done=130)]).portions == [("a", 46)]      # ends at 176
    s = StepScheduler(8, token_budget=6, portion_limit=6, page_tokens=16, row_tile=128)
    assert s.plan([prompt("a", 1000, done=2)]).portions == [("a", 6)]         # no edge within reach: as it is
    # whatever the cuts, a prompt is run completely and in order
    s = StepScheduler(8, token_budget=77, portion_limit=53, page_tokens=16, row_tile=128)
    done, seen = 0, []
    while done < 1000:
        (entry,) = s.plan([prompt("a", 1000, done=done)]).entries
        seen += entry.tokens
        done += len(entry.tokens)
        assert entry.want == ([len(entry.tokens) - 1] if done == 1000 else [])
    assert seen == list(range(1000))


def test_a_decode_step_names_the_graph_it_replays():
    s = StepScheduler(128, token_budget=128, portion_limit=8, page_tokens=16, graph_sizes=(1, 2, 4, 8, 64, 96))
    assert s.plan([decoding(i) for i in range(3)]).graph_size == 4
    assert s.plan([decoding(i) for i in range(65)]).graph_size == 96
    assert s.plan([decoding(i) for i in range(100)]).graph_size is None     # beyond the last graph: launched one by one


# ------------------------------------------------------------------ the service over a fake engine
class FakeSpec:
    vocab_size, max_positions, eos_token_id = 50, 4096, 49


class FakeModel:
    spec = FakeSpec()


class FakeEngine:
    """The next token after t is (t + 1) % 49 at the request's first logits, and so on; token 48
    is followed by 49 = eos."""

    def __init__(self, pages, page=16, slots=8):
        self.cache = CacheManager([(PagedKV(1, 16, None),)], page, pages, slots, allocate=False)
        self.model = FakeModel()
        self.steps = []

    def step(self, entries):
        opened = [e.request for e in entries if e.request not in self.cache.sequences]
        for r in opened:
            self.cache.open(r)
        try:
            self.cache.reserve([(e.request, len(e.tokens)) for e in entries])
        except OutOfPages:
            for r in opened:
                self.cache.close(r)
            raise
        rows = []
        for e in entries:
            self.cache.commit(e.request, len(e.tokens))
            for w in e.want:
                row = np.zeros(50, dtype=np.float32)
                row[(e.tokens[w] + 1) % 50] = 5.0
                rows.append(row)
        self.steps.append([(e.request, len(e.tokens), list(e.want)) for e in entries])
        self._rows = len(rows)
        return torch.tensor(np.array(rows).reshape(len(rows), 50))

    def sample(self, logits, temperature=None, uniform=None):
        return logits.argmax(-1).to(torch.int32)

    def finish(self, request):
        self.cache.close(request)

    status_word = 0          # what a kernel would have left in the device's status word

    def read_status(self):
        return self.status_word

    def clear_status(self, code):
        self.status_word = 0
        return f"device fault {code}"


def test_prompt_in_portions_then_decode_and_pages_back():
    eng = FakeEngine(pages=8)
    svc = InferenceService(eng, SchedulerConfig(max_active_requests=4, token_budget_per_cycle=16,
                                                prefill_quantum_tokens=6))
    r = svc.generate([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 20], GenerationConfig(max_new_tokens=4))
    assert r.tokens == [21, 22, 23, 24] and not r.hit_eos and r.error is None
    # 14 prompt tokens in portions of 6, 6, 2 (the last one wants logits), then 3 decode steps
    assert eng.steps == [[(0, 6, [])], [(0, 6, [])], [(0, 2, [1])], [(0, 1, [0])], [(0, 1, [0])], [(0, 1, [0])]]
    assert eng.cache.free_pages() == 8 and not eng.cache.sequences
    assert r.metrics.prompt_tokens == 14 and r.metrics.generated_tokens == 4


def test_eos_stops_and_zero_new_tokens():
    eng = FakeEngine(pages=8)
    svc = InferenceService(eng, SchedulerConfig(max_active_requests=4))
    r = svc.generate([46], GenerationConfig(max_new_tokens=10))
    assert r.tokens == [47, 48, 49] and r.hit_eos
    r = svc.generate([46], GenerationConfig(max_new_tokens=10, stop_on_eos=False))
    assert r.tokens == [47, 48, 49, 0, 1, 2, 3, 4, 5, 6]
    r = svc.generate([5, 6], GenerationConfig(max_new_tokens=0))
    assert r.tokens == [] and eng.cache.free_pages() == 8


def test_decode_beside_prompt_portions_in_one_step():
    eng = FakeEngine(pages=32)
    svc = InferenceService(eng, SchedulerConfig(max_active_requests=4, token_budget_per_cycle=8,
                                                prefill_quantum_tokens=4))
    out = svc.generate_cohort([([1, 2], GenerationConfig(max_new_tokens=6)),
                               (list(range(10, 22)), GenerationConfig(max_new_tokens=2))])
    assert out[0].tokens == [3, 4, 5, 6, 7, 8] and out[1].tokens == [22, 23]
    mixed = [s for s in eng.steps if len(s) == 2 and {n for _, n, _ in s} != {1}]
    assert mixed, "a decoded token of one request ran beside a prompt portion of the other"
    assert all(sum(n for _, n, _ in s) <= 8 for s in eng.steps)


def test_admission_waits_for_reserved_pages_and_fails_what_never_fits():
    eng = FakeEngine(pages=4)                                    # 64 tokens
    svc = InferenceService(eng, SchedulerConfig(max_active_requests=4))
    a = svc.submit(list(range(30)), GenerationConfig(max_new_tokens=10))     # 40 tokens -> 3 pages
    b = svc.submit(list(range(20)), GenerationConfig(max_new_tokens=10))     # 30 tokens -> 2 pages: must wait
    c = svc.submit(list(range(40)), GenerationConfig(max_new_tokens=40))     # 80 tokens -> 5 pages: never fits
    svc.run_cycle()
    assert [i.request_id for i in svc.active] == [a] and [i.request_id for i in svc.queued] == [b, c]
    assert svc.snapshot()["reserved_pages"] == 3
    while svc.active or svc.queued:
        svc.run_cycle()
    assert svc.finished[a].tokens == list(range(30, 40)) and svc.finished[b].tokens == list(range(20, 30))
    assert svc.finished[c].error == "insufficient KV pages for one sequence" and svc.finished[c].tokens == []
    assert eng.cache.free_pages() == 4


def test_a_fault_that_the_device_reports_fails_the_requests_of_that_step():
    """The status word is read with every step's tokens.  When a kernel has set it, the requests of that
    step end with the fault's message (and the tokens they had), their pages go back, the word is cleared,
    and requests that come later are served."""
    eng = FakeEngine(pages=16)
    svc = InferenceService(eng, SchedulerConfig(max_active_requests=4))
    a = svc.submit([1, 2, 3], GenerationConfig(max_new_tokens=8))
    b = svc.submit([4, 5], GenerationConfig(max_new_tokens=8))
    for _ in range(3):
        svc.run_cycle()
    assert len(svc.active) == 2 and all(len(i.generated) == 3 for i in svc.active)
    eng.status_word = 3
    svc.run_cycle()
    assert svc.finished[a].error == "device fault 3" and svc.finished[b].error == "device fault 3"
    assert svc.finished[a].tokens == [4, 5, 6] and eng.status_word == 0
    assert not svc.active and eng.cache.free_pages() == 16 and svc.snapshot()["failed_steps"] == 1
    r = svc.generate([7], GenerationConfig(max_new_tokens=3))
    assert r.error is None and r.tokens == [8, 9, 10]


def test_queue_is_bounded_and_requests_are_checked():
    svc = InferenceService(FakeEngine(pages=4), SchedulerConfig(max_queued_requests=2))
    svc.submit([1]); svc.submit([2])
    with pytest.raises(QueueFull):
        svc.submit([3])
    with pytest.raises(ValueError, match="vocabulary"):
        InferenceService(FakeEngine(4)).submit([50])
    with pytest.raises(ValueError, match="context"):
        InferenceService(FakeEngine(4)).submit([1] * 4000, GenerationConfig(max_new_tokens=200))
    with pytest.raises(ValueError, match="top_p"):
        InferenceService(FakeEngine(4)).submit([1], GenerationConfig(sampling=SamplingConfig(0.5, 0, 1.5, 0)))


def test_when_pages_run_out_the_youngest_is_put_back_and_computed_again():
    eng = FakeEngine(pages=4)                                    # 64 tokens in all
    svc = InferenceService(eng, SchedulerConfig(max_active_requests=4, reserve_worst_case=False,
                                                prefill_quantum_tokens=16, token_budget_per_cycle=64))
    out = svc.generate_cohort([(list(range(1, 25)), GenerationConfig(max_new_tokens=20, stop_on_eos=False)),
                               (list(range(2, 22)), GenerationConfig(max_new_tokens=20, stop_on_eos=False))])
    # both need 44 and 40 tokens: together more than the pool holds, so one was pre-empted
    assert svc.preemptions >= 1 and out[1].metrics.preemptions >= 1
    assert out[0].tokens == [(24 + i) % 50 for i in range(1, 21)]
    assert out[1].tokens == [(21 + i) % 50 for i in range(1, 21)]
    assert eng.cache.free_pages() == 4 and not eng.cache.sequences
    eng.cache.check()


def test_a_single_request_that_outgrows_the_pool_fails():
    eng = FakeEngine(pages=2)
    svc = InferenceService(eng, SchedulerConfig(reserve_worst_case=False))
    r = svc.generate(list(range(10)), GenerationConfig(max_new_tokens=30, stop_on_eos=False))
    assert r.error == "insufficient KV pages for one sequence"
    assert eng.cache.free_pages() == 2


def test_cancellation_while_queued_and_while_active():
    """A cancelled request leaves at the next admission pass: one that still waits in the queue with
    "cancelled while queued", one that is being computed with "cancelled while active" and the tokens it
    has so far; its pages go back, the others go on."""
    from air_b200.engine.service import CancellationSource
    eng = FakeEngine(pages=16)
    svc = InferenceService(eng, SchedulerConfig(max_active_requests=2, prefill_quantum_tokens=4))
    sources = [CancellationSource() for _ in range(3)]
    ids = [svc.submit([1 + i, 2, 3, 4, 5, 6], GenerationConfig(max_new_tokens=6), s.token())
           for i, s in enumerate(sources)]
    svc.run_cycle()                                   # two are admitted, the third waits
    assert len(svc.active) == 2 and len(svc.queued) == 1
    sources[2].cancel()
    svc.run_cycle()
    assert svc.finished[ids[2]].error == "request cancelled while queued" and not svc.queued
    for _ in range(3):
        svc.run_cycle()
    produced = len(svc.active[0].generated)
    assert produced >= 1
    sources[0].cancel()
    while ids[1] not in svc.finished:
        svc.run_cycle()
    first = svc.finished[ids[0]]
    assert first.error == "request cancelled while active" and len(first.tokens) in (produced, produced + 1)
    assert svc.finished[ids[1]].error is None and len(svc.finished[ids[1]].tokens) == 6
    assert svc.snapshot()["cancelled_requests"] == 2
    assert eng.cache.free_pages() == eng.cache.num_pages
    eng.cache.check()


@pytest.mark.parametrize("seed", range(12))
def test_random_requests_and_settings_keep_every_promise(seed):
    """Random settings (places, budget, portion size, pages, with and without reservation) and random
    requests over the fake engine: every request gets exactly its tokens (the fake's next token is
    predictable), no step exceeds the budget or the places, and every page and slot comes back."""
    rng = np.random.default_rng(100 + seed)
    places = int(rng.integers(1, 6))
    budget = int(rng.integers(places, 40))
    quantum = int(rng.integers(1, 24))
    reserve = bool(rng.random() < 0.5)
    reqs = []
    for _ in range(int(rng.integers(3, 16))):
        first = int(rng.integers(0, 40))
        prompt = [int(t) for t in rng.integers(0, 48, size=int(rng.integers(0, 30)))] + [first]
        reqs.append((prompt, GenerationConfig(max_new_tokens=int(rng.integers(0, 12)), stop_on_eos=False)))
    largest = max(-(-(len(p) + g.max_new_tokens) // 16) for p, g in reqs)
    eng = FakeEngine(pages=largest + int(rng.integers(0, 6)), slots=places)
    svc = InferenceService(eng, SchedulerConfig(max_active_requests=places, token_budget_per_cycle=budget,
                                                prefill_quantum_tokens=quantum, kv_page_tokens=16,
                                                reserve_worst_case=reserve, decode_ahead=False))
    out = svc.generate_cohort(reqs)
    for (prompt, g), r in zip(reqs, out):
        assert r.error is None
        assert r.tokens == [(prompt[-1] + 1 + i) % 50 for i in range(g.max_new_tokens)]
        assert r.metrics.prompt_tokens == len(prompt) and r.metrics.generated_tokens == g.max_new_tokens
    for step in eng.steps:
        assert sum(n for _, n, _ in step) <= budget and len(step) <= places
        assert len({r for r, _, _ in step}) == len(step), "a request appears once in a step"
    while svc.run_cycle():
        pass
    assert eng.cache.free_pages() == eng.cache.num_pages and not eng.cache.sequences
    eng.cache.check()


# ------------------------------------------------------------------ which attention block takes which keys
def test_segments_cover_every_stream_exactly_once():
    """Whatever the planner decides (whole items or cut streams), every (pair, head) has its stream covered from
    0 to the end without a gap or an overlap, cut items have consecutive slots of their own, and a step that would
    leave most SMs idle is cut."""
    import numpy as np
    from air_b200.parts.attention import MIN_SEGMENT, TO_THE_END, plan_segments
    rng = np.random.default_rng(5)
    cases = [([68, 68], 40), ([514], 28), ([4 * p + 4 for p in range(32)], 28), ([2], 2), ([], 4), ([1, 1, 1], 3),
             ([129], 3), ([7, 300, 9], 5)]
    cases += [(rng.integers(1, 600, size=rng.integers(1, 12)).tolist(), int(rng.integers(1, 41))) for _ in range(40)]
    n_cut = 0
    for streams, heads in cases:
        planned = plan_segments(streams, heads)
        if planned is None:          # one block per (pair, head): the kernel's own grid
            continue
        segments, items, slots = planned
        n_cut += slots > 0
        assert segments.dtype == np.int32 and items.dtype == np.int32
        by_item, seen_slots = {}, set()
        for pair, head, first, count, slot in segments.tolist():
            by_item.setdefault((pair, head), []).append((first, count, slot))
        assert set(by_item) == {(p, h) for p in range(len(streams)) for h in range(heads)}
        cut = {}
        for (pair, head), pieces in by_item.items():
            pieces.sort()
            at = 0
            for j, (first, count, slot) in enumerate(pieces):
                assert first == at
                last = j == len(pieces) - 1
                assert (count == TO_THE_END) == last
                assert last or count >= MIN_SEGMENT
                at += count
                assert (slot == -1) == (len(pieces) == 1)
                if slot >= 0:
                    assert slot not in seen_slots
                    seen_slots.add(slot)
            assert pieces[-1][0] < streams[pair]
            if len(pieces) > 1:
                cut[(pair, head)] = [s for _, _, s in pieces]
        assert seen_slots == set(range(slots))
        assert {(p, h): list(range(s0, s0 + n)) for p, h, s0, n in items.tolist()} == cut
    assert n_cut >= 10
    # a 512-token portion behind 3,840 tokens at 40 heads: 80 items would hold 80 of 148 SMs for the whole stream
    segments, items, slots = plan_segments([68, 68], 40)
    assert len(items) == 80 and 148 <= len(segments) <= 2 * 148 + 80
    work = [68 - first if count == TO_THE_END else count for _, _, first, count, _ in segments.tolist()]
    assert work == sorted(work, reverse=True), "the longest segments are launched first"
    # 224 equal items on 148 SMs: two rounds for some SMs unless the streams are cut
    assert plan_segments([518] * 8, 28) is not None
    # a whole prompt of 2,048 tokens: 224 items of graded length fill the SMs as they are; nothing to plan either
    assert plan_segments([4 * p + 4 for p in range(8)], 28) is None
    assert plan_segments([], 4) is None and plan_segments([2], 2) is None
