"""Generation through the Python entry point and the command line against the plain
implementation: greedy tokens, the first tokens of a sequence, long decoding, temperature
sampling, several requests at once."""
import dataclasses
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import util
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu


def service(name, dtype, **kw):
    from air_b200.engine.engine import Engine, EngineConfig
    from air_b200.engine.service import InferenceService, SchedulerConfig
    engine = Engine.from_folder(util.model_folder(name), EngineConfig(
        dtype=dtype, page_tokens=kw.pop("page_tokens", 16), max_tokens=kw.pop("max_tokens", 1024),
        max_requests=kw.get("max_active_requests", 8)))
    return InferenceService(engine, SchedulerConfig(**{"max_active_requests": 8, **kw}))


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain(name):
    from air_b200 import GenerationConfig
    folder = util.model_folder(name)
    cfg, tensors = util.plain_model(folder)
    svc = service(name, "float32", prefill_quantum_tokens=5, token_budget_per_cycle=12)
    prompts = [util.tokens_for(name, n, 20 + n) for n in (1, 7, 33)]
    want = [plain.greedy_generate(cfg, tensors, p, 16) for p in prompts]
    got = svc.generate_cohort([(p, GenerationConfig(max_new_tokens=16, stop_on_eos=False)) for p in prompts])
    assert [r.tokens for r in got] == want
    assert svc.engine.cache.free_pages() == svc.engine.cache.num_pages
    svc.engine.check_status()


@pytest.mark.parametrize("name", ["B", "K", "L"])
def test_first_tokens_of_a_sequence(name):
    """Positions 0, 1, 2: one key, two keys, three keys; decoded one by one from the very start, and as a
    portion of two tokens followed by single ones (K and L: the tensor-core attention kernels in bfloat16)."""
    from air_b200.engine.batch import Entry
    folder = util.model_folder(name)
    toks = util.tokens_for(name, 5, 77)
    want = util.plain_logits(folder, toks)
    for dtype, tol in (("float32", util.FP32_TOL), ("bfloat16", util.BF16_MAX_TOL)):
        svc = service(name, dtype, page_tokens=64)
        got = np.concatenate([svc.engine.step([Entry("r", [t], [0])]).cpu().numpy() for t in toks])
        assert np.abs(got - want).max() < tol * max(1.0, np.abs(want).max())
        got = [svc.engine.step([Entry("s", toks[:2], [0, 1])]).cpu().numpy()]
        got += [svc.engine.step([Entry("s", [t], [0])]).cpu().numpy() for t in toks[2:]]
        assert np.abs(np.concatenate(got) - want).max() < tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("name", ["A", "K"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_stays_on_the_plain_logits(dtype, name):
    """300 tokens decoded one by one after a short prompt (teacher-forced with the plain
    implementation's greedy tokens), across many pages (K in bfloat16: the decode attention kernel and the
    tcgen05 products inside the decode graph)."""
    from air_b200.engine.batch import Entry
    folder = util.model_folder(name)
    cfg, tensors = util.plain_model(folder)
    prompt = util.tokens_for(name, 5, 9)
    tokens = prompt + plain.greedy_generate(cfg, tensors, prompt, 40)
    tokens = (tokens * 8)[:320]                      # teacher-forced stream
    want = util.plain_logits(folder, tokens)
    svc = service(name, dtype, max_tokens=384)
    eng = svc.engine
    got = [eng.step([Entry("r", tokens[:5], range(5))]).cpu().numpy()]
    got += [eng.step([Entry("r", [t], [0])]).cpu().numpy() for t in tokens[5:]]
    got = np.concatenate(got)
    scale = max(1.0, np.abs(want).max())
    if dtype == "float32":
        assert np.abs(got - want).max() < util.FP32_TOL * scale
    else:
        assert np.abs(got - want).max() < util.BF16_MAX_TOL * scale
        assert np.abs(got - want).mean() < util.BF16_MEAN_TOL * scale


def test_device_feedback_of_sampled_tokens_equals_host_feedback():
    from air_b200.engine.batch import Entry, LAST_SAMPLED
    svc = service("B", "float32")
    eng = svc.engine
    prompt = util.tokens_for("B", 9, 5)
    ids = [int(eng.sample(eng.step([Entry("dev", prompt, [8])])).item())]
    for _ in range(10):
        ids.append(int(eng.sample(eng.step([Entry("dev", [LAST_SAMPLED], [0])])).item()))
    cfg, tensors = util.plain_model(util.model_folder("B"))
    assert ids == plain.greedy_generate(cfg, tensors, prompt, 11)


def test_temperature_sampling_mixed_batch_of_config_b():
    """Prompts of 5, 40 and 97 tokens in portions of 32 beside three requests that decode at
    temperature 0.8: tokens are reproducible per seed, differ between seeds, and every sampled
    token has a plausible probability under the plain implementation's distribution."""
    from air_b200 import GenerationConfig, SamplingConfig
    folder = util.model_folder("B")
    cfg, tensors = util.plain_model(folder)

    def run(seed):
        svc = service("B", "float32", prefill_quantum_tokens=32, token_budget_per_cycle=70)
        reqs = [(util.tokens_for("B", n, n), GenerationConfig(max_new_tokens=4, stop_on_eos=False)) for n in (5, 40, 97)]
        reqs += [(util.tokens_for("B", 3, 200 + i), GenerationConfig(
            max_new_tokens=12, stop_on_eos=False, sampling=SamplingConfig(temperature=0.8, seed=seed + i)))
            for i in range(3)]
        return reqs, svc.generate_cohort(reqs)

    reqs, first = run(100)
    _, again = run(100)
    _, other = run(500)
    assert [r.tokens for r in first] == [r.tokens for r in again]
    assert [r.tokens for r in first[3:]] != [r.tokens for r in other[3:]]
    for (prompt, g), r in zip(reqs[:3], first[:3]):
        assert r.tokens == plain.greedy_generate(cfg, tensors, prompt, 4)
    for (prompt, g), r in zip(reqs[3:], first[3:]):
        logits = plain.forward(cfg, tensors, prompt + r.tokens)[len(prompt) - 1:-1]
        p = torch.softmax(torch.tensor(logits).double() / 0.8, -1)
        chosen = p[torch.arange(len(r.tokens)), torch.tensor(r.tokens)]
        assert float(chosen.min()) > 1e-5


def test_decoding_one_step_ahead_gives_the_same_tokens():
    """The loop that launches a step before it reads the one in flight against the strictly
    alternating loop: requests that end by their token count at different times, one that ends by an
    end-of-sequence token (its id is set to a token that greedy decoding reaches), temperature
    sampling, a request that arrives while others decode, and all pages back at the end."""
    from air_b200 import GenerationConfig, SamplingConfig
    folder = util.model_folder("B")
    cfg, tensors = util.plain_model(folder)
    prompts = [util.tokens_for("B", n, 300 + n) for n in (3, 9, 17, 4)]
    greedy = plain.greedy_generate(cfg, tensors, prompts[0], 12)
    eos = greedy[6]
    stop_at = greedy.index(eos) + 1

    def run(ahead):
        svc = service("B", "float32", decode_ahead=ahead, max_active_requests=3)
        svc.engine.model.spec = dataclasses.replace(svc.engine.model.spec, eos_token_id=eos)
        reqs = [(prompts[0], GenerationConfig(max_new_tokens=12, stop_on_eos=True)),
                (prompts[1], GenerationConfig(max_new_tokens=5, stop_on_eos=False)),
                (prompts[2], GenerationConfig(max_new_tokens=9, stop_on_eos=False,
                                              sampling=SamplingConfig(temperature=0.7, seed=5))),
                (prompts[3], GenerationConfig(max_new_tokens=7, stop_on_eos=False))]   # waits for a free place
        out = svc.generate_cohort(reqs)
        assert svc.engine.cache.free_pages() == svc.engine.cache.num_pages
        svc.engine.check_status()
        return out, svc.cycles

    ahead, cycles_ahead = run(True)
    plainly, cycles = run(False)
    assert [r.tokens for r in ahead] == [r.tokens for r in plainly]
    assert [r.hit_eos for r in ahead] == [True, False, False, False]
    assert ahead[0].tokens == greedy[:stop_at]
    assert ahead[1].tokens == plain.greedy_generate(cfg, tensors, prompts[1], 5)
    assert ahead[3].tokens == plain.greedy_generate(cfg, tensors, prompts[3], 7)
    assert cycles_ahead <= cycles + 3      # at most a dropped step per request that stops by itself


def test_cancellation_with_a_step_in_flight():
    """A request cancelled while the loop decodes one step ahead: it leaves with the tokens read so far, the
    other one goes on and gets the tokens it would have got alone, all pages come back."""
    from air_b200 import GenerationConfig
    from air_b200.engine.service import CancellationSource
    folder = util.model_folder("B")
    cfg, tensors = util.plain_model(folder)
    prompts = [util.tokens_for("B", 6, 400), util.tokens_for("B", 11, 401)]
    svc = service("B", "float32")
    source = CancellationSource()
    ids = [svc.submit(prompts[0], GenerationConfig(max_new_tokens=20, stop_on_eos=False), source.token()),
           svc.submit(prompts[1], GenerationConfig(max_new_tokens=12, stop_on_eos=False))]
    for _ in range(6):
        svc.run_cycle()
    assert svc._inflight is not None, "the loop is one step ahead"
    source.cancel()
    while ids[1] not in svc.finished:
        svc.run_cycle()
    a, b = svc.finished[ids[0]], svc.finished[ids[1]]
    assert a.error == "request cancelled while active" and 1 <= len(a.tokens) < 20
    assert a.tokens == plain.greedy_generate(cfg, tensors, prompts[0], len(a.tokens))
    assert b.error is None and b.tokens == plain.greedy_generate(cfg, tensors, prompts[1], 12)
    while svc.run_cycle():
        pass
    assert svc.engine.cache.free_pages() == svc.engine.cache.num_pages
    svc.engine.check_status()


@pytest.mark.parametrize("reserve", [True, False])
def test_service_under_churn(reserve):
    """Twenty requests of random lengths through a service with four places, a small token budget and a
    pool that holds only part of them at a time (with and without worst-case reservation, i.e. with
    waiting in the queue and with preemption and recomputation): every request gets the tokens that the
    plain implementation generates for it alone, and every page comes back."""
    from air_b200 import GenerationConfig
    folder = util.model_folder("A")
    cfg, tensors = util.plain_model(folder)
    rng = np.random.default_rng(7)
    reqs = []
    for i in range(20):
        prompt = util.tokens_for("A", int(rng.integers(1, 70)), 600 + i)
        reqs.append((prompt, GenerationConfig(max_new_tokens=int(rng.integers(1, 20)), stop_on_eos=False)))
    svc = service("A", "float32", max_active_requests=4, token_budget_per_cycle=48, prefill_quantum_tokens=16,
                  max_tokens=288 if reserve else 160, reserve_worst_case=reserve)
    got = svc.generate_cohort(reqs)
    for (prompt, g), r in zip(reqs, got):
        assert r.error is None
        assert r.tokens == plain.greedy_generate(cfg, tensors, prompt, g.max_new_tokens)
    while svc.run_cycle():
        pass
    assert svc.engine.cache.free_pages() == svc.engine.cache.num_pages
    svc.engine.cache.check()
    svc.engine.check_status()
    if not reserve:
        assert svc.preemptions > 0, "the small pool ran out and the youngest request was computed again"


def test_top_k_and_top_p_on_the_device_through_the_service():
    """The default: requests with top-k / top-p are sampled on the device (and decoded one step ahead).
    Every token is one of the k most likely of the plain implementation at its place, the run repeats
    with its seed and differs with another."""
    from air_b200 import GenerationConfig, SamplingConfig
    folder = util.model_folder("B")
    cfg, tensors = util.plain_model(folder)
    prompt = util.tokens_for("B", 9, 31)

    def run(seed):
        svc = service("B", "float32")
        g = GenerationConfig(max_new_tokens=14, stop_on_eos=False,
                             sampling=SamplingConfig(temperature=1.3, top_k=5, top_p=0.95, seed=seed))
        out = svc.generate(prompt, g).tokens
        assert svc._inflight is None and svc.engine.cache.free_pages() == svc.engine.cache.num_pages
        return out

    a, b, c = run(3), run(3), run(4)
    assert a == b and a != c
    logits = plain.forward(cfg, tensors, prompt + a)[len(prompt) - 1:-1]
    for row, token in zip(logits, a):
        assert token in np.argsort(-row, kind="stable")[:5]


def test_host_sampler_path_with_top_k_and_top_p():
    from air_b200 import GenerationConfig, SamplingConfig
    folder = util.model_folder("A")
    cfg, tensors = util.plain_model(folder)
    svc = service("A", "float32", sample_cuts_on_device=False)
    prompt = util.tokens_for("A", 6, 1)
    sampling = SamplingConfig(temperature=0.9, top_k=7, top_p=0.8, seed=11)
    got = svc.generate(prompt, GenerationConfig(max_new_tokens=8, stop_on_eos=False, sampling=sampling)).tokens
    s = plain.PlainSampler(0.9, 7, 0.8, 11)
    toks = list(prompt)
    for t in got:
        logits = plain.forward(cfg, tensors, toks)[-1]
        assert s.sample(logits) == t
        toks.append(t)


def test_command_line(tmp_path):
    folder = util.model_folder("A")
    cfg, tensors = util.plain_model(folder)
    prompt = util.tokens_for("A", 7, 3)
    exe = [sys.executable, os.path.join(util.ROOT, "bin", "air-b200")]
    p = subprocess.run(exe + ["cuda", folder, ",".join(map(str, prompt)), "--tokens", "5", "--dtype", "float32",
                              "--no-stop-on-eos"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr
    assert [int(t) for t in p.stdout.strip().split(",")] == plain.greedy_generate(cfg, tensors, prompt, 5)
    p = subprocess.run(exe + ["cuda-compare", folder, ",".join(map(str, prompt))], capture_output=True, text=True,
                       timeout=300)
    assert p.returncode == 0, p.stderr
    report = json.loads(p.stdout)
    assert report["top1_parity"] and report["float32_whole_vs_token_by_token_max_abs"] <= 1e-5
    assert subprocess.run(exe + ["cuda", str(tmp_path), "1,2"], capture_output=True).returncode == 3
    assert subprocess.run(exe + ["cuda"], capture_output=True).returncode == 2
    p = subprocess.run(exe + ["cuda-info"], capture_output=True, text=True)
    assert p.returncode == 0 and "B200" in p.stdout


def test_smoke_entry():
    sys.path.insert(0, util.ROOT)
    import __graft_entry__
    __graft_entry__.smoke()
