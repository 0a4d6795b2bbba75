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


@pytest.mark.parametrize("name", ["K", "L"])
def test_bfloat16_through_the_service_follows_the_plain_implementation(name):
    """What serving runs and the benchmark times: bfloat16, the tcgen05 products and the tensor-core attention
    kernels, CUDA graphs, decoding one step ahead with the device's own choice fed back.  Greedy: every produced
    token is the plain implementation's choice at its place, or lies within twice the tolerance of it (then the
    comparison ends: the continuations differ).  Several requests of different lengths run together, so the
    decode graph sees batches that shrink."""
    from air_b200 import GenerationConfig
    folder = util.model_folder(name)
    cfg, tensors = util.plain_model(folder)
    svc = service(name, "bfloat16", page_tokens=64, max_tokens=4096, decode_ahead=True)
    assert svc.engine.use_graphs
    prompts = [util.tokens_for(name, n, 900 + n) for n in (3, 70, 150, 33)]
    new = [40, 25, 12, 40]
    out = svc.generate_cohort([(p, GenerationConfig(max_new_tokens=m, stop_on_eos=False)) for p, m in zip(prompts, new)])
    svc.engine.check_status()
    assert svc.engine.graphs, "decode steps replayed CUDA graphs"
    agreed = 0
    for prompt, m, r in zip(prompts, new, out):
        assert r.error is None and len(r.tokens) == m
        ref = util.plain_logits(folder, prompt + r.tokens)           # the logits along the produced tokens
        scale = max(1.0, float(np.abs(ref).max()))
        for i, t in enumerate(r.tokens):
            row = ref[len(prompt) - 1 + i]
            best = int(row.argmax())
            assert row[best] - row[t] <= 2 * util.BF16_MAX_TOL * scale, (name, i, t, best)
            agreed += t == best
    assert agreed >= 0.9 * sum(new), "nearly every token is the plain implementation's own choice"
    assert svc.engine.cache.free_pages() == svc.engine.cache.num_pages


@pytest.mark.parametrize("ahead", [True, False])
def test_bfloat16_temperature_runs_repeat_per_seed(ahead):
    from air_b200 import GenerationConfig, SamplingConfig
    prompt = util.tokens_for("K", 20, 950)
    runs = []
    for seed in (5, 5, 6):
        svc = service("K", "bfloat16", page_tokens=64, decode_ahead=ahead)
        g = GenerationConfig(max_new_tokens=30, stop_on_eos=False, sampling=SamplingConfig(0.9, 0, 1.0, seed))
        runs.append(svc.generate(prompt, g).tokens)
        svc.engine.check_status()
    assert runs[0] == runs[1] and runs[0] != runs[2]


@pytest.mark.parametrize("ahead", [True, False])
def test_a_fault_on_the_device_reaches_the_caller(ahead):
    """The device's status word travels with every step's tokens.  Here it is set from the host between two
    cycles, as a kernel whose bounded wait ran out would set it: the requests of the step that is read next end
    with the engine's message for that code, their pages come back, the word is cleared, and the service goes on
    serving."""
    from air_b200 import GenerationConfig
    svc = service("K", "bfloat16", page_tokens=64, decode_ahead=ahead)
    ids = [svc.submit(util.tokens_for("K", n, 960 + n), GenerationConfig(max_new_tokens=20, stop_on_eos=False))
           for n in (9, 30)]
    for _ in range(6):
        svc.run_cycle()
    assert len(svc.active) == 2
    svc.engine.status.fill_(5)
    for _ in range(3):
        svc.run_cycle()
    assert all(svc.finished[i].error == "a wait inside the decode attention kernel ran out" for i in ids)
    assert all(0 < len(svc.finished[i].tokens) < 20 for i in ids)
    assert svc.engine.read_status() == 0 and svc.snapshot()["failed_steps"] >= 1
    assert not svc.active and svc.engine.cache.free_pages() == svc.engine.cache.num_pages
    r = svc.generate(util.tokens_for("K", 12, 970), GenerationConfig(max_new_tokens=5, stop_on_eos=False))
    assert r.error is None and len(r.tokens) == 5


def test_sizes_that_the_kernels_refuse_are_unsupported_with_exit_code_3(tmp_path):
    """A head size that config.json allows and the attention kernels do not take (24): "unsupported" when the
    model is built, exit code 3 from the command line (air-cli's code for a model that cannot be loaded), no
    traceback."""
    from air_b200.config import ConfigError
    from air_b200.engine.engine import Engine, EngineConfig
    cfg = dict(util.TINY_A, hidden_size=96, num_attention_heads=4, num_key_value_heads=2)
    folder = str(tmp_path / "m")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    with pytest.raises(ConfigError, match="unsupported.*head size 24"):
        Engine.from_folder(folder, EngineConfig(dtype="bfloat16"))
    with pytest.raises(ConfigError, match="unsupported.*page size"):
        Engine.from_folder(util.model_folder("A"), EngineConfig(dtype="bfloat16", page_tokens=24))
    for cmd in (["inspect", folder], ["cuda", folder, "1,2,3"]):
        p = subprocess.run([sys.executable, os.path.join(util.ROOT, "bin", "air-b200")] + cmd, capture_output=True,
                           text=True, timeout=300)
        assert p.returncode == 3 and "unsupported" in p.stderr and "Traceback" not in p.stderr, p.stderr[-500:]


def test_a_float32_checkpoint_in_the_bfloat16_engine_runs_the_tensor_core_products(tmp_path):
    """A checkpoint stored in float32, loaded by the bfloat16 engine: matrices are rounded to bfloat16 at load
    (and the load says so), so every product runs the kernels of the bfloat16 path; keep_float32 keeps them and
    runs the CUDA-core product; both agree with the plain implementation on the rounded weights."""
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig, write_random_model
    folder = str(tmp_path / "m")
    write_random_model(folder, util.TINY_K, 3, "float32")
    rounded = str(tmp_path / "r")
    write_random_model(rounded, util.TINY_K, 3, "bfloat16")         # the same draws, rounded: what the oracle reads
    tokens = util.tokens_for("K", 90, 5)
    want = util.plain_logits(rounded, tokens)
    engine = Engine.from_folder(folder, EngineConfig(dtype="bfloat16", page_tokens=64, max_tokens=256))
    assert len(engine.load_report.rounded) > 0 and "rounded to bfloat16" in engine.load_report.summary()
    assert all(b.mixer.qkv.tc_ok and b.feed_forward.down.tc_ok for b in engine.model.blocks)
    got = np.concatenate([engine.step([Entry("r", tokens[:80], range(80))]).cpu().numpy()] +
                         [engine.step([Entry("r", [t], [0])]).cpu().numpy() for t in tokens[80:]])
    scale = max(1.0, float(np.abs(want).max()))
    assert np.abs(got - want).max() < util.BF16_MAX_TOL * scale
    kept = Engine.from_folder(folder, EngineConfig(dtype="bfloat16", page_tokens=64, max_tokens=256, keep_float32=True))
    assert not kept.model.blocks[0].mixer.qkv.tc_ok and len(kept.load_report.rounded) == 0


def test_the_pool_is_sized_from_the_memory_that_is_left():
    """Without a size the cache pool takes its share of the free device memory, at most what the allowed requests
    could ever hold; generation runs on it."""
    from air_b200 import GenerationConfig, InferenceService, SchedulerConfig
    svc = InferenceService.create(util.model_folder("K"), dtype="bfloat16",
                                  scheduler=SchedulerConfig(max_active_requests=3, kv_page_tokens=64))
    cache = svc.engine.cache
    assert cache.num_pages == 3 * (util.TINY_K["max_position_embeddings"] // 64)      # the cap: 3 requests of 512 tokens
    r = svc.generate(util.tokens_for("K", 30, 990), GenerationConfig(max_new_tokens=8, stop_on_eos=False))
    assert r.error is None and len(r.tokens) == 8
    from air_b200.engine.engine import Engine, EngineConfig
    engine = Engine.from_folder(util.model_folder("K"), EngineConfig(dtype="bfloat16", page_tokens=64, max_tokens=None,
                                                                     max_requests=4, memory_fraction=1e-6))
    assert 1 <= engine.cache.num_pages < 4 * 8, "a sliver of the free memory gives a small pool"
