"""The plain implementation against AIR's own compiled reference executor (golden
logits under tests/golden/, made by tests/golden/make_golden.py) and against itself."""
import os

import numpy as np

from plain import qwen2_plain as plain
from golden.make_golden import CONFIG, from_bf16_bits

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "air_reference_tiny.npz")


def load_golden():
    z = np.load(GOLDEN)
    names = [str(n) for n in z["names"]]
    tensors = {name: from_bf16_bits(z[f"w{i}"]).reshape(z[f"s{i}"]) for i, name in enumerate(names)}
    return tensors, z["tokens"].tolist(), z["logits"]


def test_plain_matches_air_reference_executor():
    tensors, tokens, golden = load_golden()
    logits = plain.forward(CONFIG, tensors, tokens)
    assert logits.shape == golden.shape
    assert np.abs(logits - golden).max() <= 2e-6 * max(1.0, np.abs(golden).max())
    assert (logits.argmax(-1) == golden.argmax(-1)).all()


def test_prefix_logits_do_not_depend_on_later_tokens():
    tensors, tokens, _ = load_golden()
    whole = plain.forward(CONFIG, tensors, tokens)
    part = plain.forward(CONFIG, tensors, tokens[:9])
    assert np.abs(whole[:9] - part).max() < 1e-6


def test_window_as_long_as_the_sequence_changes_nothing():
    tensors, tokens, golden = load_golden()
    cfg = dict(CONFIG, use_sliding_window=True, sliding_window=len(tokens), max_window_layers=0)
    assert np.abs(plain.forward(cfg, tensors, tokens) - golden).max() < 1e-5
    cfg["sliding_window"] = 4
    assert np.abs(plain.forward(cfg, tensors, tokens) - golden).max() > 1e-4
    # the first four positions see the same keys with and without the window
    assert np.abs(plain.forward(cfg, tensors, tokens)[:4] - golden[:4]).max() < 1e-5


def test_rope_rotates_pairs_half_a_head_apart():
    x = np.zeros((1, 1, 8), dtype=np.float32)
    x[0, 0, 1] = 1.0
    y = plain.rope(x, [3], 10000.0)
    angle = 3 / 10000.0 ** (2 / 8)
    assert np.allclose(y[0, 0, 1], np.cos(angle)) and np.allclose(y[0, 0, 5], np.sin(angle))
    assert np.count_nonzero(y) == 2


def test_attention_groups_consecutive_heads():
    rng = np.random.default_rng(0)
    q = rng.standard_normal((5, 4, 8)).astype(np.float32)
    k = rng.standard_normal((5, 2, 8)).astype(np.float32)
    v = rng.standard_normal((5, 2, 8)).astype(np.float32)
    out = plain.attention(q, k, v)
    # heads 0,1 read kv head 0; heads 2,3 read kv head 1
    k2, v2 = np.repeat(k, 2, axis=1), np.repeat(v, 2, axis=1)
    assert np.allclose(out, plain.attention(q, k2, v2), atol=1e-6)
    assert np.allclose(out[0], v2[0], atol=1e-6)  # first query sees only itself


def test_sampler_is_greedy_at_zero_and_seeded_above():
    logits = np.array([0.1, 2.0, 2.0, -1.0], dtype=np.float32)
    assert plain.PlainSampler().sample(logits) == 1  # lowest index of the maximum
    a = [plain.PlainSampler(temperature=0.8, seed=7).sample(logits) for _ in range(3)]
    assert a[0] == a[1] == a[2]
    s = plain.PlainSampler(temperature=1.0, seed=1)
    draws = [s.sample(logits) for _ in range(400)]
    p = np.exp(logits - logits.max()); p /= p.sum()
    freq = np.bincount(draws, minlength=4) / 400
    assert np.abs(freq - p).max() < 0.08
    assert plain.PlainSampler(temperature=1.0, top_k=1, seed=3).sample(logits) in (1, 2)


def test_mt19937_64_first_outputs():
    # the 10000th output of a default-seeded (5489) std::mt19937_64 is fixed by the C++ standard
    g = plain.MT19937_64(5489)
    for _ in range(9999):
        g.next()
    assert g.next() == 9981545732273789042
