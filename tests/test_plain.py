"""The plain implementation against AIR's own compiled reference executor (golden
logits under tests/golden/, made by tests/golden/make_golden.py) and against itself."""
import os

import numpy as np

from plain import qwen2_plain as plain
import pytest

from golden.make_golden import CONFIG, CONFIGS, from_bf16_bits

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "air_reference_tiny.npz")


def load_golden(which="tiny"):
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", CONFIGS[which][2]))
    names = [str(n) for n in z["names"]]
    tensors = {name: from_bf16_bits(z[f"w{i}"]).reshape(z[f"s{i}"]) for i, name in enumerate(names)}
    return tensors, z["tokens"].tolist(), z["logits"]


@pytest.mark.parametrize("which", ["tiny", "a", "b"])
def test_plain_matches_air_reference_executor(which):
    """AIR's own compiled CPU executor, token by token, on three tiny models: one of odd sizes, and the two
    tiny configurations of the engine's tests (tied and separate output matrix, groups of 2 and of 4)."""
    tensors, tokens, golden = load_golden(which)
    logits = plain.forward(CONFIGS[which][0], tensors, tokens)
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


def test_the_replay_models_would_show_a_missing_rotation_and_a_window_off_by_one():
    """A test of the tests.  The replay suite compares bfloat16 logits with the plain implementation within
    BF16_MAX_TOL / BF16_MEAN_TOL.  That can only catch a fault whose effect is larger than the tolerance, so for
    every configuration of that suite: the plain implementation without any position encoding, and (where layers
    have a window) with a window one key too wide, differs from itself by at least three times one of the two
    tolerances (a replay fails when either is exceeded).
    (With q and k drawn at N(0, 0.02) like the other matrices it does not: tests/util.py sharpen_attention.)"""
    import util
    for name in ("A", "B", "W", "K", "L", "M"):
        folder = util.model_folder(name)
        config, tensors = plain.read_model(folder)
        tokens = util.tokens_for(name, 150, 1)
        ref = plain.forward(config, tensors, tokens)
        scale = max(1.0, float(np.abs(ref).max()))
        rotate = plain.rope
        try:
            plain.rope = lambda x, positions, theta: x
            faulty = [("no rotation", plain.forward(config, tensors, tokens))]
        finally:
            plain.rope = rotate
        if config.get("use_sliding_window"):
            wider = dict(config, sliding_window=config["sliding_window"] + 1)
            faulty.append(("window + 1", plain.forward(wider, tensors, tokens)))
        for what, logits in faulty:
            diff = np.abs(logits - ref)
            assert (diff.max() > 3 * util.BF16_MAX_TOL * scale or
                    diff.mean(1).max() > 3 * util.BF16_MEAN_TOL * scale), (name, what, float(diff.max()),
                                                                           float(diff.mean(1).max()))
        # attention has something to look at: the largest probability is many times the uniform one
        p = f"model.layers.0.self_attn."
        heads, kv = config["num_attention_heads"], config["num_key_value_heads"]
        d = config["hidden_size"] // heads
        x = plain.rms_norm(plain.embed(tensors["model.embed_tokens.weight"], np.asarray(tokens)),
                           tensors["model.layers.0.input_layernorm.weight"], config["rms_norm_eps"])
        pos = np.arange(len(tokens))
        q = plain.rope(plain.linear(x, tensors[p + "q_proj.weight"], tensors[p + "q_proj.bias"]).reshape(-1, heads, d),
                       pos, config["rope_theta"])
        k = plain.rope(plain.linear(x, tensors[p + "k_proj.weight"], tensors[p + "k_proj.bias"]).reshape(-1, kv, d),
                       pos, config["rope_theta"])
        scores = (q[-1, 0].astype(np.float64) @ k[:, 0].astype(np.float64).T) / np.sqrt(d)
        prob = np.exp(scores - scores.max())
        assert prob.max() / prob.sum() > 5.0 / len(tokens), name
