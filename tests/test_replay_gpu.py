"""Trace replay on the GPU against the plain implementation: the same requests whole, with
the last 32 tokens one by one, in portions of changing size down to two tokens, and mixed with
other requests in a pool so small that pages are used again; in float32 and in bfloat16; for
the tiny configurations A and B (which differ in every size and option) and W (a window), and for K
and L, whose heads of 64 and 128 take the tensor-core attention kernels in bfloat16 (L with a window)."""
import json
import os
import tempfile

import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu

LENGTHS = {"A": (1, 7, 33, 97, 150), "B": (5, 40, 97, 131, 64, 18), "W": (3, 50, 97, 140),
           "K": (2, 65, 150, 300), "L": (9, 129, 64, 270), "M": (3, 70, 200)}


def streams_for(name):
    return {f"{name}{i}": util.tokens_for(name, n, i) for i, n in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W", "K", "L"])
def test_whole(name, dtype):
    folder, streams = util.model_folder(name), streams_for(name)
    steps = util.trace_whole(streams)
    got, _ = util.replay(folder, dtype, steps, max_tokens=util.peak_tokens(steps))
    util.check_against_plain(got, folder, streams, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W", "K", "L"])
def test_bulk_then_last_32_one_by_one(name, dtype):
    folder, streams = util.model_folder(name), streams_for(name)
    steps = util.trace_bulk_tail(streams, tail=32)
    got, _ = util.replay(folder, dtype, steps, max_tokens=util.peak_tokens(steps))
    util.check_against_plain(got, folder, streams, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W", "K", "L"])
def test_portions_of_changing_size(name, dtype):
    folder, streams = util.model_folder(name), streams_for(name)
    steps = util.trace_portions(streams)
    got, _ = util.replay(folder, dtype, steps, max_tokens=util.peak_tokens(steps))
    util.check_against_plain(got, folder, streams, dtype)


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W", "K", "L"])
def test_mixed_with_pages_used_again(name, dtype, page):
    folder = util.model_folder(name)
    lengths = LENGTHS[name] + (120, 2, 77, 101, 64, 129)
    streams = {f"{name}{i}": util.tokens_for(name, n, 50 + i) for i, n in enumerate(lengths)}
    steps = util.trace_mixed(streams, seed=3, live=4)
    peak = util.peak_tokens(steps, page=64)
    got, engine = util.replay(folder, dtype, steps, max_tokens=peak, page_tokens=page)
    util.check_against_plain(got, folder, streams, dtype)
    for group in engine.cache.groups:
        assert group.pool.takes > group.pool.num_pages, "pages were used again"


@pytest.mark.parametrize("page", [32, 128, 48, 80])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["K", "L"])
def test_mixed_with_other_page_sizes(name, dtype, page):
    """Pages of half a key tile and of two key tiles (the tensor-core kernels fetch 64 keys at a time), and
    pages of 48 and 80 tokens, in which a tile of 64 keys would straddle pages: those take the kernels
    that read key by key."""
    folder, streams = util.model_folder(name), streams_for(name)
    steps = util.trace_mixed(streams, seed=9, live=3)
    got, engine = util.replay(folder, dtype, steps, max_tokens=util.peak_tokens(steps, page=page), page_tokens=page)
    util.check_against_plain(got, folder, streams, dtype)


@pytest.mark.parametrize("name", ["A", "B", "W", "K", "L"])
def test_float32_does_not_depend_on_the_cut(name):
    """In float32 every kernel reduces in an order that depends only on the position, so the
    four ways of cutting give the same bits."""
    folder, streams = util.model_folder(name), streams_for(name)
    a, _ = util.replay(folder, "float32", util.trace_whole(streams), 1024)
    b, _ = util.replay(folder, "float32", util.trace_portions(streams), 1024)
    c, _ = util.replay(folder, "float32", util.trace_mixed(streams, seed=5), 1024, page_tokens=32)
    assert a.keys() == b.keys() == c.keys()
    for k in a:
        assert np.array_equal(a[k], b[k]) and np.array_equal(a[k], c[k]), k


@pytest.mark.parametrize("name", ["K", "L", "M"])
def test_bfloat16_heads_of_64_and_128_take_the_tensor_core_kernels(name):
    """The kernels' own trace says which attention kernels a mixed replay ran: the decode kernel and the
    tile kernel, never the 32-bit one.  (M has heads of 256: the mma.sync tile kernel.)"""
    import torch
    from air_b200.csrc import ops
    folder, streams = util.model_folder(name), streams_for(name)
    steps = util.trace_mixed(streams, seed=1, live=3)
    buf = torch.zeros(1 + 2 * 16384, dtype=torch.int64, device="cuda")
    ops.set_trace(buf)
    try:
        got, _ = util.replay(folder, "bfloat16", steps, max_tokens=util.peak_tokens(steps), page_tokens=64)
        torch.cuda.synchronize()
    finally:
        ops.set_trace(None)
    util.check_against_plain(got, folder, streams, "bfloat16")
    b = buf.cpu().tolist()
    ran = {ops.TRACE_NAMES.get(b[1 + 2 * i] % 100) for i in range(min(b[0], 16384))}
    assert {"decode_attention", "prefill_attention"} <= ran and "attention_ref" not in ran


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["K", "L"])
def test_eighty_requests_decode_in_one_step(name, dtype):
    """More single tokens in a step than the kernels for few rows take (64): the decode graph of the next
    bucket with the library's products, the output and down products adding into the stream, the attention
    kernel starting from the q/k/v product in one part."""
    folder = util.model_folder(name)
    streams = {f"r{i}": util.tokens_for(name, 9 + i % 5, 300 + i) for i in range(80)}
    ids = list(streams)
    steps, n = [], 0
    for i in range(0, 80, 8):                      # the prompts, eight requests a step, all but the last 4 tokens
        steps.append(util.step_line(n, [(r, streams[r][:-4], range(len(streams[r]) - 4)) for r in ids[i:i + 8]]))
        n += 1
    for k in range(4, 0, -1):                      # then four steps of 80 single tokens
        steps.append(util.step_line(n, [(r, [streams[r][-k]], [0]) for r in ids], end=ids if k == 1 else []))
        n += 1
    got, _ = util.replay(folder, dtype, steps, max_tokens=util.peak_tokens(steps, page=16), page_tokens=16,
                         max_requests=96)
    util.check_against_plain(got, folder, streams, dtype)


def random_configuration(rng):
    """A tiny configuration drawn at random: heads of 16 to 256 in groups of 1 to 7, widths that follow from
    them, any feed-forward width and vocabulary, with or without windowed layers."""
    d = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 256]))
    kv = int(rng.choice([1, 2, 3, 4]))
    heads = kv * int(rng.choice([1, 2, 3, 5, 7]))
    while heads * d > 1024:
        d = int(rng.choice([16, 32, 48, 64]))
    layers = int(rng.integers(1, 4))
    return dict(util.BASE, num_hidden_layers=layers, hidden_size=heads * d, num_attention_heads=heads,
                num_key_value_heads=kv, intermediate_size=int(rng.integers(8, 80)) * int(rng.choice([2, 4, 8, 16])),
                vocab_size=int(rng.integers(40, 900)), max_position_embeddings=512,
                rope_theta=float(rng.choice([1e4, 5e4, 1e6])), rms_norm_eps=float(rng.choice([1e-6, 1e-5, 3e-6])),
                tie_word_embeddings=bool(rng.random() < 0.5), use_sliding_window=bool(rng.random() < 0.4),
                sliding_window=int(rng.integers(5, 200)), max_window_layers=int(rng.integers(0, layers + 1)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(6))
def test_random_configurations_and_traces(seed, dtype):
    """Sizes, page size, number of live requests, portions and lengths all drawn at random; the pool holds just
    what the trace needs, so pages are used again."""
    from air_b200.engine.engine import write_random_model
    from plain import qwen2_plain as plain
    rng = np.random.default_rng(7000 + seed)
    cfg = random_configuration(rng)
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(folder, cfg, seed, "bfloat16")
        util.sharpen_attention(folder, cfg)
        lengths = [int(x) for x in rng.integers(1, 330, size=int(rng.integers(3, 8)))]
        streams = {f"r{i}": rng.integers(0, cfg["vocab_size"], size=m).tolist() for i, m in enumerate(lengths)}
        steps = util.trace_mixed(streams, seed=seed, live=int(rng.integers(1, 5)), tail=int(rng.integers(1, 20)),
                                 portions=tuple(int(x) for x in rng.integers(2, 90, size=6)))
        page = int(rng.choice([16, 32, 64, 128]))
        got, _ = util.replay(folder, dtype, steps, max_tokens=util.peak_tokens(steps, page=page), page_tokens=page)
        pcfg, tensors = plain.read_model(folder)
        for rid, toks in streams.items():
            ref = plain.forward(pcfg, tensors, list(toks))
            scale = max(1.0, float(np.abs(ref).max()))
            err = np.stack([np.abs(got[(rid, p)] - ref[p]) for p in range(len(toks))])
            if dtype == "float32":
                assert err.max() < util.FP32_TOL * scale, cfg
            else:
                assert err.max() < util.BF16_MAX_TOL * scale and err.mean(1).max() < util.BF16_MEAN_TOL * scale, cfg


def test_trace_run_program_writes_files_and_done_lines():
    folder = util.model_folder("B")
    streams = {"x": util.tokens_for("B", 70, 11), "y": util.tokens_for("B", 45, 12)}
    steps = [
        util.step_line(0, [("x", streams["x"][:40], [0, 39])]),
        util.step_line(1, [("x", streams["x"][40:42], []), ("y", streams["y"][:45], [44])]),   # nothing wanted of x
        util.step_line(2, [("x", streams["x"][42:70], [27])], end=["x", "y"]),
        util.step_line(3, [], end=[]),
    ]
    with tempfile.TemporaryDirectory() as out:
        util.run_trace_program(folder, "float32", steps, util.peak_tokens(steps), out)
        assert sorted(os.listdir(out)) == ["0.f32", "1.f32", "2.f32"]
        got = util.collect(steps, out, util.TINY_B["vocab_size"])
    assert sorted(got) == [("x", 0), ("x", 39), ("x", 69), ("y", 44)]
    util.check_against_plain(got, folder, streams, "float32")


def test_out_of_pages_is_an_error_that_changes_nothing():
    from air_b200.cache.manager import OutOfPages
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    folder = util.model_folder("A")
    engine = Engine.from_folder(folder, EngineConfig(dtype="float32", page_tokens=16, max_tokens=64))
    toks = util.tokens_for("A", 80, 1)
    engine.step([Entry("a", toks[:40], [39])])
    with pytest.raises(OutOfPages):
        engine.step([Entry("a", toks[40:45], [4]), Entry("b", toks[:30], [29])])
    assert engine.cache.length("a") == 40 and "b" not in engine.cache.sequences
    engine.cache.check()
    got = engine.step([Entry("a", toks[40:45], [4])]).cpu().numpy()
    ref = util.plain_logits(folder, toks[:45])
    assert np.abs(got[0] - ref[44]).max() < util.FP32_TOL * max(1, np.abs(ref).max())


# ------------------------------------------------------------------ the widths of a large model
WIDE = dict(util.BASE, num_hidden_layers=2, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
            intermediate_size=18944, vocab_size=2999, max_position_embeddings=1024, rope_theta=1e6,
            rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False)
_wide = {}


def wide_model():
    """Two layers with the layer sizes of the 7-billion-parameter shape that the benchmark runs (hidden 3584,
    28 query heads of 128 in 4 groups, feed-forward 18944) under a small vocabulary that is no multiple of
    anything: the engine's choices at these sizes (tile widths, parts of k, gate and up rows interleaved in
    blocks of 128, 256-row tiles, the decode kernel that starts from the q/k/v product at 7 heads a group) meet
    the plain implementation here and nowhere else."""
    if not _wide:
        from air_b200.engine.engine import write_random_model
        d = tempfile.TemporaryDirectory(prefix="air_b200_wide_")
        write_random_model(d.name, WIDE, 11, "bfloat16")
        util.sharpen_attention(d.name, WIDE)
        rng = np.random.default_rng(77)
        _wide["folder"], _wide["keep"] = d.name, d
        _wide["streams"] = {f"w{i}": rng.integers(0, WIDE["vocab_size"], size=n).tolist()
                            for i, n in enumerate((150, 67, 3, 200))}
    return _wide["folder"], _wide["streams"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("regime", ["whole", "bulk_tail", "portions", "mixed"])
def test_the_layer_sizes_of_the_benchmark_shape(regime, dtype):
    folder, streams = wide_model()
    steps = {"whole": util.trace_whole, "bulk_tail": util.trace_bulk_tail, "portions": util.trace_portions,
             "mixed": lambda s: util.trace_mixed(s, seed=2, live=3)}[regime](streams)
    got, engine = util.replay(folder, dtype, steps, max_tokens=util.peak_tokens(steps), page_tokens=64)
    util.check_against_plain(got, folder, streams, dtype)
    if dtype == "bfloat16":
        block = engine.model.blocks[0]
        assert block.feed_forward.gate_up.gate_up_block == 128 and block.mixer.qkv.tc_ok


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_of_more_than_4096_rows(dtype):
    """A prompt portion longer than the largest step that the fused gate/up product takes (4,096 rows): the
    library's product and the activation kernel over the interleaved rows; then a second portion and single
    tokens on top of that context.  K with room for 5,000 positions."""
    from air_b200.engine.engine import write_random_model
    cfg = dict(util.TINY_K, max_position_embeddings=5120)
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(folder, cfg, 21, "bfloat16")
        util.sharpen_attention(folder, cfg)
        toks = np.random.default_rng(5).integers(0, cfg["vocab_size"], size=4300).tolist()
        want_rows = [0, 1, 63, 64, 2047, 4095, 4096, 4199]
        steps = [util.step_line(0, [("r", toks[:4200], want_rows)]),
                 util.step_line(1, [("r", toks[4200:4290], [0, 89])])]
        steps += [util.step_line(2 + i, [("r", [toks[4290 + i]], [0])], end=["r"] if i == 9 else []) for i in range(10)]
        got, _ = util.replay(folder, dtype, steps, max_tokens=4352, page_tokens=64)
        from plain import qwen2_plain as plain
        pcfg, tensors = plain.read_model(folder)
        ref = plain.forward(pcfg, tensors, toks)
        scale = max(1.0, float(np.abs(ref).max()))
        for (rid, p), row in got.items():
            diff = np.abs(row - ref[p])
            if dtype == "float32":
                assert diff.max() <= util.FP32_TOL * scale, p
            else:
                assert diff.max() <= util.BF16_MAX_TOL * scale and diff.mean() <= util.BF16_MEAN_TOL * scale, p
        assert sorted(p for _, p in got) == want_rows + [4200, 4289] + list(range(4290, 4300))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_three_hundred_requests_decode_in_one_step(dtype):
    """More single tokens in one step than the largest captured graph holds (256): the step's kernels are launched
    one by one."""
    name = "K"
    folder = util.model_folder(name)
    streams = {f"r{i}": util.tokens_for(name, 6 + i % 7, 2000 + i) for i in range(300)}
    ids = list(streams)
    steps, n = [], 0
    for i in range(0, 300, 30):
        steps.append(util.step_line(n, [(r, streams[r][:-2], range(len(streams[r]) - 2)) for r in ids[i:i + 30]]))
        n += 1
    for k in (2, 1):
        steps.append(util.step_line(n, [(r, [streams[r][-k]], [0]) for r in ids], end=ids if k == 1 else []))
        n += 1
    got, engine = util.replay(folder, dtype, steps, max_tokens=util.peak_tokens(steps, page=16), page_tokens=16,
                              max_requests=300)
    util.check_against_plain(got, folder, streams, dtype)
    assert all(size <= 256 for size in engine.graphs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_context_of_eight_thousand_tokens(dtype):
    """A request that grows to 8,200 tokens: its prompt in four portions of about 2,000 tokens (the tile kernels over
    a long prefix, 128 pages behind one block table row), then 40 tokens one by one (the decode kernels, split over
    32 tiles and more).  The logits at the end of every portion and at every decoded token against the plain
    implementation on the whole sequence."""
    from air_b200.engine.engine import write_random_model
    from plain import qwen2_plain as plain
    cfg = dict(util.TINY_K, max_position_embeddings=8448)
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(folder, cfg, 31, "bfloat16")
        util.sharpen_attention(folder, cfg)
        toks = np.random.default_rng(8).integers(0, cfg["vocab_size"], size=8200).tolist()
        cuts = [0, 2048, 4100, 6147, 8160]
        steps = [util.step_line(i, [("r", toks[a:b], [0, b - a - 1])]) for i, (a, b) in enumerate(zip(cuts, cuts[1:]))]
        steps += [util.step_line(4 + i, [("r", [toks[8160 + i]], [0])], end=["r"] if i == 39 else []) for i in range(40)]
        got, _ = util.replay(folder, dtype, steps, max_tokens=8256, page_tokens=64, max_requests=2)
        pcfg, tensors = plain.read_model(folder)
        ref = plain.forward(pcfg, tensors, toks)
        scale = max(1.0, float(np.abs(ref).max()))
        assert len(got) == 8 + 40
        for (rid, p), row in got.items():
            diff = np.abs(row - ref[p])
            if dtype == "float32":
                assert diff.max() <= util.FP32_TOL * scale, p
            else:
                assert diff.max() <= util.BF16_MAX_TOL * scale and diff.mean() <= util.BF16_MEAN_TOL * scale, p


@pytest.mark.parametrize("name", ["K", "L"])
def test_streams_of_keys_whole_and_cut(name, monkeypatch):
    """The tcgen05 attention kernel takes a pair of row tiles with its whole stream of keys per block, or the host
    cuts the streams where whole ones would leave SMs idle (parts/attention.py, plan_segments).  Tiny models always
    fall on the first side; here the second is forced, down to one key tile a block, and both give the plain
    implementation's logits for prompts of more than 256 tokens in portions."""
    import air_b200.parts.attention as attention
    folder = util.model_folder(name)
    streams = {f"{name}{i}": util.tokens_for(name, n, 70 + i) for i, n in enumerate((300, 129, 410, 257))}
    steps = util.trace_portions(streams, sizes=(260, 2, 131, 17, 300))
    for sms, cost, shortest in ((1, 3.5, 4), (1 << 20, 0.0, 1), (attention.SMS, 0.0, 2)):
        monkeypatch.setattr(attention, "SMS", sms)
        monkeypatch.setattr(attention, "SEGMENT_COST", cost)
        monkeypatch.setattr(attention, "MIN_SEGMENT", shortest)
        assert (attention.plan_segments([5, 3], 2) is not None) == (sms > 1)
        got, _ = util.replay(folder, "bfloat16", steps, max_tokens=util.peak_tokens(steps), page_tokens=64)
        util.check_against_plain(got, folder, streams, "bfloat16")
