"""Each CUDA kernel alone against a plain float32/float64 torch or numpy reference of the same
operation, at sizes other than the engine's (widths and vocabularies that are no power of two,
head sizes in steps of 16, odd numbers of heads and groups)."""
import math

import numpy as np
import pytest
import torch

from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(x, dtype=None):
    t = torch.as_tensor(x)
    return t.to("cuda", dtype=dtype) if dtype is not None else t.to("cuda")


def ops():
    from air_b200.csrc import ops as o
    return o


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_gathers_rows_and_feeds_back_sampled_tokens(dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(1000, 200, generator=g).to(DT[dtype])
    ids = torch.tensor([0, 999, 5, -3, 17, -1], dtype=torch.int32)
    last = torch.tensor([42, 7, 500], dtype=torch.int32)
    out = torch.empty(6, 200, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops().embedding(dev(table), dev(ids), out, status=status, last_token=dev(last))
    want = table[[0, 999, 5, 500, 17, 42]].float()
    assert torch.equal(out.cpu(), want) and status.item() == 0
    ops().embedding(dev(table), dev(torch.tensor([1000], dtype=torch.int32)), out[:1], status=status)
    assert status.item() == 1 and float(out[0].abs().sum()) == 0.0
    ops().embedding(dev(table), dev(ids), out, last_token=dev(last), multiplier=14.25)       # rows times a constant
    assert torch.equal(out.cpu(), want * 14.25)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("parts", [0, 1, 5])
def test_add_parts_adds_every_form_of_delta_in_order(parts, dtype):
    """h += delta for a plain [T, E] delta (parts 0) and for partial sums [parts, T, E], added in order."""
    g = torch.Generator().manual_seed(parts)
    T, E = 37, 203
    h = torch.randn(T, E, generator=g)
    shape = (T, E) if parts == 0 else (parts, T, E)
    delta = (torch.randn(shape, generator=g) * 100).to(DT[dtype])
    got = ops().add_parts(dev(h.clone()), dev(delta)).cpu()
    want = h.clone()
    for part in (delta.float() if parts else delta.float()[None]):
        want = want + part                  # float32 additions in the order of the parts
    assert torch.equal(got, want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,parts", [(1, 3584, 5), (8, 3584, 1), (37, 200, 0), (64, 5120, 9), (3, 1000, 2)])
def test_add_prenorm_gives_the_norm_short_of_its_scale(T, E, parts, dtype):
    """h += delta; xg = bfloat16(h * w); sums of squares per chunk of 512 columns: together with the scale per row
    that follows from the sums they are what add_rmsnorm gives."""
    g = torch.Generator().manual_seed(T + E)
    h = torch.randn(T, E, generator=g)
    w = (1 + 0.1 * torch.randn(E, generator=g)).to(DT[dtype])
    delta = None if parts == 0 else torch.randn((parts, T, E) if parts > 1 else (T, E), generator=g)
    chunks = -(-E // 512)
    hd = dev(h.clone())
    xg = torch.full((T, E), 9.0, dtype=torch.bfloat16, device="cuda")
    ss = torch.full((chunks, T), -1.0, device="cuda")
    ops().add_prenorm(hd, None if delta is None else dev(delta), dev(w), xg, ss)
    want = h.clone()
    if delta is not None:
        for part in (delta if parts > 1 else delta[None]):
            want = want + part
    assert torch.equal(hd.cpu(), want)
    assert float((xg.float().cpu() - want * w.float()).abs().max()) <= 1e-2 * float((want * w.float()).abs().max())
    pad = torch.zeros(T, chunks * 512, dtype=torch.float64)
    pad[:, :E] = want.double()
    want_ss = (pad.view(T, chunks, 512) ** 2).sum(-1).T
    assert float((ss.double().cpu() - want_ss).abs().max()) <= 1e-5 * float(want_ss.abs().max())
    # the scale that a consumer derives is the norm's
    eps = 1e-6
    scale = torch.rsqrt(ss.double().cpu().sum(0) / E + eps)
    normed = torch.empty(T, E, dtype=torch.float32, device="cuda")
    ops().add_rmsnorm(dev(h.clone()), None if delta is None else dev(delta), dev(w), eps, normed)
    assert float((xg.double().cpu() * scale[:, None] - normed.double().cpu()).abs().max()) <= \
        1e-2 * float(normed.abs().max())


def test_logits_post_adds_scales_and_caps():
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(9, 1001, generator=g) * 20
    bias = torch.randn(1001, generator=g)
    got = ops().logits_post(dev(logits.clone()), dev(bias), 0.125, 3.0).cpu().double()
    want = 3.0 * torch.tanh((logits.double() + bias.double()) * 0.125 / 3.0)
    assert float((got - want).abs().max()) < 2e-6 and float(got.abs().max()) <= 3.0
    plain_scale = ops().logits_post(dev(logits.clone()), None, 0.5, 0.0).cpu()
    assert torch.equal(plain_scale, logits * 0.5)


@pytest.mark.parametrize("E", [200, 1000, 3584, 5120, 9000])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("R", [37, 150, 1100])      # (few rows, many, and very many take different kernels)
def test_add_rmsnorm(E, dtype, R):
    g = torch.Generator().manual_seed(E)
    h = torch.randn(R, E, generator=g) * 3
    delta = torch.randn(R, E, generator=g).to(DT[dtype])
    w = (1 + 0.1 * torch.randn(E, generator=g)).to(DT[dtype])
    eps = 1e-5
    x = h + delta.float()
    want = plain.rms_norm(x.numpy(), w.float().numpy(), eps)
    hd = dev(h.clone())
    out = torch.empty(R, E, dtype=DT[dtype], device="cuda")
    ops().add_rmsnorm(hd, dev(delta), dev(w), eps, out)
    assert torch.equal(hd.cpu(), x), "the residual stream is updated in float32"
    tol = 2e-6 if dtype == "float32" else 1e-2
    assert np.abs(out.float().cpu().numpy() - want).max() <= tol * np.abs(want).max()
    # without delta, and on chosen rows only (h stays as it is)
    rows = torch.tensor([36, 0, 5], dtype=torch.int32)
    out2 = torch.empty(3, E, dtype=DT[dtype], device="cuda")
    before = hd.clone()
    ops().add_rmsnorm(hd, None, dev(w), eps, out2, rows=dev(rows))
    assert torch.equal(hd, before)
    # the same bits, whichever kernel the number of rows chose (up to 4,096 wide; beyond, to rounding)
    same = torch.equal if E <= 4096 else (lambda a, b: torch.allclose(a.float(), b.float(), rtol=2e-2 if dtype == "bfloat16" else 1e-5, atol=1e-6))
    assert same(out2.cpu(), out.cpu()[rows.long()])
    out3 = torch.empty(3, E, dtype=DT[dtype], device="cuda")
    ops().add_rmsnorm(dev(h.clone()), dev(delta), dev(w), eps, out3, rows=dev(rows))
    assert same(out3.cpu(), out.cpu()[rows.long()])
    # nothing to add (the stream as the products' epilogues left it): for many rows the kernel that the copy
    # engine feeds, the same bits again
    out5 = torch.full((R, E), 5.0, dtype=DT[dtype], device="cuda")
    ops().add_rmsnorm(hd, None, dev(w), eps, out5)
    assert torch.equal(hd, before) and same(out5.cpu(), out.cpu())
    # partial sums of a split product are added in their order
    three = torch.randn(3, R, E, generator=g)
    h3 = dev(h.clone())
    out4 = torch.empty(R, E, dtype=DT[dtype], device="cuda")
    ops().add_rmsnorm(h3, dev(three), dev(w), eps, out4)
    x3 = ((h + three[0]) + three[1]) + three[2]
    assert torch.equal(h3.cpu(), x3)
    want3 = plain.rms_norm(x3.numpy(), w.float().numpy(), eps)
    assert np.abs(out4.float().cpu().numpy() - want3).max() <= tol * np.abs(want3).max()


@pytest.mark.parametrize("M,N,K", [(1, 130, 75), (37, 130, 75), (64, 64, 16), (65, 257, 1000), (3, 9, 3584)])
def test_gemm_f32_is_true_32_bit_and_rows_do_not_depend_on_the_batch(M, N, K):
    g = torch.Generator().manual_seed(M * N)
    a, w, b = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g), torch.randn(N, generator=g)
    out = torch.empty(M, N, device="cuda")
    ops().gemm_f32(dev(a), dev(w), dev(b), out)
    want = (a.double() @ w.double().T + b.double())
    err = (out.cpu().double() - want).abs().max() / want.abs().max()
    assert err < 5e-7 * math.sqrt(K), "an error of TF32 size (1e-3) would show a reduced-precision mode"
    one = torch.empty(1, N, device="cuda")
    ops().gemm_f32(dev(a[M // 2:M // 2 + 1].contiguous()), dev(w), dev(b), one)
    assert torch.equal(one[0], out[M // 2]), "a row alone gives the same bits as in the batch"
    nobias = torch.empty(M, N, device="cuda")
    ops().gemm_f32(dev(a), dev(w), None, nobias)
    assert torch.allclose(nobias.cpu() + b, out.cpu(), atol=1e-5)


def rope_reference(x, positions, theta, rot):
    """x [T, heads, d]: rotate the first `rot` elements of every head (plain formula)."""
    y = x.copy()
    y[..., :rot] = plain.rope(x[..., :rot], positions, theta)
    return y


@pytest.mark.parametrize("H,K,d,rot", [(5, 1, 48, 48), (6, 3, 80, 80), (4, 2, 128, 64), (3, 3, 16, 16), (28, 4, 128, 128),
                                       (40, 8, 128, 128)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n0,n1", [(14, 9), (70, 40), (700, 400)])       # (few tokens, many and very many take different kernels)
def test_qkv_rope_store(H, K, d, rot, dtype, n0, n1):
    from air_b200.parts.rope import RopeHalf
    from air_b200.parts.spec import PartSpec
    from air_b200.parts.base import Runtime
    P, T, theta = 16, n0 + n1, 12345.0
    rng = np.random.default_rng(d)
    qkv = rng.standard_normal((T, (H + 2 * K) * d)).astype(np.float32)
    bias = rng.standard_normal((H + 2 * K) * d).astype(np.float32)
    # two requests: the first tokens are request 0's at positions 30.., the others request 1's at 0..
    positions = np.array(list(range(30, 30 + n0)) + list(range(n1)), dtype=np.int32)
    token_seq = np.array([0] * n0 + [1] * n1, dtype=np.int32)
    block_table = np.array([[7, 2, 9, 0, 11, 5, 3], [4, 8, 1, -1, -1, -1, -1]], dtype=np.int32)
    pages = 12
    if T > 112:         # more pages than the hand-made table has: shuffled ones
        need = [-(-(30 + n0) // P), -(-n1 // P)]
        pages = sum(need) + 2
        perm = rng.permutation(pages)
        block_table = np.full((2, max(need)), -1, dtype=np.int32)
        block_table[0, :need[0]], block_table[1, :need[1]] = perm[:need[0]], perm[need[0]:sum(need)]
    pe = RopeHalf(PartSpec("rope_half", {"rotary_dim": rot, "theta": theta, "max_positions": 30 + n0 + 8}))
    pe.load({}, Runtime(torch.device("cuda"), DT[dtype], P))
    q_out = torch.zeros(T, H, d, dtype=DT[dtype], device="cuda")
    cache = torch.zeros(pages, 2, K, P, d, dtype=DT[dtype], device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops().qkv_rope_store(dev(qkv), dev(bias), pe.table(), dev(positions), dev(token_seq), dev(block_table),
                         q_out, cache, H, K, d, status=status)
    x = (qkv + bias).reshape(T, H + 2 * K, d)
    q_want = rope_reference(x[:, :H], positions, theta, rot)
    k_want = rope_reference(x[:, H:H + K], positions, theta, rot)
    v_want = x[:, H + K:]
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert np.abs(q_out.float().cpu().numpy() - q_want).max() < tol * np.abs(q_want).max()
    c = cache.float().cpu().numpy()
    touched = np.zeros(c.shape[:1] + c.shape[3:4], dtype=bool)
    for t in range(T):
        page = block_table[token_seq[t], positions[t] // P]
        off = positions[t] % P
        touched[page, off] = True
        assert np.abs(c[page, 0, :, off] - k_want[t]).max() < tol * np.abs(k_want).max()
        assert np.abs(c[page, 1, :, off] - v_want[t]).max() < tol * np.abs(v_want).max()
    untouched = ~touched[:, None, None, :, None]
    assert np.abs(c * untouched).sum() == 0, "no other place of any page is written"
    assert status.item() == 0
    # a run that reads another run's cache writes q only
    cache2 = torch.zeros_like(cache)
    ops().qkv_rope_store(dev(qkv), dev(bias), pe.table(), dev(positions), dev(token_seq), dev(block_table),
                         q_out, cache2, H, K, d, write_kv=False)
    assert float(cache2.abs().sum()) == 0.0


def attention_reference(q, k_all, v_all, positions, seq_of, window):
    """q [T, H, d]; k_all/v_all: per request [len, K, d] (float64 softmax, plain formula)."""
    T, H, d = q.shape
    out = np.zeros_like(q)
    for t in range(T):
        p = positions[t]
        lo = 0 if not window else max(0, p - window + 1)
        k, v = k_all[seq_of[t]][lo:p + 1], v_all[seq_of[t]][lo:p + 1]
        for h in range(H):
            g = h * k.shape[1] // H
            s = (k[:, g].astype(np.float64) @ q[t, h].astype(np.float64)) / math.sqrt(d)
            e = np.exp(s - s.max())
            out[t, h] = ((e / e.sum()).astype(np.float32)[:, None] * v[:, g]).sum(0)
    return out


def paged_case(H, K, d, P, lens, q_lens, dtype, seed, num_pages=40):
    """Requests with `lens` tokens in the cache in shuffled pages; the last q_lens are queries."""
    rng = np.random.default_rng(seed)
    perm = rng.permutation(num_pages)
    cache = np.zeros((num_pages, 2, K, P, d), dtype=np.float32)
    width = max(-(-n // P) for n in lens)
    bt = -np.ones((len(lens), width), dtype=np.int32)
    ks, vs, used = [], [], 0
    for s, n in enumerate(lens):
        k = rng.standard_normal((n, K, d)).astype(np.float32)
        v = rng.standard_normal((n, K, d)).astype(np.float32)
        if dtype == "bfloat16":
            k, v = plain.round_bf16(k), plain.round_bf16(v)
        ks.append(k); vs.append(v)
        for b in range(-(-n // P)):
            bt[s, b] = perm[used]; used += 1
            m = min(P, n - b * P)
            cache[bt[s, b], 0, :, :m] = k[b * P:b * P + m].transpose(1, 0, 2)
            cache[bt[s, b], 1, :, :m] = v[b * P:b * P + m].transpose(1, 0, 2)
    positions = np.concatenate([np.arange(n - ql, n) for n, ql in zip(lens, q_lens)]).astype(np.int32)
    seq_of = np.concatenate([[s] * ql for s, ql in enumerate(q_lens)]).astype(np.int32)
    q = rng.standard_normal((len(positions), H, d)).astype(np.float32)
    if dtype == "bfloat16":
        q = plain.round_bf16(q)
    return q, cache, bt, positions, seq_of, ks, vs


@pytest.mark.parametrize("H,K,d,P", [(6, 2, 48, 16), (7, 1, 80, 32), (4, 4, 128, 64), (2, 1, 256, 16), (3, 3, 16, 16)])
@pytest.mark.parametrize("window", [0, 21])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_paged_attention_ref(H, K, d, P, window, dtype):
    lens, q_lens = [150, 1, 64, 33], [37, 1, 1, 33]
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, lens, q_lens, dtype, seed=d + window)
    out = torch.empty(q.shape, dtype=DT[dtype], device="cuda")
    ops().paged_attention_ref(dev(q, DT[dtype]), dev(cache, DT[dtype]), dev(bt), dev(seq_of), dev(positions), out,
                              window, 1.0 / math.sqrt(d))
    want = attention_reference(q, ks, vs, positions, seq_of, window)
    tol = 2e-6 if dtype == "float32" else 1e-2
    assert np.abs(out.float().cpu().numpy() - want).max() < tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("far", [0, 15, 16, 17, 63, 64, 300, 447])
def test_attention_finds_one_far_key_among_hundreds(far):
    """One key is made to match the query so that its score stands out: the output must be that
    key's value, wherever in the pages the key lies (a page's first or last place, a far page)."""
    H, K, d, P, n = 4, 2, 64, 16, 448
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, [n], [1], "float32", seed=far)
    q[:] = 0
    q[0, :, :] = 0.5
    page, off = bt[0, far // P], far % P
    cache[page, 0, :, off, :] = 40.0          # score 0.5*40*64/8 = 160 against |score| < 20 elsewhere
    ks[0][far] = 40.0
    out = torch.empty(q.shape, device="cuda")
    ops().paged_attention_ref(dev(q), dev(cache), dev(bt), dev(seq_of), dev(positions), out, 0, 1.0 / math.sqrt(d))
    got = out.cpu().numpy()[0]
    for h in range(H):
        assert np.abs(got[h] - vs[0][far, h * K // H]).max() < 1e-4


def test_window_edge_is_exact():
    """With a window of w the key at distance w - 1 counts and the key at distance w does not."""
    H, K, d, P, n, w = 2, 1, 32, 16, 100, 37
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, [n], [1], "float32", seed=1)
    q[:] = 0.5
    for key, visible in ((n - w, True), (n - w - 1, False)):
        c = cache.copy()
        c[bt[0, key // P], 0, :, key % P, :] = 40.0
        out = torch.empty(q.shape, device="cuda")
        ops().paged_attention_ref(dev(q), dev(c), dev(bt), dev(seq_of), dev(positions), out, w, 1.0 / math.sqrt(d))
        hit = np.abs(out.cpu().numpy()[0, 0] - vs[0][key, 0]).max() < 1e-4
        assert hit == visible


@pytest.mark.parametrize("T,I", [(1, 352), (37, 1000), (5, 18944)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul(T, I, dtype):
    g = torch.Generator().manual_seed(I)
    x = (torch.randn(T, 2 * I, generator=g) * 3).to(DT[dtype])
    out = torch.empty(T, I, dtype=DT[dtype], device="cuda")
    ops().silu_mul(dev(x), out)
    xf = x.float().numpy()
    want = plain.silu(xf[:, :I]) * xf[:, I:]
    tol = 2e-6 if dtype == "float32" else 1e-2
    assert np.abs(out.float().cpu().numpy() - want).max() <= tol * np.abs(want).max()


def test_argmax_takes_the_lowest_index_of_the_maximum():
    V = 50001
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(5, V, generator=g)
    logits[0, 40000] = logits[0, 123] = 9.0
    logits[1, V - 1] = 11.0
    logits[2, 0] = 11.0
    logits[3] = -3.0                      # all equal: index 0
    out = torch.empty(5, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    slots = torch.tensor([2, 0, 1, 4, 3], dtype=torch.int32, device="cuda")
    last = torch.zeros(6, dtype=torch.int32, device="cuda")
    ops().sample(dev(logits), None, None, out, status=status, slots=slots, last_token=last)
    assert out.tolist() == [123, V - 1, 0, 0, int(logits[4].argmax())] and status.item() == 0
    assert last.tolist() == [V - 1, 0, 123, out[4].item(), 0, 0]
    logits[4, 77] = float("nan")
    ops().sample(dev(logits), None, None, out, status=status)
    assert status.item() == 3


def test_temperature_sampling_follows_the_distribution_and_the_uniform_number():
    V, R = 1003, 4000
    g = torch.Generator().manual_seed(1)
    row = torch.randn(V, generator=g) * 2
    temp = 0.7
    p = torch.softmax(row.double() / temp, 0)
    cdf = torch.cumsum(p, 0)
    u = torch.rand(R, generator=g)
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops().sample(dev(row.repeat(R, 1)), dev(torch.full((R,), temp)), dev(u), out)
    got = out.cpu().long()
    want = torch.searchsorted(cdf, u.double()).clamp(max=V - 1)
    # the walk is in index order: the drawn index is where the cumulative sum passes u (up to rounding)
    near = (got - want).abs() <= 1
    assert near.float().mean() > 0.995
    agree = (got == want).float().mean()
    assert agree > 0.97
    # rows with temperature 0 among them are greedy
    t = torch.tensor([0.0, 0.7, 0.0])
    out3 = torch.empty(3, dtype=torch.int32, device="cuda")
    ops().sample(dev(row.repeat(3, 1)), dev(t), dev(torch.tensor([0.3, 0.999999, 0.5])), out3)
    assert out3[0].item() == out3[2].item() == int(row.argmax())


def kept_like_the_host_sampler(row, temp, k, p):
    """The indices that AIR's sampler keeps, in its order (src/runtime/sampling.cpp:23-53): weights
    exp((x - max) / T), a stable descending sort, the k largest (0: all), then the shortest prefix whose
    weights reach p of the remaining total (at least one)."""
    w = np.exp((row.astype(np.float64) - row.max()) / temp)
    order = np.argsort(-w, kind="stable")
    if k and k < order.size:
        order = order[:k]
    if p < 1.0:
        total, cum, keep = w[order].sum(), 0.0, 0
        for i in order:
            cum += w[i]
            keep += 1
            if cum >= p * total:
                break
        order = order[:keep]
    return order, w


@pytest.mark.parametrize("V,R", [(1500, 3000), (50257, 400), (152064, 200), (33, 500)])
@pytest.mark.parametrize("k,p", [(0, 0.8), (7, 1.0), (50, 0.6), (3, 0.999), (1, 0.5), (0, 0.05), (2000, 0.9), (3000, 0.97)])
def test_top_k_and_top_p_on_the_device_keep_what_the_host_sampler_keeps(k, p, V, R):
    """Draws with many uniform numbers: every drawn index is one that AIR's sampler keeps, every kept index
    is drawn, and the index is where the cumulative weight of the kept indices passes the uniform number:
    in AIR's descending order where the kernel cuts among its candidates in shared memory (k of up to 2,048
    is always so), in index order where it cuts over the whole row (k above that; a share that the 1,024 to
    2,048 largest do not reach).  The logits have ties at the cut's value, which a stable sort keeps in
    index order."""
    temp = 0.8
    g = torch.Generator().manual_seed(k * 10 + int(p * 100) + V)
    row = (torch.randn(V, generator=g) * 2).round(decimals=1)          # one decimal: many exact ties
    order, w = kept_like_the_host_sampler(row.numpy(), temp, k, p)
    kept = np.sort(order)
    u = torch.rand(R, generator=g)
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops().sample(dev(row.repeat(R, 1)), dev(torch.full((R,), temp)), dev(u), out,
                 top_k=dev(torch.full((R,), k, dtype=torch.int32)), top_p=dev(torch.full((R,), p)))
    got = out.cpu().numpy()
    assert set(got.tolist()) <= set(kept.tolist()), "an index outside the kept set was drawn"
    if len(kept) * 50 <= R:
        assert set(got.tolist()) == set(kept.tolist()), "a kept index was never drawn"

    def walk(indices):
        cdf = np.cumsum(w[indices]) / w[indices].sum()
        return (got == indices[np.minimum(np.searchsorted(cdf, u.double().numpy()), len(indices) - 1)]).mean()
    as_air, by_index = walk(order), walk(kept)
    if 0 < k < V and k <= 100:                   # (with ties at the 2,000th there are too many candidates)
        assert as_air > 0.97
    elif k > 2048 and k < V:
        assert by_index > 0.97
    else:
        assert max(as_air, by_index) > 0.97


def test_many_equal_logits_are_cut_in_index_order():
    """More ties at the cut's value than the kernel's candidates hold: the whole-row path keeps the first k of
    them in index order, as a stable sort does."""
    V, R, k = 20000, 400, 5
    row = torch.zeros(V)
    row[7], row[11000] = 1.0, 1.0
    kept = [7, 11000, 0, 1, 2]
    u = torch.rand(R, generator=torch.Generator().manual_seed(3))
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops().sample(dev(row.repeat(R, 1)), dev(torch.full((R,), 1.0)), dev(u), out,
                 top_k=dev(torch.full((R,), k, dtype=torch.int32)), top_p=dev(torch.full((R,), 0.99)))
    assert set(out.cpu().tolist()) == set(kept)


def test_kernels_refuse_what_they_cannot_take():
    o = ops()
    q = torch.zeros(2, 2, 24, device="cuda")
    with pytest.raises(o.KernelError, match="multiples of 16"):
        o.paged_attention_ref(q, torch.zeros(1, 2, 1, 16, 24, device="cuda"), torch.zeros(1, 1, dtype=torch.int32, device="cuda"),
                              torch.zeros(2, dtype=torch.int32, device="cuda"), torch.zeros(2, dtype=torch.int32, device="cuda"),
                              torch.empty_like(q), 0, 1.0)
    with pytest.raises(o.KernelError, match="CUDA tensor"):
        o.silu_mul(torch.zeros(2, 8), torch.zeros(2, 4))
    with pytest.raises(o.KernelError, match="shape"):
        o.gemm_f32(torch.zeros(2, 8, device="cuda"), torch.zeros(3, 9, device="cuda"), None, torch.zeros(2, 3, device="cuda"))
    # pages of 80 tokens: a tile of 64 keys would straddle two pages, the copy-engine kernels refuse them
    qb = torch.zeros(16, 2, 128, dtype=torch.bfloat16, device="cuda")
    cb = torch.zeros(4, 2, 1, 80, 128, dtype=torch.bfloat16, device="cuda")
    tiles = torch.zeros(16, 4, dtype=torch.int32, device="cuda")
    table = torch.zeros(1, 4, dtype=torch.int32, device="cuda")
    for kernel in (o.prefill_attention, o.prefill_attention_tc):
        with pytest.raises(o.KernelError, match="neither a divisor nor a multiple of 64"):
            kernel(qb, cb, table, tiles, torch.empty_like(qb), 0, 1.0)
    assert o.tile_pages(16) and o.tile_pages(64) and o.tile_pages(192) and not o.tile_pages(48) and not o.tile_pages(96)


@pytest.mark.parametrize("H,K,d,P", [(28, 4, 128, 64), (6, 2, 64, 16), (4, 4, 128, 16), (40, 2, 64, 32), (8, 1, 256, 16)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("engine", ["tma", "ldg"])
def test_decode_attention(H, K, d, P, window, splits, engine):
    """One query per request, groups of 1 to 20 query heads per kv head, contexts from one key
    to several pages, any number of splits (also more splits than tiles)."""
    lens = [700, 1, 16, 17, 333, 64]
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, lens, [1] * len(lens), "bfloat16", seed=H + splits,
                                                         num_pages=80)
    # a padded token in the middle is skipped
    q = np.insert(q, 2, 0, axis=0)
    positions = np.insert(positions, 2, 0).astype(np.int32)
    seq_of = np.insert(seq_of, 2, -1).astype(np.int32)
    out = torch.full(q.shape, 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops().decode_attention(dev(q, torch.bfloat16), dev(cache, torch.bfloat16), dev(bt), dev(seq_of), dev(positions), out,
                           window, 1.0 / math.sqrt(d), splits=splits, status=status, engine=engine)
    assert status.item() == 0
    keep = seq_of >= 0
    want = attention_reference(q[keep], ks, vs, positions[keep], seq_of[keep], window)
    got = out.float().cpu().numpy()
    assert np.abs(got[keep] - want).max() < 1e-2 * max(1.0, np.abs(want).max())
    assert (got[~keep] == 7.0).all()


@pytest.mark.parametrize("H,K,d,P", [(28, 4, 128, 64), (6, 2, 64, 16), (40, 2, 64, 32), (8, 1, 256, 16), (4, 4, 128, 128)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_decode_attention_from_the_product(H, K, d, P, window, splits):
    """The decode kernel that takes the q/k/v product's partial sums (adds them and the bias, rotates, writes the
    new keys and values, attends) against the two kernels that do the same one after the other; the place of
    the new key in the cache holds other numbers beforehand, so a kernel that attended to what the copy
    engine brought would show.  Contexts that end at a tile's first and last row and in the middle of a page."""
    from air_b200.parts.rope import RopeHalf
    from air_b200.parts.spec import PartSpec
    from air_b200.parts.base import Runtime
    lens = [700, 1, 64, 65, 333, 128, 17]
    _, cache, bt, positions, seq_of, _, _ = paged_case(H, K, d, P, lens, [1] * len(lens), "bfloat16", seed=H + splits,
                                                       num_pages=120)
    positions = np.insert(positions, 2, 0).astype(np.int32)        # a padded token in the middle is skipped
    seq_of = np.insert(seq_of, 2, -1).astype(np.int32)
    T, width = len(positions), (H + 2 * K) * d
    g = torch.Generator().manual_seed(d + window)
    qkv = (torch.randn(3, T, width, generator=g) * 0.6).cuda()
    bias = torch.randn(width, generator=g).cuda()
    pe = RopeHalf(PartSpec("rope_half", {"rotary_dim": d, "theta": 10000.0, "max_positions": 1024}))
    pe.load({}, Runtime(torch.device("cuda"), torch.bfloat16, P))
    o = ops()
    args = (dev(bt), dev(seq_of), dev(positions))
    scale = 1.0 / math.sqrt(d)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # one after the other
    cache_two = dev(cache, torch.bfloat16)
    q = torch.zeros(T, H, d, dtype=torch.bfloat16, device="cuda")
    o.qkv_rope_store(qkv, bias, pe.table(), args[2], args[1], args[0], q, cache_two, H, K, d, status=status)
    want = torch.full((T, H, d), 7.0, dtype=torch.bfloat16, device="cuda")
    o.decode_attention(q, cache_two, *args, want, window, scale, splits=splits, status=status)
    # in one
    cache_one = dev(cache, torch.bfloat16)
    got = torch.full((T, H, d), 7.0, dtype=torch.bfloat16, device="cuda")
    o.decode_attention_fresh(qkv, bias, pe.table(), cache_one, *args, got, H, window, scale, splits=splits, status=status)
    assert status.item() == 0
    assert float((cache_one.float() - cache_two.float()).abs().max()) <= 1e-2 * float(cache_two.float().abs().max())
    assert not torch.equal(cache_one, dev(cache, torch.bfloat16))
    assert float((got.float() - want.float()).abs().max()) <= 2e-2 * max(1.0, float(want.float().abs().max()))
    assert (got[2] == 7.0).all()
    # a run that reads another run's cache: nothing is written, the keys are the ones that lie there
    cache_read = cache_two.clone()
    got2 = torch.empty((T, H, d), dtype=torch.bfloat16, device="cuda")
    o.decode_attention_fresh(qkv, bias, pe.table(), cache_read, *args, got2, H, window, scale, write_kv=False,
                             splits=splits, status=status)
    assert torch.equal(cache_read, cache_two)
    keep = torch.from_numpy(seq_of >= 0).cuda()
    assert float((got2.float() - want.float())[keep].abs().max()) <= 2e-2 * max(1.0, float(want.float().abs().max()))


@pytest.mark.parametrize("far,n", [(0, 2048), (15, 2048), (16, 2048), (63, 2048), (64, 2048), (1000, 2048), (2047, 2048),
                                   (0, 32768), (20001, 32768), (32767, 32768)])
def test_decode_attention_finds_one_far_key(far, n):
    """One key among thousands (up to the 32,768 positions of a long context, 512 pages) stands out: the output is
    its value, wherever it lies."""
    H, K, d, P = 14, 2, 128, 64
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, [n], [1], "bfloat16", seed=far, num_pages=n // P + 8)
    q[:] = 0.5
    cache[bt[0, far // P], 0, :, far % P, :] = 8.0       # score 0.5*8*128/sqrt(128) = 45 against |score| < 6
    out = torch.empty(q.shape, dtype=torch.bfloat16, device="cuda")
    ops().decode_attention(dev(q, torch.bfloat16), dev(cache, torch.bfloat16), dev(bt), dev(seq_of), dev(positions), out,
                           0, 1.0 / math.sqrt(d))
    got = out.float().cpu().numpy()[0]
    for h in range(H):
        assert np.abs(got[h] - vs[0][far, h * K // H]).max() < 2e-2


def tiles_for(lens, q_lens):
    tiles, tok = [], 0
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        for i in range(0, ql, 16):
            tiles.append([s, tok + i, n - ql + i, min(16, ql - i)])
        while len(tiles) % 16:
            tiles.append([s, 0, 0, 0])          # groups of 16 tiles per request
        tok += ql
    return np.array(tiles, dtype=np.int32)


@pytest.mark.parametrize("H,K,d,P", [(28, 4, 128, 64), (6, 2, 64, 16), (3, 3, 128, 16), (20, 2, 64, 32), (4, 1, 256, 16),
                                     (8, 4, 128, 128), (24, 2, 64, 64)])
@pytest.mark.parametrize("window", [0, 21, 100])
def test_prefill_attention(H, K, d, P, window):
    """Portions of 1 to 150 tokens at any offset in their requests, groups of 1 to 10 heads."""
    lens, q_lens = [150, 1, 64, 33, 333, 200], [150, 1, 1, 33, 18, 77]
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, lens, q_lens, "bfloat16", seed=H + window,
                                                         num_pages=90)
    out = torch.full(q.shape, 7.0, dtype=torch.bfloat16, device="cuda")
    ops().prefill_attention(dev(q, torch.bfloat16), dev(cache, torch.bfloat16), dev(bt), dev(tiles_for(lens, q_lens)),
                            out, window, 1.0 / math.sqrt(d))
    want = attention_reference(q, ks, vs, positions, seq_of, window)
    assert np.abs(out.float().cpu().numpy() - want).max() < 1e-2 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("far", [0, 15, 16, 63, 64, 500, 1023])
def test_prefill_attention_finds_one_far_key(far):
    H, K, d, P, n = 8, 2, 128, 64, 1040
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, [n], [16], "bfloat16", seed=far, num_pages=20)
    q[:] = 0.5
    cache[bt[0, far // P], 0, :, far % P, :] = 8.0
    out = torch.empty(q.shape, dtype=torch.bfloat16, device="cuda")
    ops().prefill_attention(dev(q, torch.bfloat16), dev(cache, torch.bfloat16), dev(bt), dev(tiles_for([n], [16])), out,
                            0, 1.0 / math.sqrt(d))
    got = out.float().cpu().numpy()
    for t in range(16):
        for h in range(H):
            assert np.abs(got[t, h] - vs[0][far, h * K // H]).max() < 2e-2


@pytest.mark.parametrize("T,I,block", [(3, 352, 32), (37, 1024, 128), (5, 208, 208), (9, 120, 24), (2, 18944, 128)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul_with_gate_and_up_in_blocks(T, I, block, dtype):
    g = torch.Generator().manual_seed(I + block)
    gate = (torch.randn(T, I, generator=g) * 3).to(DT[dtype])
    up = (torch.randn(T, I, generator=g) * 3).to(DT[dtype])
    x = torch.stack([gate.view(T, I // block, block), up.view(T, I // block, block)], dim=2).reshape(T, 2 * I)
    out = torch.empty(T, I, dtype=DT[dtype], device="cuda")
    ops().silu_mul(dev(x.contiguous()), out, block=block)
    want = plain.silu(gate.float().numpy()) * up.float().numpy()
    tol = 2e-6 if dtype == "float32" else 1e-2
    assert np.abs(out.float().cpu().numpy() - want).max() <= tol * np.abs(want).max()


@pytest.mark.parametrize("H,K,d,P", [(28, 4, 128, 64), (6, 2, 64, 16), (3, 3, 128, 16), (20, 2, 64, 32), (8, 4, 128, 128)])
@pytest.mark.parametrize("window", [0, 21, 100])
def test_prefill_attention_tc(H, K, d, P, window):
    """The tcgen05 attention: portions of 1 to 150 tokens at any offset in their requests."""
    lens, q_lens = [150, 1, 64, 33, 333, 200], [150, 1, 1, 33, 18, 77]
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, lens, q_lens, "bfloat16", seed=H + window,
                                                         num_pages=90)
    out = torch.full(q.shape, 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops().prefill_attention_tc(dev(q, torch.bfloat16), dev(cache, torch.bfloat16), dev(bt), dev(tiles_for(lens, q_lens)),
                               out, window, 1.0 / math.sqrt(d), status=status)
    assert status.item() == 0
    want = attention_reference(q, ks, vs, positions, seq_of, window)
    assert np.abs(out.float().cpu().numpy() - want).max() < 1e-2 * max(1.0, np.abs(want).max())


def streams_of(tiles, window):
    """Key tiles in the stream of every pair of a tile list (as the kernel counts them)."""
    out = []
    for p in range(len(tiles) // 16):
        grp = tiles[16 * p: 16 * p + 16]
        pos0, rows = int(grp[0, 2]), int(grp[:, 3].sum())
        lowest = max(0, pos0 - window + 1) if window else 0
        out.append((pos0 + rows - 1) // 64 + 1 - lowest // 64)
    return out


def pieces_of(streams, heads, piece, whole_every=3):
    """A hand-made list of segments: every (pair, head) cut into pieces of `piece` key tiles, except every third
    item, which stays whole (slot -1).  The last piece says `to the end`; the order is scrambled."""
    segments, items, slot = [], [], 0
    for p, n in enumerate(streams):
        for h in range(heads):
            if (p * heads + h) % whole_every == 0 or n <= piece:
                segments.append([p, h, 0, 1 << 30, -1])
                continue
            starts = list(range(0, n, piece))
            items.append([p, h, slot, len(starts)])
            for j, first in enumerate(starts):
                segments.append([p, h, first, piece if j + 1 < len(starts) else 1 << 30, slot])
                slot += 1
    order = np.random.default_rng(len(segments)).permutation(len(segments))
    return (np.array(segments, dtype=np.int32)[order], np.array(items, dtype=np.int32).reshape(-1, 4), slot)


@pytest.mark.parametrize("H,K,d,P", [(28, 4, 128, 64), (6, 2, 64, 16), (3, 3, 128, 16), (20, 2, 64, 32), (8, 4, 128, 128)])
@pytest.mark.parametrize("window", [0, 21, 100])
@pytest.mark.parametrize("piece", [1, 3])
def test_prefill_attention_tc_in_segments(H, K, d, P, window, piece):
    """The same portions with the streams of keys cut into pieces of one and of three key tiles, each piece a block
    of its own that writes partial sums, merged by the second kernel; some items stay whole.  Pieces fall before a
    window's start and behind the causal edge of the pair's first row tile (a row tile with no key in its piece)."""
    lens, q_lens = [150, 1, 64, 33, 333, 200, 700], [150, 1, 1, 33, 18, 77, 260]
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, lens, q_lens, "bfloat16", seed=H + window,
                                                         num_pages=120)
    tiles = tiles_for(lens, q_lens)
    segments, items, slots = pieces_of(streams_of(tiles, window), H, piece)
    assert slots > 0
    out = torch.full(q.shape, 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops().prefill_attention_tc(dev(q, torch.bfloat16), dev(cache, torch.bfloat16), dev(bt), dev(tiles), out, window,
                               1.0 / math.sqrt(d), status=status, segments=dev(segments), items=dev(items), slots=slots)
    assert status.item() == 0
    want = attention_reference(q, ks, vs, positions, seq_of, window)
    assert np.abs(out.float().cpu().numpy() - want).max() < 1e-2 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("lens,q_lens,H", [([6000], [80], 6), ([3000, 5000], [300, 130], 10), ([40000], [130], 4)])
def test_prefill_attention_tc_with_the_planner_s_segments(lens, q_lens, H):
    """Short portions on top of long prefixes: the planner cuts the streams (asserted), the result is the plain one."""
    from air_b200.parts.attention import plan_segments
    K, d, P = 2, 128, 64
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, lens, q_lens, "bfloat16", seed=H,
                                                         num_pages=sum(-(-n // P) for n in lens) + 2)
    tiles = tiles_for(lens, q_lens)
    planned = plan_segments(streams_of(tiles, 0), H)
    assert planned is not None, "the planner is expected to cut these streams"
    segments, items, slots = planned
    assert slots > 0 and len(segments) > len(tiles) // 16 * H
    out = torch.full(q.shape, 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops().prefill_attention_tc(dev(q, torch.bfloat16), dev(cache, torch.bfloat16), dev(bt), dev(tiles), out, 0,
                               1.0 / math.sqrt(d), status=status, segments=dev(segments), items=dev(items), slots=slots)
    assert status.item() == 0
    want = attention_reference(q, ks, vs, positions, seq_of, 0)
    assert np.abs(out.float().cpu().numpy() - want).max() < 1e-2 * max(1.0, np.abs(want).max())


def test_prefill_attention_tc_reports_a_segment_that_names_no_pair():
    H, K, d, P = 4, 2, 64, 64
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, [100], [100], "bfloat16", seed=3, num_pages=4)
    segments = np.array([[0, h, 0, 1 << 30, -1] for h in range(H)] + [[1, 0, 0, 4, -1]], dtype=np.int32)
    out = torch.zeros(q.shape, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops().prefill_attention_tc(dev(q, torch.bfloat16), dev(cache, torch.bfloat16), dev(bt), dev(tiles_for([100], [100])),
                               out, 0, 1.0 / math.sqrt(d), status=status, segments=dev(segments))
    assert status.item() == 8


def test_prefill_attention_tc_reports_a_list_that_is_not_in_pairs():
    """Two requests with one group of 8 tiles each, one after the other: the second group does not go on
    where the first ends, so the kernel flags status 8 instead of mixing the requests."""
    H, K, d, P = 4, 2, 64, 64
    lens, q_lens = [100, 90], [100, 90]
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, lens, q_lens, "bfloat16", seed=3, num_pages=8)
    tiles, tok = [], 0
    for s_, n in enumerate(q_lens):
        for i in range(0, n, 16):
            tiles.append([s_, tok + i, i, min(16, n - i)])
        while len(tiles) % 8:
            tiles.append([s_, 0, 0, 0])
        tok += n
    assert len(tiles) == 16
    out = torch.zeros(q.shape, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops().prefill_attention_tc(dev(q, torch.bfloat16), dev(cache, torch.bfloat16), dev(bt),
                               dev(np.array(tiles, dtype=np.int32)), out, 0, 1.0 / math.sqrt(d), status=status)
    assert status.item() == 8


@pytest.mark.parametrize("kernel", ["decode", "decode_ldg", "fresh", "prefill", "prefill_tc"])
@pytest.mark.parametrize("n,w", [(300, 37), (300, 64), (257, 129), (200, 200), (70, 1), (129, 2)])
@pytest.mark.parametrize("P,holes", [(64, False), (16, True), (32, True)])
def test_window_edge_is_exact_in_the_tensor_core_kernels(kernel, n, w, P, holes):
    """The key at distance w - 1 from the last query counts, the key at distance w does not: one of them
    at a time is made to stand out, and the last token's output either is its value or is not.  The
    window's edge falls inside a tile of keys, on a tile's first key and on a page's first key.  With
    `holes` the table has -1 where the cache manager has taken pages back: below the first block that the
    query can see.  Every kernel that generation runs is here: the decode kernel fed by the copy engine and
    the one whose warps load the keys themselves, the decode kernel that starts from the q/k/v product, and
    the two tile kernels."""
    H, K, d = 4, 2, 128 if kernel != "prefill" else 256
    q_len = 1 if kernel in ("decode", "decode_ldg", "fresh") else 40
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, [n], [q_len], "bfloat16", seed=n + w,
                                                         num_pages=-(-n // P) + 3)
    q[:] = 0.5
    last = n - 1
    if holes:       # what the manager gives back: blocks that no query of this step can see
        first_query = n - q_len
        bt[0, : max(0, first_query - w + 1) // P] = -1
    scale = 1.0 / math.sqrt(d)
    for key, visible in ((last - w + 1, True), (last - w, False)):
        if key < 0 or bt[0, key // P] < 0:
            continue
        c = cache.copy()
        c[bt[0, key // P], 0, :, key % P, :] = 8.0
        out = torch.empty(q.shape, dtype=torch.bfloat16, device="cuda")
        args = (dev(q, torch.bfloat16), dev(c, torch.bfloat16), dev(bt))
        if kernel in ("decode", "decode_ldg"):
            ops().decode_attention(*args, dev(seq_of), dev(positions), out, w, scale,
                                   engine="tma" if kernel == "decode" else "ldg")
        elif kernel == "fresh":
            # the product's output: q, and the last token's own key and value, which the kernel writes itself;
            # a table that rotates by nothing, so that q and the keys stay what they are
            own_k = np.full((K, d), 8.0, dtype=np.float32) if key == last else ks[0][last]
            qkv = np.concatenate([q[0].reshape(-1), own_k.reshape(-1), vs[0][last].reshape(-1)])[None, :]
            table = np.concatenate([np.ones((n, d // 2)), np.zeros((n, d // 2))], axis=1)     # cos | sin
            c[bt[0, last // P], :, :, last % P, :] = -3.0          # what lies at the new token's place beforehand
            ops().decode_attention_fresh(dev(qkv.astype(np.float32)), None, dev(table.astype(np.float32)),
                                         dev(c, torch.bfloat16), dev(bt), dev(seq_of), dev(positions), out, H, w, scale)
        elif kernel == "prefill":
            ops().prefill_attention(*args, dev(tiles_for([n], [q_len])), out, w, scale)
        else:
            ops().prefill_attention_tc(*args, dev(tiles_for([n], [q_len])), out, w, scale)
        hit = np.abs(out.float().cpu().numpy()[-1, 0] - vs[0][key, 0]).max() < 3e-2
        assert hit == visible, (key, visible)


@pytest.mark.parametrize("far,n", [(0, 1040), (15, 1040), (63, 1040), (64, 1040), (500, 1040), (1023, 1040), (3, 16400),
                                   (16383, 16400)])
@pytest.mark.parametrize("cut", [False, True])
def test_prefill_attention_tc_finds_one_far_key(far, n, cut):
    """One key among thousands stands out; with `cut` the stream is cut into pieces of four key tiles (the key
    lies in one of many pieces, and the merge has to give that piece all the weight)."""
    H, K, d, P = 8, 2, 128, 64
    q, cache, bt, positions, seq_of, ks, vs = paged_case(H, K, d, P, [n], [16], "bfloat16", seed=far, num_pages=n // P + 4)
    q[:] = 0.5
    cache[bt[0, far // P], 0, :, far % P, :] = 8.0
    out = torch.empty(q.shape, dtype=torch.bfloat16, device="cuda")
    more = {}
    if cut:
        segments, items, slots = pieces_of(streams_of(tiles_for([n], [16]), 0), H, 4, whole_every=1 << 30)
        assert slots > 0
        more = dict(segments=dev(segments), items=dev(items), slots=slots)
    ops().prefill_attention_tc(dev(q, torch.bfloat16), dev(cache, torch.bfloat16), dev(bt), dev(tiles_for([n], [16])),
                               out, 0, 1.0 / math.sqrt(d), **more)
    got = out.float().cpu().numpy()
    for t in range(16):
        for h in range(H):
            assert np.abs(got[t, h] - vs[0][far, h * K // H]).max() < 2e-2
