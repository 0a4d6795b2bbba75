"""The tcgen05 matrix products against a float64 product of the same bfloat16 inputs: every
tile width, every epilogue, sizes with tails in M, N and K, one token to thousands; with few
tokens both kernels (tokens as the M side of the instruction, weights as the M side)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def ops():
    from air_b200.csrc import ops as o
    return o


def inputs(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(M, K, generator=g)).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    return a.cuda(), w.cuda(), a.double() @ w.double().T


def close(got, want, K):
    tol = 2e-6 * K ** 0.5 + 1e-6
    return float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max()) + 1e-5


@pytest.mark.parametrize("bn", [32, 64, 128, 256])
@pytest.mark.parametrize("M,N,K", [(8, 64, 64), (1, 256, 128), (16, 512, 192), (37, 388, 352), (128, 256, 256),
                                   (200, 1000, 1000), (64, 4608, 3584), (600, 1000, 1000), (515, 260, 136),
                                   (17, 520, 328), (33, 300, 72), (64, 132, 4096)])
@pytest.mark.parametrize("rows_as_m", [False, True])
def test_float32_output(bn, M, N, K, rows_as_m):
    o = ops()
    if rows_as_m and not o.small_rows(M, N, bn, o.EPI_F32):
        pytest.skip("one kernel only for this size")
    a, w, want = inputs(M, N, K, M + N)
    out = torch.full((M, N), 9.0, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o.gemm_tc(a, w, out, bn, o.EPI_F32, status=status, force_rows_as_m=rows_as_m)
    assert status.item() == 0
    assert close(out, want, K)


@pytest.mark.parametrize("bn,splits", [(32, 2), (64, 3), (128, 5), (64, 1), (256, 4)])
@pytest.mark.parametrize("M", [8, 40])
@pytest.mark.parametrize("rows_as_m", [False, True])
def test_partial_sums_over_k(bn, splits, M, rows_as_m):
    o = ops()
    N, K = 3584, 18944 // 8
    if rows_as_m and not o.small_rows(M, N, bn, o.EPI_PARTIAL):
        pytest.skip("one kernel only for this size")
    a, w, want = inputs(M, N, K, splits)
    out = torch.zeros(splits, M, N, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o.gemm_tc(a, w, out, bn, o.EPI_PARTIAL, splits=splits, status=status, force_rows_as_m=rows_as_m)
    assert status.item() == 0
    assert close(out.sum(0), want, K)
    if splits > 1:
        assert float(out[1].abs().max()) > 0


@pytest.mark.parametrize("bn", [64, 128, 256])
@pytest.mark.parametrize("M", [3, 20, 64, 130, 700])   # (from 512 rows on, 256-wide tiles take 256 rows)
@pytest.mark.parametrize("rows_as_m", [False, True])
def test_silu_epilogue_with_interleaved_gate_and_up(bn, M, rows_as_m):
    o = ops()
    if rows_as_m and not o.small_rows(M, 6 * bn, bn, o.EPI_SILU):
        pytest.skip("one kernel only for this size")
    I, K = 3 * bn, 320
    g = torch.Generator().manual_seed(bn + M)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    gate = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16)
    up = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16)
    half = bn // 2
    w = torch.cat([torch.cat([gate[i:i + half], up[i:i + half]]) for i in range(0, I, half)])
    out = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
    o.gemm_tc(a.cuda(), w.cuda(), out, bn, o.EPI_SILU, force_rows_as_m=rows_as_m)
    gd, ud = a.double() @ gate.double().T, a.double() @ up.double().T
    want = gd / (1 + torch.exp(-gd)) * ud
    assert float((out.double().cpu() - want).abs().max()) < 1e-2 * float(want.abs().max())


def test_bfloat16_output_and_many_tiles():
    o = ops()
    M, N, K = 2048, 1536, 512
    a, w, want = inputs(M, N, K, 5)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o.gemm_tc(a, w, out, 256, o.EPI_BF16, status=status)
    assert status.item() == 0
    assert float((out.double().cpu() - want).abs().max()) < 1e-2 * float(want.abs().max())
    # fewer blocks than tiles: every block walks several tiles, both accumulators in turn
    out2 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    o.gemm_tc(a, w, out2, 128, o.EPI_BF16, status=status, max_blocks=7)
    assert status.item() == 0 and torch.equal(out2, out)


@pytest.mark.parametrize("M", [5, 48])
def test_bfloat16_output_with_few_tokens(M):
    o = ops()
    N, K = 1000, 520
    a, w, want = inputs(M, N, K, M)
    for bn in (128, 256):
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        o.gemm_tc(a, w, out, bn, o.EPI_BF16, status=status, max_blocks=3)
        assert status.item() == 0
        assert float((out.double().cpu() - want).abs().max()) < 1e-2 * float(want.abs().max())


def test_refusals():
    o = ops()
    a = torch.zeros(4, 36, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(8, 36, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(o.KernelError, match="multiple of 8"):
        o.gemm_tc(a, w, torch.zeros(4, 8, device="cuda"), 32, o.EPI_F32)
    # 16 k-tiles in 5 parts would be 4 + 4 + 4 + 4 + 0: an empty part's accumulator is never written
    a = torch.zeros(8, 1024, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(256, 1024, dtype=torch.bfloat16, device="cuda")
    for bn in (64, 128):            # both kernels
        with pytest.raises(o.KernelError, match="size or dtype"):
            o.gemm_tc(a, w, torch.zeros(5, 8, 256, device="cuda"), bn, o.EPI_PARTIAL, splits=5)


# ------------------------------------------------------------------ an RMSNorm's scale applied by the product
@pytest.mark.parametrize("T", [3, 30, 64])
@pytest.mark.parametrize("epi", ["partial", "f32", "silu"])
def test_scale_per_row_from_sums_of_squares(T, epi):
    """The products for few rows multiply their accumulators by rsqrt(sum of the parts of ss / K + eps) per row:
    with x = h * g as input they give what the product of the RMSNorm of h gives."""
    o = ops()
    N, K, eps, tiles = 1024, 896, 1e-5, 7
    g = torch.Generator().manual_seed(T)
    h = torch.randn(T, K, generator=g) * 3
    gw = 1 + 0.1 * torch.randn(K, generator=g)
    x = (h * gw).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    ss = (h.view(T, tiles, 128) ** 2).sum(-1).T.contiguous()
    scale = torch.rsqrt((h.double() ** 2).mean(-1, keepdim=True) + eps)
    want = (x.double() @ w.double().T) * scale
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    if epi == "partial":
        out = torch.zeros(3, T, N, device="cuda")
        o.gemm_tc(x.cuda(), w.cuda(), out, 128, o.EPI_PARTIAL, splits=3, status=status, row_ss=ss.cuda(), eps=eps)
        got = out.sum(0).double().cpu()
    elif epi == "f32":
        out = torch.zeros(T, N, device="cuda")
        o.gemm_tc(x.cuda(), w.cuda(), out, 256, o.EPI_F32, status=status, row_ss=ss.cuda(), eps=eps)
        got = out.double().cpu()
    else:
        out = torch.zeros(T, N // 2, dtype=torch.bfloat16, device="cuda")
        o.gemm_tc(x.cuda(), w.cuda(), out, 256, o.EPI_SILU, status=status, row_ss=ss.cuda(), eps=eps)
        got = out.double().cpu()
        blocks = want.view(T, N // 256, 2, 128)
        gate, up = blocks[:, :, 0].reshape(T, -1), blocks[:, :, 1].reshape(T, -1)
        want = gate / (1 + torch.exp(-gate)) * up
    assert status.item() == 0
    assert float((got - want).abs().max()) <= (1e-2 if epi == "silu" else 1e-4) * float(want.abs().max())
    with pytest.raises(o.KernelError, match="up to 64 rows"):
        o.gemm_tc(torch.zeros(100, K, dtype=torch.bfloat16, device="cuda"), w.cuda(), torch.zeros(100, N, device="cuda"),
                  256, o.EPI_F32, row_ss=torch.zeros(tiles, 100, device="cuda"), eps=eps)
