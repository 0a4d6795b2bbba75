"""y = x W^T for a weight stored [out, in], the layout of the checkpoint and of AIR's
tensors (src/reference/tensor_reader.cpp:369-394), so nothing is transposed at load.

bfloat16 weights, few rows (decoding): this package's tcgen05 kernel (csrc/gemm_tc.cu), which
keeps every SM streaming weights by splitting the k range and hands the partial sums
[parts, rows, out] to the consumer's kernel, or applies SiLU(gate)*up in its epilogue.
bfloat16 weights, many rows (prompts): the library's tensor-core product (cuBLAS through
torch.mm), as AIR's engine calls cuBLAS for its dense products
(src/cuda/cuda_backend.cu:1981-1989, 2037-2043); accumulation is 32-bit.
float32 weights: this package's CUDA-core kernel with fused multiply-adds in a fixed order, no
tensor cores and no reduced-precision mode; a bfloat16 input is widened first.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from .base import PreNormed

SMALL_ROWS = 64      # up to this many rows the tcgen05 kernel is used
SMS = 148


def choose_tile(out_features: int, in_features: int, may_split: bool = True):
    """(tile width, parts of k) for a product with few rows: as many blocks as SMs, whole waves,
    wide tiles and few parts preferred, at least 8 k-steps per part."""
    k_tiles = -(-in_features // 64)
    if out_features >= 256 * SMS:
        return 128, 1        # several waves of tiles: the tail does not matter (measured: 128 before 256)
    best = None
    # (tiles of 128 or 256 rows of W run with the weights as the M side of the instruction, which is what a
    # step of few tokens wants; narrower tiles are for matrices smaller than that)
    for bn in ((256, 128) if out_features >= 128 else (64, 32)):
        for s in range(1, 9 if may_split else 2):
            if s > 1 and k_tiles // s < 8:
                continue
            blocks = -(-out_features // bn) * s
            eff = blocks / (-(-blocks // SMS) * SMS)
            score = eff - 0.02 * s - (0.05 if bn == 32 else 0.0)
            if best is None or score > best[0] + 1e-9:
                best = (score, bn, s)
    return best[1], best[2]


class Linear:
    def __init__(self, weight: torch.Tensor, status: Optional[torch.Tensor] = None, gate_up_block: int = 0):
        assert weight.dim() == 2
        self.weight = weight
        self.status = status
        self.out_features, self.in_features = weight.shape
        self.gate_up_block = gate_up_block       # > 0: rows are blocks of gate rows and up rows in turn
        self.tc_ok = (weight.dtype == torch.bfloat16 and weight.is_cuda and self.in_features % 8 == 0
                      and self.out_features % 4 == 0)
        self.tile = 0
        if self.tc_ok:
            self.tile, self.parts = choose_tile(self.out_features, self.in_features)

    def rows(self, begin: int, end: int) -> "Linear":
        """The product with a band of output rows (a view, nothing is copied)."""
        return Linear(self.weight[begin:end], self.status)

    def small(self, x) -> bool:
        return self.tc_ok and x.dtype == torch.bfloat16 and x.shape[0] <= SMALL_ROWS

    def takes_prenormed(self, rows: int, silu: bool = False) -> bool:
        """Whether this product (partial sums, or with the activation) can apply an RMSNorm's scale per row to
        its accumulators (PreNormed input): only the kernel for few rows does."""
        if not self.tc_ok or rows > SMALL_ROWS:
            return False
        if silu:
            return self.gate_up_block > 0 and ops.small_rows(rows, self.out_features, 2 * self.gate_up_block, ops.EPI_SILU)
        return ops.small_rows(rows, self.out_features, self.tile, ops.EPI_PARTIAL)

    @staticmethod
    def _scaled(x):
        """(rows, keyword arguments of the scale per row) of a plain or a PreNormed input."""
        if isinstance(x, PreNormed):
            return x.x, {"row_ss": x.ss, "eps": x.eps}
        return x, {}

    def partial(self, x) -> torch.Tensor:
        """float32 [parts, rows, out]: partial sums over parts of k, for a consumer that adds them."""
        x, scale = self._scaled(x)
        out = torch.empty((self.parts, x.shape[0], self.out_features), dtype=torch.float32, device=x.device)
        return ops.gemm_tc(x, self.weight, out, self.tile, ops.EPI_PARTIAL, splits=self.parts, status=self.status,
                           **scale)

    def full(self, x) -> torch.Tensor:
        """float32 [rows, out] in one pass of the tcgen05 kernel."""
        x, scale = self._scaled(x)
        bn, _ = choose_tile(self.out_features, self.in_features, may_split=False)
        out = torch.empty((x.shape[0], self.out_features), dtype=torch.float32, device=x.device)
        return ops.gemm_tc(x, self.weight, out, bn, ops.EPI_F32, status=self.status, **scale)

    def silu_mul(self, x) -> torch.Tensor:
        """bfloat16 [rows, out / 2] = silu(gate) * up, in the epilogue of the tcgen05 kernel."""
        x, scale = self._scaled(x)
        out = torch.empty((x.shape[0], self.out_features // 2), dtype=torch.bfloat16, device=x.device)
        return ops.gemm_tc(x, self.weight, out, 2 * self.gate_up_block, ops.EPI_SILU, status=self.status, **scale)

    def adds_into(self, x: torch.Tensor, residual) -> bool:
        """Whether add_into() applies: 16-bit weights, a float32 stream of this product's shape."""
        return (residual is not None and self.weight.dtype != torch.float32 and x.dtype == self.weight.dtype
                and x.is_cuda and residual.dtype == torch.float32
                and tuple(residual.shape) == (x.shape[0], self.out_features))

    def add_into(self, x: torch.Tensor, residual: torch.Tensor) -> None:
        """residual += x W^T, the sum taken in 32-bit in the library product's epilogue (the product is not
        rounded to 16 bits first, and is not written and read again by the norm that follows)."""
        torch.addmm(residual, x, self.weight.t(), out_dtype=torch.float32, out=residual)

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype, bias=None) -> torch.Tensor:
        w = self.weight
        if w.dtype == torch.float32:
            if x.dtype != torch.float32:
                x = ops.convert(x, torch.empty(x.shape, dtype=torch.float32, device=x.device))
            out = torch.empty((x.shape[0], self.out_features), dtype=torch.float32, device=x.device)
            ops.gemm_f32(x, w, bias, out)
            if out_dtype != torch.float32:
                out = ops.convert(out, torch.empty(out.shape, dtype=out_dtype, device=x.device))
            return out
        if x.dtype != w.dtype:
            raise ops.KernelError(f"Linear: input {x.dtype} with weight {w.dtype}")
        if bias is not None:
            raise ops.KernelError("Linear: a bias with 16-bit weights is added by the consumer's kernel")
        if not x.is_cuda:
            raise ops.KernelError("Linear: input must be a CUDA tensor")
        return torch.mm(x, w.t(), out_dtype=out_dtype)
