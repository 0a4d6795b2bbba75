"""y = x W^T for a weight stored [out, in], the layout of the checkpoint and of AIR's
tensors (src/reference/tensor_reader.cpp:369-394), so nothing is transposed at load.

bfloat16 weights: the tensor-core product of the library (cuBLAS through torch.mm), as AIR's
engine calls cuBLAS for its dense products (src/cuda/cuda_backend.cu:1981-1989, 2037-2043);
accumulation is 32-bit and the result may be asked for in float32.
float32 weights: this package's own CUDA-core kernel with fused multiply-adds in a fixed
order, no tensor cores and no reduced-precision mode; a bfloat16 input is widened first.
"""
from __future__ import annotations

import torch

from ..csrc import ops


class Linear:
    def __init__(self, weight: torch.Tensor):
        assert weight.dim() == 2
        self.weight = weight
        self.out_features, self.in_features = weight.shape

    def rows(self, begin: int, end: int) -> "Linear":
        """The product with a band of output rows (a view, nothing is copied)."""
        return Linear(self.weight[begin:end])

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
