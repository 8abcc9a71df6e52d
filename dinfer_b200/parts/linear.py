"""``y = x W^T`` for a weight in the PyTorch ``[out, in]`` layout (crates/layers/src/nn.rs:16-76).

Which product runs follows from the dtypes at hand:
  * float32 activations (the true 32-bit engine): 32-bit multiply-adds on the CUDA cores;
  * bfloat16 activations and weight: the tensor-core path (the library product, where the
    reference's engine uses cuBLASLt: crates/kernels/src/gemm.rs:649-690, or this package's own
    kernels once they are selected for the shape);
  * bfloat16 activations and a weight the file stores in 32-bit: the 32-bit product, the
    activations widened on the fly.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from ..kernels.lib import add_launches


class Linear:
    def __init__(self, weight: torch.Tensor):
        if weight.dim() != 2:
            raise ValueError("a linear weight is 2-D [out, in]")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape

    def kernel_libraries(self):
        return ["gemm_f32"] if self.weight.dtype == torch.float32 else []

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out_dtype = out_dtype or x.dtype
        if out is None:
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype, device=x.device)
        w = self.weight
        if x.dtype == torch.float32 or w.dtype == torch.float32:
            return ops.gemm_f32(x, w, out)
        # bfloat16 x bfloat16, f32 accumulation
        add_launches(1)
        if out.dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
        else:
            torch.mm(x, w.t(), out_dtype=out.dtype, out=out)
        return out
