"""``y = x W^T`` for a weight in the PyTorch ``[out, in]`` layout (crates/layers/src/nn.rs:16-76).

Which product runs follows from the dtypes and the number of rows at hand:
  * float32 activations (the true 32-bit engine): 32-bit multiply-adds on the CUDA cores;
  * bfloat16 activations and a weight the file stores in 32-bit: the same 32-bit product, the
    activations widened on the fly;
  * bfloat16 activations and weight, up to ``TC_MAX_DECODE_TOKENS`` rows (decode steps): this
    package's tcgen05 / TMA kernel with the operands swapped, so that the weight is streamed from
    memory exactly once (where the reference uses its own small-M kernels,
    crates/kernels/cuda/gemm_small_m.cu:148-285);
  * bfloat16 with more rows (prompts): the library product, where the reference's engine uses
    cuBLASLt (crates/kernels/src/gemm.rs:649-690), or the tcgen05 kernel when ``PROMPT_BACKEND`` says so;
    the gated pair product of the feed-forward is this package's two-SM tcgen05 kernel from
    ``TC_MIN_GATED_PROMPT_TOKENS`` rows on, with silu(gate) * up in its epilogue.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import gemm_ops, ops
from ..kernels.lib import add_launches
from .base import HalfNormed

# rows up to which a bfloat16 product takes the swapped-operand tcgen05 kernel
TC_MAX_DECODE_TOKENS = 32
# "library" or "tc": who multiplies prompts (more rows than the decode threshold)
PROMPT_BACKEND = "library"
# rows from which the gated pair product runs on the two-SM tcgen05 kernel with the gate in its epilogue; between
# the two thresholds the library product followed by the gate kernel is faster (measured at the 0.6B, 8B and 32B
# shapes: 38.7 against 42.7 us at 33 rows, 43.4 against 55.4 at 128, even at 512, 280 against 300 at 2048)
TC_MIN_GATED_PROMPT_TOKENS = 512


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        """``bias`` [out] is added behind the product by a kernel of its own (the Qwen3 dense model has none; with
        one, the fused epilogues (gate, norm halves) step aside for the plain product)."""
        if weight.dim() != 2:
            raise ValueError("a linear weight is 2-D [out, in]")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        if bias is not None and tuple(bias.shape) != (self.out_features,):
            raise ValueError(f"a bias of {tuple(bias.shape)} does not fit {self.out_features} outputs")
        self.bias = None if bias is None else bias.contiguous()

    def kernel_libraries(self):
        return (["gemm_f32"] if self.weight.dtype == torch.float32 else ["gemm_tc"]) + (["elementwise"] if self.bias is not None else [])

    def fuses_gate(self, x: torch.Tensor) -> bool:
        """Whether ``gated_pairs`` runs as one kernel for these rows: the tcgen05 product with the gate in its
        epilogue, for decode steps and for prompt portions that are long enough."""
        rows = x.shape[0]
        return (self.bias is None and x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16
                and (rows <= TC_MAX_DECODE_TOKENS or rows >= TC_MIN_GATED_PROMPT_TOKENS)
                and self.out_features % 2 == 0 and gemm_ops.supported(x, self.weight))

    def fuses_norm(self, rows: int, act_dtype: torch.dtype) -> bool:
        """Whether this product can take one half of an RMSNorm for ``rows`` rows (the decode product with its
        residual or row-scale epilogue): bfloat16 throughout and rows that TMA can address."""
        w = self.weight
        return (self.bias is None and act_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < rows <= TC_MAX_DECODE_TOKENS
                and self.in_features % 8 == 0 and self.out_features % 8 == 0 and w.data_ptr() % 16 == 0)

    def gated_pairs(self, x) -> torch.Tensor:
        """For a weight whose rows are (gate, up) pairs: ``silu(x gate_j^T) * (x up_j^T)``, [rows, out/2].
        One kernel where ``fuses_gate``, else the product followed by the gate kernel."""
        if isinstance(x, HalfNormed):
            act = torch.empty((x.shape[0], self.out_features // 2), dtype=x.xw.dtype, device=x.xw.device)
            return gemm_ops.gemm_tc(x.xw, self.weight, act, gated=True, row_scale=(x.sums, x.parts, x.size, x.eps))
        act = torch.empty((x.shape[0], self.out_features // 2), dtype=x.dtype, device=x.device)
        if self.fuses_gate(x):
            return gemm_ops.gemm_tc(x, self.weight, act, gated=True)
        return ops.silu_mul(self(x), act, pairs=True)

    def into_residual(self, x: torch.Tensor, residual: torch.Tensor, norm) -> HalfNormed:
        """``residual += x W^T`` and the half-normed rows for the product behind ``norm`` (an RMSNorm over
        ``out_features``), in one kernel.  Only where ``fuses_norm``."""
        rows = x.shape[0]
        parts = gemm_ops.residual_parts(rows, self.out_features, self.in_features)
        sums = torch.empty((parts, rows), dtype=torch.float32, device=x.device)
        xw = torch.empty((rows, self.out_features), dtype=x.dtype, device=x.device)
        gemm_ops.gemm_tc(x, self.weight, xw, residual=residual, norm_weight=norm.weight, sums=sums)
        return HalfNormed(xw, sums, parts, norm.size, norm.eps)

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if isinstance(x, HalfNormed):                      # the product finishes the norm (see HalfNormed)
            if out is None:
                out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype or x.xw.dtype, device=x.xw.device)
            return gemm_ops.gemm_tc(x.xw, self.weight, out, row_scale=(x.sums, x.parts, x.size, x.eps))
        out = self._product(x, out_dtype, out)
        return out if self.bias is None else ops.add_bias(out, self.bias)

    def _product(self, x: torch.Tensor, out_dtype: Optional[torch.dtype], out: Optional[torch.Tensor]) -> torch.Tensor:
        out_dtype = out_dtype or x.dtype
        if out is None:
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype, device=x.device)
        w = self.weight
        if x.dtype == torch.float32 or w.dtype == torch.float32:
            return ops.gemm_f32(x, w, out)
        # bfloat16 x bfloat16, f32 accumulation
        rows = x.shape[0]
        use_tc = rows <= TC_MAX_DECODE_TOKENS or PROMPT_BACKEND == "tc"
        if use_tc and gemm_ops.supported(x, w):
            return gemm_ops.gemm_tc(x, w, out)
        add_launches(1)
        if out.dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
        else:
            torch.mm(x, w.t(), out_dtype=out.dtype, out=out)
        return out
