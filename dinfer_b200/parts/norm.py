"""RMSNorm over the residual stream, fused with the residual add and the gather of rows."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import NORMS, Norm
from .spec import TensorDecl


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """params: ``size``, ``eps``, ``weight`` (tensor name after the prefix).

    ``out = T(v * rsqrt(mean(v^2) + eps) * w)`` with ``v = residual (+ delta)`` in 32-bit
    (crates/kernels/cuda/norm.cu:54-115, crates/layers/src/nn.rs:78-111)."""

    def __init__(self, params, env, prefix=""):
        super().__init__(params, env, prefix)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight_name = prefix + params.get("weight", "weight")
        self.weight: Optional[torch.Tensor] = None

    def declare(self) -> List[TensorDecl]:
        return [TensorDecl(self.weight_name, (self.size,), init="ones")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def kernel_libraries(self):
        return ["norm"]

    def forward(self, residual, delta=None, rows=None):
        n = rows.numel() if rows is not None else residual.shape[0]
        out = torch.empty((n, self.size), dtype=self.env.act_dtype, device=residual.device)
        return ops.rmsnorm(residual, self.weight, self.eps, out, delta=delta, rows=rows)
