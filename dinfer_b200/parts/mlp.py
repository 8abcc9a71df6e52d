"""Dense gated feed-forward: ``down( silu(gate(x)) * up(x) )``.

gate and up are stacked once at load into one ``[2I, h]`` matrix, gate rows first, so one
product feeds the gate kernel (crates/layers/src/nn.rs:288-311,373-381)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import FEED_FORWARDS, FeedForward
from .linear import Linear
from .spec import TensorDecl


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """params: ``intermediate_size``, optional tensor names ``gate_proj``, ``up_proj``, ``down_proj``."""

    def __init__(self, params, env, prefix=""):
        super().__init__(params, env, prefix)
        self.hidden = env.hidden_size
        self.inter = int(params["intermediate_size"])
        n = lambda key, default: prefix + params.get(key, default)
        self.names = {"g": n("gate_proj", "gate_proj.weight"), "u": n("up_proj", "up_proj.weight"),
                      "d": n("down_proj", "down_proj.weight")}
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def declare(self) -> List[TensorDecl]:
        return [TensorDecl(self.names["g"], (self.inter, self.hidden)),
                TensorDecl(self.names["u"], (self.inter, self.hidden)),
                TensorDecl(self.names["d"], (self.hidden, self.inter))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors[self.names["g"]], tensors[self.names["u"]]
        dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.gate_up = Linear(torch.cat([g.to(dt), u.to(dt)], dim=0))
        self.down = Linear(tensors[self.names["d"]])

    def kernel_libraries(self):
        return ["elementwise"] + self.gate_up.kernel_libraries() + self.down.kernel_libraries()

    def forward(self, x: torch.Tensor, ctx=None) -> torch.Tensor:
        gu = self.gate_up(x)
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        ops.silu_mul(gu, act)
        return self.down(act)
