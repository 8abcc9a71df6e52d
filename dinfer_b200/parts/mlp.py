"""Dense gated feed-forward: ``down( silu(gate(x)) * up(x) )``.

gate and up are stacked once at load into one ``[2I, h]`` matrix whose rows are (gate_j, up_j) pairs, so
that one product feeds the gate (the reference stacks them as two halves and runs the gate as its own
kernel: crates/layers/src/nn.rs:288-311,373-381).  With the pairs in neighbouring rows the decode
product applies the gate in its epilogue; prompts run the product and then the gate kernel."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

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
        # row 2j = gate_j, row 2j + 1 = up_j
        self.gate_up = Linear(torch.stack([g.to(dt), u.to(dt)], dim=1).reshape(2 * self.inter, self.hidden))
        self.down = Linear(tensors[self.names["d"]])

    def kernel_libraries(self):
        return ["elementwise"] + self.gate_up.kernel_libraries() + self.down.kernel_libraries()

    def takes_half_normed(self, rows: int) -> bool:
        return self.gate_up.fuses_norm(rows, self.env.act_dtype) and self.gate_up.out_features % 2 == 0

    def adds_into_residual(self, rows: int) -> bool:
        return self.down.fuses_norm(rows, self.env.act_dtype)

    def forward(self, x, ctx=None, sink=None):
        act = self.gate_up.gated_pairs(x)
        if sink is not None:                               # (residual, the norm behind this feed-forward)
            return self.down.into_residual(act, sink[0], sink[1])
        return self.down(act)
