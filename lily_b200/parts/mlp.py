"""Dense SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``, no bias.

gate and up are one matrix ``[2 * inter, hidden]`` (gate rows first) so that one product feeds the
SiLU*mul kernel: lily/models/llama.py:31-47, stacking llama.py:164-165.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch

from lily_b200.parts.base import BuildContext, FeedForward, TensorSpec, register_part


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, spec: SwiGLUSpec, prefix: str, ctx: BuildContext):
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.w_gate_up = None
        self.w_down = None

    def tensors(self) -> Dict[str, TensorSpec]:
        h, i, p = self.spec.hidden_size, self.spec.intermediate_size, self.prefix
        return {f"{p}.gate_proj.weight": TensorSpec((i, h)), f"{p}.up_proj.weight": TensorSpec((i, h)),
                f"{p}.down_proj.weight": TensorSpec((h, i))}

    def load(self, get) -> None:
        p, i = self.prefix, self.spec.intermediate_size
        gate = get(f"{p}.gate_proj.weight")
        self.w_gate_up = torch.empty((2 * i, self.spec.hidden_size), dtype=gate.dtype, device=gate.device)
        self.w_gate_up[:i].copy_(gate)
        del gate
        self.w_gate_up[i:].copy_(get(f"{p}.up_proj.weight"))
        self.w_down = get(f"{p}.down_proj.weight").contiguous()

    def forward(self, x, batch):
        ops = self.ctx.ops
        product = getattr(ops, "linear_auto", ops.linear)        # partial sums for a few tokens, else [M, N]
        return product(ops.silu_mul(product(x, self.w_gate_up), x.dtype), self.w_down)
