"""Dense SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``, no bias.

gate and up are one matrix ``[2 * inter, hidden]`` so that one product feeds the SiLU*mul
(lily/models/llama.py:31-47, stacking llama.py:164-165).  In bfloat16, when the intermediate size
is a multiple of 128, the rows alternate between 128 gate rows and the 128 up rows of the same
outputs: a 256-row tile of the product then holds both halves of 128 outputs, and for more than a
few tokens the tcgen05 kernel applies SiLU*mul in its epilogue, so the ``[tokens, 2 * inter]``
intermediate never reaches memory.  Otherwise gate rows come first, then up rows.  For up to 8
tokens (decode) one weight-streaming kernel forms both sums and SiLU*mul from either layout; the
reference streams these products through its own kernel as well (lily/csrc/bf16_skinny.cu:45-96).
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
        self.block = None          # rows of gate / up alternate in runs of this many (None: all gate, then all up)

    def tensors(self) -> Dict[str, TensorSpec]:
        h, i, p = self.spec.hidden_size, self.spec.intermediate_size, self.prefix
        return {f"{p}.gate_proj.weight": TensorSpec((i, h)), f"{p}.up_proj.weight": TensorSpec((i, h)),
                f"{p}.down_proj.weight": TensorSpec((h, i))}

    def load(self, get) -> None:
        p, i = self.prefix, self.spec.intermediate_size
        gate = get(f"{p}.gate_proj.weight")
        h = self.spec.hidden_size
        self.w_gate_up = torch.empty((2 * i, h), dtype=gate.dtype, device=gate.device)
        self.block = b = self.ctx.ops.gate_up_interleave(gate.dtype, i)
        if b:
            runs = self.w_gate_up.view(i // b, 2, b, h)
            runs[:, 0].copy_(gate.view(i // b, b, h))
            del gate
            runs[:, 1].copy_(get(f"{p}.up_proj.weight").view(i // b, b, h))
        else:
            self.w_gate_up[:i].copy_(gate)
            del gate
            self.w_gate_up[i:].copy_(get(f"{p}.up_proj.weight"))
        self.w_down = get(f"{p}.down_proj.weight").contiguous()

    def forward(self, x, batch):
        ops = self.ctx.ops
        product = ops.linear_auto                                # partial sums for a few tokens, else [M, N]
        few = ops.swiglu_skinny_need(x.shape[0], self.spec.intermediate_size, self.spec.hidden_size, x.dtype, self.block)
        if few is not None and batch.workspace is not None:
            # a few tokens: one kernel streams the fused matrix and applies SiLU*mul to its own sums
            act = ops.swiglu_skinny(x, self.w_gate_up, self.block, batch.workspace.floats("swiglu", few[0]),
                                    batch.workspace.counters("swiglu", few[1]))
        elif self.block and ops.gate_up_fused_pays(x.shape[0], self.w_gate_up.shape[0]) and ops.gemm_tc_takes(x, self.w_gate_up):
            act = ops.gemm_tc(x, self.w_gate_up, silu_mul_block=True)
        else:
            act = ops.silu_mul(product(x, self.w_gate_up), x.dtype, block=self.block)
        return product(act, self.w_down)
