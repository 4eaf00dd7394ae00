"""RMSNorm fused with the residual add.

``forward(residual, delta)`` adds ``delta`` into the float32 residual stream in place and
returns the normalised activations in the compute dtype: the fused-add convention of
lily/layers/layernorm.py:11-47 with the sum kept in float32.  With ``rows`` only those rows are
normalised (the final norm before the logits).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

from lily_b200.parts.base import BuildContext, Norm, TensorSpec, register_part


@dataclass(frozen=True)
class RMSNormSpec:
    size: int
    eps: float
    kind: str = "rmsnorm"


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec: RMSNormSpec, prefix: str, ctx: BuildContext):
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.weight = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {f"{self.prefix}.weight": TensorSpec((self.spec.size,), role="vector", init="gain")}

    def load(self, get) -> None:
        self.weight = get(f"{self.prefix}.weight")

    def forward(self, residual, delta=None, delta_bias=None, rows=None, write_residual=True):
        if delta_bias is not None:
            raise NotImplementedError("rmsnorm takes no separate bias; add it in the producing linear")
        return self.ctx.ops.add_rmsnorm(residual, delta, self.weight, self.spec.eps, self.ctx.dtype, rows=rows,
                                        write_residual=write_residual)
