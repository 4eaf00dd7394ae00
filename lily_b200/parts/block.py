"""The pre-norm block: ``r += mixer(norm_in(r)); r += feed_forward(norm_post(r))``.

The residual stream ``r`` is float32 and updated in place; each add is fused into the norm that
follows it, so a block receives the pending delta of the block before it and returns its own
(lily/models/llama.py:108-117 with the fused-add convention of lily/layers/layernorm.py:34-36).
"""

from __future__ import annotations

from typing import Dict

from lily_b200.parts.base import Block, BlockSpec, BuildContext, RunSlots, TensorSpec, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    def __init__(self, spec: BlockSpec, prefix: str, ctx: BuildContext):
        self.spec = spec
        p = spec.prefix
        self.norm_in = build_part("norm", spec.norm_in, f"{p}.{spec.norm_in_name}", ctx)
        self.mixer = build_part("mixer", spec.mixer, f"{p}.{spec.mixer_name}", ctx)
        self.norm_post = build_part("norm", spec.norm_post, f"{p}.{spec.norm_post_name}", ctx)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, f"{p}.{spec.feed_forward_name}", ctx)
        self.mixers = (self.mixer,)
        self.parts = (self.norm_in, self.mixer, self.norm_post, self.feed_forward)

    def tensors(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self.parts:
            out.update(part.tensors())
        return out

    def load(self, get) -> None:
        for part in self.parts:
            part.load(get)

    def forward(self, residual, delta, batch, run: RunSlots):
        x = self.norm_in.forward(residual, delta)
        a = self.mixer.forward(x, batch, run.caches[0], run.states[0], run.write_cache)
        y = self.norm_post.forward(residual, a)
        return self.feed_forward.forward(y, batch)
