"""What a part is, and the registries parts are chosen from.

A model is put together from parts that know nothing of the model they are in:

* a **mixer** moves information between the tokens of a request (attention here);
* a **feed-forward** works on each token alone (dense SwiGLU here; experts would go here);
* a **norm** normalises the residual stream and, fused with it, adds the pending delta;
* a **position encoding** is a parameter of the mixer that uses it (rotary tables here);
* a **block** arranges one mixer, one feed-forward and their norms around the residual stream.

Each part is described by a *spec* (a dataclass with a ``kind`` string and every size and
constant the part needs) and built from it by ``build_part``.  The specs of a model's blocks
and the order in which the blocks run are plain data (``ModelSpec``), produced by the
architecture's ``build_spec`` from its typed configuration, layer by layer, so that one model
may use different mixers and feed-forwards in different layers.

Interfaces
----------
``Part.tensors()``   -> {checkpoint tensor name: TensorSpec}; what the loader must find.
``Part.load(get)``   -> fetch each tensor with ``get(name)`` (already on the device, in the
                        dtype its role gives) and pack it for the kernels.
``Mixer.cache_need()`` -> ``CacheNeed`` (paged keys/values) or None.
``Mixer.state_need()`` -> ``StateNeed`` (fixed-size per-request state) or None.
``Mixer.forward(x, batch, cache, state, write_cache)`` -> [tokens, hidden] delta.
``FeedForward.forward(x, batch)`` -> [tokens, hidden] delta.
``Mixer.forward`` reads the step from ``batch`` (device tensors; host lists when it is not
                        ``graph_safe``) and may keep a plan of its own there (``batch.plan``).
``FeedForward.forward(x, batch)`` -> [tokens, hidden] delta.
``Norm.forward(residual, delta, delta_bias, rows, write_residual)`` -> normed activations.
``Block.mixers``     -> the mixers of the block, in a fixed order; each run of the block gets a
                        cache layer and a state tensor for each of them (``RunSlots``).
``Block.forward(residual, delta, batch, run)`` -> next pending delta.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch


# --------------------------------------------------------------------------- tensors

@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part expects.

    role  "matrix": a GEMM operand or embedding table; held in the compute dtype.
          "vector": gains and biases; a tensor stored in 32-bit stays 32-bit, anything
                    else is held in the compute dtype.
          "table":  integer tables; held as int32.
    init  how the random-weights mode draws it: "normal" N(0, std), "gain" 1 + N(0, jitter),
          "zeros".
    short_rows  vocabulary tables: a checkpoint saved before the vocabulary was padded holds fewer rows; they
          are taken and the missing rows are zero (lily/layers/vocab_embedding.py:29-35).
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    short_rows: bool = False      # the checkpoint may hold fewer rows than ``shape[0]``; the rest is zero


# --------------------------------------------------------------------------- needs of a mixer

@dataclass(frozen=True)
class CacheNeed:
    """Paged keys and values.  Layers whose needs are equal share a cache group
    (one pool of pages and one block table per request); ``window`` None keeps all keys,
    an integer keeps the last ``window`` of them and lets older pages go."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size for each live request: ``shape`` per request, zero when a request
    starts, carried from one step to the next in the request's slot."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# --------------------------------------------------------------------------- build context

@dataclass
class BuildContext:
    """What a part may rely on while it is built and run."""

    device: torch.device
    dtype: torch.dtype                 # compute dtype: torch.bfloat16 or torch.float32
    ops: Any                           # lily_b200.csrc.ops (the kernels), or a stand-in in CPU tests
    page_size: int = 64
    max_position: int = 4096           # positions the position tables must cover


class Part:
    kind: str = ""

    def tensors(self) -> Dict[str, TensorSpec]:
        return {}

    def load(self, get: Callable[[str], torch.Tensor]) -> None:
        pass


class Mixer(Part):
    # True when ``forward`` reads the batch's device tensors only (never its host lists), so that a
    # decode step may be captured once in a CUDA graph and replayed with new contents.
    graph_safe: bool = False

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, x, batch, cache, state, write_cache: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, batch):
        raise NotImplementedError


class Norm(Part):
    def forward(self, residual, delta=None, delta_bias=None, rows=None, write_residual=True):
        raise NotImplementedError


@dataclass
class RunSlots:
    """What one run of a block (one position of the schedule) owns: for each mixer of the block, in the
    order of ``Block.mixers``, its layer of the paged cache (or None) and its per-request state tensor
    ``[slots + 1, *shape]`` (or None); ``write_cache`` False when the run reads another run's cache."""

    caches: List[Any]
    states: List[Any]
    write_cache: bool = True


class Block(Part):
    """An arrangement of mixers, feed-forwards and norms around the residual stream.  A block kind is built
    from a spec of its own (any dataclass with ``kind`` and ``prefix``); the model asks it only for
    ``mixers``, ``parts``, ``tensors``, ``load`` and ``forward``."""

    mixers: Tuple[Mixer, ...] = ()
    parts: Tuple[Part, ...] = ()

    def forward(self, residual, delta, batch, run: RunSlots):
        raise NotImplementedError


# --------------------------------------------------------------------------- registries

_REGISTRIES: Dict[str, Dict[str, Callable[..., Part]]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
}


def register_part(family: str, kind: str):
    """Class decorator: ``@register_part("mixer", "attention")``.  The class is built as
    ``cls(spec, prefix, ctx)`` where ``prefix`` is the part's checkpoint name prefix."""
    if family not in _REGISTRIES:
        raise ValueError(f"unknown part family {family!r}; have {sorted(_REGISTRIES)}")

    def deco(cls):
        cls.kind = kind
        _REGISTRIES[family][kind] = cls
        return cls
    return deco


def build_part(family: str, spec: Any, prefix: str, ctx: BuildContext) -> Part:
    _load_builtin_parts()
    table = _REGISTRIES[family]
    kind = getattr(spec, "kind", None)
    if kind not in table:
        raise ValueError(f"no {family} of kind {kind!r}; have {sorted(table)}")
    return table[kind](spec, prefix, ctx)


def registered(family: str) -> List[str]:
    _load_builtin_parts()
    return sorted(_REGISTRIES[family])


_BUILTINS = False


def _load_builtin_parts() -> None:
    global _BUILTINS
    if not _BUILTINS:
        _BUILTINS = True
        from lily_b200.parts import attention, block, mlp, norm, rope  # noqa: F401


# --------------------------------------------------------------------------- model description

@dataclass
class BlockSpec:
    """The pre-norm block (kind "prenorm"): its checkpoint prefix and the specs of its parts.  Another block
    kind brings a spec class of its own; ``ModelSpec.blocks`` takes any mix of them."""

    prefix: str
    mixer: Any
    feed_forward: Any
    norm_in: Any
    norm_post: Any
    kind: str = "prenorm"
    mixer_name: str = "self_attn"                 # names of the parts under the block's prefix
    feed_forward_name: str = "mlp"
    norm_in_name: str = "input_layernorm"
    norm_post_name: str = "post_attention_layernorm"


@dataclass
class ScheduleEntry:
    """One run of a block.  ``reads`` names an earlier position of the schedule whose cache
    this run reads instead of writing one of its own (shared keys and values)."""

    block: int
    reads: Optional[int] = None


@dataclass
class ModelSpec:
    """A whole model as data: the blocks, and the order in which they run (a block may be
    named more than once; each run has a cache and a state of its own unless it ``reads``)."""

    architecture: str
    vocab_size: int
    hidden_size: int
    blocks: List[Any]                                 # BlockSpec, or the spec of any registered block kind
    schedule: List[ScheduleEntry]
    final_norm: Any
    embed_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm"
    head_name: Optional[str] = "lm_head.weight"      # None: the head reads the embedding table
    max_position: int = 4096
    eos_token_ids: List[int] = field(default_factory=list)
    ignored_tensors: Tuple[str, ...] = ("rotary_emb.inv_freq",)   # lily/models/llama.py:217-218
    embed_scale: float = 1.0                          # the embedding rows are multiplied by this
    logit_scale: float = 1.0                          # logits = logit_scale * (x . head^T) ...
    logit_softcap: Optional[float] = None             # ... then cap * tanh(. / cap) when given
