"""A model put together from a ``ModelSpec``: embedding, the scheduled blocks, final norm, head.

The schedule is walked as data.  For each position of the schedule, every mixer of its block that
asks for paged keys and values gets a layer of its own in the cache group that matches the need
(or, with ``reads``, borrows the layer of the same mixer at an earlier position and writes
nothing); every mixer that asks for per-request state gets a state tensor of its own.  The same
block may therefore run twice with separate caches.  The embedding may be scaled and the logits
scaled and soft-capped (``ModelSpec.embed_scale``, ``logit_scale``, ``logit_softcap``).

Embedding and logits follow lily/layers/vocab_embedding.py:37-39,84-96 (logits in float32, a
tied head reads the embedding table: lily/models/llama.py:175-176); the wanted rows are gathered
before the final norm, as lily/models/llama.py:199-205 gathers the last row of each request.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from lily_b200.parts.attention import LayerCache
from lily_b200.parts.base import BuildContext, CacheNeed, ModelSpec, RunSlots, StateNeed, TensorSpec, build_part


class AssembledModel:
    def __init__(self, spec: ModelSpec, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.blocks = [build_part("block", b, b.prefix, ctx) for b in spec.blocks]
        self.final_norm = build_part("norm", spec.final_norm, spec.final_norm_prefix, ctx)
        self.embed: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

        # cache and state layout, in schedule order: one entry per (schedule position, mixer of its block)
        self.cache_groups: List[Tuple[CacheNeed, int]] = []
        self.entry_cache: List[List[Optional[Tuple[int, int, bool]]]] = []      # (group, layer, writes)
        self.state_needs: List[StateNeed] = []
        self.entry_state: List[List[Optional[int]]] = []
        group_of: Dict[CacheNeed, int] = {}
        counts: List[int] = []
        for pos, entry in enumerate(spec.schedule):
            if not (0 <= entry.block < len(self.blocks)):
                raise ValueError(f"schedule position {pos} names block {entry.block} of {len(self.blocks)}")
            mixers = self.blocks[entry.block].mixers
            if entry.reads is not None and not (0 <= entry.reads < pos):
                raise ValueError(f"schedule position {pos} reads the cache of position {entry.reads}, "
                                 "which must be an earlier position")
            caches: List[Optional[Tuple[int, int, bool]]] = []
            states: List[Optional[int]] = []
            for k, mixer in enumerate(mixers):
                need = mixer.cache_need()
                if need is None:
                    caches.append(None)
                elif entry.reads is not None:
                    owners = self.blocks[spec.schedule[entry.reads].block].mixers
                    lent = self.entry_cache[entry.reads][k] if k < len(owners) else None
                    if lent is None:
                        raise ValueError(f"schedule position {pos} reads the cache of position {entry.reads}, "
                                         f"whose mixer {k} has none")
                    other = owners[k].cache_need()
                    if (other.kv_heads, other.head_dim) != (need.kv_heads, need.head_dim):
                        raise ValueError(f"schedule position {pos} cannot read a cache of another shape")
                    if other.window is not None and (need.window is None or need.window > other.window):
                        # the owner's group gives pages back once its window has passed them
                        raise ValueError(f"schedule position {pos} looks back {need.window or 'over all'} keys but reads "
                                         f"a cache that keeps the last {other.window}")
                    caches.append((lent[0], lent[1], False))
                else:
                    if need not in group_of:
                        group_of[need] = len(counts)
                        counts.append(0)
                    g = group_of[need]
                    caches.append((g, counts[g], True))
                    counts[g] += 1
                sneed = mixer.state_need()
                if sneed is None:
                    states.append(None)
                else:
                    states.append(len(self.state_needs))
                    self.state_needs.append(sneed)
            self.entry_cache.append(caches)
            self.entry_state.append(states)
        self.cache_groups = [(need, counts[g]) for need, g in sorted(group_of.items(), key=lambda kv: kv[1])]

    @property
    def graph_safe(self) -> bool:
        return all(m.graph_safe for b in self.blocks for m in b.mixers)

    # ---- weights -------------------------------------------------------------------

    def tensors(self) -> Dict[str, TensorSpec]:
        s = self.spec
        out = {s.embed_name: TensorSpec((s.vocab_size, s.hidden_size), short_rows=True)}
        for b in self.blocks:
            out.update(b.tensors())
        out.update(self.final_norm.tensors())
        if s.head_name is not None:
            out[s.head_name] = TensorSpec((s.vocab_size, s.hidden_size), short_rows=True)
        return out

    def ignorable(self, name: str) -> bool:
        """Checkpoint tensors that may be present without being used."""
        if any(tag in name for tag in self.spec.ignored_tensors):
            return True
        return self.spec.head_name is None and name == "lm_head.weight"    # tied: llama.py:219-220

    def load(self, get) -> None:
        self.embed = get(self.spec.embed_name).contiguous()
        for b in self.blocks:
            b.load(get)
        self.final_norm.load(get)
        self.head = self.embed if self.spec.head_name is None else get(self.spec.head_name).contiguous()

    def weight_bytes(self) -> int:
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen and not getattr(v, "_is_table", False):
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        visit(self)
        for b in self.blocks:
            for part in b.parts:
                visit(part)
        visit(self.final_norm)
        return total

    # ---- one step ------------------------------------------------------------------

    def forward(self, batch, cache) -> torch.Tensor:
        """Runs the batch's tokens through the schedule and returns float32 logits
        ``[len(batch.logit_rows), vocab]``."""
        ops, spec = self.ctx.ops, self.spec
        residual = ops.embed(self.embed, batch.token_ids, future=batch.future_tokens, scale=spec.embed_scale)
        delta = None
        for pos, entry in enumerate(spec.schedule):
            caches = [LayerCache(ec[0], cache.groups[ec[0]].data[ec[1]]) if ec is not None else None
                      for ec in self.entry_cache[pos]]
            states = [cache.states[es] if es is not None else None for es in self.entry_state[pos]]
            writes = all(ec[2] for ec in self.entry_cache[pos] if ec is not None)
            delta = self.blocks[entry.block].forward(residual, delta, batch, RunSlots(caches, states, writes))
        if batch.logit_rows.numel() == 0:
            return torch.empty((0, spec.vocab_size), dtype=torch.float32, device=residual.device)
        x = self.final_norm.forward(residual, delta, rows=batch.logit_rows)
        logits = ops.logits(x, self.head)
        if spec.logit_scale != 1.0 or spec.logit_softcap is not None:
            ops.logit_transform(logits, spec.logit_scale, spec.logit_softcap)
        return logits
