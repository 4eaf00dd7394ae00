"""A model put together from a ``ModelSpec``: embedding, the scheduled blocks, final norm, head.

The schedule is walked as data.  Each position of the schedule whose mixer asks for paged keys
and values gets a layer of its own in the cache group that matches the need (or, with ``reads``,
borrows the layer of an earlier position and writes nothing); each position whose mixer asks for
per-request state gets a state tensor of its own.  The same block may therefore run twice with
separate caches.

Embedding and logits follow lily/layers/vocab_embedding.py:37-39,84-96 (logits in float32, a
tied head reads the embedding table: lily/models/llama.py:175-176); the wanted rows are gathered
before the final norm, as lily/models/llama.py:199-205 gathers the last row of each request.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from lily_b200.parts.attention import LayerCache
from lily_b200.parts.base import BuildContext, CacheNeed, ModelSpec, StateNeed, TensorSpec, build_part


class AssembledModel:
    def __init__(self, spec: ModelSpec, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.blocks = [build_part("block", b, b.prefix, ctx) for b in spec.blocks]
        self.final_norm = build_part("norm", spec.final_norm, spec.final_norm_prefix, ctx)
        self.embed: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

        # cache and state layout, in schedule order
        self.cache_groups: List[Tuple[CacheNeed, int]] = []
        self.entry_cache: List[Optional[Tuple[int, int, bool]]] = []      # (group, layer, writes)
        self.state_needs: List[StateNeed] = []
        self.entry_state: List[Optional[int]] = []
        group_of: Dict[CacheNeed, int] = {}
        counts: List[int] = []
        for pos, entry in enumerate(spec.schedule):
            if not (0 <= entry.block < len(self.blocks)):
                raise ValueError(f"schedule position {pos} names block {entry.block} of {len(self.blocks)}")
            mixer = self.blocks[entry.block].mixer
            need = mixer.cache_need()
            if need is None:
                self.entry_cache.append(None)
            elif entry.reads is not None:
                if not (0 <= entry.reads < pos) or self.entry_cache[entry.reads] is None:
                    raise ValueError(f"schedule position {pos} reads the cache of position {entry.reads}, "
                                     "which must be an earlier position that has one")
                g, layer, _ = self.entry_cache[entry.reads]
                other = self.blocks[spec.schedule[entry.reads].block].mixer.cache_need()
                if (other.kv_heads, other.head_dim) != (need.kv_heads, need.head_dim):
                    raise ValueError(f"schedule position {pos} cannot read a cache of another shape")
                self.entry_cache.append((g, layer, False))
            else:
                if need not in group_of:
                    group_of[need] = len(counts)
                    counts.append(0)
                g = group_of[need]
                self.entry_cache.append((g, counts[g], True))
                counts[g] += 1
            sneed = mixer.state_need()
            if sneed is None:
                self.entry_state.append(None)
            else:
                self.entry_state.append(len(self.state_needs))
                self.state_needs.append(sneed)
        self.cache_groups = [(need, counts[g]) for need, g in sorted(group_of.items(), key=lambda kv: kv[1])]

    @property
    def graph_safe(self) -> bool:
        return all(b.mixer.graph_safe for b in self.blocks)

    # ---- weights -------------------------------------------------------------------

    def tensors(self) -> Dict[str, TensorSpec]:
        s = self.spec
        out = {s.embed_name: TensorSpec((s.vocab_size, s.hidden_size))}
        for b in self.blocks:
            out.update(b.tensors())
        out.update(self.final_norm.tensors())
        if s.head_name is not None:
            out[s.head_name] = TensorSpec((s.vocab_size, s.hidden_size))
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
        ops = self.ctx.ops
        future = getattr(batch, "future_tokens", None)
        residual = ops.embed(self.embed, batch.token_ids) if future is None else ops.embed(self.embed, batch.token_ids, future=future)
        delta = None
        for pos, entry in enumerate(self.spec.schedule):
            ec, es = self.entry_cache[pos], self.entry_state[pos]
            layer_cache = LayerCache(ec[0], cache.groups[ec[0]].data[ec[1]]) if ec is not None else None
            state = cache.states[es] if es is not None else None
            delta = self.blocks[entry.block].forward(residual, delta, batch, layer_cache, state,
                                                     ec[2] if ec is not None else True)
        if batch.logit_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=residual.device)
        x = self.final_norm.forward(residual, delta, rows=batch.logit_rows)
        split = getattr(ops, "linear_split", None)
        if split is not None:                     # a few rows: stream the head once, float32 out
            parts = split(x, self.head)
            if parts is not None and parts.shape[0] == 1:
                return parts[0]
        return ops.linear(x, self.head, out_dtype=torch.float32)
