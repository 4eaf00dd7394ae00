"""Grouped-query attention over the paged cache.

q, k and v come from one product with the stacked matrix ``[q rows | k rows | v rows]``; one fused
kernel then normalises each q and k head (when ``qk_norm``), rotates them by the position tables,
leaves q in a buffer and writes k and v into the token's page; attention runs over the cache
(split-key decode kernel for requests that bring one token, prefill kernel for portions); the
output projection closes the part.  How a step's attention is cut (key ranges, kernel forms, tile
lists) is this part's own plan, made once a step from the batch's host fields by asking the kernels
(``ops.plan_decode_attention``, ``ops.prefill_tile_rows``, ``ops.prefill_tiles``); the step function
knows nothing of it.  Sizes, eps, scale, window and the position encoding are
parameters of the spec; nothing here knows which model it serves.

Formulas: lily/models/llama.py:50-90 (projections, scale = head_dim^-0.5 unless the spec gives
one), lily/models/qwen3.py:17-32 (per-head q/k RMSNorm before the rotation),
lily/layers/attention/triton_backend.py:110-141 (cache write before attention).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch

from lily_b200.parts.base import BuildContext, CacheNeed, Mixer, TensorSpec, build_part, register_part


@dataclass(frozen=True)
class AttentionSpec:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qk_norm: bool = False
    norm_eps: float = 1e-6
    bias: bool = False
    window: Optional[int] = None          # None: all keys; n: the last n keys
    scale: Optional[float] = None         # None: head_dim ** -0.5
    position: Any = None                  # a position spec (e.g. RopeSpec) or None
    kind: str = "attention"


@dataclass
class AttentionPlan:
    """One step's attention for one set of sizes: the decode rows' plan (``ops.plan_decode_attention``) and,
    when requests bring portions, the prefill kernel's tile height and its (request, offset) lists."""

    decode: Any
    tile_rows: Optional[int]
    tiles: Any


@dataclass
class LayerCache:
    """The cache one run of a mixer reads and writes: its group and its layer's pages."""

    group: int
    data: torch.Tensor            # [pages + 1, 2, kv_heads, page_size, head_dim]


@register_part("mixer", "attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec: AttentionSpec, prefix: str, ctx: BuildContext):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads do not group over {spec.num_kv_heads} kv heads")
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.scale = spec.scale if spec.scale is not None else spec.head_dim ** -0.5
        self.position = build_part("position", spec.position, prefix, ctx) if spec.position is not None else None
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_gain = self.k_gain = None

    # ---- what it needs ----------------------------------------------------------

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def tensors(self) -> Dict[str, TensorSpec]:
        s, p = self.spec, self.prefix
        q, kv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        out = {f"{p}.q_proj.weight": TensorSpec((q, s.hidden_size)),
               f"{p}.k_proj.weight": TensorSpec((kv, s.hidden_size)),
               f"{p}.v_proj.weight": TensorSpec((kv, s.hidden_size)),
               f"{p}.o_proj.weight": TensorSpec((s.hidden_size, q))}
        if s.bias:
            out.update({f"{p}.q_proj.bias": TensorSpec((q,), role="matrix"),
                        f"{p}.k_proj.bias": TensorSpec((kv,), role="matrix"),
                        f"{p}.v_proj.bias": TensorSpec((kv,), role="matrix"),
                        f"{p}.o_proj.bias": TensorSpec((s.hidden_size,), role="matrix")})
        if s.qk_norm:
            out.update({f"{p}.q_norm.weight": TensorSpec((s.head_dim,), role="vector", init="gain"),
                        f"{p}.k_norm.weight": TensorSpec((s.head_dim,), role="vector", init="gain")})
        return out

    def load(self, get) -> None:
        s, p = self.spec, self.prefix
        q, kv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        wq = get(f"{p}.q_proj.weight")
        self.w_qkv = torch.empty((q + 2 * kv, s.hidden_size), dtype=wq.dtype, device=wq.device)
        self.w_qkv[:q].copy_(wq)
        del wq
        self.w_qkv[q:q + kv].copy_(get(f"{p}.k_proj.weight"))
        self.w_qkv[q + kv:].copy_(get(f"{p}.v_proj.weight"))
        self.w_o = get(f"{p}.o_proj.weight").contiguous()
        if s.bias:
            self.b_qkv = torch.cat([get(f"{p}.{n}_proj.bias") for n in "qkv"]).contiguous()
            self.b_o = get(f"{p}.o_proj.bias").contiguous()
        if s.qk_norm:
            self.q_gain = get(f"{p}.q_norm.weight")
            self.k_gain = get(f"{p}.k_norm.weight")
            if self.q_gain.dtype != self.k_gain.dtype:
                self.q_gain, self.k_gain = self.q_gain.float(), self.k_gain.float()

    # ---- one step ----------------------------------------------------------------

    def _plan(self, batch, group: int, dtype, page: int):
        """How this step's attention runs for this mixer's sizes in cache group ``group``; made once a step and
        shared by every layer with the same sizes (``batch.plan``)."""
        s, ops = self.spec, self.ctx.ops
        key = ("attention", group, s.num_heads, s.num_kv_heads, s.head_dim, dtype, page)

        def make(b):
            nd = b.num_decode
            decode = ops.plan_decode_attention(dtype, nd, s.num_heads, s.num_kv_heads, s.head_dim, b.max_decode_len,
                                               even=b.decode_even)
            if decode != ops.plan_decode_attention(dtype, nd, s.num_heads, s.num_kv_heads, s.head_dim, b.max_decode_len,
                                                   even=not b.decode_even):
                b.even_asked = True              # a captured step with this plan serves batches of this kind only
            rows = tiles = None
            if b.num_requests > nd:
                rows = ops.prefill_tile_rows(dtype, s.head_dim, page, b.num_tokens - nd)
                tiles = ops.prefill_tiles(b.h_prefix_lens, b.h_new_lens, nd, rows, b.token_ids.device)
            return AttentionPlan(decode, rows, tiles)
        return batch.plan(key, make)

    def forward(self, x, batch, cache: LayerCache, state=None, write_cache: bool = True):
        s, ops = self.spec, self.ctx.ops
        page = cache.data.shape[3]
        table = batch.block_tables[cache.group]
        plan = self._plan(batch, cache.group, cache.data.dtype, page)
        qkv = ops.linear_auto(x, self.w_qkv, self.b_qkv)
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        nd, dec = batch.num_decode, plan.decode
        scratch = batch.workspace.floats("attention_decode", dec.scratch_floats) if nd and dec.scratch_floats else None
        if nd == batch.num_tokens and dec.fused:
            # every request brings one token: the decode attention kernel finishes q, k and v itself
            out = torch.empty((nd, s.num_heads * s.head_dim), dtype=cache.data.dtype, device=cache.data.device)
            ops.attention_decode_fused(qkv, self.q_gain, self.k_gain, s.norm_eps, cos, sin, cache.data, table, batch.seq_lens,
                                       out, scratch, dec.splits, s.num_heads, s.num_kv_heads, s.head_dim, rotary_dim, page,
                                       self.scale, s.window, write_kv=write_cache, stages=dec.stages)
            return ops.linear_auto(out, self.w_o, self.b_o)
        q = ops.qk_norm_rope_write(qkv, self.q_gain, self.k_gain, s.norm_eps, cos, sin, batch.positions,
                                   batch.token_req, table, cache.data, s.num_heads, s.num_kv_heads, s.head_dim,
                                   rotary_dim, page, write_kv=write_cache)
        out = torch.empty_like(q)       # [tokens, heads * head_dim]
        if nd:
            ops.attention_decode(q[:nd], cache.data, table, batch.seq_lens, out[:nd], scratch, dec.splits,
                                 s.num_heads, s.num_kv_heads, s.head_dim, page, self.scale, s.window, stages=dec.stages)
        if batch.num_requests > nd:
            tile_req, tile_start = plan.tiles
            ops.attention_prefill(q, cache.data, table, batch.cu_seqlens, batch.prefix_lens, tile_req, tile_start,
                                  out, s.num_heads, s.num_kv_heads, s.head_dim, page, self.scale, s.window,
                                  tile_rows=plan.tile_rows)
        return ops.linear_auto(out, self.w_o, self.b_o)
