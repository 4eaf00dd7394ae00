"""Parts that are no part of any real model, defined here and registered without touching the
framework's files: a mixer with per-request state of its own, a feed-forward with routing, another
position encoding, a schedule that names a block twice and lets a run read another run's cache,
and a windowed attention layer beside a full one (two cache groups).  A second toy has what decodes
through CUDA graphs: a mixer whose state a captured step reaches through the slots on the device, two
attention groups of different head sizes, a block kind with a spec class of its own, a windowed cache read
by a layer with a shorter window, a scaled embedding and scaled, soft-capped logits.

Each toy is checked against a plain whole-sequence statement written beside it.  The CPU variants
use the kernels' PyTorch statements as ops; the ``gpu`` variants use the CUDA kernels.
"""

from dataclasses import dataclass

import pytest
import torch

import kernel_refs
import plain_impl
import tiny_models
from harness import run_mixed, run_portions, run_whole
from lily_b200.config.registry import register_architecture
from lily_b200.config.server_args import ServerArgs
from lily_b200.engine.runner import ModelRunner
from lily_b200.parts.attention import AttentionSpec
from lily_b200.parts.base import (Block, BlockSpec, FeedForward, Mixer, ModelSpec, RunSlots, ScheduleEntry, StateNeed,
                                  TensorSpec, build_part, register_part)
from lily_b200.parts.mlp import SwiGLUSpec
from lily_b200.parts.norm import RMSNormSpec
from lily_b200.parts.rope import RopeSpec, RotaryTable
from lily_b200.weights.random_init import RandomSource, expected_tensors

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


# ------------------------------------------------------------------ a mixer with state of its own

@dataclass(frozen=True)
class MeanMixerSpec:
    hidden_size: int
    inner: int
    kind: str = "toy_running_mean"


@register_part("mixer", "toy_running_mean")
class MeanMixer(Mixer):
    """out_t = W_out . mean_{s <= t}(W_in . x_s): the state is the running sum and the count."""

    def __init__(self, spec, prefix, ctx):
        self.spec, self.prefix, self.ctx = spec, prefix, ctx

    def state_need(self):
        return StateNeed((self.spec.inner + 1,), torch.float32)

    def tensors(self):
        return {f"{self.prefix}.w_in": TensorSpec((self.spec.inner, self.spec.hidden_size)),
                f"{self.prefix}.w_out": TensorSpec((self.spec.hidden_size, self.spec.inner))}

    def load(self, get):
        self.w_in, self.w_out = get(f"{self.prefix}.w_in"), get(f"{self.prefix}.w_out")

    def forward(self, x, batch, cache, state, write_cache=True):
        ops = self.ctx.ops
        u = ops.linear(x, self.w_in).float()
        mean = torch.empty_like(u)
        at = 0
        for slot, n in zip(batch.h_slots, batch.h_new_lens):
            run = state[slot, :-1] + torch.cumsum(u[at:at + n], 0)
            count = state[slot, -1] + torch.arange(1, n + 1, device=u.device)
            mean[at:at + n] = run / count[:, None]
            state[slot, :-1] = run[-1]
            state[slot, -1] = count[-1]
            at += n
        return ops.linear(mean.to(x.dtype), self.w_out)


# ------------------------------------------------------------------ the same state, reachable inside a CUDA graph

@dataclass(frozen=True)
class DeviceMeanMixerSpec:
    hidden_size: int
    inner: int
    kind: str = "toy_running_mean_on_device"


@register_part("mixer", "toy_running_mean_on_device")
class DeviceMeanMixer(MeanMixer):
    """The running mean again, but a step in which every request brings one token reads and writes the state
    through ``batch.slots`` on the device alone, so that such a step can be captured once and replayed
    (rows that pad a captured batch name slot 0, which belongs to no request)."""

    graph_safe = True

    def forward(self, x, batch, cache, state, write_cache=True):
        if batch.num_decode != batch.num_tokens:
            return super().forward(x, batch, cache, state, write_cache)
        ops = self.ctx.ops
        u = ops.linear(x, self.w_in).float()
        slots = batch.slots.long()
        now = state.index_select(0, slots)
        now[:, :-1] += u
        now[:, -1] += 1.0
        state.index_copy_(0, slots, now)
        return ops.linear((now[:, :-1] / now[:, -1:]).to(x.dtype), self.w_out)


# ------------------------------------------------------------------ a block kind with a spec of its own

@dataclass(frozen=True)
class ParallelBlockSpec:
    """r += mixer(n(r)) + feed_forward(n(r)): one norm, both parts read it (a parallel-residual block)."""

    prefix: str
    mixer: object
    feed_forward: object
    norm: object
    kind: str = "toy_parallel"


@register_part("block", "toy_parallel")
class ParallelBlock(Block):
    def __init__(self, spec, prefix, ctx):
        self.norm = build_part("norm", spec.norm, f"{prefix}.ln", ctx)
        self.mixer = build_part("mixer", spec.mixer, f"{prefix}.attn", ctx)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, f"{prefix}.ff", ctx)
        self.mixers = (self.mixer,)
        self.parts = (self.norm, self.mixer, self.feed_forward)

    def tensors(self):
        out = {}
        for part in self.parts:
            out.update(part.tensors())
        return out

    def load(self, get):
        for part in self.parts:
            part.load(get)

    def forward(self, residual, delta, batch, run: RunSlots):
        x = self.norm.forward(residual, delta)
        a = self.mixer.forward(x, batch, run.caches[0], run.states[0], run.write_cache)
        f = self.feed_forward.forward(x, batch)
        a = a.sum(0) if a.dim() == 3 else a                       # a few tokens' products come as partial sums
        f = f.sum(0) if f.dim() == 3 else f
        return (a.float() + f.float()).to(x.dtype)


# ------------------------------------------------------------------ a feed-forward with routing

@dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    inner: int
    experts: int
    kind: str = "toy_routed"


@register_part("feed_forward", "toy_routed")
class Routed(FeedForward):
    """Top-1 of `experts` two-matrix experts, router logits in float32."""

    def __init__(self, spec, prefix, ctx):
        self.spec, self.prefix, self.ctx = spec, prefix, ctx

    def tensors(self):
        s, p = self.spec, self.prefix
        out = {f"{p}.router": TensorSpec((s.experts, s.hidden_size), role="vector")}
        for e in range(s.experts):
            out[f"{p}.experts.{e}.up"] = TensorSpec((s.inner, s.hidden_size))
            out[f"{p}.experts.{e}.down"] = TensorSpec((s.hidden_size, s.inner))
        return out

    def load(self, get):
        p = self.prefix
        self.router = get(f"{p}.router").float()
        self.up = [get(f"{p}.experts.{e}.up") for e in range(self.spec.experts)]
        self.down = [get(f"{p}.experts.{e}.down") for e in range(self.spec.experts)]

    def forward(self, x, batch):
        ops = self.ctx.ops
        choice = torch.argmax(x.float() @ self.router.t(), dim=-1)
        out = torch.zeros_like(x)
        for e in range(self.spec.experts):
            rows = torch.nonzero(choice == e).flatten()
            if rows.numel():
                h = torch.relu(ops.linear(x[rows].contiguous(), self.up[e]))
                out[rows] = ops.linear(h, self.down[e])
        return out


# ------------------------------------------------------------------ another position encoding

@dataclass(frozen=True)
class HalfSpeedRopeSpec:
    head_dim: int
    rotary_dim: int
    theta: float
    kind: str = "toy_half_speed_rope"


@register_part("position", "toy_half_speed_rope")
class HalfSpeedRope(RotaryTable):
    """Rotation tables whose angles advance half as fast (position interpolation by 2)."""

    def __init__(self, spec, prefix, ctx):
        inv = plain_impl.rope_inv_freq(spec.rotary_dim, spec.theta)
        freqs = torch.outer(torch.arange(ctx.max_position, dtype=torch.float32) / 2.0, inv)
        self.spec, self.ctx, self.rotary_dim = spec, ctx, spec.rotary_dim
        self._cos, self._sin = freqs.cos().to(ctx.device), freqs.sin().to(ctx.device)


# ------------------------------------------------------------------ a toy architecture of its own

@dataclass
class ToyConfig:
    width: int
    vocab: int
    heads: int
    kv_heads: int
    head: int
    inner: int
    experts: int
    window: int
    positions: int
    eps: float

    @classmethod
    def from_dict(cls, cfg, generation=None, architecture=None):
        return cls(**{k: cfg[f"toy_{k}"] for k in cls.__dataclass_fields__})


def toy_spec(c: ToyConfig) -> ModelSpec:
    norm = RMSNormSpec(c.width, c.eps)
    full = AttentionSpec(c.width, c.heads, c.kv_heads, c.head, qk_norm=True, norm_eps=c.eps,
                         position=HalfSpeedRopeSpec(c.head, c.head // 2, 777.0))
    windowed = AttentionSpec(c.width, c.heads, c.kv_heads, c.head, window=c.window, scale=0.2,
                             position=RopeSpec(c.head, c.head, 1000.0))
    nope = AttentionSpec(c.width, c.heads, c.kv_heads, c.head)        # no position encoding at all
    blocks = [
        BlockSpec("toy.0", full, SwiGLUSpec(c.width, c.inner), norm, norm),
        BlockSpec("toy.1", MeanMixerSpec(c.width, c.inner), RoutedSpec(c.width, c.inner, c.experts), norm, norm,
                  mixer_name="mean", feed_forward_name="routed"),
        BlockSpec("toy.2", windowed, SwiGLUSpec(c.width, c.inner), norm, norm),
        BlockSpec("toy.3", nope, SwiGLUSpec(c.width, c.inner), norm, norm),
    ]
    # block 1 runs twice (two states), block 3 runs twice: once with its own cache, once reading block 0's
    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(3), ScheduleEntry(1),
                ScheduleEntry(3, reads=0)]
    return ModelSpec("ToyForCausalLM", c.vocab, c.width, blocks, schedule, norm, embed_name="toy.embed",
                     final_norm_prefix="toy.final", head_name="toy.head", max_position=c.positions)


register_architecture("ToyForCausalLM", ToyConfig.from_dict, toy_spec)

TOY = {"architectures": ["ToyForCausalLM"], "toy_width": 72, "toy_vocab": 211, "toy_heads": 6, "toy_kv_heads": 2,
       "toy_head": 16, "toy_inner": 40, "toy_experts": 3, "toy_window": 21, "toy_positions": 200, "toy_eps": 1e-5}


def plain_toy(c: ToyConfig, w, ids):
    """The toy model on a whole sequence, from plain_impl's parts."""
    t = len(ids)
    r = w["toy.embed"].float()[torch.tensor(ids)]
    pos = torch.arange(t)

    def attn(r, p, kv=None, qk_norm=False, cos_sin=None, rd=0, window=None, scale=None):
        x = plain_impl.rms_norm(r, w[f"{p}.input_layernorm.weight"], c.eps)
        q = (x @ w[f"{p}.self_attn.q_proj.weight"].float().t()).view(t, c.heads, c.head)
        k = (x @ w[f"{p}.self_attn.k_proj.weight"].float().t()).view(t, c.kv_heads, c.head)
        v = (x @ w[f"{p}.self_attn.v_proj.weight"].float().t()).view(t, c.kv_heads, c.head)
        if qk_norm:
            q = plain_impl.rms_norm(q, w[f"{p}.self_attn.q_norm.weight"], c.eps)
            k = plain_impl.rms_norm(k, w[f"{p}.self_attn.k_norm.weight"], c.eps)
        if cos_sin is not None:
            q = plain_impl.apply_rope_neox(q, *cos_sin, rd)
            k = plain_impl.apply_rope_neox(k, *cos_sin, rd)
        own = (k, v)
        if kv is not None:
            k, v = kv
        o = plain_impl.causal_attention(q, k, v, scale or c.head ** -0.5, window)
        return r + o.reshape(t, -1) @ w[f"{p}.self_attn.o_proj.weight"].float().t(), own

    def swiglu(r, p):
        y = plain_impl.rms_norm(r, w[f"{p}.post_attention_layernorm.weight"], c.eps)
        return r + plain_impl.swiglu_part(y, w, f"{p}.mlp")

    def mean_block(r):
        p = "toy.1"
        x = plain_impl.rms_norm(r, w[f"{p}.input_layernorm.weight"], c.eps)
        u = x @ w[f"{p}.mean.w_in"].float().t()
        r = r + (torch.cumsum(u, 0) / torch.arange(1, t + 1)[:, None]) @ w[f"{p}.mean.w_out"].float().t()
        y = plain_impl.rms_norm(r, w[f"{p}.post_attention_layernorm.weight"], c.eps)
        choice = torch.argmax(y @ w[f"{p}.routed.router"].float().t(), -1)
        out = torch.zeros_like(y)
        for e in range(c.experts):
            sel = choice == e
            out[sel] = torch.relu(y[sel] @ w[f"{p}.routed.experts.{e}.up"].float().t()) @ w[f"{p}.routed.experts.{e}.down"].float().t()
        return r + out

    half = plain_impl.rope_cos_sin(pos / 2.0, plain_impl.rope_inv_freq(c.head // 2, 777.0))
    r, kv0 = attn(r, "toy.0", qk_norm=True, cos_sin=half, rd=c.head // 2)
    r = swiglu(r, "toy.0")
    r = mean_block(r)
    r, _ = attn(r, "toy.2", cos_sin=plain_impl.rope_cos_sin(pos, plain_impl.rope_inv_freq(c.head, 1000.0)), rd=c.head,
                window=c.window, scale=0.2)
    r = swiglu(r, "toy.2")
    r, _ = attn(r, "toy.3")
    r = swiglu(r, "toy.3")
    r = mean_block(r)
    r, _ = attn(r, "toy.3", kv=kv0)
    r = swiglu(r, "toy.3")
    return plain_impl.rms_norm(r, w["toy.final.weight"], c.eps) @ w["toy.head"].float().t()


@pytest.mark.parametrize("device", DEVICES)
def test_toy_architecture_builds_and_steps(device):
    from lily_b200.config.registry import resolve_architecture
    arch = resolve_architecture(TOY["architectures"])
    cfg = arch.config_from_dict(TOY, {}, architecture=arch.name)
    specs = expected_tensors(cfg, arch)
    source = RandomSource(specs, seed=3, dtype=torch.float32, device="cpu", std=0.08, gain_jitter=0.05)
    weights = {n: source.get(n) for n in specs}
    args = ServerArgs(dtype="float32", device=device, max_total_tokens=12 * 8, page_size=8, max_running_requests=4)
    runner = ModelRunner(arch.build_spec(cfg), source, args, ops=kernel_refs if device == "cpu" else None)
    # two cache groups (the two full-attention blocks share one need; the windowed block has its own), two states
    assert len(runner.cache.groups) == 2 and [n for _, n in runner.model.cache_groups] == [2, 1]
    assert len(runner.cache.states) == 2 and runner.cache.states[0].shape == (5, 41)
    reqs = {k: tiny_models.random_tokens(n, 211, 130 + i) for i, (k, n) in enumerate({"a": 60, "b": 35, "c": 50}.items())}
    plain = {k: plain_toy(cfg, weights, ids) for k, ids in reqs.items()}
    tol = 2e-4
    assert float((run_whole(runner, reqs["a"]) - plain["a"]).abs().max()) < tol
    assert float((run_portions(runner, reqs["a"], [28] + [1] * 32) - plain["a"]).abs().max()) < tol
    assert float((run_portions(runner, reqs["c"], [7, 2, 19, 3, 2]) - plain["c"]).abs().max()) < tol
    plan = [{"a": 30}, {"a": 1, "b": 20}, {"b": 15, "a": 1, "c": 9}, {"a": 28, "c": 2}, {"c": 39}]
    got = run_mixed(runner, reqs, plan, {2: ["b"], 3: ["a"]})
    for k in reqs:
        assert float((got[k] - plain[k]).abs().max()) < tol, k
    # the windowed group gave pages back while requests lived, and everything is back at the end
    assert runner.cache.held_pages() == [0, 0] and runner.cache.slots.available == 4


# ------------------------------------------------------------------ a second toy: what decodes through CUDA graphs

@dataclass
class Toy2Config:
    width: int
    vocab: int
    inner: int
    positions: int
    eps: float

    @classmethod
    def from_dict(cls, cfg, generation=None, architecture=None):
        return cls(**{k: cfg[f"toy2_{k}"] for k in cls.__dataclass_fields__})


def toy2_spec(c: Toy2Config) -> ModelSpec:
    """Two attention groups of different head sizes (6 x 16 over 2 kv heads; 2 x 32 over 1), a mixer with state
    that a captured step can reach, a parallel-residual block with a spec class of its own, a windowed layer whose
    cache a layer with a shorter window reads, a scaled embedding and scaled, soft-capped logits."""
    norm = RMSNormSpec(c.width, c.eps)
    small = AttentionSpec(c.width, 6, 2, 16, position=RopeSpec(16, 16, 1000.0))
    wide = AttentionSpec(c.width, 2, 1, 32, qk_norm=True, norm_eps=c.eps, position=RopeSpec(32, 32, 5000.0))
    owner = AttentionSpec(c.width, 6, 2, 16, window=21, position=RopeSpec(16, 16, 1000.0))
    reader = AttentionSpec(c.width, 6, 2, 16, window=10)
    ff = SwiGLUSpec(c.width, c.inner)
    blocks = [
        BlockSpec("t2.0", small, ff, norm, norm),
        BlockSpec("t2.1", DeviceMeanMixerSpec(c.width, c.inner), ff, norm, norm, mixer_name="mean"),
        ParallelBlockSpec("t2.2", wide, ff, norm),
        BlockSpec("t2.3", owner, ff, norm, norm),
        BlockSpec("t2.4", reader, ff, norm, norm),
    ]
    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(3), ScheduleEntry(1),
                ScheduleEntry(4, reads=3)]
    return ModelSpec("Toy2ForCausalLM", c.vocab, c.width, blocks, schedule, norm, embed_name="t2.embed",
                     final_norm_prefix="t2.final", head_name=None, max_position=c.positions,
                     embed_scale=3.0, logit_scale=0.5, logit_softcap=2.0)


register_architecture("Toy2ForCausalLM", Toy2Config.from_dict, toy2_spec)

TOY2 = {"architectures": ["Toy2ForCausalLM"], "toy2_width": 64, "toy2_vocab": 173, "toy2_inner": 128,
        "toy2_positions": 256, "toy2_eps": 1e-5}


def plain_toy2(c: Toy2Config, w, ids):
    t = len(ids)
    r = 3.0 * w["t2.embed"].float()[torch.tensor(ids)]
    pos = torch.arange(t)

    def attention(x, p, heads, kv_heads, head, theta=None, qk_norm=False, window=None, kv=None):
        q = (x @ w[f"{p}.q_proj.weight"].float().t()).view(t, heads, head)
        k = (x @ w[f"{p}.k_proj.weight"].float().t()).view(t, kv_heads, head)
        v = (x @ w[f"{p}.v_proj.weight"].float().t()).view(t, kv_heads, head)
        if qk_norm:
            q = plain_impl.rms_norm(q, w[f"{p}.q_norm.weight"], c.eps)
            k = plain_impl.rms_norm(k, w[f"{p}.k_norm.weight"], c.eps)
        if theta is not None:
            cs = plain_impl.rope_cos_sin(pos, plain_impl.rope_inv_freq(head, theta))
            q, k = plain_impl.apply_rope_neox(q, *cs, head), plain_impl.apply_rope_neox(k, *cs, head)
        own = (k, v)
        if kv is not None:
            k, v = kv
        o = plain_impl.causal_attention(q, k, v, head ** -0.5, window)
        return o.reshape(t, -1) @ w[f"{p}.o_proj.weight"].float().t(), own

    def prenorm(r, p, mixer):
        a, own = mixer(plain_impl.rms_norm(r, w[f"{p}.input_layernorm.weight"], c.eps))
        r = r + a
        y = plain_impl.rms_norm(r, w[f"{p}.post_attention_layernorm.weight"], c.eps)
        return r + plain_impl.swiglu_part(y, w, f"{p}.mlp"), own

    def mean(x):
        u = x @ w["t2.1.mean.w_in"].float().t()
        return (torch.cumsum(u, 0) / torch.arange(1, t + 1)[:, None]) @ w["t2.1.mean.w_out"].float().t(), None

    r, _ = prenorm(r, "t2.0", lambda x: attention(x, "t2.0.self_attn", 6, 2, 16, theta=1000.0))
    r, _ = prenorm(r, "t2.1", mean)
    x = plain_impl.rms_norm(r, w["t2.2.ln.weight"], c.eps)
    r = r + attention(x, "t2.2.attn", 2, 1, 32, theta=5000.0, qk_norm=True)[0] + plain_impl.swiglu_part(x, w, "t2.2.ff")
    r, kv3 = prenorm(r, "t2.3", lambda x: attention(x, "t2.3.self_attn", 6, 2, 16, theta=1000.0, window=21))
    r, _ = prenorm(r, "t2.1", mean)
    r, _ = prenorm(r, "t2.4", lambda x: attention(x, "t2.4.self_attn", 6, 2, 16, window=10, kv=kv3))
    logits = 0.5 * (plain_impl.rms_norm(r, w["t2.final.weight"], c.eps) @ w["t2.embed"].float().t())
    return 2.0 * torch.tanh(logits / 2.0)


@pytest.mark.parametrize("device", DEVICES)
def test_second_toy_decodes_through_graphs(device):
    from lily_b200.config.registry import resolve_architecture
    arch = resolve_architecture(TOY2["architectures"])
    cfg = arch.config_from_dict(TOY2, {}, architecture=arch.name)
    specs = expected_tensors(cfg, arch)
    source = RandomSource(specs, seed=5, dtype=torch.float32, device="cpu", std=0.08, gain_jitter=0.05)
    weights = {n: source.get(n) for n in specs}
    args = ServerArgs(dtype="float32", device=device, max_total_tokens=40 * 8, page_size=8, max_running_requests=6)
    runner = ModelRunner(arch.build_spec(cfg), source, args, ops=kernel_refs if device == "cpu" else None)
    # three cache groups: 2 x 16 all keys, 1 x 32 all keys, 2 x 16 over a window (the reading layer has no layer of
    # its own); two states (the mean block runs twice)
    assert [(n.kv_heads, n.head_dim, n.window, layers) for n, layers in runner.model.cache_groups] == \
        [(2, 16, None, 1), (1, 32, None, 1), (2, 16, 21, 1)]
    assert len(runner.cache.states) == 2 and runner.model.graph_safe
    reqs = {k: tiny_models.random_tokens(n, 173, 230 + i) for i, (k, n) in enumerate({"a": 80, "b": 55, "c": 64}.items())}
    plain = {k: plain_toy2(cfg, weights, ids) for k, ids in reqs.items()}
    tol = 2e-4
    assert float((run_whole(runner, reqs["a"]) - plain["a"]).abs().max()) < tol
    before = runner.graph_steps
    assert float((run_portions(runner, reqs["a"], [48] + [1] * 32) - plain["a"]).abs().max()) < tol
    assert float((run_portions(runner, reqs["c"], [7, 2, 19, 3, 2]) - plain["c"]).abs().max()) < tol
    # three live requests decoding side by side (the state rows of their slots, a padded fourth row on slot 0)
    plan = [{"a": 30, "b": 20, "c": 41}] + [{"a": 1, "b": 1, "c": 1}] * 23 + [{"a": 27, "b": 12}]
    got = run_mixed(runner, reqs, plan)
    for k in reqs:
        assert float((got[k] - plain[k]).abs().max()) < tol, k
    if device == "cuda":
        assert runner.graph_steps - before == 32 + 23         # every all-decode step was a replay
    assert runner.cache.held_pages() == [0, 0, 0] and runner.cache.slots.available == 6


def test_a_wider_look_back_may_not_read_a_windowed_cache():
    """A windowed group gives pages back as its window passes them: a layer that looks further back than the
    owner keeps (or over all keys) must not read that cache."""
    from lily_b200.models.assembled import AssembledModel
    from lily_b200.parts.base import BuildContext
    c = Toy2Config.from_dict(TOY2)
    spec = toy2_spec(c)
    ctx = BuildContext(device=torch.device("cpu"), dtype=torch.float32, ops=kernel_refs, page_size=8, max_position=64)
    AssembledModel(spec, ctx)                                                   # window 10 reads window 21: fine
    for window in (None, 22):
        spec.blocks[4] = BlockSpec("t2.4", AttentionSpec(c.width, 6, 2, 16, window=window), SwiGLUSpec(c.width, c.inner),
                                   RMSNormSpec(c.width, c.eps), RMSNormSpec(c.width, c.eps))
        with pytest.raises(ValueError, match="reads a cache that keeps the last 21"):
            AssembledModel(spec, ctx)
