"""Each part of the model alone on the GPU (norm, position tables, attention mixer over the paged
cache, feed-forward, block), built through the registry from its spec, against the plain
implementation's function for that part, in float32 and in bfloat16."""

import pytest
import torch

import plain_impl
import tiny_models
from lily_b200.cache.kv_cache import KVCacheManager
from lily_b200.config.model_config import RopeScaling
from lily_b200.engine.batch import StepEntry, Workspace, build_step_batch
from lily_b200.parts.attention import AttentionSpec, LayerCache
from lily_b200.parts.base import BlockSpec, BuildContext, RunSlots, build_part
from lily_b200.parts.mlp import SwiGLUSpec
from lily_b200.parts.norm import RMSNormSpec
from lily_b200.parts.rope import RopeSpec

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]


def ctx(dtype, max_position=512):
    from lily_b200.csrc import ops
    return BuildContext(device=DEV, dtype=dtype, ops=ops, page_size=16, max_position=max_position)


def tol(dtype):
    return dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)


def loader(weights, dtype):
    return lambda name: weights[name].to(device=DEV, dtype=dtype if weights[name].dim() > 1 else torch.float32)


def rnd(g, *shape, scale=1.0):
    return torch.randn(*shape, generator=g) * scale


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    g = torch.Generator().manual_seed(0)
    w = {"n.weight": 1 + 0.1 * rnd(g, 136)}
    part = build_part("norm", RMSNormSpec(136, 3e-6), "n", ctx(dtype))
    part.load(loader(w, dtype))
    resid, delta = rnd(g, 9, 136), rnd(g, 9, 136).to(dtype)
    r = resid.to(DEV)
    out = part.forward(r, delta.to(DEV))
    want_r = resid + delta.float()
    torch.testing.assert_close(r.cpu(), want_r, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(out.float().cpu(), plain_impl.rms_norm(want_r, w["n.weight"], 3e-6), **tol(dtype))
    rows = torch.tensor([8, 2], dtype=torch.int32, device=DEV)
    out = part.forward(r, None, rows=rows)
    torch.testing.assert_close(out.float().cpu(), plain_impl.rms_norm(want_r[[8, 2]], w["n.weight"], 3e-6), **tol(dtype))


def test_rope_tables_part():
    scaling = RopeScaling("llama3", 8.0, 1.0, 4.0, 64)
    part = build_part("position", RopeSpec(32, 24, 500000.0, scaling), "p", ctx(torch.float32, 300))
    cos, sin = part.tables()
    inv = plain_impl.llama3_inv_freq(plain_impl.rope_inv_freq(24, 500000.0), 8.0, 1.0, 4.0, 64)
    c, s = plain_impl.rope_cos_sin(torch.arange(300), inv)
    assert cos.shape == (300, 12) and part.rotary_dim == 24
    torch.testing.assert_close(cos.cpu(), c, atol=1e-6, rtol=0)
    torch.testing.assert_close(sin.cpu(), s, atol=1e-6, rtol=0)


def attention_weights(g, hidden, nq, nkv, d, qk_norm, bias, prefix="a"):
    w = {f"{prefix}.q_proj.weight": rnd(g, nq * d, hidden, scale=hidden ** -0.5),
         f"{prefix}.k_proj.weight": rnd(g, nkv * d, hidden, scale=hidden ** -0.5),
         f"{prefix}.v_proj.weight": rnd(g, nkv * d, hidden, scale=hidden ** -0.5),
         f"{prefix}.o_proj.weight": rnd(g, hidden, nq * d, scale=(nq * d) ** -0.5)}
    if bias:
        for n, rows in (("q", nq * d), ("k", nkv * d), ("v", nkv * d), ("o", hidden)):
            w[f"{prefix}.{n}_proj.bias"] = rnd(g, rows, scale=0.1)
    if qk_norm:
        w[f"{prefix}.q_norm.weight"] = 1 + 0.1 * rnd(g, d)
        w[f"{prefix}.k_norm.weight"] = 1 + 0.1 * rnd(g, d)
    return w


def one_request_batch(cache, tokens_per_step, prefix_len, slot):
    """A StepBatch that brings `tokens_per_step` tokens of the request in `slot` after `prefix_len` cached ones."""
    cache.grow(slot, prefix_len + tokens_per_step)
    tables = [[cache.block_table(g, slot)] for g in range(len(cache.groups))]
    return build_step_batch([StepEntry(slot, [0] * tokens_per_step, [])], [prefix_len], tables, DEV,
                            workspace=Workspace(DEV))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,nq,nkv,d,qk_norm,bias,window,rotary", [
    (64, 4, 2, 16, True, False, None, 16), (120, 5, 1, 80, False, True, None, 40), (256, 8, 2, 128, True, False, 37, 128),
    (96, 6, 3, 64, False, False, None, 0)])
def test_attention_part_over_the_cache(dtype, hidden, nq, nkv, d, qk_norm, bias, window, rotary):
    g = torch.Generator().manual_seed(1)
    c = ctx(dtype)
    pos = RopeSpec(d, rotary, 10000.0) if rotary else None
    spec = AttentionSpec(hidden, nq, nkv, d, qk_norm=qk_norm, norm_eps=1e-5, bias=bias, window=window, position=pos)
    part = build_part("mixer", spec, "a", c)
    w = attention_weights(g, hidden, nq, nkv, d, qk_norm, bias)
    if dtype == torch.bfloat16:
        w = {k: (v.bfloat16().float() if v.dim() > 1 or "bias" in k else v) for k, v in w.items()}
    part.load(loader(w, dtype))
    need = part.cache_need()
    assert (need.kv_heads, need.head_dim, need.window) == (nkv, d, window)
    cache = KVCacheManager([(need, 1)], [], page_size=16, num_pages=12, max_requests=2, max_context=192, dtype=dtype, device=DEV)
    t = 150
    x = rnd(g, t, hidden).to(dtype)
    # plain: whole sequence
    pc = dict(heads=nq, kv_heads=nkv, head_dim=d, qk_norm=qk_norm, eps=1e-5, rotary_dim=rotary)
    cos, sin = plain_impl.rope_cos_sin(torch.arange(t), plain_impl.rope_inv_freq(rotary, 10000.0)) if rotary else (torch.ones(t, 0), torch.zeros(t, 0))
    want = plain_impl.attention_part(x.float(), w, "a", pc, cos, sin, window)
    # engine part: a portion, then two tokens, then one by one (decode kernel), over the paged cache
    slot = cache.open_request()
    got, done = [], 0
    for n in [97, 2] + [1] * (t - 99):
        batch = one_request_batch(cache, n, done, slot)
        got.append(part.forward(x[done:done + n].to(DEV).contiguous(), batch, LayerCache(0, cache.groups[0].data[0])))
        if got[-1].dim() == 3:
            got[-1] = got[-1].sum(0)
        done += n
        cache.advance(slot, done)
    torch.testing.assert_close(torch.cat(got).float().cpu(), want, **tol(dtype))
    cache.close_request(slot)
    assert cache.held_pages() == [0]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,inter,tokens", [(64, 128, 5), (136, 200, 70), (256, 384, 130), (512, 1408, 9)])
def test_swiglu_part(dtype, hidden, inter, tokens):
    g = torch.Generator().manual_seed(2)
    w = {"m.gate_proj.weight": rnd(g, inter, hidden, scale=hidden ** -0.5), "m.up_proj.weight": rnd(g, inter, hidden, scale=hidden ** -0.5),
         "m.down_proj.weight": rnd(g, hidden, inter, scale=inter ** -0.5)}
    if dtype == torch.bfloat16:
        w = {k: v.bfloat16().float() for k, v in w.items()}
    part = build_part("feed_forward", SwiGLUSpec(hidden, inter), "m", ctx(dtype))
    part.load(loader(w, dtype))
    x = rnd(g, tokens, hidden).to(dtype)
    from types import SimpleNamespace
    step = SimpleNamespace(workspace=Workspace(DEV))              # what the part asks of a step: scratch for its kernels
    out = part.forward(x.to(DEV), step)
    if out.dim() == 3:
        out = out.sum(0)
    torch.testing.assert_close(out.float().cpu(), plain_impl.swiglu_part(x.float(), w, "m"), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block(dtype):
    cfg = tiny_models.TINY_QWEN3
    weights = tiny_models.make_weights(cfg, 5, std=0.1, norm_jitter=0.1)
    if dtype == torch.bfloat16:
        weights = {k: (v.bfloat16().float() if v.dim() > 1 else v) for k, v in weights.items()}
    pc = plain_impl.read_config(cfg)
    rope = RopeSpec(16, 16, 10000.0)
    spec = BlockSpec("model.layers.1", AttentionSpec(64, 4, 2, 16, qk_norm=True, norm_eps=1e-6, position=rope),
                     SwiGLUSpec(64, 128), RMSNormSpec(64, 1e-6), RMSNormSpec(64, 1e-6))
    c = ctx(dtype)
    block = build_part("block", spec, spec.prefix, c)
    assert sorted(block.tensors()) == sorted(k for k in weights if k.startswith("model.layers.1."))
    block.load(loader(weights, dtype))
    cache = KVCacheManager([(block.mixer.cache_need(), 1)], [], page_size=16, num_pages=8, max_requests=2, max_context=128, dtype=dtype, device=DEV)
    g = torch.Generator().manual_seed(3)
    t = 40
    r0, d0 = rnd(g, t, 64), rnd(g, t, 64).to(dtype)
    cos, sin = plain_impl.rope_cos_sin(torch.arange(t), plain_impl.rope_inv_freq(16, 10000.0))
    want_r = plain_impl.decoder_block(r0 + d0.float(), weights, 1, pc, cos, sin)
    slot = cache.open_request()
    batch = one_request_batch(cache, t, 0, slot)
    r = r0.to(DEV)
    delta = block.forward(r, d0.to(DEV), batch, RunSlots([LayerCache(0, cache.groups[0].data[0])], [None]))
    if delta.dim() == 3:
        delta = delta.sum(0)
    torch.testing.assert_close((r + delta.float()).cpu(), want_r, **tol(dtype))
