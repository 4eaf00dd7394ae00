"""Plain, slow implementation of the Llama / Qwen3 dense decoder, for tests only.

Whole sequences, no cache, one function per part; float32 on the CPU unless the
weights lie on another device (it follows them) or ``precision(torch.float64)`` is
in force (the rounding-free yardstick for large layer sizes).  It is
written from the formulas of CodeMan62/lily (each function cites the file and
lines it restates) and shares no code with ``lily_b200``: it reads the raw
``config.json`` dictionary and the checkpoint's own tensor names
(``model.layers.N.self_attn.q_proj.weight`` ...), never the engine's typed
configuration, loader, packed weights or kernels.

``tests/golden/make_golden.py`` compares it once with the reference's own model
code on the CPU for two tiny random models; the outputs of that run are stored
beside the script and checked by ``tests/test_plain_impl.py``.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

Tensor = torch.Tensor

_COMPUTE = [torch.float32]


class precision:
    """``with precision(torch.float64):`` sums and activations in that dtype (the rotation angles stay float32,
    as lily/layers/rotary.py:49-56 computes them)."""

    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        _COMPUTE.append(self.dtype)

    def __exit__(self, *exc):
        _COMPUTE.pop()


def _c(t: Tensor) -> Tensor:
    return t.to(_COMPUTE[-1])


# --------------------------------------------------------------------------- config

def read_config(cfg: dict) -> dict:
    """Numbers the model needs, with the reference's defaults.

    lily/models/model_config.py:85-170 (head_dim default :98, kv heads :99,
    rope_theta and rope_parameters :101-105, ``type`` alias :108-109, eps :148,
    tie :147, max positions :128,153, partial rotary :151-152 (the key itself, else
    the one inside rope_parameters), bias :156).
    QK-norm is switched by the architecture name, lily/models/qwen3.py:17-37.
    """
    text = cfg.get("text_config", cfg)
    heads = text["num_attention_heads"]
    hidden = text["hidden_size"]
    rope_scaling = text.get("rope_scaling")
    rope_params = text.get("rope_parameters")
    theta = text.get("rope_theta", 10000.0)
    if rope_params:
        theta = rope_params.get("rope_theta", theta)
        if rope_params.get("rope_type", "default") != "default":
            rope_scaling = dict(rope_params)
    if rope_scaling is not None and "rope_type" not in rope_scaling and "type" in rope_scaling:
        rope_scaling = {**rope_scaling, "rope_type": rope_scaling["type"]}
    head_dim = text.get("head_dim") or hidden // heads
    return dict(
        arch=cfg.get("architectures", [""])[0],
        hidden=hidden,
        layers=text["num_hidden_layers"],
        heads=heads,
        kv_heads=text.get("num_key_value_heads") or heads,
        head_dim=head_dim,
        inter=text["intermediate_size"],
        vocab=text["vocab_size"],
        eps=text.get("rms_norm_eps", 1e-6),
        theta=float(theta),
        rope_scaling=rope_scaling,
        rotary_dim=int(head_dim * float(text.get("partial_rotary_factor",
                                                 (rope_params or {}).get("partial_rotary_factor", 1.0)))),
        tie=bool(text.get("tie_word_embeddings", cfg.get("tie_word_embeddings", False))),
        bias=bool(text.get("attention_bias", False)),
        act=text.get("hidden_act", "silu"),
        qk_norm=cfg.get("architectures", [""])[0] == "Qwen3ForCausalLM",
    )


# --------------------------------------------------------------------------- norm

def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """lily/layers/layernorm.py:37-44: variance over the last axis in float32,
    ``x * rsqrt(var + eps)``, then the weight."""
    xf = _c(x)
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    return _c(weight) * (xf * torch.rsqrt(var + eps))


# --------------------------------------------------------------------------- rotary

def rope_inv_freq(rotary_dim: int, base: float) -> Tensor:
    """lily/layers/rotary.py:49-50."""
    return 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))


def llama3_inv_freq(inv_freq: Tensor, factor: float, low_freq_factor: float,
                    high_freq_factor: float, original_max_position: int) -> Tensor:
    """lily/layers/rotary.py:99-119: long wavelengths are slowed by ``factor``,
    short ones kept, the band between them blended."""
    low_wavelen = original_max_position / low_freq_factor
    high_wavelen = original_max_position / high_freq_factor
    wavelen = 2 * math.pi / inv_freq
    if low_freq_factor != high_freq_factor:
        smooth = (original_max_position / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    else:
        smooth = 0
    blended = (1 - smooth) * inv_freq / factor + smooth * inv_freq
    return torch.where(wavelen < high_wavelen, inv_freq,
                       torch.where(wavelen > low_wavelen, inv_freq / factor, blended))


def model_inv_freq(c: dict) -> Tensor:
    """Selection of the scaling, lily/layers/rotary.py:196-207."""
    inv = rope_inv_freq(c["rotary_dim"], c["theta"])
    rs = c["rope_scaling"]
    if rs is None or rs.get("rope_type", "default") == "default":
        return inv
    if rs["rope_type"] == "llama3":
        return llama3_inv_freq(inv, rs["factor"], rs["low_freq_factor"], rs["high_freq_factor"],
                               rs["original_max_position_embeddings"])
    raise ValueError(f"plain implementation has no rope type {rs['rope_type']!r}")


def rope_cos_sin(positions: Tensor, inv_freq: Tensor):
    """lily/layers/rotary.py:52-56: angle = position * inv_freq in float32."""
    freqs = torch.outer(positions.to(torch.float32), inv_freq.to(positions.device))
    return _c(freqs.cos()), _c(freqs.sin())


def apply_rope_neox(x: Tensor, cos: Tensor, sin: Tensor, rotary_dim: int) -> Tensor:
    """lily/layers/rotary.py:18-20,70-87: rotate-half over the first
    ``rotary_dim`` features of each head; the rest passes through.
    x: [T, heads, head_dim]; cos, sin: [T, rotary_dim/2]."""
    rot, rest = x[..., :rotary_dim], x[..., rotary_dim:]
    c = torch.cat((cos, cos), dim=-1).unsqueeze(1)
    s = torch.cat((sin, sin), dim=-1).unsqueeze(1)
    x1, x2 = rot.chunk(2, dim=-1)
    rotated = torch.cat((-x2, x1), dim=-1)
    return torch.cat((rot * c + rotated * s, rest), dim=-1)


# --------------------------------------------------------------------------- attention

def causal_attention(q: Tensor, k: Tensor, v: Tensor, scale: float,
                     window: Optional[int] = None) -> Tensor:
    """lily/layers/attention/torch_native_backend.py:31-37,52-64 with the whole
    sequence as the portion: query head h reads kv head ``h // (heads/kv_heads)``,
    scores ``q.k * scale``, a key is seen when its position is <= the query's
    (and, with ``window``, > query - window), softmax over keys, then ``p.v``.
    q: [T, heads, d]; k, v: [T, kv_heads, d] -> [T, heads, d]."""
    t, heads, d = q.shape
    rep = heads // k.shape[1]
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, kk) * scale
    pos = torch.arange(t, device=q.device)
    seen = pos[None, :] <= pos[:, None]
    if window is not None:
        seen &= pos[None, :] > pos[:, None] - window
    scores = scores.masked_fill(~seen[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vv)


def attention_part(x: Tensor, w: Dict[str, Tensor], prefix: str, c: dict, cos: Tensor, sin: Tensor,
                   window: Optional[int] = None) -> Tensor:
    """lily/models/llama.py:85-90 and lily/models/qwen3.py:24-32: projections,
    per-head q/k RMSNorm (Qwen3 only) before the rotation, attention with
    scale head_dim^-0.5 (llama.py:65), output projection."""
    t = x.shape[0]
    nq, nkv, d = c["heads"], c["kv_heads"], c["head_dim"]

    def proj(name, inp):
        out = inp @ _c(w[f"{prefix}.{name}.weight"]).t()
        b = w.get(f"{prefix}.{name}.bias")
        return out if b is None else out + _c(b)

    q = proj("q_proj", x).view(t, nq, d)
    k = proj("k_proj", x).view(t, nkv, d)
    v = proj("v_proj", x).view(t, nkv, d)
    if c["qk_norm"]:
        q = rms_norm(q, w[f"{prefix}.q_norm.weight"], c["eps"])
        k = rms_norm(k, w[f"{prefix}.k_norm.weight"], c["eps"])
    q = apply_rope_neox(q, cos, sin, c["rotary_dim"])
    k = apply_rope_neox(k, cos, sin, c["rotary_dim"])
    o = causal_attention(q, k, v, d ** -0.5, window)
    return proj("o_proj", o.reshape(t, nq * d))


# --------------------------------------------------------------------------- feed-forward

def swiglu_part(x: Tensor, w: Dict[str, Tensor], prefix: str) -> Tensor:
    """lily/models/llama.py:42-47: ``down(silu(gate(x)) * up(x))``, no bias."""
    g = x @ _c(w[f"{prefix}.gate_proj.weight"]).t()
    u = x @ _c(w[f"{prefix}.up_proj.weight"]).t()
    return (torch.nn.functional.silu(g) * u) @ _c(w[f"{prefix}.down_proj.weight"]).t()


# --------------------------------------------------------------------------- block and model

def decoder_block(r: Tensor, w: Dict[str, Tensor], layer: int, c: dict, cos: Tensor, sin: Tensor) -> Tensor:
    """lily/models/llama.py:108-117 with the fused-add convention unrolled:
    ``r += attn(norm_in(r)); r += mlp(norm_post(r))``."""
    p = f"model.layers.{layer}"
    r = r + attention_part(rms_norm(r, w[f"{p}.input_layernorm.weight"], c["eps"]), w, f"{p}.self_attn", c, cos, sin)
    r = r + swiglu_part(rms_norm(r, w[f"{p}.post_attention_layernorm.weight"], c["eps"]), w, f"{p}.mlp")
    return r


def hidden_states(cfg: dict, w: Dict[str, Tensor], token_ids: Sequence[int]) -> Tensor:
    """lily/models/llama.py:136-147: embedding rows, the blocks in order, final norm."""
    c = read_config(cfg)
    if c["act"] != "silu":
        raise ValueError(c["act"])  # lily/models/llama.py:39-40
    table = w["model.embed_tokens.weight"]
    ids = torch.tensor(list(token_ids), dtype=torch.long, device=table.device)
    r = _c(table[ids])
    cos, sin = rope_cos_sin(torch.arange(len(ids), device=table.device), model_inv_freq(c))
    for layer in range(c["layers"]):
        r = decoder_block(r, w, layer, c, cos, sin)
    return rms_norm(r, w["model.norm.weight"], c["eps"])


def all_logits(cfg: dict, w: Dict[str, Tensor], token_ids: Sequence[int]) -> Tensor:
    """Logits at every position, [T, vocab] float32.  lily/layers/vocab_embedding.py:89-96;
    a tied head reads the embedding table (lily/models/llama.py:175-176)."""
    c = read_config(cfg)
    head = w["model.embed_tokens.weight"] if c["tie"] else w["lm_head.weight"]
    return hidden_states(cfg, w, token_ids) @ _c(head).t()


def greedy_generate(cfg: dict, w: Dict[str, Tensor], prompt: Sequence[int], n: int) -> List[int]:
    """lily/engine.py:113-131 without the cache: argmax of the last position,
    append, run the whole sequence again."""
    ids = list(prompt)
    out: List[int] = []
    for _ in range(n):
        tok = int(torch.argmax(all_logits(cfg, w, ids)[-1]))
        out.append(tok)
        ids.append(tok)
    return out


# --------------------------------------------------------------------------- sampling

def penalised(logits: Tensor, seen: Sequence[int], repetition: float = 1.0, frequency: float = 0.0,
              presence: float = 0.0, bias: Optional[Dict[int, float]] = None) -> Tensor:
    """lily/layers/sampler.py:64-87 for one row: repetition penalty on the set of
    seen tokens, then frequency and presence penalties by count, then the bias."""
    x = logits.clone().float()
    if repetition != 1.0 and seen:
        u = torch.tensor(sorted(set(seen)))
        vals = x[u]
        x[u] = torch.where(vals > 0, vals / repetition, vals * repetition)
    if (frequency or presence) and seen:
        counts = torch.bincount(torch.tensor(list(seen)), minlength=x.shape[-1]).float()
        x = x - counts * frequency - (counts > 0).float() * presence
    if bias:
        for k, b in bias.items():
            x[int(k)] += float(b)
    return x


def filtered_probs(logits: Tensor, temperature: float, top_k: int = -1, top_p: float = 1.0,
                   min_p: float = 0.0) -> Tensor:
    """lily/layers/sampler.py:97-112 for one row, returned in vocabulary order:
    ``logits / max(T, 1e-5)``, keep the top_k largest, softmax over them, keep the
    sorted prefix whose mass before each member is < top_p, drop what is below
    ``min_p * max``, renormalise."""
    vocab = logits.shape[-1]
    x = logits.float() / max(temperature, 1e-5)
    if 0 < top_k < vocab:
        values, indices = torch.topk(x, top_k)
    else:
        values, indices = torch.sort(x, descending=True)
    probs = torch.softmax(values, dim=-1)
    if top_p < 1.0:
        cum = torch.cumsum(probs, dim=-1)
        keep = cum - probs < top_p
        keep[0] = True
        probs = torch.where(keep, probs, torch.zeros_like(probs))
    if min_p > 0.0:
        probs = torch.where(probs >= min_p * probs.max(), probs, torch.zeros_like(probs))
    probs = probs / probs.sum()
    out = torch.zeros(vocab)
    out[indices] = probs
    return out


def inverse_cdf_pick(probs: Tensor, u: float) -> int:
    """The draw the engine specifies for itself (the reference draws with
    ``torch.multinomial`` and a per-request generator, lily/layers/sampler.py:114):
    the first token, in vocabulary order, whose cumulative probability exceeds ``u``."""
    cum = torch.cumsum(probs.double(), dim=-1)
    idx = int(torch.searchsorted(cum, torch.tensor(u, dtype=torch.float64) * cum[-1], right=True))
    nz = torch.nonzero(probs > 0).flatten()
    return min(max(idx, int(nz[0])), int(nz[-1]))
