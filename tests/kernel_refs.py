"""Plain PyTorch statements of what each CUDA kernel computes, with the kernels' signatures.

Two uses, both in tests only: (1) each kernel is compared with its function here on the GPU, at
sizes other than the engine's; (2) handed to the engine as ``ops`` on the CPU they let the cache
manager, batch packing, step function, scheduler and replay be tested without a device.  They
compute in float32 and round once to the output dtype.  Nothing in ``lily_b200`` imports this.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

launches = {"count": 0}        # the kernels' Python faces count their launches here; these statements launch nothing
TC_MIN_ROWS = 65               # as the kernels: products of this many rows and more take the fused gate/up epilogue


def gate_up_fused_pays(rows, fused_rows):
    return rows >= TC_MIN_ROWS
FUSE_DECODE = True             # tests flip this to send all-decode steps through either form of the attention


def library():
    return None


def sm_count():
    return 148


def _sum(t):
    """Kernels that take a product take it whole or as float32 partial sums [splits, rows, cols]."""
    return t.sum(0) if t.dim() == 3 else t


def embed(table, ids, out=None, future=None, scale=1.0):
    ids = ids.long()
    if future is not None:
        ids = torch.where(ids < 0, future.long()[(-ids - 1).clamp(min=0)], ids)
    return table[ids].float() * scale


def logit_transform(logits, scale=1.0, softcap=None):
    logits.mul_(scale)
    if softcap:
        logits.copy_(softcap * torch.tanh(logits / softcap))
    return logits


def scatter_tokens(tokens, logit_rows, token_req, slots, future):
    n = tokens.numel()
    future[slots.long()[token_req.long()[logit_rows.long()[:n]]]] = tokens.to(future.dtype)


def add_rmsnorm(resid, delta, weight, eps, out_dtype, rows=None, write_residual=True, out=None):
    if delta is not None:
        delta = _sum(delta)
    if rows is not None:
        v = resid[rows.long()]
        if delta is not None:
            v = v + delta[rows.long()].float()
    else:
        if delta is not None:
            if write_residual:
                resid += delta.float()
                v = resid
            else:
                v = resid + delta.float()
        else:
            v = resid
    var = v.pow(2).mean(-1, keepdim=True)
    return ((v * torch.rsqrt(var + eps)) * weight.float()).to(out_dtype)


def silu_mul(gate_up, out_dtype=None, out=None, block=None):
    out_dtype = out_dtype or gate_up.dtype
    gate_up = _sum(gate_up)
    i = gate_up.shape[1] // 2
    if block:
        runs = gate_up.view(gate_up.shape[0], i // block, 2, block)
        g, u = runs[:, :, 0].reshape(-1, i).float(), runs[:, :, 1].reshape(-1, i).float()
    else:
        g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
    return ((g / (1 + torch.exp(-g))) * u).to(out_dtype)


def qk_norm_rope_write(qkv, q_gain, k_gain, eps, cos, sin, positions, token_req, block_table, kv_layer, nq, nkv, d,
                       rotary_dim, page_size, write_kv=True, q_out=None):
    qkv = _sum(qkv)
    n = qkv.shape[0]
    x = qkv.float().view(n, nq + 2 * nkv, d)
    q, k, v = x[:, :nq], x[:, nq:nq + nkv], x[:, nq + nkv:]

    def norm(t, gain):
        if gain is None:
            return t
        return (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)) * gain.float()

    def rot(t):
        if cos is None:
            return t
        half = rotary_dim // 2
        c = cos[positions.long()].unsqueeze(1)
        s = sin[positions.long()].unsqueeze(1)
        x1, x2, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
        return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, rest), dim=-1)

    q = rot(norm(q, q_gain))
    if write_kv:
        k = rot(norm(k, k_gain))
        pos = positions.long()
        page = block_table[token_req.long(), pos // page_size].long()
        within = pos % page_size
        kv_layer[page, 0, :, within] = k.to(kv_layer.dtype)
        kv_layer[page, 1, :, within] = v.to(kv_layer.dtype)
    return q.reshape(n, nq * d).to(kv_layer.dtype)


def cast(x, dtype):
    return x.to(dtype)


def linear(x, weight, bias=None, out_dtype=None):
    out = x.float() @ weight.float().t()
    if bias is not None:
        out = out + bias.float()
    return out.to(out_dtype or x.dtype)


def linear_split(x, weight, splits=None):
    """For a few tokens the product comes as float32 partial sums over slices of K (here: two halves)."""
    m, k = x.shape
    if m > 16 or k % 2 or (splits is not None and splits < 1):
        return None
    n = splits or 2
    if k % n:
        return None
    xs, ws = x.float().view(m, n, k // n), weight.float().view(-1, n, k // n)
    return torch.einsum("msk,nsk->smn", xs, ws).contiguous()


def linear_auto(x, weight, bias=None):
    if bias is None:
        parts = linear_split(x, weight)
        if parts is not None:
            return parts
    return linear(x, weight, bias)


def swiglu_skinny_need(tokens, intermediate, hidden, dtype, block=None, whenever_possible=False):
    return (16, 4) if dtype == torch.bfloat16 and tokens <= 8 and hidden % 64 == 0 else None


def swiglu_skinny(x, gate_up, block, scratch, counters, out=None):
    assert int(counters.abs().sum()) == 0           # the kernel finds them zero and leaves them zero
    return silu_mul(linear(x, gate_up, out_dtype=torch.float32), x.dtype, block=block)


def logits(x, head):
    return linear(x, head, out_dtype=torch.float32)


def gate_up_interleave(dtype, intermediate):
    return 128 if dtype == torch.bfloat16 and intermediate % 128 == 0 else None


def gemm_tc_takes(x, weight):
    return x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0


def gemm_tc(x, weight, bias=None, silu_mul_block=False):
    out = linear(x, weight, bias, out_dtype=torch.float32)
    return silu_mul(out, x.dtype, block=128) if silu_mul_block else out.to(x.dtype)


def uses_tensor_cores(dtype, d):
    return dtype == torch.bfloat16 and d in (64, 128, 192, 256)


def prefill_tile_rows(dtype=None, d=0, page_size=0, new_tokens=0):
    return 32


def prefill_tiles(prefix_lens, new_lens, first, rows, device):
    pairs = [(r, s) for r in range(first, len(new_lens)) for s in range(0, new_lens[r], rows)]
    both = torch.tensor([[r for r, _ in pairs], [s for _, s in pairs]], dtype=torch.int32).reshape(2, -1).to(device)
    return both[0].contiguous(), both[1].contiguous()


def decode_clusters(d, splits, group):
    return 0


@dataclass(frozen=True)
class DecodePlan:
    splits: int
    fused: bool
    scratch_floats: int
    arm: str
    stages: int = 0


def plan_decode_attention(dtype, requests, nq, nkv, d, max_seq_len, even=False):
    if requests == 0:
        return DecodePlan(1, False, 0, "single")
    splits = 2 if max_seq_len >= 32 else 1
    return DecodePlan(splits, FUSE_DECODE, decode_scratch_floats(requests, nq, d, splits), "wave" if splits > 1 else "single")


def decode_scratch_floats(requests, nq, d, splits):
    return requests * nq * splits * (d + 2) if splits > 1 else 0


def _gather_kv(kv_layer, table_row, length, page_size):
    pos = torch.arange(length, device=kv_layer.device)
    page = table_row[(pos // page_size)].long()
    k = kv_layer[page, 0, :, pos % page_size]          # [length, nkv, d]
    v = kv_layer[page, 1, :, pos % page_size]
    return k.float(), v.float()


def _attend(q, k, v, q_pos, scale, window):
    """q [rows, nq, d] at positions q_pos [rows]; k, v [keys, nkv, d] at positions 0..keys-1."""
    rep = q.shape[1] // k.shape[1]
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = torch.einsum("qhd,khd->hqk", q, kk) * scale
    kpos = torch.arange(k.shape[0], device=q.device)
    seen = kpos[None, :] <= q_pos[:, None]
    if window:
        seen &= kpos[None, :] > q_pos[:, None] - window
    s = s.masked_fill(~seen[None], float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv)


def attention_prefill(q, kv_layer, block_table, cu_seqlens, prefix_lens, tile_req, tile_start, out, nq, nkv, d,
                      page_size, scale, window=None, tile_rows=None, heads_per_block=0):
    for r in sorted(set(tile_req.tolist())):
        t0, t1 = int(cu_seqlens[r]), int(cu_seqlens[r + 1])
        prefix = int(prefix_lens[r])
        k, v = _gather_kv(kv_layer, block_table[r], prefix + t1 - t0, page_size)
        qpos = torch.arange(prefix, prefix + t1 - t0, device=q.device)
        o = _attend(q[t0:t1].float().view(-1, nq, d), k, v, qpos, scale, window)
        out[t0:t1] = o.reshape(t1 - t0, nq * d).to(out.dtype)


def attention_decode(q, kv_layer, block_table, seq_lens, out, scratch, splits, nq, nkv, d, page_size, scale,
                     window=None, stages=0):
    for r in range(q.shape[0]):
        n = int(seq_lens[r])
        k, v = _gather_kv(kv_layer, block_table[r], n, page_size)
        o = _attend(q[r:r + 1].float().view(1, nq, d), k, v, torch.tensor([n - 1], device=q.device), scale, window)
        out[r] = o.reshape(nq * d).to(out.dtype)


def attention_decode_fused(qkv, q_gain, k_gain, eps, cos, sin, kv_layer, block_table, seq_lens, out, scratch, splits, nq, nkv,
                           d, rotary_dim, page_size, scale, window=None, write_kv=True, stages=0):
    """What the one kernel does, as the two statements it replaces: every request brings one token, at position
    seq_len - 1."""
    qkv = _sum(qkv)
    n = qkv.shape[0]
    q = qk_norm_rope_write(qkv, q_gain, k_gain, eps, cos, sin, (seq_lens - 1).to(torch.int32),
                           torch.arange(n, dtype=torch.int32, device=qkv.device), block_table, kv_layer, nq, nkv, d, rotary_dim,
                           page_size, write_kv=write_kv)
    attention_decode(q.to(out.dtype), kv_layer, block_table, seq_lens, out, scratch, splits, nq, nkv, d, page_size, scale, window)


def argmax(logits, out=None):
    return torch.argmax(logits, dim=-1).to(torch.int32)


def apply_penalties(logits, entry_row, entry_token, entry_count, entry_bias, repetition, frequency, presence):
    for e in range(entry_row.numel()):
        r, t, c = int(entry_row[e]), int(entry_token[e]), int(entry_count[e])
        v = logits[r, t]
        if c > 0:
            rep = repetition[r]
            if rep != 1.0:
                v = v / rep if v > 0 else v * rep
            v = v - c * frequency[r] - presence[r]
        logits[r, t] = v + entry_bias[e]


def sample(logits, temperature, top_k, top_p, min_p, uniform, want_logprob=False):
    import plain_impl

    toks, lps = [], []
    for r in range(logits.shape[0]):
        t, k = float(temperature[r]), int(top_k[r])
        if t == 0 or k == 1:
            tok = int(torch.argmax(logits[r]))
            lp = float(torch.log_softmax(logits[r].float(), -1)[tok])
        else:
            probs = plain_impl.filtered_probs(logits[r].cpu(), t, k, float(top_p[r]), float(min_p[r]))
            tok = plain_impl.inverse_cdf_pick(probs, float(uniform[r]))
            lp = float(torch.log(probs[tok]))
        toks.append(tok)
        lps.append(lp)
    dev = logits.device
    return (torch.tensor(toks, dtype=torch.int32, device=dev),
            torch.tensor(lps, dtype=torch.float32, device=dev) if want_logprob else None)


def top_logprobs_cap():
    return 128


def top_logprobs(logits, k):
    rows, vocab = logits.shape
    cap = top_logprobs_cap()
    tokens = torch.zeros((rows, cap), dtype=torch.int32, device=logits.device)
    logprobs = torch.zeros((rows, cap), dtype=torch.float32, device=logits.device)
    counts = torch.zeros((rows,), dtype=torch.int32, device=logits.device)
    lp = torch.log_softmax(logits.float(), -1)
    for r in range(rows):
        kk = min(int(k[r]), cap, vocab)
        if kk <= 0:
            continue
        kth = torch.topk(lp[r], kk).values[-1]
        idx = torch.nonzero(lp[r] >= kth).flatten()[:cap]
        counts[r] = idx.numel()
        tokens[r, :idx.numel()] = idx.to(torch.int32)
        logprobs[r, :idx.numel()] = lp[r, idx]
    return tokens, logprobs, counts
