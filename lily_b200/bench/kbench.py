"""Per-kernel timing against the roofline, in the manner of the reference's bench/kbench.py:1-15:
CUDA-event timing after warm-up, inputs rotated through several copies so that nothing is served
from L2, results as achieved GB/s or TFLOP/s and as a fraction of the measured peaks.

    python -m lily_b200.bench.kbench attention_decode --batch 8 --ctx 4096
    python -m lily_b200.bench.kbench attention_decode_fused --batch 8 --ctx 4096   (from the qkv product's partial sums)
    python -m lily_b200.bench.kbench attention_prefill --tokens 2048
    python -m lily_b200.bench.kbench add_rmsnorm --tokens 8
    python -m lily_b200.bench.kbench silu_mul --tokens 2048
    python -m lily_b200.bench.kbench rope --tokens 2048
    python -m lily_b200.bench.kbench linear --tokens 8 --n 4096 --k 12288          (library product)
    python -m lily_b200.bench.kbench linear_split --tokens 8 --n 4096 --k 12288    (this package's decode product)
    python -m lily_b200.bench.kbench swiglu_skinny --tokens 8 --n 24576 --k 4096   (decode gate/up product + SiLU*mul)
    python -m lily_b200.bench.kbench gemm_tc --tokens 2048 --n 6144 --k 4096       (tcgen05 product)
    python -m lily_b200.bench.kbench gemm_tc_silu --tokens 2048 --n 24576 --k 4096 (tcgen05 product + SiLU*mul)

Sizes default to the Qwen3-8B layer (32 query heads, 8 kv heads, head size 128, width 4096,
intermediate 12288); every size is a flag.  ``--reps 1 --copies 1`` gives a run small enough for a
profiler capture.

The launches of a timing loop follow one another under programmatic dependent launch, so the blocks of the next
launch fill the places that a ragged last round of this one leaves idle: a kernel that runs in one and a bit rounds
of blocks looks better here than between other kernels of a step (decode attention of 64 rows in one block a row:
168 us here, 179 us in the step).  What decides a plan is the step (``bench.step_profile``).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))

            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif k in ("hbm_gbs", "bf16_tflops") and isinstance(v, (int, float)):
                        out[k] = float(v)
                        out["source"] = "measured"
            walk(raw)
        except (OSError, ValueError):
            pass
    return out


def time_ms(fns, reps, warmup=3, graph=False):
    """Mean milliseconds of one call, cycling through ``fns`` (copies of the same work on different
    memory).  With ``graph`` the calls are captured once and replayed, which takes the host's launch
    cost out of the time of a kernel of a few microseconds."""
    for i in range(max(warmup, len(fns))):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        rounds = max(1, reps // len(fns))
        start.record()
        for _ in range(rounds):
            g.replay()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / (rounds * len(fns))
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(reps):
        fns[i % len(fns)]()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / reps


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["attention_decode", "attention_decode_fused", "attention_prefill", "add_rmsnorm", "silu_mul", "rope", "linear", "linear_split", "gemm_tc", "gemm_tc_silu", "swiglu_skinny", "swiglu_library"])
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--prefix", type=int, default=0)
    ap.add_argument("--nq", type=int, default=32)
    ap.add_argument("--nkv", type=int, default=8)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=12288)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--page", type=int, default=64)
    ap.add_argument("--splits", type=int, default=0, help="0: the engine's choice")
    ap.add_argument("--stages", type=int, default=0, help="attention_decode: key/value tiles a block holds (0: the default; 3)")
    ap.add_argument("--reps", type=int, default=50)
    ap.add_argument("--copies", type=int, default=4)
    ap.add_argument("--no-graph", action="store_true", help="launch from the host each time instead of replaying a graph")
    ap.add_argument("--rows64", action="store_true", help="attention_prefill: the mma.sync kernel (tiles of 64 rows) where the tcgen05 kernel would run")
    a = ap.parse_args()

    from lily_b200.csrc import ops
    from lily_b200.csrc.ops import choose_decode_splits

    dev = "cuda"
    dt = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    item = 2 if dt == torch.bfloat16 else 4
    pk = peaks()
    g = torch.Generator(device=dev).manual_seed(0)
    fns, bytes_moved, flops = [], 0.0, 0.0

    if a.kernel in ("attention_decode", "attention_decode_fused", "attention_prefill"):
        decode = a.kernel != "attention_prefill"
        reqs = a.batch if decode else 1
        total_len = a.ctx if decode else a.prefix + a.tokens
        width = -(-total_len // a.page)
        for _ in range(a.copies):
            cache = torch.randn(reqs * width + 1, 2, a.nkv, a.page, a.d, device=dev, generator=g).to(dt)
            table = (torch.randperm(reqs * width, device=dev, generator=g) + 1).view(reqs, width).to(torch.int32)
            if decode:
                q = torch.randn(reqs, a.nq * a.d, device=dev, generator=g).to(dt)
                out = torch.empty_like(q)
                seq = torch.full((reqs,), a.ctx, device=dev, dtype=torch.int32)
                splits = a.splits or choose_decode_splits(reqs, a.nkv, a.ctx, clusters=lambda n: ops.decode_clusters(a.d, n, a.nq // a.nkv))
                scratch = torch.empty(max(1, ops.decode_scratch_floats(reqs, a.nq, a.d, splits)), device=dev)
                if a.kernel == "attention_decode_fused":
                    # the projection's result as the skinny product leaves it: float32 partial sums over 6 slices of k
                    qkv = torch.randn(6, reqs, (a.nq + 2 * a.nkv) * a.d, device=dev, generator=g)
                    gain = torch.ones(a.d, device=dev, dtype=dt)
                    cos = torch.rand(a.ctx, a.d // 2, device=dev, generator=g)
                    sin = torch.rand(a.ctx, a.d // 2, device=dev, generator=g)
                    fns.append(lambda qkv=qkv, gain=gain, cos=cos, sin=sin, cache=cache, table=table, seq=seq, out=out,
                               scratch=scratch: ops.attention_decode_fused(qkv, gain, gain, 1e-6, cos, sin, cache, table, seq, out,
                                                                           scratch, splits, a.nq, a.nkv, a.d, a.d, a.page, a.d ** -0.5,
                                                                           stages=a.stages))
                    continue
                fns.append(lambda q=q, cache=cache, table=table, seq=seq, out=out, scratch=scratch: ops.attention_decode(
                    q, cache, table, seq, out, scratch, splits, a.nq, a.nkv, a.d, a.page, a.d ** -0.5, stages=a.stages))
            else:
                q = torch.randn(a.tokens, a.nq * a.d, device=dev, generator=g).to(dt)
                out = torch.empty_like(q)
                rows = ops.prefill_tile_rows(dt, a.d) if a.rows64 else ops.prefill_tile_rows(dt, a.d, a.page, a.tokens)
                starts = list(range(0, a.tokens, rows))
                treq = torch.zeros(len(starts), device=dev, dtype=torch.int32)
                tstart = torch.tensor(starts, device=dev, dtype=torch.int32)
                cu = torch.tensor([0, a.tokens], device=dev, dtype=torch.int32)
                pre = torch.tensor([a.prefix], device=dev, dtype=torch.int32)
                fns.append(lambda q=q, cache=cache, table=table, out=out, treq=treq, tstart=tstart, cu=cu, pre=pre:
                           ops.attention_prefill(q, cache, table, cu, pre, treq, tstart, out, a.nq, a.nkv, a.d, a.page,
                                                 a.d ** -0.5, tile_rows=rows))
        if decode:
            bytes_moved = reqs * a.ctx * 2 * a.nkv * a.d * item + 2 * reqs * a.nq * a.d * item
            flops = 4.0 * reqs * a.nq * a.d * a.ctx
            extra = {"splits": splits}
        else:
            pairs = a.tokens * a.prefix + a.tokens * (a.tokens + 1) / 2
            flops = 4.0 * a.nq * a.d * pairs
            bytes_moved = (a.prefix + a.tokens) * 2 * a.nkv * a.d * item + 2 * a.tokens * a.nq * a.d * item
            extra = {"tile_rows": rows}
    elif a.kernel == "add_rmsnorm":
        for _ in range(a.copies):
            r = torch.randn(a.tokens, a.hidden, device=dev, generator=g)
            dlt = torch.randn(a.tokens, a.hidden, device=dev, generator=g).to(dt)
            w = torch.ones(a.hidden, device=dev, dtype=dt)
            fns.append(lambda r=r, dlt=dlt, w=w: ops.add_rmsnorm(r, dlt, w, 1e-6, dt))
            if a.splits > 1:       # the delta as float32 partial sums of a split-k product
                parts = torch.randn(a.splits, a.tokens, a.hidden, device=dev, generator=g)
                fns[-1] = lambda r=r, parts=parts, w=w: ops.add_rmsnorm(r, parts, w, 1e-6, dt)
        bytes_moved = a.tokens * a.hidden * (8 + 2 * item)
        extra = {}
    elif a.kernel == "silu_mul":
        for _ in range(a.copies):
            gu = torch.randn(a.tokens, 2 * a.inter, device=dev, generator=g).to(dt)
            fns.append(lambda gu=gu: ops.silu_mul(gu))
        bytes_moved = a.tokens * 3 * a.inter * item
        extra = {}
    elif a.kernel == "rope":
        width = -(-a.tokens // a.page)
        for _ in range(a.copies):
            qkv = torch.randn(a.tokens, (a.nq + 2 * a.nkv) * a.d, device=dev, generator=g).to(dt)
            cache = torch.zeros(width + 1, 2, a.nkv, a.page, a.d, device=dev, dtype=dt)
            table = (torch.arange(width, device=dev, dtype=torch.int32) + 1).view(1, width)
            pos = torch.arange(a.tokens, device=dev, dtype=torch.int32)
            req = torch.zeros(a.tokens, device=dev, dtype=torch.int32)
            cos = torch.rand(a.tokens, a.d // 2, device=dev, generator=g)
            sin = torch.rand(a.tokens, a.d // 2, device=dev, generator=g)
            gain = torch.ones(a.d, device=dev, dtype=dt)
            fns.append(lambda qkv=qkv, cache=cache, table=table, pos=pos, req=req, cos=cos, sin=sin, gain=gain:
                       ops.qk_norm_rope_write(qkv, gain, gain, 1e-6, cos, sin, pos, req, table, cache, a.nq, a.nkv, a.d,
                                              a.d, a.page))
        bytes_moved = a.tokens * ((a.nq + 2 * a.nkv) * a.d * item * 2 + a.d * 4)
        extra = {}
    else:
        for _ in range(a.copies):
            x = torch.randn(a.tokens, a.k, device=dev, generator=g).to(dt)
            w = torch.randn(a.n, a.k, device=dev, generator=g).to(dt)
            if a.kernel == "swiglu_skinny":          # n is the fused matrix's height, 2 x intermediate
                need = ops.swiglu_skinny_need(a.tokens, a.n // 2, a.k, dt, 128, whenever_possible=True)
                scratch = torch.empty(need[0], device=dev)
                counters = torch.zeros(need[1], device=dev, dtype=torch.int32)
                fns.append(lambda x=x, w=w, scratch=scratch, counters=counters: ops.swiglu_skinny(x, w, 128, scratch, counters))
            elif a.kernel == "swiglu_library":       # what it replaces: the library product and the SiLU*mul kernel
                fns.append(lambda x=x, w=w: ops.silu_mul(ops.linear(x, w), block=128))
            elif a.kernel == "linear_split":
                fns.append(lambda x=x, w=w: ops.linear_split(x, w, splits=a.splits or None))
            elif a.kernel == "gemm_tc":
                fns.append(lambda x=x, w=w: ops.gemm_tc(x, w))
            elif a.kernel == "gemm_tc_silu":
                fns.append(lambda x=x, w=w: ops.gemm_tc(x, w, silu_mul_block=True))
            else:
                fns.append(lambda x=x, w=w: ops.linear(x, w))
        bytes_moved = (a.n * a.k + a.tokens * (a.n + a.k)) * item
        flops = 2.0 * a.tokens * a.n * a.k
        extra = {}

    ms = time_ms(fns, a.reps, graph=not a.no_graph)
    out = {"kernel": a.kernel, "dtype": a.dtype, "ms": round(ms, 5), "GB/s": round(bytes_moved / ms / 1e6, 1),
           "hbm_frac": round(bytes_moved / ms / 1e6 / pk["hbm_gbs"], 4), "peaks": pk["source"], **extra}
    if flops:
        out["TFLOP/s"] = round(flops / ms / 1e9, 2)
        out["tensor_frac"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 4)
    out["args"] = {k: v for k, v in vars(a).items() if k != "kernel"}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
