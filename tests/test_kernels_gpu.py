"""Each CUDA kernel alone against its plain PyTorch statement (tests/kernel_refs.py), at sizes
other than the engine's: odd widths, head sizes in steps of 16, any grouping, windows, page edges."""

import os

import pytest
import torch

import kernel_refs as ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from lily_b200.csrc import ops as o
    return o


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


DTYPES = [torch.float32, torch.bfloat16]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(64, 256), (136, 331), (4096, 1009)])
def test_embed(dtype, hidden, vocab):
    g = torch.Generator(device=DEV).manual_seed(0)
    table = torch.randn(vocab, hidden, device=DEV, generator=g).to(dtype)
    ids = torch.randint(0, vocab, (37,), device=DEV, generator=g, dtype=torch.int32)
    assert torch.equal(ops().embed(table, ids), ref.embed(table, ids))
    # ids below zero name request slots whose token the sampler left on the device
    future = torch.randint(0, vocab, (9,), device=DEV, generator=g, dtype=torch.int32)
    mixed = ids.clone()
    mixed[::3] = -(torch.arange(0, 13, device=DEV, dtype=torch.int32) % 9 + 1)
    assert torch.equal(ops().embed(table, mixed, future=future), ref.embed(table, mixed, future=future))
    assert torch.equal(ops().embed(table, mixed, future=future)[0], table[future[0].long()].float())


def test_scatter_tokens():
    g = torch.Generator(device=DEV).manual_seed(17)
    tokens = torch.randint(0, 1000, (5,), device=DEV, generator=g, dtype=torch.int32)
    logit_rows = torch.tensor([0, 1, 2, 9, 30], device=DEV, dtype=torch.int32)        # three decode tokens, two portions' ends
    token_req = torch.tensor([0, 1, 2] + [3] * 7 + [4] * 21, device=DEV, dtype=torch.int32)
    slots = torch.tensor([4, 1, 7, 2, 5], device=DEV, dtype=torch.int32)
    a = torch.full((9,), -5, device=DEV, dtype=torch.int32)
    b = a.clone()
    ops().scatter_tokens(tokens, logit_rows, token_req, slots, a)
    ref.scatter_tokens(tokens, logit_rows, token_req, slots, b)
    assert torch.equal(a, b) and a[4] == tokens[0] and a[5] == tokens[4] and a[0] == -5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("wdtype", DTYPES)
@pytest.mark.parametrize("hidden", [64, 136, 1000, 4096, 12288])
def test_add_rmsnorm(dtype, wdtype, hidden):
    if dtype == torch.float32 and wdtype == torch.bfloat16:
        pytest.skip("float32 activations keep float32 gains")
    g = torch.Generator(device=DEV).manual_seed(1)
    n = 19
    resid = torch.randn(n, hidden, device=DEV, generator=g) * 3
    delta = torch.randn(n, hidden, device=DEV, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, device=DEV, generator=g)).to(wdtype)
    for d in (delta, None):
        r1, r2 = resid.clone(), resid.clone()
        got = ops().add_rmsnorm(r1, d, w, 1e-5, dtype)
        want = ref.add_rmsnorm(r2, d, w, 1e-5, dtype)
        torch.testing.assert_close(r1, r2, atol=0, rtol=0)
        torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
    rows = torch.tensor([18, 0, 7, 7], device=DEV, dtype=torch.int32)
    r1 = resid.clone()
    got = ops().add_rmsnorm(r1, delta, w, 1e-6, dtype, rows=rows)
    want = ref.add_rmsnorm(resid.clone(), delta, w, 1e-6, dtype, rows=rows)
    assert torch.equal(r1, resid)                       # gathered rows leave the residual alone
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [128, 200, 352, 12288])
def test_silu_mul(dtype, inter):
    g = torch.Generator(device=DEV).manual_seed(2)
    gu = (torch.randn(23, 2 * inter, device=DEV, generator=g) * 2).to(dtype)
    torch.testing.assert_close(ops().silu_mul(gu).float(), ref.silu_mul(gu).float(), **tol(dtype))


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (7, 331, 136), (65, 129, 200), (33, 1009, 4096), (300, 24, 17)])
def test_gemm_fp32_is_true_fp32(m, n, k):
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn(m, k, device=DEV, generator=g)
    w = torch.randn(n, k, device=DEV, generator=g)
    b = torch.randn(n, device=DEV, generator=g)
    want = (x.double() @ w.double().t() + b.double()).float()
    got = ops().linear(x, w, b)
    # float32 accumulation error grows like sqrt(k) * 2^-24 * |x||w|; TF32 would be ~1e-3 relative
    assert float((got - want).abs().max()) < 4e-6 * (k ** 0.5) * 4
    # a row's result does not depend on the other rows in the batch
    assert torch.equal(ops().linear(x[:1].contiguous(), w, b), got[:1])


def test_linear_bf16_and_fp32_logits():
    g = torch.Generator(device=DEV).manual_seed(4)
    x = torch.randn(9, 136, device=DEV, generator=g).bfloat16()
    w = torch.randn(331, 136, device=DEV, generator=g).bfloat16()
    b = torch.randn(331, device=DEV, generator=g).bfloat16()
    want = x.float() @ w.float().t()
    torch.testing.assert_close(ops().linear(x, w).float(), want, atol=0.1, rtol=2e-2)
    out = ops().linear(x, w, out_dtype=torch.float32)
    assert out.dtype == torch.float32
    torch.testing.assert_close(out, want, atol=1e-3, rtol=1e-4)       # logits keep the accumulator's precision
    # the product may be rounded to bfloat16 before the bias is added: half an ulp at its magnitude (~64)
    torch.testing.assert_close(ops().linear(x, w, b).float(), want + b.float(), atol=0.5, rtol=2e-2)


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (8, 6144, 4096), (8, 4096, 12288), (5, 331, 128), (16, 1000, 256),
                                   (17, 136, 64), (33, 2000, 1024), (64, 4096, 1024), (3, 24576, 4096), (64, 24, 64),
                                   (8, 5120, 25600), (16, 4096, 12288),                                     # a long slice of x
                                   (1, 5120, 25600), (2, 5120, 25600), (3, 10240, 8192), (3, 300, 16384)])   # x read from global memory
def test_skinny_gemm_partial_sums(m, n, k):
    g = torch.Generator(device=DEV).manual_seed(11)
    x = torch.randn(m, k, device=DEV, generator=g).bfloat16()
    w = torch.randn(n, k, device=DEV, generator=g).bfloat16()
    parts = ops().linear_split(x, w, splits=max(1, min(5, k // 512)))
    assert parts is not None and parts.dtype == torch.float32 and parts.shape[1:] == (m, n)
    auto = ops().linear_split(x, w)                     # the kernel's own rule may leave the shape to the library
    if auto is not None:
        torch.testing.assert_close(auto.sum(0), parts.sum(0), atol=2e-5 * (k ** 0.5) * 4, rtol=1e-4)       # other slices, other rounding
    want = x.double() @ w.double().t()
    got = parts.double().sum(0)
    assert float((got - want).abs().max()) < 2e-5 * (k ** 0.5) * 4      # float32 accumulation of exact products
    # a token's result does not depend on the other tokens in the batch
    alone = ops().linear_split(x[:1].contiguous(), w, splits=parts.shape[0])
    assert torch.equal(alone[:, 0], parts[:, 0])
    # shapes the kernel does not take are left to the library product
    assert ops().linear_split(torch.zeros(65, k, device=DEV).bfloat16(), w) is None
    assert ops().linear_split(torch.zeros(2, 72, device=DEV).bfloat16(), torch.zeros(8, 72, device=DEV).bfloat16()) is None
    assert ops().linear_split(x.float(), w.float()) is None


SWIGLU_SHAPES = [(8, 12288, 4096, 128), (1, 12288, 4096, 128), (5, 1408, 512, 128), (8, 200, 64, None),
                 (3, 264, 1088, 8), (7, 25600, 5120, 128), (8, 352, 128, None), (2, 128, 12288, 64)]


def test_skinny_swiglu_with_x_from_global_memory():
    """The kernel's other form (the lanes read x from global memory; taken when x of a block's stretch does not fit
    beside the rings) on every shape: the form is chosen by an environment variable read once, so a fresh process."""
    import subprocess, sys
    code = (f"import sys; sys.path.insert(0, {os.path.dirname(os.path.abspath(__file__))!r}); import test_kernels_gpu as t\n"
            "for shape in t.SWIGLU_SHAPES: t.test_skinny_swiglu(*shape)")
    done = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, LILY_B200_SWIGLU_X="global"),
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]


@pytest.mark.parametrize("m,inter,k,run", SWIGLU_SHAPES)
def test_skinny_swiglu(m, inter, k, run):
    """The gate/up product with SiLU*mul in one weight-streaming kernel against the plain statement: tall and low
    matrices (row blocks finished by one block or by several, whose stretches end anywhere), deep k (more units a
    block than a row block has), both layouts of the fused matrix, 1 to 8 tokens; twice over the same scratch, and a
    token's result does not depend on its neighbours."""
    o = ops()
    g = torch.Generator(device=DEV).manual_seed(12)
    x = torch.randn(m, k, device=DEV, generator=g).bfloat16()
    w = (torch.randn(2 * inter, k, device=DEV, generator=g) * k ** -0.5).bfloat16()
    need = o.swiglu_skinny_need(m, inter, k, torch.bfloat16, run, whenever_possible=True)
    assert need is not None
    scratch = torch.full((need[0],), float("nan"), device=DEV)
    counters = torch.zeros(need[1], device=DEV, dtype=torch.int32)
    got = o.swiglu_skinny(x, w, run, scratch, counters)
    gu = x.double() @ w.double().t()
    want = ref.silu_mul(gu.float(), torch.float32, block=run)
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)
    assert float((got.float() - want).abs().mean()) < 2e-3
    assert int(counters.abs().sum()) == 0
    again = o.swiglu_skinny(x, w, run, scratch, counters)
    assert torch.equal(again, got) and int(counters.abs().sum()) == 0
    alone = o.swiglu_skinny(x[:1].contiguous(), w, run, scratch, counters)
    assert torch.equal(alone[0], got[0])
    assert o.swiglu_skinny_need(9, inter, k, torch.bfloat16, run) is None
    # several tokens of an input too wide to stage beside the rings: the kernel takes it, the library pair is preferred
    from_global = os.environ.get("LILY_B200_SWIGLU_X") == "global" or (m, inter, k) == (7, 25600, 5120)
    assert (o.swiglu_skinny_need(m, inter, k, torch.bfloat16, run) is None) == (from_global and m * k > 3 * 8192)
    assert o.swiglu_skinny_need(m, inter, k, torch.float32, run) is None
    assert o.swiglu_skinny_need(m, inter, k + 8, torch.bfloat16, run) is None


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (2048, 6144, 4096), (300, 1000, 136), (65, 331, 200), (1, 24, 8),
                                   (777, 512, 4096), (129, 257, 72), (1100, 5000, 520), (2048, 4096, 12288), (4100, 2500, 72)])
def test_gemm_tcgen05(m, n, k):
    o = ops()
    g = torch.Generator(device=DEV).manual_seed(13)
    x = torch.randn(m, k, device=DEV, generator=g).bfloat16()
    w = torch.randn(n, k, device=DEV, generator=g).bfloat16()
    b = torch.randn(n, device=DEV, generator=g).bfloat16()
    want = x.float() @ w.float().t()
    got = o.gemm_tc(x, w)
    assert o.gemm_tc_status() == 0
    # exact bfloat16 products summed in float32, rounded once to bfloat16
    torch.testing.assert_close(got.float(), want, atol=2e-2 * (k ** 0.5), rtol=1e-2)
    assert float((got.float() - want).abs().max()) <= float(want.abs().max()) * 2 ** -7
    torch.testing.assert_close(o.gemm_tc(x, w, b).float(), want + b.float(), atol=2e-2 * (k ** 0.5) + 0.1, rtol=1e-2)
    assert o.gemm_tc_status() == 0
    assert torch.equal(o.gemm_tc(x, w), got) and o.gemm_tc_status() == 0          # again: the same bits


@pytest.mark.parametrize("m,inter,k", [(128, 128, 64), (2048, 12288, 4096), (300, 384, 136), (70, 256, 4096)])
def test_gemm_tcgen05_silu_mul_epilogue(m, inter, k):
    o = ops()
    g = torch.Generator(device=DEV).manual_seed(14)
    x = (torch.randn(m, k, device=DEV, generator=g) * 0.5).bfloat16()
    gate = (torch.randn(inter, k, device=DEV, generator=g) * (k ** -0.5)).bfloat16()
    up = (torch.randn(inter, k, device=DEV, generator=g) * (k ** -0.5)).bfloat16()
    mixed = torch.stack((gate.view(inter // 128, 128, k), up.view(inter // 128, 128, k)), dim=1).reshape(2 * inter, k).contiguous()
    gt, ut = x.float() @ gate.float().t(), x.float() @ up.float().t()
    want = torch.nn.functional.silu(gt) * ut
    got = o.gemm_tc(x, mixed, silu_mul_block=True)
    assert o.gemm_tc_status() == 0 and got.shape == (m, inter)
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)
    # the same interleaved product through the unfused path: library product, then SiLU*mul in runs of 128
    two = o.linear(x, mixed)
    torch.testing.assert_close(o.silu_mul(two, block=128).float(), want, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(o.silu_mul(two, block=128).float(), ref.silu_mul(two, block=128).float(), atol=2e-2, rtol=2e-2)


def test_kernels_add_up_partial_sums():
    o = ops()
    g = torch.Generator(device=DEV).manual_seed(12)
    m, h, nq, nkv, d, page = 7, 136, 4, 2, 16, 16
    parts = torch.randn(3, m, h, device=DEV, generator=g)
    whole = (parts[0] + parts[1]) + parts[2]
    w = (1 + 0.1 * torch.randn(h, device=DEV, generator=g)).bfloat16()
    r1, r2 = torch.randn(m, h, device=DEV, generator=g), None
    r2 = r1.clone()
    a = o.add_rmsnorm(r1, parts, w, 1e-6, torch.bfloat16)
    b = o.add_rmsnorm(r2, whole, w, 1e-6, torch.bfloat16)
    assert torch.equal(a, b) and torch.equal(r1, r2)
    gu = torch.randn(3, m, 2 * 200, device=DEV, generator=g)
    assert torch.equal(o.silu_mul(gu, torch.bfloat16), o.silu_mul((gu[0] + gu[1]) + gu[2], torch.bfloat16))
    torch.testing.assert_close(o.silu_mul(gu, torch.bfloat16).float(),
                               ref.silu_mul(gu.sum(0)).float(), atol=2e-2, rtol=2e-2)
    qkv = torch.randn(3, m, (nq + 2 * nkv) * d, device=DEV, generator=g)
    pos = torch.arange(m, device=DEV, dtype=torch.int32) + 5
    req = torch.zeros(m, device=DEV, dtype=torch.int32)
    table = torch.tensor([[2, 1]], device=DEV, dtype=torch.int32)
    cos, sin = torch.rand(32, d // 2, device=DEV, generator=g), torch.rand(32, d // 2, device=DEV, generator=g)
    gain = torch.ones(d, device=DEV).bfloat16()
    c1 = torch.zeros(3, 2, nkv, page, d, device=DEV).bfloat16()
    c2 = c1.clone()
    q1 = o.qk_norm_rope_write(qkv, gain, gain, 1e-6, cos, sin, pos, req, table, c1, nq, nkv, d, d, page)
    q2 = o.qk_norm_rope_write((qkv[0] + qkv[1]) + qkv[2], gain, gain, 1e-6, cos, sin, pos, req, table, c2, nq, nkv, d, d, page)
    assert q1.dtype == torch.bfloat16 and torch.equal(q1, q2) and torch.equal(c1, c2) and float(c1.abs().max()) > 0


def _cache(pages, nkv, page_size, d, dtype, g):
    return (torch.randn(pages + 1, 2, nkv, page_size, d, device=DEV, generator=g)).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rd,norm", [(4, 2, 16, 16, True), (8, 2, 32, 32, False), (6, 2, 48, 24, True),
                                               (5, 1, 80, 80, False), (32, 8, 128, 128, True), (3, 3, 256, 64, True),
                                               (7, 7, 64, 64, True), (2, 1, 256, 256, True), (9, 3, 128, 128, False)])
def test_qk_norm_rope_write(dtype, nq, nkv, d, rd, norm):
    g = torch.Generator(device=DEV).manual_seed(5)
    page, n, reqs = 16, 50, 3
    qkv = torch.randn(n, (nq + 2 * nkv) * d, device=DEV, generator=g).to(dtype)
    token_req = torch.tensor([i % reqs for i in range(n)], device=DEV, dtype=torch.int32)
    # distinct (request, position) pairs so that no two tokens write the same place
    positions = torch.arange(n, device=DEV, dtype=torch.int32) + 3
    table = (torch.randperm(reqs * 6, device=DEV, generator=g) + 1).view(reqs, 6).to(torch.int32)
    cos = torch.rand(128, rd // 2, device=DEV, generator=g)
    sin = torch.rand(128, rd // 2, device=DEV, generator=g)
    qg = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)).to(dtype) if norm else None
    kg = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)).to(dtype) if norm else None
    c1 = _cache(18, nkv, page, d, dtype, g)
    c0, c2 = c1.clone(), c1.clone()
    got = ops().qk_norm_rope_write(qkv, qg, kg, 1e-6, cos, sin, positions, token_req, table, c1, nq, nkv, d, rd, page)
    want = ref.qk_norm_rope_write(qkv, qg, kg, 1e-6, cos, sin, positions, token_req, table, c2, nq, nkv, d, rd, page)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
    torch.testing.assert_close(c1.float(), c2.float(), **tol(dtype))
    assert not torch.equal(c1, c0)
    # without rotation tables and without the cache write
    c3 = c1.clone()
    got = ops().qk_norm_rope_write(qkv, qg, kg, 1e-6, None, None, positions, token_req, table, c3, nq, nkv, d, 0, page,
                                   write_kv=False)
    want = ref.qk_norm_rope_write(qkv, qg, kg, 1e-6, None, None, positions, token_req, table, c2.clone(), nq, nkv, d,
                                  0, page, write_kv=False)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
    assert torch.equal(c3, c1)


def _attention_case(dtype, nq, nkv, d, page, prefixes, news, window, seed=6, spike=False):
    g = torch.Generator(device=DEV).manual_seed(seed)
    reqs = len(prefixes)
    width = max(-(-(p + n) // page) for p, n in zip(prefixes, news))
    pages = reqs * width
    cache = _cache(pages, nkv, page, d, dtype, g)
    table = (torch.randperm(pages, device=DEV, generator=g) + 1).view(reqs, width).to(torch.int32)
    total = sum(news)
    q = torch.randn(total, nq * d, device=DEV, generator=g).to(dtype)
    if spike:
        # one far key per request dominates: its key is a scaled copy of the first query of that request
        at = 0
        for r, (p, n) in enumerate(zip(prefixes, news)):
            far = 1 if p + n > 2 else 0
            pg, off = int(table[r, far // page]), far % page
            for h in range(nkv):
                cache[pg, 0, h, off] = (q[at].view(nq, d)[h * (nq // nkv)].float() * 4).to(dtype)
            at += n
    cu = torch.tensor([0] + list(torch.tensor(news).cumsum(0)), device=DEV, dtype=torch.int32)
    pre = torch.tensor(prefixes, device=DEV, dtype=torch.int32)
    return cache, table, q, cu, pre


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page,window", [
    (4, 2, 16, 16, None), (8, 2, 32, 16, None), (6, 2, 48, 8, 40), (5, 1, 80, 32, None), (32, 8, 128, 64, None),
    (2, 2, 256, 16, 100), (16, 2, 64, 16, 33), (40, 1, 32, 16, None), (40, 2, 64, 16, None), (6, 2, 192, 32, 500),
    (8, 8, 128, 8, 64)])
def test_attention_prefill(dtype, nq, nkv, d, page, window):
    prefixes, news = [0, 17, 130, 5, 300, 64], [1, 70, 33, 200, 129, 2]      # lengths of the reference's own test
    cache, table, q, cu, pre = _attention_case(dtype, nq, nkv, d, page, prefixes, news, window, spike=True)
    rows = ops().prefill_tile_rows(dtype, d)
    treq = [r for r, n in enumerate(news) for _ in range(0, n, rows)]
    tstart = [s for r, n in enumerate(news) for s in range(0, n, rows)]
    treq_t = torch.tensor(treq, device=DEV, dtype=torch.int32)
    tstart_t = torch.tensor(tstart, device=DEV, dtype=torch.int32)
    got, want = torch.zeros_like(q), torch.zeros_like(q)
    ops().attention_prefill(q, cache, table, cu, pre, treq_t, tstart_t, got, nq, nkv, d, page, d ** -0.5, window)
    ref.attention_prefill(q, cache, table, cu, pre, treq_t, tstart_t, want, nq, nkv, d, page, d ** -0.5, window)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))


def _tiles_of(news, rows):
    treq = [r for r, n in enumerate(news) for _ in range(0, n, rows)]
    tstart = [s for r, n in enumerate(news) for s in range(0, n, rows)]
    return (torch.tensor(treq, device=DEV, dtype=torch.int32), torch.tensor(tstart, device=DEV, dtype=torch.int32))


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("nq,nkv,page,window", [(8, 2, 64, None), (4, 4, 128, None), (6, 1, 256, None), (4, 2, 64, 200),
                                                 (2, 1, 64, 100), (4, 2, 128, 129), (6, 2, 64, None), (3, 3, 64, 70)])
def test_attention_prefill_tcgen05(nq, nkv, page, window, d):
    """The tcgen05 kernel (tiles of 128 rows; head sizes 128 and 64) against the plain statement: cached prefixes
    that end inside a page and inside a key tile, portions shorter and longer than a tile, one token."""
    o, dtype = ops(), torch.bfloat16
    rows = o.prefill_tile_rows(dtype, d, page, 10 ** 6)
    assert rows == 128 and o.uses_tcgen05_attention(dtype, d, page, 4096) and not o.uses_tcgen05_attention(dtype, d, 16, 4096)
    prefixes, news = [0, 17, 130, 5, 700, 64, 1000], [1, 70, 333, 200, 129, 2, 640]
    cache, table, q, cu, pre = _attention_case(dtype, nq, nkv, d, page, prefixes, news, window, spike=True)
    treq_t, tstart_t = _tiles_of(news, rows)
    got, want = torch.zeros_like(q), torch.zeros_like(q)
    o.attention_prefill(q, cache, table, cu, pre, treq_t, tstart_t, got, nq, nkv, d, page, d ** -0.5, window, tile_rows=rows,
                        heads_per_block=1)
    assert o.attention_tc_status() == 0
    ref.attention_prefill(q, cache, table, cu, pre, treq_t, tstart_t, want, nq, nkv, d, page, d ** -0.5, window)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
    if (nq // nkv) % 2 == 0:
        # the form with two heads of a kv head a block
        both = torch.zeros_like(q)
        o.attention_prefill(q, cache, table, cu, pre, treq_t, tstart_t, both, nq, nkv, d, page, d ** -0.5, window, tile_rows=rows,
                            heads_per_block=2)
        assert o.attention_tc_status() == 0
        torch.testing.assert_close(both.float(), want.float(), **tol(dtype))
    else:
        with pytest.raises(o.KernelError, match="heads a block"):
            o.attention_prefill(q, cache, table, cu, pre, treq_t, tstart_t, torch.zeros_like(q), nq, nkv, d, page, d ** -0.5,
                                window, tile_rows=rows, heads_per_block=2)
    # the mma.sync kernel on the same case, cut into its own tiles, agrees too
    base = o.prefill_tile_rows(dtype, d)
    breq, bstart = _tiles_of(news, base)
    other = torch.zeros_like(q)
    o.attention_prefill(q, cache, table, cu, pre, breq, bstart, other, nq, nkv, d, page, d ** -0.5, window)
    torch.testing.assert_close(got.float(), other.float(), **tol(dtype))


@pytest.mark.parametrize("d", [128, 64])
def test_attention_prefill_tcgen05_rising_scores(d):
    """Scores that grow by far more than 2^8 from one key tile to the next, for every row: the kernel
    must rescale the output in tensor memory each time (the path that ordinary data rarely takes)."""
    o, dtype, nq, nkv, page = ops(), torch.bfloat16, 4, 2, 64
    g = torch.Generator(device=DEV).manual_seed(21)
    prefixes, news = [300, 0], [520, 700]
    cache, table, q, cu, pre = _attention_case(dtype, nq, nkv, d, page, prefixes, news, None, seed=22)
    u = torch.randn(d, device=DEV, generator=g)
    q = (0.5 * q.float().view(-1, nq, d) + u).view(q.shape).to(dtype)
    for r, (p, n) in enumerate(zip(prefixes, news)):
        for pos, c in ((40, 0.25), (190, 0.5), (330, 1.0), (470, 1.5), (p + n - 90, 2.5), (p + n - 3, 4.0)):
            pg, off = int(table[r, pos // page]), pos % page
            cache[pg, 0, :, off] = (c * u).to(dtype)
            cache[pg, 1, :, off] = c
    rows = o.prefill_tile_rows(dtype, d, page, 10 ** 6)
    treq_t, tstart_t = _tiles_of(news, rows)
    want = torch.zeros_like(q)
    ref.attention_prefill(q, cache, table, cu, pre, treq_t, tstart_t, want, nq, nkv, d, page, d ** -0.5, None)
    for heads in (1, 2):
        got = torch.zeros_like(q)
        o.attention_prefill(q, cache, table, cu, pre, treq_t, tstart_t, got, nq, nkv, d, page, d ** -0.5, None, tile_rows=rows,
                            heads_per_block=heads)
        assert o.attention_tc_status() == 0
        torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
    assert float(want.float()[-1].view(nq, d)[0].mean()) > 3.5          # the last row sees the strongest key


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [1, 3, 6, 7, 8, 12, 40, 300])         # 300: past what the combine kernel stages in shared memory
@pytest.mark.parametrize("nq,nkv,d,page,window", [
    (4, 2, 16, 16, None), (8, 2, 32, 16, None), (6, 2, 48, 8, 40), (5, 1, 80, 32, None), (32, 8, 128, 64, None),
    (2, 2, 256, 16, 100), (40, 1, 32, 16, None), (16, 16, 64, 16, 7), (40, 2, 64, 16, None), (6, 2, 192, 32, 500),
    (8, 8, 128, 8, 64)])
def test_attention_decode(dtype, splits, nq, nkv, d, page, window):
    seqs = [1, 8, 65, 500, 1000, 3, 257]                                     # prefixes up to 999, as the reference tests
    prefixes, news = [s - 1 for s in seqs], [1] * len(seqs)
    cache, table, q, cu, pre = _attention_case(dtype, nq, nkv, d, page, prefixes, news, window, seed=7, spike=True)
    seq_t = torch.tensor(seqs, device=DEV, dtype=torch.int32)
    need = ops().decode_scratch_floats(len(seqs), nq, d, splits)
    scratch = torch.full((max(need, 1),), float("nan"), device=DEV)
    got, want = torch.zeros_like(q), torch.zeros_like(q)
    ops().attention_decode(q, cache, table, seq_t, got, scratch, splits, nq, nkv, d, page, d ** -0.5, window)
    ref.attention_decode(q, cache, table, seq_t, want, None, splits, nq, nkv, d, page, d ** -0.5, window)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("from_projection", [False, True])
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("nq,nkv,d,page,window", [(32, 8, 128, 64, None), (8, 2, 64, 16, None), (40, 2, 64, 16, 70), (5, 1, 128, 8, 300)])
def test_attention_decode_with_three_stages(from_projection, splits, nq, nkv, d, page, window):
    """The tensor-core kernel with three key/value tiles a block (the plan's form for many rows of about one length):
    rows of one tile, of two, of exactly the three that are asked for ahead, and longer; a spike in every row; from
    finished queries and from the projection, where the block with the new position writes its key and value first."""
    o = ops()
    dtype = torch.bfloat16
    seqs = [1, 64, 65, 128, 129, 192, 193, 500, 1000, 3, 257]
    cache, table, q, cu, pre = _attention_case(dtype, nq, nkv, d, page, [n - 1 for n in seqs], [1] * len(seqs), window, seed=17, spike=True)
    seq_t = torch.tensor(seqs, device=DEV, dtype=torch.int32)
    scratch = torch.full((max(o.decode_scratch_floats(len(seqs), nq, d, splits), 1),), float("nan"), device=DEV)
    got, want = torch.zeros_like(q), torch.zeros_like(q)
    if not from_projection:
        o.attention_decode(q, cache, table, seq_t, got, scratch, splits, nq, nkv, d, page, d ** -0.5, window, stages=3)
        ref.attention_decode(q, cache, table, seq_t, want, None, splits, nq, nkv, d, page, d ** -0.5, window)
    else:
        g = torch.Generator(device=DEV).manual_seed(171)
        qkv = torch.cat([q, torch.randn(len(seqs), 2 * nkv * d, device=DEV, generator=g).to(dtype)], 1)
        gain = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)).to(dtype)
        cos, sin = torch.rand(1100, d // 2, device=DEV, generator=g), torch.rand(1100, d // 2, device=DEV, generator=g)
        one, two = cache.clone(), cache.clone()
        o.attention_decode_fused(qkv, gain, gain, 1e-6, cos, sin, one, table, seq_t, got, scratch, splits, nq, nkv, d, d, page,
                                 d ** -0.5, window, stages=3)
        o.attention_decode_fused(qkv, gain, gain, 1e-6, cos, sin, two, table, seq_t, want, scratch, splits, nq, nkv, d, d, page,
                                 d ** -0.5, window)
        ref_out = torch.zeros_like(q)
        ref.attention_decode_fused(qkv, gain, gain, 1e-6, cos, sin, cache.clone(), table, seq_t, ref_out, None, splits, nq, nkv, d,
                                   d, page, d ** -0.5, window)
        assert torch.equal(one, two)                                   # the same key and value written
        torch.testing.assert_close(want.float(), ref_out.float(), **tol(dtype))
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
    with pytest.raises(Exception, match="stages"):
        o.attention_decode(q, cache, table, seq_t, got, scratch, splits, nq, nkv, d, page, d ** -0.5, window, stages=4)


def test_three_stages_are_refused_where_they_do_not_fit():
    o = ops()
    nq, nkv, d, page = 2, 2, 256, 16
    cache, table, q, cu, pre = _attention_case(torch.bfloat16, nq, nkv, d, page, [99], [1], None, seed=3)
    seq_t = torch.tensor([100], device=DEV, dtype=torch.int32)
    with pytest.raises(Exception, match="stages"):
        o.attention_decode(q, cache, table, seq_t, torch.zeros_like(q), None, 1, nq, nkv, d, page, d ** -0.5, stages=3)
    cache, table, q, cu, pre = _attention_case(torch.float32, 4, 2, 16, 16, [99], [1], None, seed=3)
    with pytest.raises(Exception, match="stages"):
        o.attention_decode(q, cache, table, seq_t, torch.zeros_like(q), None, 1, 4, 2, 16, 16, 0.25, stages=3)


@pytest.mark.parametrize("requests,longest", [(1, 40000), (2, 30000), (4, 20000)])
def test_attention_decode_of_a_few_long_rows(requests, longest):
    """A few rows of tens of thousands of keys: the plan leaves the clusters (16 blocks a row at most) for one full
    wave of ranges through scratch and the combine kernel, from the qkv product as the engine would run it; one far
    key among them carries the row (its key is the query scaled up)."""
    o = ops()
    dtype, nq, nkv, d, page = torch.bfloat16, 32, 8, 128, 64
    plan = o.plan_decode_attention(dtype, requests, nq, nkv, d, longest)
    assert plan.arm == "wave" and plan.splits > 16 // requests + 8 and plan.fused and plan.scratch_floats > 0
    seqs = [longest - 1777 * i for i in range(requests)]
    cache, table, _, cu, pre = _attention_case(dtype, nq, nkv, d, page, [n - 1 for n in seqs], [1] * requests, None, seed=10)
    g = torch.Generator(device=DEV).manual_seed(92)
    qkv = torch.randn(3, requests, (nq + 2 * nkv) * d, device=DEV, generator=g) * 0.6
    far = 12345                                                     # a position in the middle of some range
    q_sum = qkv.sum(0)
    for r in range(requests):
        pg, off = int(table[r, far // page]), far % page
        for h in range(nkv):
            cache[pg, 0, h, off] = (q_sum[r].view(nq + 2 * nkv, d)[h * (nq // nkv)] * 3).to(dtype)
    seq_t = torch.tensor(seqs, device=DEV, dtype=torch.int32)
    scratch = torch.full((plan.scratch_floats,), float("nan"), device=DEV)
    got, want = (torch.zeros(requests, nq * d, device=DEV, dtype=dtype) for _ in range(2))
    one, two = cache.clone(), cache.clone()
    o.attention_decode_fused(qkv, None, None, 1e-6, None, None, one, table, seq_t, got, scratch, plan.splits, nq, nkv, d, 0,
                             page, d ** -0.5)
    ref.attention_decode_fused(qkv, None, None, 1e-6, None, None, two, table, seq_t, want, None, plan.splits, nq, nkv, d, 0,
                                page, d ** -0.5)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
    torch.testing.assert_close(one.float(), two.float(), atol=2 ** -7, rtol=2 ** -7)
    # the far key matters: without it the heads that look at it give another result
    cache2 = cache.clone()
    for r in range(requests):
        cache2[int(table[r, far // page]), 0, :, far % page] = 0
    other = torch.zeros_like(got)
    o.attention_decode_fused(qkv, None, None, 1e-6, None, None, cache2, table, seq_t, other, scratch, plan.splits, nq, nkv, d, 0,
                             page, d ** -0.5)
    assert float((other.float() - got.float()).abs().max()) > 0.05


@pytest.mark.parametrize("planes", [1, 3])
@pytest.mark.parametrize("splits", [1, 4, 6, 12])
@pytest.mark.parametrize("nq,nkv,d,page,window,rd,gains", [
    (32, 8, 128, 64, None, 128, True), (8, 2, 64, 16, None, 64, False), (40, 2, 64, 16, 70, 32, True),
    (6, 2, 192, 32, None, 0, True), (2, 2, 256, 16, 100, 256, False), (5, 1, 128, 8, None, 128, True)])
def test_attention_decode_from_the_projection(planes, splits, nq, nkv, d, page, window, rd, gains):
    """One kernel from the qkv product to the attention output (bfloat16, tensor-core head sizes) against the two
    kernels it replaces: the same output and the same cache afterwards, with per-head gains or without, full,
    partial or no rotation, a window, the product as bfloat16 or as float32 partial sums, and sequence lengths whose
    new position opens a page, ends one, or is the only one.  (Up to a last bit of bfloat16: the two sum a head's
    squares in different orders.)"""
    o = ops()
    dtype = torch.bfloat16
    seqs = [1, 8, 65, 500, 1000, 3, 257, 64, 129]
    prefixes, news = [n - 1 for n in seqs], [1] * len(seqs)
    cache, table, _, cu, pre = _attention_case(dtype, nq, nkv, d, page, prefixes, news, window, seed=8)
    g = torch.Generator(device=DEV).manual_seed(81)
    n, width = len(seqs), (nq + 2 * nkv) * d
    qkv = torch.randn(planes, n, width, device=DEV, generator=g) * 0.7 if planes > 1 else \
        torch.randn(n, width, device=DEV, generator=g).to(dtype)
    qg = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)).to(dtype) if gains else None
    kg = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)).to(dtype) if gains else None
    cos = torch.rand(1100, rd // 2, device=DEV, generator=g) if rd else None
    sin = torch.rand(1100, rd // 2, device=DEV, generator=g) if rd else None
    seq_t = torch.tensor(seqs, device=DEV, dtype=torch.int32)
    pos = seq_t - 1
    req = torch.arange(n, device=DEV, dtype=torch.int32)
    scratch = torch.full((max(o.decode_scratch_floats(n, nq, d, splits), 1),), float("nan"), device=DEV)
    two, one = cache.clone(), cache.clone()
    q = o.qk_norm_rope_write(qkv, qg, kg, 1e-6, cos, sin, pos, req, table, two, nq, nkv, d, rd, page)
    want = torch.zeros(n, nq * d, device=DEV, dtype=dtype)
    o.attention_decode(q, two, table, seq_t, want, scratch, splits, nq, nkv, d, page, d ** -0.5, window)
    got = torch.zeros_like(want)
    o.attention_decode_fused(qkv, qg, kg, 1e-6, cos, sin, one, table, seq_t, got, scratch, splits, nq, nkv, d, rd, page,
                             d ** -0.5, window)
    last_bit = dict(atol=2 ** -7, rtol=2 ** -7)
    torch.testing.assert_close(one.float(), two.float(), **last_bit, msg="the cache after the step")
    assert float((one.float() - two.float()).abs().gt(0).float().mean()) < 1e-3        # and nearly everywhere the same bits
    torch.testing.assert_close(got.float(), want.float(), **last_bit)
    # and against the plain statement of the fused step itself (float32 inside, rounded once)
    plain_cache, plain_out = cache.clone(), torch.zeros_like(want)
    ref.attention_decode_fused(qkv, qg, kg, 1e-6, cos, sin, plain_cache, table, seq_t, plain_out, None, splits, nq, nkv, d, rd,
                                page, d ** -0.5, window)
    torch.testing.assert_close(one.float(), plain_cache.float(), **last_bit, msg="the cache against the plain statement")
    torch.testing.assert_close(got.float(), plain_out.float(), atol=2e-2, rtol=2e-2)
    # a layer that reads another layer's cache: nothing is written
    kept = two.clone()
    o.attention_decode_fused(qkv * 0.5 if planes > 1 else qkv, qg, kg, 1e-6, cos, sin, kept, table, seq_t, got, scratch, splits,
                             nq, nkv, d, rd, page, d ** -0.5, window, write_kv=False)
    assert torch.equal(kept, two)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page", [(4, 2, 16, 16), (8, 2, 128, 64), (6, 2, 48, 8)])
def test_attention_window_edge_and_page_edge(dtype, nq, nkv, d, page):
    """A key that dominates every score, placed first just inside and then just outside the window
    of the last query (and on the last slot of a page): inside it owns the output, outside it must
    not be seen at all.  Prefill and decode kernels, same cache."""
    o = ops()
    window, seq = 2 * page + 3, 5 * page + 2
    g = torch.Generator(device=DEV).manual_seed(15)
    width = -(-seq // page)
    table = (torch.randperm(width, device=DEV, generator=g) + 1).view(1, width).to(torch.int32)
    q = torch.randn(1, nq * d, device=DEV, generator=g).to(dtype)
    qpos = seq - 1
    for key_pos, inside in ((qpos - window + 1, True), (qpos - window, False), (3 * page - 1, True)):
        cache = (torch.randn(width + 1, 2, nkv, page, d, device=DEV, generator=g) * 0.1).to(dtype)
        pg, off = int(table[0, key_pos // page]), key_pos % page
        for h in range(nkv):
            cache[pg, 0, h, off] = (q.view(nq, d)[h * (nq // nkv)].float() * 8).to(dtype)
            cache[pg, 1, h, off] = 7.0
        for decode in (True, False):
            got, want = torch.zeros_like(q), torch.zeros_like(q)
            seq_t = torch.tensor([seq], device=DEV, dtype=torch.int32)
            if decode:
                scratch = torch.empty(max(1, o.decode_scratch_floats(1, nq, d, 2)), device=DEV)
                o.attention_decode(q, cache, table, seq_t, got, scratch, 2, nq, nkv, d, page, d ** -0.5, window)
                ref.attention_decode(q, cache, table, seq_t, want, None, 2, nq, nkv, d, page, d ** -0.5, window)
            else:
                cu = torch.tensor([0, 1], device=DEV, dtype=torch.int32)
                pre = torch.tensor([seq - 1], device=DEV, dtype=torch.int32)
                z = torch.zeros(1, device=DEV, dtype=torch.int32)
                o.attention_prefill(q, cache, table, cu, pre, z, z, got, nq, nkv, d, page, d ** -0.5, window)
                ref.attention_prefill(q, cache, table, cu, pre, z, z, want, nq, nkv, d, page, d ** -0.5, window)
            torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
            first_head = got.view(nq, d)[0].float()
            if inside:
                assert float((first_head - 7.0).abs().max()) < 0.5, (key_pos, decode)
            else:
                assert float(first_head.abs().max()) < 1.0, (key_pos, decode)


def test_attention_refuses_what_it_cannot_do():
    o = ops()
    q = torch.zeros(1, 2 * 272, device=DEV)
    cache = torch.zeros(2, 2, 2, 16, 272, device=DEV)
    table = torch.ones(1, 1, device=DEV, dtype=torch.int32)
    seq = torch.ones(1, device=DEV, dtype=torch.int32)
    with pytest.raises(o.KernelError, match="head_dim"):
        o.attention_decode(q, cache, table, seq, torch.zeros_like(q), None, 1, 2, 2, 272, 16, 1.0)
    with pytest.raises(o.KernelError, match="CUDA"):
        o.silu_mul(torch.zeros(2, 4))


@pytest.mark.parametrize("vocab", [256, 331, 1009, 151936])
def test_argmax_and_penalties(vocab):
    g = torch.Generator(device=DEV).manual_seed(8)
    logits = torch.randn(5, vocab, device=DEV, generator=g)
    logits[2, vocab - 1] = 50.0
    logits[3, 7] = logits[3, 100] = 40.0                         # a tie goes to the lower index
    got = ops().argmax(logits)
    assert got.tolist() == torch.argmax(logits, -1).tolist() and got[3] == 7 and got[2] == vocab - 1
    rows = torch.tensor([0, 0, 1, 4], device=DEV, dtype=torch.int32)
    toks = torch.tensor([3, 9, 3, vocab - 1], device=DEV, dtype=torch.int32)
    cnt = torch.tensor([2, 0, 1, 5], device=DEV, dtype=torch.int32)
    bias = torch.tensor([0.0, 1.5, -2.0, 0.0], device=DEV)
    rep = torch.tensor([1.3, 1.0, 1.0, 1.0, 2.0], device=DEV)
    freq = torch.tensor([0.1, 0.2, 0.0, 0.0, 0.05], device=DEV)
    pres = torch.tensor([0.5, 0.0, 0.0, 0.0, 0.25], device=DEV)
    a, b = logits.clone(), logits.clone()
    ops().apply_penalties(a, rows, toks, cnt, bias, rep, freq, pres)
    ref.apply_penalties(b, rows, toks, cnt, bias, rep, freq, pres)
    torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("vocab", [256, 1009, 151936])
def test_top_logprobs(vocab):
    g = torch.Generator(device=DEV).manual_seed(23)
    logits = torch.randn(5, vocab, device=DEV, generator=g) * 3
    logits[1, 7] = logits[1, 11] = float(logits[1].max()) + 1.0          # a tie at the top
    ks = [0, 2, 5, 20, 64]
    tokens, lps, counts = ops().top_logprobs(logits, torch.tensor(ks, device=DEV, dtype=torch.int32))
    want = torch.log_softmax(logits.double(), -1)
    for r, k in enumerate(ks):
        n = int(counts[r])
        if k == 0:
            assert n == 0
            continue
        assert k <= n <= ops().top_logprobs_cap()
        got = sorted(zip(tokens[r, :n].tolist(), lps[r, :n].tolist()), key=lambda tv: (-tv[1], tv[0]))[:k]
        top = torch.topk(want[r], k)
        assert sorted(t for t, _ in got) == sorted(top.indices.tolist())
        for t, v in got:
            assert abs(v - float(want[r, t])) < 1e-4
    rt, rl, rc = ref.top_logprobs(logits, torch.tensor(ks, device=DEV, dtype=torch.int32))
    assert rc.tolist() == counts.tolist()


@pytest.mark.parametrize("vocab,copies", [(256, 1), (1009, 1), (151936, 1), (151936, 4)])
def test_sample_matches_filtered_distribution(vocab, copies):
    """(Four copies of the cases at the large vocabulary: more blocks than the device holds at once, which the
    launcher gives half the threads each.)"""
    import plain_impl

    g = torch.Generator(device=DEV).manual_seed(9)
    cases = [(0.7, -1, 1.0, 0.0), (1.0, 5, 1.0, 0.0), (1.3, -1, 0.6, 0.0), (0.9, 50, 0.8, 0.05), (1.0, -1, 1.0, 0.2),
             (0.0, -1, 1.0, 0.0), (1.0, 1, 1.0, 0.0), (2.0, -1, 0.05, 0.0)] * copies
    rows = len(cases)
    logits = torch.randn(rows, vocab, device=DEV, generator=g) * 3
    t = torch.tensor([c[0] for c in cases], device=DEV)
    k = torch.tensor([c[1] for c in cases], device=DEV, dtype=torch.int32)
    p = torch.tensor([c[2] for c in cases], device=DEV)
    mp = torch.tensor([c[3] for c in cases], device=DEV)
    for u_val in (0.0, 0.123, 0.5, 0.77, 0.999999):
        u = torch.full((rows,), u_val, device=DEV)
        toks, lps = ops().sample(logits, t, k, p, mp, u, want_logprob=True)
        for r, (temp, kk, pp, mm) in enumerate(cases):
            tok = int(toks[r])
            if temp == 0 or kk == 1:
                assert tok == int(torch.argmax(logits[r]))
                assert abs(float(lps[r]) - float(torch.log_softmax(logits[r], -1)[tok])) < 1e-4
                continue
            probs = plain_impl.filtered_probs(logits[r].cpu(), temp, kk, pp, mm).double()
            assert probs[tok] > 0, (r, tok)
            cum = torch.cumsum(probs, 0)
            lo, hi = float(cum[tok] - probs[tok]), float(cum[tok])
            assert lo - 1e-5 <= u_val < hi + 1e-5, (r, u_val, lo, hi)      # the drawn token's interval holds u
            assert abs(float(lps[r]) - float(torch.log(probs[tok]))) < 1e-3


def test_sample_frequencies():
    # chi-square of many draws against the softmax, as the reference tests its sampler
    # (tests/test_engine.py:157-184 there): 12 tokens, temperature 1, 40000 draws.
    g = torch.Generator(device=DEV).manual_seed(10)
    vocab, draws = 12, 40000
    row = torch.randn(vocab, device=DEV, generator=g)
    logits = row.repeat(draws, 1).contiguous()
    u = torch.rand(draws, device=DEV, generator=g)
    ones = torch.ones(draws, device=DEV)
    toks, _ = ops().sample(logits, ones, torch.full((draws,), -1, device=DEV, dtype=torch.int32), ones,
                           torch.zeros(draws, device=DEV), u)
    counts = torch.bincount(toks.long(), minlength=vocab).double().cpu()
    expect = torch.softmax(row.double().cpu(), 0) * draws
    chi2 = float(((counts - expect) ** 2 / expect).sum())
    assert chi2 < 31.26                                         # df = 11, p = 0.001
