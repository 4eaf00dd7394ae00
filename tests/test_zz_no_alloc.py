"""The allocation-free decode-attention entry point (lily_b200/csrc/no_alloc.h), called the way
a host program without an allocator would call it: through its exported C symbol, with raw
device pointers.  Its output is compared with the existing entry point's (which takes a scratch
buffer from the caller) on two calls in a row that share the static scratch.

This file is collected last, so a run that stops at the first failure has run everything else.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
MAX_FLOATS = 2 * 1024 * 1024


def entry():
    from lily_b200.csrc import build
    lib = build.load()
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn = lib.lily_attention_decode_static
    fn.argtypes = [vp, vp, vp, vp, i, vp, i, i, i, i, i, i, i, f, i, vp]
    fn.restype = i
    lib.lily_attention_decode_static_fits.argtypes = [i, i, i, i]
    lib.lily_attention_decode_static_fits.restype = i
    lib.lily_last_error.restype = ctypes.c_char_p
    return lib, fn


def case(dtype, nq, nkv, d, page, seqs, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    reqs = len(seqs)
    width = max(-(-s // page) for s in seqs)
    cache = torch.randn(reqs * width + 1, 2, nkv, page, d, device=DEV, generator=g).to(dtype)
    table = (torch.randperm(reqs * width, device=DEV, generator=g) + 1).view(reqs, width).to(torch.int32)
    q = torch.randn(reqs, nq * d, device=DEV, generator=g).to(dtype)
    return cache, table, q, torch.tensor(seqs, device=DEV, dtype=torch.int32)


@pytest.mark.parametrize("dtype,nq,nkv,d,page,splits,through_scratch", [
    (torch.bfloat16, 32, 8, 128, 64, 6, False),    # tensor-core kernels; these few pairs merge inside clusters
    (torch.bfloat16, 32, 8, 128, 64, 20, True),    # more ranges than a cluster has blocks: the array and the combine kernel
    (torch.float32, 6, 2, 48, 16, 4, True),        # CUDA-core kernels
    (torch.bfloat16, 8, 2, 64, 16, 1, False),      # one split: no scratch at all
])
def test_static_scratch_entry_matches_the_allocating_one(dtype, nq, nkv, d, page, splits, through_scratch):
    from lily_b200.csrc import ops
    lib, fn = entry()
    code = 1 if dtype == torch.bfloat16 else 0
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    stream = torch.cuda.current_stream().cuda_stream
    if through_scratch:
        # which form runs is the kernels' own choice: make sure this case is one that goes through the array
        pairs = 5 * nkv * -(-(nq // nkv) // 16)
        assert not (ops.uses_tensor_cores(dtype, d) and pairs <= ops.decode_clusters(d, splits, nq // nkv))
        # leave NaN in the array (a call over a cache whose values are NaN): the calls below must overwrite all they read
        cache, table, q, seq_t = case(dtype, nq, nkv, d, page, [700, 3, 1025, 64, 333], 9)
        cache[:, 1] = float("nan")
        junk = torch.zeros_like(q)
        rc = fn(q.data_ptr(), cache.data_ptr(), junk.data_ptr(), table.data_ptr(), table.shape[1], seq_t.data_ptr(), 5,
                splits, nq, nkv, d, page, 0, d ** -0.5, code, stream)
        assert rc == 0, lib.lily_last_error().decode()
        torch.cuda.synchronize()
        assert bool(torch.isnan(junk.float()).any())
    free_before = None
    # two calls in a row share the array: the second must not see what the first left
    for seqs, seed in (([700, 3, 1025, 64, 333], 1), ([5, 1999, 130], 2)):
        cache, table, q, seq_t = case(dtype, nq, nkv, d, page, seqs, seed)
        want = torch.zeros_like(q)
        need = ops.decode_scratch_floats(len(seqs), nq, d, splits)
        scratch = torch.empty(max(need, 1), device=DEV)
        ops.attention_decode(q, cache, table, seq_t, want, scratch, splits, nq, nkv, d, page, d ** -0.5)
        got = torch.zeros_like(q)
        before = torch.cuda.memory_allocated()
        rc = fn(q.data_ptr(), cache.data_ptr(), got.data_ptr(), table.data_ptr(), table.shape[1], seq_t.data_ptr(),
                len(seqs), splits, nq, nkv, d, page, 0, d ** -0.5, code, stream)
        assert rc == 0, lib.lily_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before                 # nothing taken from torch's allocator ...
        torch.testing.assert_close(got.float(), want.float(), **tol)
        if free_before is None:
            free_before = torch.cuda.mem_get_info()[0]                 # ... nor, once warm, from the device itself
            rc = fn(q.data_ptr(), cache.data_ptr(), got.data_ptr(), table.data_ptr(), table.shape[1], seq_t.data_ptr(),
                    len(seqs), splits, nq, nkv, d, page, 0, d ** -0.5, code, stream)
            torch.cuda.synchronize()
            assert rc == 0 and torch.cuda.mem_get_info()[0] == free_before


def test_sizes_beyond_the_static_scratch_are_refused():
    lib, fn = entry()
    assert lib.lily_attention_decode_static_fits(8, 8, 32, 128) == 1
    assert lib.lily_attention_decode_static_fits(64, 64, 32, 128) == 0
    assert lib.lily_attention_decode_static_fits(1 << 20, 1, 32, 128) == 1          # one split needs none
    assert 64 * 64 * 32 * 130 > MAX_FLOATS
    cache, table, q, seq_t = case(torch.bfloat16, 32, 8, 128, 64, [10] * 64, 3)
    out = torch.zeros_like(q)
    rc = fn(q.data_ptr(), cache.data_ptr(), out.data_ptr(), table.data_ptr(), table.shape[1], seq_t.data_ptr(),
            64, 64, 32, 8, 128, 64, 0, 1.0, 1, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = lib.lily_last_error().decode()
    assert "static array holds" in msg and "fewer splits" in msg
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0                                             # nothing ran
