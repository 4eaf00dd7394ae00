"""Python faces of the CUDA kernels in this folder.

Every function takes CUDA tensors, checks dtypes, shapes and contiguity, and launches on the
current stream.  There is no CPU path and no library stand-in: a tensor that is not on a CUDA
device, or a library that cannot be built, raises.  bfloat16 matrix products go to cuBLAS through
``torch.mm`` where the reference's engine uses a library product (lily/layers/quantization/
base.py:69-72); float32 products use this folder's own FFMA kernel so that no reduced-precision
matrix mode can slip in.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Callable, Optional, Sequence, Tuple

import torch

from lily_b200.csrc import build as _build

_F32, _BF16 = 0, 1
_vp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t

_SIGNATURES = {
    "lily_embed": [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "lily_logit_transform": [_vp, _sz, _f, _f, _vp],
    "lily_scatter_tokens": [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "lily_add_rmsnorm": [_vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _i, _i, _i, _i, _sz, _vp],
    "lily_silu_mul": [_vp, _vp, _i, _i, _i, _i, _i, _i, _sz, _vp],
    "lily_gemm_tc": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "lily_qk_norm_rope_write": [_vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i,
                                _i, _i, _i, _i, _i, _sz, _vp],
    "lily_skinny_gemm": [_vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "lily_skinny_swiglu": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "lily_cast": [_vp, _i, _vp, _i, _sz, _vp],
    "lily_gemm_fp32": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "lily_attention_prefill_simt": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "lily_attention_decode_simt": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "lily_attention_combine": [_vp, _vp, _i, _i, _i, _i, _i, _vp],
    "lily_attention_prefill_mma": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp],
    "lily_attention_prefill_tc": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _vp],
    "lily_attention_decode_mma": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "lily_attention_decode_mma_fused": [_vp, _i, _sz, _i, _vp, _vp, _i, _f, _vp, _vp, _i, _i, _vp, _vp, _vp, _i, _vp, _vp,
                                        _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "lily_argmax": [_vp, _vp, _vp, _vp, _i, _i, _vp],
    "lily_apply_penalties": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "lily_top_logprobs": [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "lily_sample": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
}

_lib = None


class KernelError(RuntimeError):
    pass


def library():
    """Loads (building first if needed) the kernel library and declares its entry points."""
    global _lib
    if _lib is None:
        lib = _build.load()
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _i
        lib.lily_attention_prefill_simt_rows.restype = _i
        lib.lily_argmax_chunks.argtypes = [_i, _i]
        lib.lily_argmax_chunks.restype = _i
        lib.lily_skinny_gemm_max_rows.restype = _i
        lib.lily_skinny_gemm_splits.argtypes = [_i, _i, _i]
        lib.lily_skinny_gemm_splits.restype = _i
        lib.lily_skinny_swiglu_need.argtypes = [_i, _i, _i, _i, ctypes.POINTER(_sz), ctypes.POINTER(_i)]
        lib.lily_skinny_swiglu_need.restype = _i
        lib.lily_attention_prefill_mma_rows.restype = _i
        lib.lily_attention_prefill_tc_rows.restype = _i
        lib.lily_attention_prefill_tc_takes.argtypes = [_i, _i]
        lib.lily_attention_prefill_tc_takes.restype = _i
        lib.lily_attention_mma_supports.argtypes = [_i]
        lib.lily_attention_mma_supports.restype = _i
        lib.lily_top_logprobs_cap.restype = _i
        lib.lily_attention_decode_scratch_floats.argtypes = [_i, _i, _i, _i]
        lib.lily_attention_decode_scratch_floats.restype = _sz
        _lib = lib
    return _lib


launches = {"count": 0}          # kernels of this package launched so far (bench.py reports the difference)


def _call(name: str, *args) -> None:
    lib = library()
    launches["count"] += 1
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(f"{name}: {lib.lily_last_error().decode(errors='replace')}")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _dev(*tensors) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError("lily_b200 kernels run on a CUDA device only; got a tensor on " + str(t.device))
        if not t.is_contiguous():
            raise KernelError(f"kernels take contiguous tensors (shape {tuple(t.shape)}, strides {t.stride()})")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _i32(t: Optional[torch.Tensor], name: str):
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")
    return _p(t)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle.  The step launches a few hundred kernels from Python, so the two
    C calls are used directly where this torch has them (the public route builds a Stream object a call)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


# ------------------------------------------------------------------------------ elementwise

def embed(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None,
          future: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """Rows of ``table`` [vocab, hidden] at ``ids`` [tokens], times ``scale``, as float32 (the residual
    stream).  With ``future`` (int32, one entry per request slot) an id ``-(slot + 1)`` stands for the
    token that ``scatter_tokens`` stored for that slot."""
    _dev(table, ids, out, future)
    n, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _call("lily_embed", _p(table), _dt(table), _i32(ids, "ids"), _i32(future, "future") if future is not None else None,
          _p(out), n, hidden, vocab, float(scale), _stream())
    return out


def logit_transform(logits: torch.Tensor, scale: float = 1.0, softcap: Optional[float] = None) -> torch.Tensor:
    """In place on float32 ``logits``: times ``scale``, then ``softcap * tanh(. / softcap)`` when a cap is given."""
    _dev(logits)
    if logits.dtype != torch.float32:
        raise KernelError("logit_transform takes float32 logits")
    _call("lily_logit_transform", _p(logits), logits.numel(), float(scale), float(softcap or 0.0), _stream())
    return logits


def scatter_tokens(tokens: torch.Tensor, logit_rows: torch.Tensor, token_req: torch.Tensor, slots: torch.Tensor,
                   future: torch.Tensor) -> None:
    """``future[slots[token_req[logit_rows[i]]]] = tokens[i]``: each sampled token goes to the entry
    of its request's slot, where the next step's ``embed`` finds it."""
    _dev(tokens, logit_rows, token_req, slots, future)
    n = tokens.numel()
    if logit_rows.numel() < n:
        raise KernelError(f"scatter_tokens: {n} tokens for {logit_rows.numel()} logit rows")
    _call("lily_scatter_tokens", _i32(tokens, "tokens"), _i32(logit_rows, "logit_rows"), _i32(token_req, "token_req"),
          _i32(slots, "slots"), _i32(future, "future"), n, future.numel(), _stream())


def _summed(t: torch.Tensor, rows: int, cols: int, what: str):
    """(splits, stride) of a kernel input that is either [rows, cols] in the activation dtype or
    float32 partial sums [splits, rows, cols] of a split-k product."""
    if t.dim() == 3:
        if t.dtype != torch.float32 or tuple(t.shape[1:]) != (rows, cols):
            raise KernelError(f"{what}: partial sums must be float32 [splits, {rows}, {cols}], got {t.dtype} {tuple(t.shape)}")
        return t.shape[0], rows * cols
    if tuple(t.shape) != (rows, cols):
        raise KernelError(f"{what}: expected [{rows}, {cols}], got {tuple(t.shape)}")
    return 1, 0


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, write_residual: bool = True,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``resid += delta`` (float32, in place when ``write_residual``), then RMSNorm with ``weight``.
    ``delta`` is [tokens, hidden] in the activation dtype or float32 partial sums [splits, tokens,
    hidden].  With ``rows`` only those rows are normalised (and the residual is left as it is)."""
    _dev(resid, delta, weight, rows, out)
    if resid.dtype != torch.float32:
        raise KernelError("the residual stream is float32")
    hidden = resid.shape[-1]
    m = resid.shape[0] if rows is None else rows.numel()
    if rows is not None:
        write_residual = False
    if out is None:
        out = torch.empty((m, hidden), dtype=out_dtype, device=resid.device)
    splits, stride = (1, 0) if delta is None else _summed(delta, resid.shape[0], hidden, "add_rmsnorm delta")
    if delta is not None and delta.dtype not in (out.dtype, torch.float32):
        raise KernelError(f"delta {delta.dtype} does not match out {out.dtype}")
    if weight.numel() != hidden:
        raise KernelError(f"norm gain has {weight.numel()} entries, rows have {hidden}")
    _call("lily_add_rmsnorm", _p(resid), _p(delta), _p(weight), _p(out), _i32(rows, "rows"), m, hidden, float(eps),
          int(write_residual), _dt(out), _dt(weight), _dt(delta) if delta is not None else _dt(out), splits, stride,
          _stream())
    return out


def silu_mul(gate_up: torch.Tensor, out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
             block: Optional[int] = None) -> torch.Tensor:
    """``silu(gate) * up`` of ``gate_up`` [tokens, 2I] = [all gate | all up], or, with ``block``,
    alternating runs of ``block`` gate and ``block`` up columns.  ``gate_up`` may be float32 partial
    sums [splits, tokens, 2I], in which case ``out_dtype`` says what to write."""
    _dev(gate_up, out)
    n, two_i = gate_up.shape[-2:]
    splits, stride = _summed(gate_up, n, two_i, "silu_mul")
    if out is None:
        out = torch.empty((n, two_i // 2), dtype=out_dtype or gate_up.dtype, device=gate_up.device)
    _call("lily_silu_mul", _p(gate_up), _p(out), n, two_i // 2, int(block or two_i // 2), _dt(out), _dt(gate_up), splits,
          stride, _stream())
    return out


def qk_norm_rope_write(qkv: torch.Tensor, q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor],
                       eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                       positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                       kv_layer: torch.Tensor, nq: int, nkv: int, d: int, rotary_dim: int, page_size: int,
                       write_kv: bool = True, q_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-head RMSNorm of q and k (when gains are given), rotation by the tables, q to ``q_out``
    [tokens, nq * d], k and v into the token's place in its page of ``kv_layer``.  ``qkv`` is
    [tokens, (nq + 2 nkv) d] in the cache's dtype or float32 partial sums [splits, tokens, ...]."""
    _dev(qkv, q_gain, k_gain, cos, sin, positions, token_req, block_table, kv_layer, q_out)
    n = qkv.shape[-2]
    splits, stride = _summed(qkv, n, (nq + 2 * nkv) * d, "qk_norm_rope_write qkv")
    if qkv.dtype not in (kv_layer.dtype, torch.float32):
        raise KernelError(f"cache dtype {kv_layer.dtype} differs from activations {qkv.dtype}")
    if tuple(kv_layer.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError(f"cache layer shape {tuple(kv_layer.shape)} does not fit kv_heads={nkv} page={page_size} d={d}")
    if cos is not None and (cos.dtype != torch.float32 or cos.shape[-1] != rotary_dim // 2):
        raise KernelError("rotation tables must be float32 [positions, rotary_dim / 2]")
    if q_gain is not None and q_gain.dtype != k_gain.dtype:
        raise KernelError("q and k gains must share a dtype")
    if q_out is None:
        q_out = torch.empty((n, nq * d), dtype=kv_layer.dtype, device=qkv.device)
    _call("lily_qk_norm_rope_write", _p(qkv), _p(q_gain), _p(k_gain), float(eps), _p(cos), _p(sin),
          _i32(positions, "positions"), _i32(token_req, "token_req"), _i32(block_table, "block_table"),
          block_table.shape[-1], _p(kv_layer), _p(q_out), n, nq, nkv, d, rotary_dim, page_size, int(write_kv),
          _dt(kv_layer), _dt(q_gain) if q_gain is not None else _F32, _dt(qkv), splits, stride, _stream())
    return q_out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _dev(x)
    if x.dtype == dtype:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _call("lily_cast", _p(x), _dt(x), _p(out), _dt(out), x.numel(), _stream())
    return out


# ------------------------------------------------------------------------------ matrix products

def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x [M, K] . weight [N, K]^T (+ bias)``.  float32: this package's FFMA kernel.
    bfloat16: cuBLAS with float32 accumulation; ``out_dtype=float32`` keeps the accumulator's
    precision (used for the logits)."""
    _dev(x, weight, bias)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or weight.dtype != x.dtype:
        raise KernelError(f"linear: x {tuple(x.shape)} {x.dtype} against weight {tuple(weight.shape)} {weight.dtype}")
    if x.dtype == torch.float32:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
        if bias is not None and bias.dtype != torch.float32:
            raise KernelError("float32 linear takes a float32 bias")
        _call("lily_gemm_fp32", _p(x), _p(weight), _p(bias), _p(out), m, n, k, k, n, _stream())
        return out
    if _OWN_PLAIN_GEMM and out_dtype is None and m >= TC_MIN_ROWS and gemm_tc_takes(x, weight):
        return gemm_tc(x, weight, bias.to(x.dtype) if bias is not None else None)
    if out_dtype == torch.float32:
        out = torch.mm(x, weight.t(), out_dtype=torch.float32)
        if bias is not None:
            out += bias.float()
        return out
    if bias is not None:
        return torch.addmm(bias.to(x.dtype), x, weight.t())
    return torch.mm(x, weight.t())


TC_MIN_ROWS = 65          # products of more rows than this go to the tcgen05 kernel when it takes the shape


def gate_up_fused_pays(rows: int, fused_rows: int) -> bool:
    """Whether the tcgen05 gate/up product with the SiLU*mul epilogue is the faster way for ``rows`` tokens and a
    fused matrix of ``fused_rows`` rows (gate and up together), against the library product followed by the SiLU*mul
    kernel.  It is, except for 129 to 256 tokens where its 256-wide tiles fill the last round of block pairs badly
    (Qwen3-8B, 96 tiles on 74 pairs: 56 against 47 us at 192 tokens, 57 against 54 at 256; equal from 65 to 128 and
    from 384 on, where the epilogue saves the [tokens, 2 I] intermediate)."""
    if rows < TC_MIN_ROWS:
        return False
    if 128 < rows <= 256:
        tiles, pairs = -(-fused_rows // 256), max(1, sm_count() // 2)
        return -(-tiles // pairs) * pairs < 1.3 * tiles
    return True
# LILY_B200_PLAIN_GEMM=tcgen05 sends the plain bfloat16 products of 65 rows and more (QKV, output, down in prefill) to
# this package's tcgen05 kernel too instead of the library, which is 8 to 10 % faster on them and therefore the default.
_OWN_PLAIN_GEMM = os.environ.get("LILY_B200_PLAIN_GEMM", "") == "tcgen05"


def gemm_tc_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
            silu_mul_block: bool = False) -> torch.Tensor:
    """``x [M, K] . weight [N, K]^T`` in bfloat16 on the tcgen05 tensor cores (TMA-fed, accumulator
    in tensor memory).  With ``silu_mul_block`` the rows of ``weight`` alternate between 128 gate
    rows and the 128 up rows of the same outputs and the result is ``silu(gate) * up`` [M, N / 2]."""
    _dev(x, weight, bias)
    m, k = x.shape
    n = weight.shape[0]
    if not gemm_tc_takes(x, weight) or weight.shape[1] != k:
        raise KernelError(f"gemm_tc: x {tuple(x.shape)} {x.dtype} against weight {tuple(weight.shape)} {weight.dtype}")
    out = torch.empty((m, n // 2 if silu_mul_block else n), dtype=torch.bfloat16, device=x.device)
    _call("lily_gemm_tc", _p(x), _p(weight), _p(out), _p(bias), m, n, k, k, out.shape[1], 1 if silu_mul_block else 0,
          _stream())
    return out


def gemm_tc_status() -> int:
    """0, or a code from the first bounded wait that gave up in a tcgen05 kernel (synchronises)."""
    return int(library().lily_gemm_tc_status())


def linear_split(x: torch.Tensor, weight: torch.Tensor, splits: Optional[int] = None) -> Optional[torch.Tensor]:
    """``x [M, K] . weight [N, K]^T`` for a few tokens (decode) by this package's weight-streaming
    kernel, as float32 partial sums ``[splits, M, N]`` over slices of K that the consuming kernel
    (``add_rmsnorm``, ``silu_mul``, ``qk_norm_rope_write``) adds up.  Without ``splits`` the kernel's
    own rule decides, and None comes back for shapes it leaves to the library product (wide
    outputs, more than 16 tokens) or cannot take (K not a multiple of 64, not bfloat16); the caller
    then uses ``linear``.  With ``splits`` given the kernel runs whenever it can (up to 64 tokens)."""
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        return None
    m, k = x.shape
    n = weight.shape[0]
    lib = library()
    if m > lib.lily_skinny_gemm_max_rows() or m < 1 or weight.shape[1] != k or k % 64:
        return None
    if splits is None:
        splits = int(lib.lily_skinny_gemm_splits(m, n, k))
    if splits < 1:
        return None
    _dev(x, weight)
    parts = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
    _call("lily_skinny_gemm", _p(x), _p(weight), _p(parts), m, n, k, splits, _stream())
    return parts


def linear_auto(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The product in whichever form is fastest for the shape: float32 partial sums from
    ``linear_split`` for a few tokens, else ``linear``'s [M, N].  For producers whose consumer is
    one of the kernels that take either form."""
    if bias is None:
        parts = linear_split(x, weight)
        if parts is not None:
            return parts
    return linear(x, weight, bias)


def swiglu_skinny_need(tokens: int, intermediate: int, hidden: int, dtype: torch.dtype,
                       block: Optional[int] = None, whenever_possible: bool = False) -> Optional[Tuple[int, int]]:
    """(float32 of scratch, int32 counters) that ``swiglu_skinny`` wants for this shape, or None when it does not
    take it (more than 8 tokens, not bfloat16, K not a multiple of 64) or, unless ``whenever_possible``, when the
    library product followed by SiLU*mul is the faster pair for it (several tokens of a very wide input): the caller
    then forms the product and SiLU*mul separately.  ``LILY_B200_SWIGLU=library`` always answers None."""
    if dtype != torch.bfloat16 or _LIBRARY_SWIGLU:
        return None
    floats, counters = _sz(0), _i(0)
    verdict = library().lily_skinny_swiglu_need(int(tokens), int(intermediate), int(hidden), int(block or intermediate),
                                                ctypes.byref(floats), ctypes.byref(counters))
    if verdict == 0 or (verdict == 2 and not whenever_possible):
        return None
    return int(floats.value), int(counters.value)


_LIBRARY_SWIGLU = os.environ.get("LILY_B200_SWIGLU", "") == "library"


def swiglu_skinny(x: torch.Tensor, gate_up: torch.Tensor, block: Optional[int], scratch: torch.Tensor,
                  counters: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(x . gate^T) * (x . up^T)`` [tokens, I] for up to 8 tokens in one kernel that streams the fused
    gate/up matrix [2 I, K] once (rows in alternating runs of ``block`` gate and up rows; None: all gate, then all
    up).  ``scratch`` (float32) and ``counters`` (int32, zero before the first call; the kernel leaves them zero)
    are sized by ``swiglu_skinny_need``."""
    _dev(x, gate_up, scratch, counters, out)
    m, k = x.shape
    inter = gate_up.shape[0] // 2
    need = swiglu_skinny_need(m, inter, k, x.dtype, block, whenever_possible=True)
    if need is None or gate_up.dtype != torch.bfloat16 or gate_up.shape[1] != k:
        raise KernelError(f"swiglu_skinny: x {tuple(x.shape)} {x.dtype} against {tuple(gate_up.shape)} {gate_up.dtype}")
    if scratch.dtype != torch.float32 or scratch.numel() < need[0] or counters.dtype != torch.int32 or counters.numel() < need[1]:
        raise KernelError(f"swiglu_skinny: {need[0]} float32 of scratch and {need[1]} int32 counters needed")
    if out is None:
        out = torch.empty((m, inter), dtype=torch.bfloat16, device=x.device)
    _call("lily_skinny_swiglu", _p(x), _p(gate_up), _p(out), _p(scratch), _p(counters), m, inter, k, int(block or inter),
          _stream())
    return out


def logits(x: torch.Tensor, head: torch.Tensor) -> torch.Tensor:
    """``x [rows, hidden] . head [vocab, hidden]^T`` as float32 [rows, vocab]: for a few rows the head is
    streamed once by this package's kernel when one slice of K serves, else a product that keeps the
    accumulator's precision (lily/layers/vocab_embedding.py:89-96 casts a model-dtype product)."""
    parts = linear_split(x, head)
    if parts is not None and parts.shape[0] == 1:
        return parts[0]
    return linear(x, head, out_dtype=torch.float32)


def gate_up_interleave(dtype: torch.dtype, intermediate: int) -> Optional[int]:
    """How a fused gate/up matrix should be laid out for these kernels: None for all gate rows, then all up
    rows; a number for alternating runs of that many gate rows and the up rows of the same outputs (what the
    tcgen05 product's SiLU*mul epilogue wants: both halves of 128 outputs inside one 256-row tile)."""
    return 128 if dtype == torch.bfloat16 and intermediate % 128 == 0 else None


# ------------------------------------------------------------------------------ attention

def uses_tensor_cores(dtype: torch.dtype, d: int) -> bool:
    """Whether attention of this precision and head size runs on the mma.sync kernels
    (bfloat16, head sizes 64, 128, 192, 256); everything else runs on the CUDA-core kernels."""
    return dtype == torch.bfloat16 and bool(library().lily_attention_mma_supports(int(d)))


# A step with fewer new tokens than this in its prompt portions runs them through the mma.sync kernel
# (tiles of 64 rows); from here on the tcgen05 kernel's tiles of 128 rows are worth filling.
TC_ATTENTION_MIN_TOKENS = 128


def uses_tcgen05_attention(dtype: torch.dtype, d: int, page_size: int, new_tokens: int) -> bool:
    """Whether prefill attention of this precision, head size, page size and number of new tokens
    runs on the tcgen05 kernel (bfloat16, head size 128 or 64, pages of a multiple of 64 positions)."""
    return (dtype == torch.bfloat16 and new_tokens >= TC_ATTENTION_MIN_TOKENS
            and bool(library().lily_attention_prefill_tc_takes(int(d), int(page_size))))


def prefill_tile_rows(dtype: torch.dtype = torch.float32, d: int = 0, page_size: int = 0, new_tokens: int = 0) -> int:
    """New tokens per tile of the prefill kernel that will take this precision, head size, page
    size and number of new tokens."""
    lib = library()
    if uses_tcgen05_attention(dtype, d, page_size, new_tokens):
        return int(lib.lily_attention_prefill_tc_rows())
    return int(lib.lily_attention_prefill_mma_rows() if uses_tensor_cores(dtype, d) else lib.lily_attention_prefill_simt_rows())


def attention_tc_status() -> int:
    """0, or a code from the first bounded wait that gave up in the tcgen05 attention kernel (synchronises)."""
    return int(library().lily_attention_tc_status())


def attention_prefill(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, cu_seqlens: torch.Tensor,
                      prefix_lens: torch.Tensor, tile_req: torch.Tensor, tile_start: torch.Tensor, out: torch.Tensor,
                      nq: int, nkv: int, d: int, page_size: int, scale: float, window: Optional[int] = None,
                      tile_rows: Optional[int] = None, heads_per_block: int = 0) -> None:
    """Causal attention of each request's new tokens over its cached prefix and themselves.
    ``q`` and ``out`` are [tokens, nq * d] indexed by ``cu_seqlens``; tiles list (request, offset)
    in steps of ``tile_rows`` (default: ``prefill_tile_rows(q.dtype, d)``), which also names the
    kernel: the tcgen05 kernel takes tiles of its own size, the others theirs.  ``heads_per_block``
    (tcgen05 only) 1 or 2 picks between its one-head and its two-head form; 0 lets the launcher choose."""
    _dev(q, kv_layer, block_table, cu_seqlens, prefix_lens, tile_req, tile_start, out)
    if q.dtype != kv_layer.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, cache and out must share a dtype")
    common = (_p(q), _p(kv_layer), _p(out), _i32(block_table, "block_table"), block_table.shape[-1],
              _i32(cu_seqlens, "cu_seqlens"), _i32(prefix_lens, "prefix_lens"), _i32(tile_req, "tile_req"),
              _i32(tile_start, "tile_start"), tile_req.numel(), nq, nkv, d, page_size, int(window or 0), float(scale))
    lib = library()
    base_rows = int(lib.lily_attention_prefill_mma_rows() if uses_tensor_cores(q.dtype, d) else lib.lily_attention_prefill_simt_rows())
    if tile_rows is not None and tile_rows != base_rows:
        if not (tile_rows == int(lib.lily_attention_prefill_tc_rows()) and q.dtype == torch.bfloat16
                and lib.lily_attention_prefill_tc_takes(int(d), int(page_size))):
            raise KernelError(f"attention_prefill: no kernel with tiles of {tile_rows} rows for {q.dtype}, head size {d}, "
                              f"page size {page_size}")
        if not (q.is_contiguous() and out.is_contiguous() and kv_layer.is_contiguous()):
            raise KernelError("attention_prefill: the tcgen05 kernel takes contiguous q, out and cache")
        _call("lily_attention_prefill_tc", *common, q.shape[0], kv_layer.shape[0], int(heads_per_block), _stream())
    elif uses_tensor_cores(q.dtype, d):
        _call("lily_attention_prefill_mma", *common, _stream())
    else:
        _call("lily_attention_prefill_simt", *common, _dt(q), _stream())


def decode_clusters(d: int, splits: int, group: int) -> int:
    """How many (request, kv head) pairs the tensor-core decode attention can merge inside clusters of
    ``splits`` blocks at once (0: it would use scratch and the combine kernel)."""
    return int(library().lily_attention_decode_mma_clusters(int(d), int(splits), int(group)))


def decode_scratch_floats(requests: int, nq: int, d: int, splits: int) -> int:
    return int(library().lily_attention_decode_scratch_floats(requests, nq, d, splits))


def attention_decode(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                     out: torch.Tensor, scratch: Optional[torch.Tensor], splits: int, nq: int, nkv: int, d: int,
                     page_size: int, scale: float, window: Optional[int] = None, stages: int = 0) -> None:
    """One query token per request (rows of ``q`` [requests, nq * d]) over ``seq_lens`` cached
    positions, keys cut into ``splits`` ranges merged through ``scratch`` (float32).  ``stages`` (tensor-core
    kernel only): the key/value tiles a block holds, 0 for the default (``DecodePlan.stages``)."""
    _dev(q, kv_layer, block_table, seq_lens, out, scratch)
    requests = q.shape[0]
    if q.dtype != kv_layer.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, cache and out must share a dtype")
    need = decode_scratch_floats(requests, nq, d, splits)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        raise KernelError(f"attention_decode: scratch of {need} float32 needed")
    common = (_p(q), _p(kv_layer), _p(out), _i32(block_table, "block_table"), block_table.shape[-1],
              _i32(seq_lens, "seq_lens"), _p(scratch), requests, splits, nq, nkv, d, page_size, int(window or 0),
              float(scale))
    if uses_tensor_cores(q.dtype, d):
        _call("lily_attention_decode_mma", *common, int(stages), _stream())   # merges the splits itself (cluster, or combine behind)
        if splits > 1 and (stages or requests * nkv * -(-(nq // nkv) // 16) > decode_clusters(d, splits, nq // nkv)):
            launches["count"] += 1                                   # the combine kernel, launched inside
    else:
        if stages:
            raise KernelError(f"attention_decode: {stages} stages are the tensor-core kernel's; {q.dtype}, head size {d} runs on CUDA cores")
        _call("lily_attention_decode_simt", *common, _dt(q), _stream())
        if splits > 1:
            launches["count"] += 1          # the combine kernel, launched inside


def sm_count() -> int:
    """Streaming multiprocessors of the current device (148 on a B200)."""
    return int(library().lily_sm_count())


def choose_decode_splits(num_decode: int, kv_heads: int, max_seq_len: int, sm_count: int = 148,
                         blocks_per_sm: int = 3, min_keys: int = 256, max_splits: int = 32,
                         clusters: Optional[Callable[[int], int]] = None) -> int:
    """How many ranges the keys of a decode row are cut into.  One block works on one (request, kv
    head, range); the device holds ``sm_count * blocks_per_sm`` blocks at a time.

    ``clusters(s)`` says how many clusters of ``s`` blocks the attention kernel can have resident at
    once (``decode_clusters``): while every (request, kv head) pair gets one, the blocks of a pair
    merge their ranges through distributed shared memory and no combine kernel follows, and the
    most ranges that allow this are the fastest (measured on a B200, head size 128, 8 kv heads:
    batch 1 and 2: 16 ranges; 4: 10; 8: 6; 16: 3; 24: 2; sizes past 8 want a tenth of room to spare:
    24 pairs in clusters of 15, of which exactly 24 fit, took 21 us against 16 us in clusters of 13).
    A cluster has at most 16 blocks, so a few long rows leave most of the device idle (one row of 131,072 keys:
    128 blocks, 168 us, half of the memory's speed); from 16 k keys on, where one wave of ranges of at least 512
    keys through scratch and the combine kernel has a quarter more blocks than the clusters, the wave is taken
    (measured, 8 kv heads, clusters against the wave: one row of 16 k keys 28 / 23 us, of 24 k 38 / 27, of 131 k
    168 / 88; two rows of 16 k 36 / 32; four rows of 16 k 53 / 51, of 8 k 31 / 32; five rows and more fill the
    device with clusters).
    Without clusters (float32, other head sizes, more pairs than clusters of two): the single wave that
    comes closest to filling the device, and when the rows alone overfill it, about four waves
    (batch 64: 4 ranges).  The reference fixes 32 splits with a floor of 64 keys
    (lily/layers/attention/triton_backend.py:21, decode_attention.py:68,172)."""
    if num_decode == 0:
        return 1
    limit = max(1, min(max_splits, max_seq_len // min_keys))
    pairs, held = num_decode * kv_heads, sm_count * blocks_per_sm
    if clusters is not None:
        full = max(1, min(64, max_seq_len // 512, held // pairs))           # ranges that fill the device once
        for s in range(min(limit, 16), 1, -1):
            room = clusters(s)
            if pairs <= (room if s <= 8 else 0.9 * room):
                if full * 4 >= s * 5 and max_seq_len >= 16384:
                    return full
                return s
    one_wave = min(limit, held // pairs)
    if one_wave >= 1 and (pairs * one_wave >= 0.7 * held or one_wave == limit):
        return one_wave
    return max(1, min(limit, -(-4 * held // pairs)))


@dataclass(frozen=True)
class DecodePlan:
    """How the decode attention of a step runs (the same for every layer of a cache group)."""

    splits: int                 # key ranges per (request, kv head)
    fused: bool                 # the attention kernel starts from the qkv product (norm, rotation, cache write inside)
    scratch_floats: int         # float32 scratch the split ranges are merged through (0: merged inside clusters)
    arm: str                    # which rule chose the splits: "cluster", "wave", "single" or "whole rows"
    stages: int = 0             # key/value tiles a block of the tensor-core kernel holds (0: its default)


def whole_rows_pay(pairs: int, sm_count: int = 148) -> bool:
    """Whether ``pairs`` blocks of the tensor-core kernel with three key/value stages, one block for all keys of a
    (request, kv head), beat ranges of two stages: two such blocks fit a SM, and they keep the memory busy once three
    quarters of those places are taken.  A last round that is less than 45 % full costs more than it saves (a block
    alone on its SM takes about 1.2 us a tile of 64 keys whatever the others do), and past three and a half rounds
    the ranges of two stages are as good or better.
    Measured on a B200, head size 128, 8 kv heads of 4 query heads, decode steps of Qwen3-8B sizes with and without
    (same run, ms): context 4,096: 28 rows 6.66 / 6.45, 32 rows 7.02 / 6.72, 64 rows 10.51 / 10.37, 96 rows 14.36 / 14.13,
    128 rows 17.33 / 17.60; context 1,024: 32 rows 4.67 / 4.44, 64 rows 5.85 / 5.58, 128 rows 7.93 / 7.77, 256 rows 11.94 /
    12.22.  The kernel alone, us, against the best plan of two stages: 32 rows of 4,096 keys 82 against 96, of 1,024 keys
    24 against 32, 64 rows of 1,024 keys 48 against 58; 20 rows of 4,096 keys 79 against 61 (too few blocks)."""
    places = 2 * sm_count
    if pairs < 0.75 * places or pairs > 3.5 * places:
        return False
    last = pairs % places
    return last == 0 or last >= 0.45 * places


def plan_decode_attention(dtype: torch.dtype, requests: int, nq: int, nkv: int, d: int, max_seq_len: int,
                          even: bool = False) -> DecodePlan:
    """The plan for ``requests`` rows that bring one token each, none longer than ``max_seq_len`` positions.
    A step in which every request brings one token may hand the qkv product straight to the attention kernel
    (``fused``): every block then finishes its own queries, which costs less than a kernel of its own while all
    blocks are resident at once (three a SM) and more when they run in several rounds (measured at batch 64:
    2 % of the step).
    ``even``: the caller knows that the rows are about equally long (the longest at most an eighth over their
    mean).  Then, and when ``whole_rows_pay``, a block
    takes all keys of its row with three stages; rows of very different lengths keep their ranges, which spread a
    long row over many blocks."""
    if requests == 0:
        return DecodePlan(1, False, 0, "single")
    group = nq // nkv
    tensor_cores = uses_tensor_cores(dtype, d)
    row_blocks = -(-group // 16)                 # the tensor-core kernel takes 16 query heads of a kv head a block
    pairs = requests * nkv * row_blocks
    if even and tensor_cores and d <= 128 and _WHOLE_ROWS and whole_rows_pay(pairs, sm_count()):
        return DecodePlan(1, pairs <= 2 * sm_count(), 0, "whole rows", 3)
    room = (lambda s: decode_clusters(d, s, group)) if tensor_cores else None
    splits = choose_decode_splits(requests, nkv, max_seq_len, sm_count=sm_count(), clusters=room)
    in_clusters = tensor_cores and splits > 1 and pairs <= decode_clusters(d, splits, group)
    fused = tensor_cores and pairs * splits <= 3 * sm_count()
    arm = "single" if splits == 1 else ("cluster" if in_clusters else "wave")
    return DecodePlan(splits, fused, decode_scratch_floats(requests, nq, d, splits), arm)


_WHOLE_ROWS = os.environ.get("LILY_B200_DECODE_WHOLE_ROWS", "1") != "0"



def prefill_tiles(prefix_lens: Sequence[int], new_lens: Sequence[int], first: int, rows: int,
                  device) -> Tuple[torch.Tensor, torch.Tensor]:
    """(request, offset) of each tile of ``rows`` new tokens over the requests from ``first`` on, as two int32
    device tensors, in the order of the keys a tile attends to (the prefill kernels start with the last,
    longest ones)."""
    pairs = [(prefix_lens[r] + s, r, s) for r in range(first, len(new_lens)) for s in range(0, new_lens[r], rows)]
    pairs.sort()
    both = torch.tensor([[r for _, r, _ in pairs], [s for _, _, s in pairs]], dtype=torch.int32).reshape(2, -1)
    both = both.to(device, non_blocking=True)
    return both[0].contiguous(), both[1].contiguous()


def attention_decode_fused(qkv: torch.Tensor, q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                           cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], kv_layer: torch.Tensor,
                           block_table: torch.Tensor, seq_lens: torch.Tensor, out: torch.Tensor,
                           scratch: Optional[torch.Tensor], splits: int, nq: int, nkv: int, d: int, rotary_dim: int,
                           page_size: int, scale: float, window: Optional[int] = None, write_kv: bool = True,
                           stages: int = 0) -> None:
    """``qk_norm_rope_write`` and ``attention_decode`` of a step in which every request brings one token, as one
    kernel: ``qkv`` is the projection's result ([requests, (nq + 2 nkv) d] in the cache's dtype, or float32 partial
    sums [splits, requests, ...]); the attention blocks finish their own query heads, and the block whose key range
    holds the new position finishes the key and the value and writes them to the cache before it reads them."""
    _dev(qkv, q_gain, k_gain, cos, sin, kv_layer, block_table, seq_lens, out, scratch)
    requests = qkv.shape[-2]
    planes, stride = _summed(qkv, requests, (nq + 2 * nkv) * d, "attention_decode_fused qkv")
    if not uses_tensor_cores(kv_layer.dtype, d) or out.dtype != kv_layer.dtype or qkv.dtype not in (kv_layer.dtype, torch.float32):
        raise KernelError(f"attention_decode_fused: cache {kv_layer.dtype}, qkv {qkv.dtype}, out {out.dtype}, head size {d}")
    if tuple(kv_layer.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError(f"cache layer shape {tuple(kv_layer.shape)} does not fit kv_heads={nkv} page={page_size} d={d}")
    if cos is not None and (cos.dtype != torch.float32 or cos.shape[-1] != rotary_dim // 2):
        raise KernelError("rotation tables must be float32 [positions, rotary_dim / 2]")
    if q_gain is not None and q_gain.dtype != k_gain.dtype:
        raise KernelError("q and k gains must share a dtype")
    need = decode_scratch_floats(requests, nq, d, splits)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        raise KernelError(f"attention_decode: scratch of {need} float32 needed")
    _call("lily_attention_decode_mma_fused", _p(qkv), planes, stride, _dt(qkv), _p(q_gain), _p(k_gain),
          _dt(q_gain) if q_gain is not None else _F32, float(eps), _p(cos), _p(sin), int(rotary_dim), int(write_kv),
          _p(kv_layer), _p(out), _i32(block_table, "block_table"), block_table.shape[-1], _i32(seq_lens, "seq_lens"),
          _p(scratch), requests, splits, nq, nkv, d, page_size, int(window or 0), float(scale), int(stages), _stream())
    if splits > 1 and (stages or requests * nkv * -(-(nq // nkv) // 16) > decode_clusters(d, splits, nq // nkv)):
        launches["count"] += 1                                       # the combine kernel, launched inside


# ------------------------------------------------------------------------------ sampling

def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _dev(logits, out)
    if logits.dtype != torch.float32:
        raise KernelError("argmax takes float32 logits")
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    chunks = int(library().lily_argmax_chunks(rows, vocab))
    pv = pi = None
    if chunks > 1:          # a large vocabulary: many blocks per row, then a merge
        pv = torch.empty((rows * chunks,), dtype=torch.float32, device=logits.device)
        pi = torch.empty((rows * chunks,), dtype=torch.int32, device=logits.device)
        launches["count"] += 1
    _call("lily_argmax", _p(logits), _i32(out, "out"), _p(pv), _p(pi), rows, vocab, _stream())
    return out


def apply_penalties(logits: torch.Tensor, entry_row: torch.Tensor, entry_token: torch.Tensor,
                    entry_count: torch.Tensor, entry_bias: torch.Tensor, repetition: torch.Tensor,
                    frequency: torch.Tensor, presence: torch.Tensor) -> None:
    _dev(logits, entry_row, entry_token, entry_count, entry_bias, repetition, frequency, presence)
    rows, vocab = logits.shape
    _call("lily_apply_penalties", _p(logits), _i32(entry_row, "entry_row"), _i32(entry_token, "entry_token"),
          _i32(entry_count, "entry_count"), _p(entry_bias), _p(repetition), _p(frequency), _p(presence),
          entry_row.numel(), vocab, _stream())


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor, want_logprob: bool = False):
    """One token per row of float32 ``logits``; per-row parameters are float32 (``top_k`` int32).
    Returns (tokens int32, logprobs float32 or None)."""
    _dev(logits, temperature, top_k, top_p, min_p, uniform)
    rows, vocab = logits.shape
    for t, name in ((temperature, "temperature"), (top_p, "top_p"), (min_p, "min_p"), (uniform, "uniform")):
        if t.dtype != torch.float32 or t.numel() != rows:
            raise KernelError(f"sample: {name} must be float32 [rows]")
    tokens = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    logprob = torch.empty((rows,), dtype=torch.float32, device=logits.device) if want_logprob else None
    _call("lily_sample", _p(logits), _p(temperature), _i32(top_k, "top_k"), _p(top_p), _p(min_p), _p(uniform),
          _p(tokens), _p(logprob), rows, vocab, _stream())
    return tokens, logprob


def top_logprobs_cap() -> int:
    """The most entries a row of ``top_logprobs`` can return."""
    return int(library().lily_top_logprobs_cap())


def top_logprobs(logits: torch.Tensor, k: torch.Tensor):
    """The ``k[r]`` most probable tokens of each row of float32 ``logits`` with their log-probabilities
    (log-softmax of the logits as given).  Returns (tokens int32 [rows, cap], logprobs float32 [rows, cap],
    counts int32 [rows]): row r holds ``counts[r] >= k[r]`` entries in no particular order (ties at the
    k-th value are all kept, up to cap); rows with ``k[r] <= 0`` hold none."""
    _dev(logits, k)
    if logits.dtype != torch.float32:
        raise KernelError("top_logprobs takes float32 logits")
    rows, vocab = logits.shape
    cap = top_logprobs_cap()
    tokens = torch.empty((rows, cap), dtype=torch.int32, device=logits.device)
    logprobs = torch.empty((rows, cap), dtype=torch.float32, device=logits.device)
    counts = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _call("lily_top_logprobs", _p(logits), _i32(k, "k"), _p(tokens), _p(logprobs), _p(counts), rows, vocab, _stream())
    return tokens, logprobs, counts
