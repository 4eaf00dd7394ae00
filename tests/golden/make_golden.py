"""Compare the plain implementation with CodeMan62/lily's own model code, once, on the CPU.

Usage (from the repository root, with the reference checkout at hand):

    python tests/golden/make_golden.py /path/to/lily-checkout

For each tiny configuration it writes a seeded random checkpoint into a temporary
folder, loads it with the reference's ``ModelConfig`` / ``get_model`` in float32 on
the CPU, runs a prompt through the reference model over the reference's own pools
and its plain PyTorch attention backend (whole, and cut into portions), and stores
the reference's logits in ``tests/golden/<name>.safetensors`` together with the
prompt.  ``tests/test_plain_impl.py`` rebuilds the same weights from the seed and
requires the plain implementation to reproduce these logits.

The reference's CUDA wrappers are switched off (``LILY_DISABLE_CUDA_KERNELS=1``):
its RMSNorm and rotary layers then take their PyTorch branches
(lily/layers/layernorm.py:34-47, lily/layers/rotary.py:70-87).
"""

from __future__ import annotations

import os
import sys
import tempfile
from types import SimpleNamespace

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

SEEDS = {"tiny_qwen3": 11, "tiny_llama": 12, "odd_qwen3": 13, "odd_llama": 14, "partial_qwen3": 15, "partial_llama": 16}
PROMPT_LEN = {"tiny_qwen3": 40, "tiny_llama": 70, "odd_qwen3": 33, "odd_llama": 48, "partial_qwen3": 45, "partial_llama": 52}
PORTIONS = (8, 2, 30, 17, 43)


def reference_logits(ref_root: str, model_dir: str, ids, portions=None) -> torch.Tensor:
    os.environ["LILY_DISABLE_CUDA_KERNELS"] = "1"
    os.environ["HF_HUB_OFFLINE"] = "1"
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    from lily.layers.attention.torch_native_backend import TorchNativeAttnBackend
    from lily.mem_cache.allocator import TokenToKVPoolAllocator
    from lily.mem_cache.memory_pool import MHATokenToKVPool, ReqToTokenPool
    from lily.model_executor.forward_batch_info import ForwardBatch
    from lily.models.loader import get_model
    from lily.models.model_config import ModelConfig

    mc = ModelConfig.from_pretrained(model_dir, dtype="float32")
    model = get_model(mc, device="cpu", dtype=torch.float32)
    req_pool = ReqToTokenPool(4, mc.context_len + 4, "cpu")
    kv_pool = MHATokenToKVPool(2048, 1, torch.float32, mc.num_key_value_heads, mc.head_dim,
                               mc.num_hidden_layers, "cpu")
    alloc = TokenToKVPoolAllocator(2048, torch.float32, "cpu", kv_pool)
    runner = SimpleNamespace(req_to_token_pool=req_pool, token_to_kv_pool=kv_pool)
    backend = TorchNativeAttnBackend(runner)
    req = req_pool.alloc(1)[0]
    cuts = [len(ids)] if portions is None else []
    if portions is not None:
        left = len(ids)
        for p in portions:
            if left <= 0:
                break
            cuts.append(min(p, left))
            left -= cuts[-1]
        if left > 0:
            cuts.append(left)
    rows, done = [], 0
    with torch.inference_mode():
        for n in cuts:
            loc = alloc.alloc(n)
            req_pool.write((req, slice(done, done + n)), loc.to(torch.int32))
            fb = ForwardBatch.for_extend([list(ids[done:done + n])], [done], [req], "cpu", out_cache_loc=loc)
            fb.attn_backend, fb.req_to_token_pool, fb.token_to_kv_pool = backend, req_pool, kv_pool
            fb.return_all_logits = True
            rows.append(model(fb.input_ids, fb.positions, fb).next_token_logits.float())
            done += n
    return torch.cat(rows)


def main() -> None:
    if len(sys.argv) < 2 or not os.path.isfile(os.path.join(sys.argv[1], "lily", "engine.py")):
        sys.exit("usage: python tests/golden/make_golden.py /path/to/lily-checkout")
    ref_root = sys.argv[1]
    from safetensors.torch import save_file

    import plain_impl
    import tiny_models

    for name, cfg in tiny_models.CONFIGS.items():
        weights = tiny_models.make_weights(cfg, SEEDS[name])
        ids = tiny_models.random_tokens(PROMPT_LEN[name], cfg["vocab_size"], SEEDS[name] + 100)
        with tempfile.TemporaryDirectory() as tmp:
            tiny_models.write_model_dir(tmp, cfg, weights)
            whole = reference_logits(ref_root, tmp, ids)
            cut = reference_logits(ref_root, tmp, ids, PORTIONS)
        plain = plain_impl.all_logits(cfg, weights, ids)
        print(f"{name}: reference whole vs portions {float((whole - cut).abs().max()):.3e}; "
              f"plain vs reference {float((plain - whole).abs().max()):.3e}; "
              f"logit scale {float(whole.abs().max()):.3f}")
        save_file({"logits": whole.contiguous(), "ids": torch.tensor(ids, dtype=torch.int32)},
                  os.path.join(HERE, f"{name}.safetensors"))


if __name__ == "__main__":
    main()
