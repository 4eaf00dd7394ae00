"""Tiny configurations and seeded random checkpoints for the tests.

Two configurations of the Llama / Qwen3 dense decoder that differ in every size
and option (heads and groups, head size, width, depth, vocabulary, eps, rope base
and scaling, QK-norm, tied head, bias), plus two more with sizes that are no power
of two.  The weights are drawn on the CPU from a seeded generator, under the
checkpoint's own tensor names, and saved with the ``safetensors`` package, so that
this file shares no code with ``lily_b200``'s loader or random-weights mode.
"""

from __future__ import annotations

import json
import os
from typing import Dict

import torch

TINY_QWEN3 = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "intermediate_size": 128,
    "vocab_size": 256,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "max_position_embeddings": 256,
    "hidden_act": "silu",
    "torch_dtype": "float32",
}

TINY_LLAMA = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 3,
    "hidden_size": 128,
    "num_attention_heads": 8,
    "num_key_value_heads": 2,
    "head_dim": 32,
    "intermediate_size": 352,
    "vocab_size": 384,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 512,
    "hidden_act": "silu",
    "torch_dtype": "float32",
}

# Sizes that are no power of two anywhere: 3 query heads per kv head, head size 48,
# width 136, odd vocabulary, bias on, head_dim absent from the file (hidden // heads).
ODD_QWEN3 = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 288,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "intermediate_size": 200,
    "vocab_size": 331,
    "rope_parameters": {"rope_theta": 30000.0, "rope_type": "default"},
    "rms_norm_eps": 3e-6,
    "attention_bias": True,
    "tie_word_embeddings": False,
    "max_position_embeddings": 640,
    "torch_dtype": "float32",
}

# One kv head (multi-query), head size 80, 5 heads, width that differs from heads*head_dim.
ODD_LLAMA = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 1,
    "hidden_size": 120,
    "num_attention_heads": 5,
    "num_key_value_heads": 1,
    "head_dim": 80,
    "intermediate_size": 264,
    "vocab_size": 1009,
    "rope_theta": 1000000.0,
    "rope_scaling": {"type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 2.0, "original_max_position_embeddings": 128},
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True,
    "max_position_embeddings": 1024,
    "torch_dtype": "float32",
}

# Rotation over a part of each head only: the first half of 32 features (the key beside the other sizes), and the
# first quarter of 64 with the factor given inside rope_parameters together with llama3 scaling.
PARTIAL_QWEN3 = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 80,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 32,
    "partial_rotary_factor": 0.5,
    "intermediate_size": 136,
    "vocab_size": 300,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "max_position_embeddings": 384,
    "torch_dtype": "float32",
}

PARTIAL_LLAMA = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 128,
    "num_attention_heads": 2,
    "num_key_value_heads": 1,
    "head_dim": 64,
    "intermediate_size": 200,
    "vocab_size": 500,
    "rope_parameters": {"rope_theta": 50000.0, "rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                        "high_freq_factor": 2.0, "original_max_position_embeddings": 32,
                        "partial_rotary_factor": 0.25},
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 512,
    "torch_dtype": "float32",
}

# Head size 128 and widths in multiples of 128, small enough for the CPU: the sizes at which the
# tensor-core attention, the tcgen05 gate/up kernel and the weight-streaming decode product run
# inside the engine (the tiny configurations above mostly take the CUDA-core kernels).
MID_QWEN3 = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 512,
    "num_attention_heads": 8,
    "num_key_value_heads": 2,
    "head_dim": 128,
    "intermediate_size": 1408,
    "vocab_size": 2000,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False,
    "max_position_embeddings": 1024,
    "torch_dtype": "float32",
}

def random_config(seed: int) -> dict:
    """A configuration drawn from everything the architecture's config.json can say: 1 to 4 kv heads with 1 to 8
    query heads each, head sizes from 16 to 256 in steps of 16, widths and intermediate sizes in steps of 8,
    any vocabulary, 1 to 3 layers, either family, with or without llama3 rope scaling, bias and a tied head."""
    import random
    r = random.Random(seed)
    qwen = r.random() < 0.5
    nkv = r.choice([1, 2, 3, 4])
    cfg = {
        "architectures": ["Qwen3ForCausalLM" if qwen else "LlamaForCausalLM"], "model_type": "qwen3" if qwen else "llama",
        "num_hidden_layers": r.randint(1, 3), "hidden_size": 8 * r.randint(8, 80),
        "num_attention_heads": nkv * r.choice([1, 2, 3, 4, 5, 8]), "num_key_value_heads": nkv,
        "head_dim": r.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 192, 256]),
        "intermediate_size": 8 * r.randint(8, 200), "vocab_size": r.randint(100, 3000),
        "rope_theta": r.choice([1e4, 3e4, 5e5, 1e6]), "rms_norm_eps": r.choice([1e-6, 3e-6, 1e-5]),
        "tie_word_embeddings": r.random() < 0.5, "max_position_embeddings": 1024, "torch_dtype": "float32",
    }
    if r.random() < 0.4:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": r.choice([2.0, 4.0, 8.0]), "low_freq_factor": 1.0,
                               "high_freq_factor": r.choice([2.0, 4.0]), "original_max_position_embeddings": r.choice([32, 64, 128])}
    if r.random() < 0.3:
        cfg["attention_bias"] = True
    return cfg


CONFIGS = {"tiny_qwen3": TINY_QWEN3, "tiny_llama": TINY_LLAMA, "odd_qwen3": ODD_QWEN3, "odd_llama": ODD_LLAMA,
           "partial_qwen3": PARTIAL_QWEN3, "partial_llama": PARTIAL_LLAMA}


def make_weights(cfg: dict, seed: int, std: float = 0.02, norm_jitter: float = 0.01,
                 dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    """Seeded N(0, std) matrices, norm gains 1 + N(0, norm_jitter), biases N(0, std)."""
    g = torch.Generator().manual_seed(seed)
    h = cfg["hidden_size"]
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nq
    d = cfg.get("head_dim") or h // nq
    inter, vocab = cfg["intermediate_size"], cfg["vocab_size"]
    qk_norm = cfg["architectures"][0] == "Qwen3ForCausalLM"
    bias = bool(cfg.get("attention_bias", False))

    def mat(*shape):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    def gain(n):
        return (1.0 + torch.randn(n, generator=g) * norm_jitter).to(dtype)

    w: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": mat(vocab, h)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        w[f"{p}.input_layernorm.weight"] = gain(h)
        w[f"{p}.self_attn.q_proj.weight"] = mat(nq * d, h)
        w[f"{p}.self_attn.k_proj.weight"] = mat(nkv * d, h)
        w[f"{p}.self_attn.v_proj.weight"] = mat(nkv * d, h)
        w[f"{p}.self_attn.o_proj.weight"] = mat(h, nq * d)
        if bias:
            w[f"{p}.self_attn.q_proj.bias"] = mat(nq * d)
            w[f"{p}.self_attn.k_proj.bias"] = mat(nkv * d)
            w[f"{p}.self_attn.v_proj.bias"] = mat(nkv * d)
            w[f"{p}.self_attn.o_proj.bias"] = mat(h)
        if qk_norm:
            w[f"{p}.self_attn.q_norm.weight"] = gain(d)
            w[f"{p}.self_attn.k_norm.weight"] = gain(d)
        w[f"{p}.post_attention_layernorm.weight"] = gain(h)
        w[f"{p}.mlp.gate_proj.weight"] = mat(inter, h)
        w[f"{p}.mlp.up_proj.weight"] = mat(inter, h)
        w[f"{p}.mlp.down_proj.weight"] = mat(h, inter)
    w["model.norm.weight"] = gain(h)
    if not cfg.get("tie_word_embeddings", False):
        w["lm_head.weight"] = mat(vocab, h)
    return w


def write_model_dir(path: str, cfg: dict, weights: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(path, "model.safetensors"))
    return path


def random_tokens(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
