"""The Llama / Qwen3 dense decoder as a ``ModelSpec``.

Every layer is a pre-norm block of grouped-query attention with rotary positions and a SwiGLU
feed-forward; Qwen3 adds the per-head q/k RMSNorm.  Tensor names are the checkpoint's own
(lily/models/llama.py:93-150,153-245; lily/models/qwen3.py:17-37).
"""

from __future__ import annotations

from lily_b200.config.model_config import DenseDecoderConfig
from lily_b200.config.registry import register_architecture
from lily_b200.parts.attention import AttentionSpec
from lily_b200.parts.base import BlockSpec, ModelSpec, ScheduleEntry
from lily_b200.parts.mlp import SwiGLUSpec
from lily_b200.parts.norm import RMSNormSpec
from lily_b200.parts.rope import RopeSpec


def build_spec(cfg: DenseDecoderConfig) -> ModelSpec:
    rope = RopeSpec(cfg.head_dim, cfg.rotary_dim, cfg.rope_theta, cfg.rope_scaling)
    blocks = []
    for i in range(cfg.num_hidden_layers):
        blocks.append(BlockSpec(
            prefix=f"model.layers.{i}",
            mixer=AttentionSpec(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                qk_norm=cfg.qk_norm, norm_eps=cfg.rms_norm_eps, bias=cfg.attention_bias,
                                position=rope),
            feed_forward=SwiGLUSpec(cfg.hidden_size, cfg.intermediate_size),
            norm_in=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps),
            norm_post=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps)))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, blocks=blocks,
        schedule=[ScheduleEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps),
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        max_position=cfg.max_position_embeddings, eos_token_ids=list(cfg.eos_token_ids))


for _name in ("LlamaForCausalLM", "Qwen3ForCausalLM"):
    register_architecture(_name, DenseDecoderConfig.from_dict, build_spec)
