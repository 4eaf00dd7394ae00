"""Configuration, registry, safetensors reading and the loader's one error."""

import json
import os
import tempfile

import pytest
import torch
from safetensors.torch import load_file, save_file

import tiny_models
from lily_b200.config import ConfigError, DenseDecoderConfig, ServerArgs, resolve_architecture, supported_architectures
from lily_b200.models.assembled import AssembledModel
from lily_b200.parts.base import BuildContext, TensorSpec
from lily_b200.weights.loader import CheckpointSource, WeightsError, kept_dtype, load_model_weights
from lily_b200.weights.random_init import RandomSource, expected_tensors, write_random_model
from lily_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors


def test_config_reads_its_own_keys_with_the_reference_defaults():
    c = DenseDecoderConfig.from_dict(tiny_models.TINY_LLAMA)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 128, 8, 2, 32)
    assert c.rope_scaling.rope_type == "llama3" and c.rope_scaling.original_max_position_embeddings == 64
    assert not c.qk_norm and not c.tie_word_embeddings and c.rms_norm_eps == 1e-5
    q = DenseDecoderConfig.from_dict(tiny_models.ODD_QWEN3)
    assert q.qk_norm and q.head_dim == 288 // 6 and q.rope_theta == 30000.0 and q.attention_bias
    assert q.rope_scaling.rope_type == "default" and q.rotary_dim == 48
    o = DenseDecoderConfig.from_dict(tiny_models.ODD_LLAMA)            # "type" is read as "rope_type"
    assert o.rope_scaling.rope_type == "llama3" and o.rope_scaling.factor == 4.0
    minimal = {"architectures": ["LlamaForCausalLM"], "hidden_size": 32, "num_hidden_layers": 1,
               "num_attention_heads": 4, "intermediate_size": 64, "vocab_size": 100}
    m = DenseDecoderConfig.from_dict(minimal, {"eos_token_id": [2, 3]})
    assert (m.num_key_value_heads, m.head_dim, m.rope_theta, m.rms_norm_eps, m.max_position_embeddings) == (4, 8, 10000.0, 1e-6, 4096)
    assert m.eos_token_ids == [2, 3] and not m.tie_word_embeddings
    assert DenseDecoderConfig.from_dict(m.to_hf_dict()) == m
    nested = {"architectures": ["Qwen3ForCausalLM"], "text_config": dict(minimal, eos_token_id=7)}
    assert DenseDecoderConfig.from_dict(nested).eos_token_ids == [7]


@pytest.mark.parametrize("patch,msg", [
    ({"hidden_act": "gelu"}, "Unsupported activation"), ({"num_key_value_heads": 3}, "multiple"),
    ({"vocab_size": None}, "vocab_size"), ({"rope_scaling": {"rope_type": "yarn", "factor": 2}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2}}, "low_freq_factor"),
    ({"partial_rotary_factor": 0.3}, "rotary_dim"), ({"num_hidden_layers": 0}, "positive")])
def test_config_errors(patch, msg):
    bad = dict(tiny_models.TINY_LLAMA, **patch)
    with pytest.raises(ConfigError, match=msg):
        DenseDecoderConfig.from_dict(bad)


def test_registry():
    assert {"LlamaForCausalLM", "Qwen3ForCausalLM"} <= set(supported_architectures())   # tests may add toys
    assert resolve_architecture(["Nope", "Qwen3ForCausalLM"]).name == "Qwen3ForCausalLM"
    with pytest.raises(ValueError, match="No registered model.*LlamaForCausalLM"):
        resolve_architecture(["GPT2LMHeadModel"])


def test_files_of_real_checkpoints_parse_and_foreign_options_are_refused():
    """The keys a published Qwen3 / Llama-3.1 config.json carries beside the sizes (dropout, window switches that are off,
    library version, a null rope_scaling, a list of end tokens) are read or passed over; an option this architecture's
    code does not have is refused when it is switched on."""
    qwen = {"architectures": ["Qwen3ForCausalLM"], "attention_bias": False, "attention_dropout": 0.0, "bos_token_id": 151643,
            "eos_token_id": 151645, "head_dim": 128, "hidden_act": "silu", "hidden_size": 4096, "initializer_range": 0.02,
            "intermediate_size": 12288, "max_position_embeddings": 40960, "max_window_layers": 36, "model_type": "qwen3",
            "num_attention_heads": 32, "num_hidden_layers": 36, "num_key_value_heads": 8, "rms_norm_eps": 1e-06,
            "rope_scaling": None, "rope_theta": 1000000, "sliding_window": None, "tie_word_embeddings": False,
            "torch_dtype": "bfloat16", "transformers_version": "4.51.0", "use_cache": True, "use_sliding_window": False,
            "vocab_size": 151936}
    llama = {"architectures": ["LlamaForCausalLM"], "attention_bias": False, "attention_dropout": 0.0, "bos_token_id": 128000,
             "eos_token_id": [128001, 128008, 128009], "hidden_act": "silu", "hidden_size": 4096, "initializer_range": 0.02,
             "intermediate_size": 14336, "max_position_embeddings": 131072, "mlp_bias": False, "model_type": "llama",
             "num_attention_heads": 32, "num_hidden_layers": 32, "num_key_value_heads": 8, "pretraining_tp": 1,
             "rms_norm_eps": 1e-05, "rope_scaling": {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                                     "original_max_position_embeddings": 8192, "rope_type": "llama3"},
             "rope_theta": 500000.0, "tie_word_embeddings": False, "torch_dtype": "bfloat16", "use_cache": True, "vocab_size": 128256}
    q = DenseDecoderConfig.from_dict(qwen)
    assert (q.qk_norm, q.head_dim, q.rope_theta, q.rope_scaling.rope_type, q.eos_token_ids) == (True, 128, 1e6, "default", [151645])
    l = DenseDecoderConfig.from_dict(llama)
    assert (l.qk_norm, l.head_dim, l.rope_scaling.rope_type, l.rope_scaling.factor, l.eos_token_ids) == \
        (False, 128, "llama3", 8.0, [128001, 128008, 128009])
    newer = {k: v for k, v in qwen.items() if k not in ("torch_dtype", "rope_theta", "rope_scaling")}
    newer.update(dtype="bfloat16", rope_parameters={"rope_theta": 1000000, "rope_type": "default"}, layer_types=["full_attention"] * 36)
    assert DenseDecoderConfig.from_dict(newer) == q
    for bad, word in (({**llama, "mlp_bias": True}, "mlp_bias"), ({**qwen, "use_sliding_window": True, "sliding_window": 4096}, "sliding"),
                      ({**qwen, "hidden_act": "gelu"}, "activation"), ({**llama, "rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "yarn")):
        with pytest.raises(ConfigError, match=word):
            DenseDecoderConfig.from_dict(bad)


def test_server_args_flags_and_checks():
    a = ServerArgs.parse(["--model-path", "x", "--dtype", "float32", "--chunked-prefill-size", "64",
                          "--max-total-tokens", "4096", "--disable-cuda-graph", "--cuda-graph-bs", "1", "8"])
    assert (a.model_path, a.dtype, a.chunked_prefill_size, a.max_total_tokens, a.disable_cuda_graph, a.cuda_graph_bs) == \
        ("x", "float32", 64, 4096, True, [1, 8])
    assert a.max_prefill_tokens == 16384 and a.schedule_policy == "fcfs"
    for kw in ({"mem_fraction_static": 1.5}, {"dtype": "float16"}, {"schedule_policy": "lpm"}, {"page_size": 48},
               {"chunked_prefill_size": 0}):
        with pytest.raises(ValueError):
            ServerArgs(**kw)


def test_safetensors_round_trip_against_the_library():
    g = torch.Generator().manual_seed(0)
    tensors = {"a.weight": torch.randn(3, 5, generator=g), "b": torch.randn(7, generator=g).bfloat16(),
               "t": torch.arange(6, dtype=torch.int32).view(2, 3), "empty": torch.zeros(0, 4)}
    with tempfile.TemporaryDirectory() as tmp:
        mine, theirs = os.path.join(tmp, "mine.safetensors"), os.path.join(tmp, "theirs.safetensors")
        write_safetensors(mine, tensors, {"k": "v"})
        save_file(tensors, theirs)
        back = load_file(mine)                                   # the library reads what this package wrote
        f = SafetensorsFile(theirs)                              # this package reads what the library wrote
        for k, v in tensors.items():
            assert torch.equal(back[k], v) and torch.equal(f.tensor(k), v) and f.entries[k] == (v.dtype, tuple(v.shape))
        assert SafetensorsFile(mine).metadata == {"k": "v"}
        with open(os.path.join(tmp, "bad.safetensors"), "wb") as fh:
            fh.write(b"\xff" * 16)
        with pytest.raises(SafetensorsError):
            SafetensorsFile(os.path.join(tmp, "bad.safetensors"))


def test_loader_lists_missing_unexpected_and_wrong_shapes_in_one_error():
    cfg = tiny_models.TINY_QWEN3
    w = tiny_models.make_weights(cfg, 1)
    del w["model.layers.1.mlp.up_proj.weight"], w["model.norm.weight"]
    w["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(17)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)      # ignorable (llama.py:217-218)
    w["lm_head.weight"] = torch.zeros(256, 64)                              # ignorable when tied
    w["model.layers.0.self_attn.extra"] = torch.zeros(2)
    with tempfile.TemporaryDirectory() as tmp:
        tiny_models.write_model_dir(tmp, cfg, w)
        arch = resolve_architecture(cfg["architectures"])
        model = AssembledModel(arch.build_spec(arch.config_from_dict(cfg, {}, architecture=arch.name)),
                               BuildContext(torch.device("cpu"), torch.float32, None, max_position=8))
        with pytest.raises(WeightsError) as e:
            load_model_weights(model, CheckpointSource(tmp), torch.float32, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.extra"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_norm.weight", (17,), (16,))]
    text = str(err)
    for needle in ("2 missing", "model.norm.weight", "1 unexpected", "self_attn.extra", "wrong shape", "[17]", "[16]"):
        assert needle in text
    with pytest.raises(FileNotFoundError):
        CheckpointSource(tempfile.mkdtemp())


def test_short_vocabulary_tables_are_padded_with_zeros():
    """A checkpoint saved with fewer vocabulary rows than config.json's vocab_size loads; the missing rows of the
    embedding and of the head are zero (lily/layers/vocab_embedding.py:29-35).  More rows, or another width, do not."""
    import kernel_refs
    cfg = tiny_models.TINY_LLAMA
    w = tiny_models.make_weights(cfg, 2)
    w["model.embed_tokens.weight"] = w["model.embed_tokens.weight"][:380].clone()
    w["lm_head.weight"] = w["lm_head.weight"][:377].clone()
    arch = resolve_architecture(cfg["architectures"])
    spec = arch.build_spec(arch.config_from_dict(cfg, {}, architecture=arch.name))
    ctx = BuildContext(torch.device("cpu"), torch.float32, kernel_refs, max_position=8)
    with tempfile.TemporaryDirectory() as tmp:
        tiny_models.write_model_dir(tmp, cfg, w)
        model = AssembledModel(spec, ctx)
        load_model_weights(model, CheckpointSource(tmp), torch.float32, "cpu")
    assert model.embed.shape == (384, 128) and model.head.shape == (384, 128)
    assert torch.equal(model.embed[:380], w["model.embed_tokens.weight"]) and float(model.embed[380:].abs().max()) == 0
    assert torch.equal(model.head[:377], w["lm_head.weight"]) and float(model.head[377:].abs().max()) == 0
    w["lm_head.weight"] = torch.zeros(385, 128)
    w["model.embed_tokens.weight"] = torch.zeros(380, 127)
    with tempfile.TemporaryDirectory() as tmp:
        tiny_models.write_model_dir(tmp, cfg, w)
        with pytest.raises(WeightsError) as e:
            load_model_weights(AssembledModel(spec, ctx), CheckpointSource(tmp), torch.float32, "cpu")
    assert [n for n, _, _ in e.value.wrong_shape] == ["lm_head.weight", "model.embed_tokens.weight"]


def test_kept_dtypes():
    mat, vec, tab = TensorSpec((2, 2)), TensorSpec((2,), role="vector"), TensorSpec((2,), role="table")
    bf, f32 = torch.bfloat16, torch.float32
    assert kept_dtype(mat, bf, bf) == bf and kept_dtype(mat, f32, bf) == bf and kept_dtype(mat, bf, f32) == f32
    assert kept_dtype(vec, f32, bf) == f32 and kept_dtype(vec, bf, bf) == bf      # 32-bit stays 32-bit
    assert kept_dtype(tab, torch.int64, bf) == torch.int32


def test_random_weights_mode_writes_a_loadable_folder():
    with tempfile.TemporaryDirectory() as tmp:
        write_random_model(tmp, tiny_models.TINY_LLAMA, seed=4, dtype="bfloat16", gain_jitter=0.01)
        cfg = json.load(open(os.path.join(tmp, "config.json")))
        assert cfg["torch_dtype"] == "bfloat16" and cfg["num_hidden_layers"] == 3
        a = load_file(os.path.join(tmp, "model.safetensors"))
        arch = resolve_architecture(cfg["architectures"])
        specs = expected_tensors(arch.config_from_dict(cfg, {}, architecture=arch.name), arch)
        assert set(a) == set(specs) and all(tuple(a[k].shape) == specs[k].shape for k in a)
        assert all(v.dtype == torch.bfloat16 for v in a.values())
        assert abs(float(a["model.embed_tokens.weight"].float().std()) - 0.02) < 2e-3
        assert abs(float(a["model.norm.weight"].float().mean()) - 1.0) < 0.01
        # the same seed gives the same tensors whatever else is made; another seed differs
        src = RandomSource(specs, 4, torch.bfloat16, gain_jitter=0.01)
        assert torch.equal(src.get("lm_head.weight"), a["lm_head.weight"])
        assert not torch.equal(RandomSource(specs, 5, torch.bfloat16).get("lm_head.weight"), a["lm_head.weight"])
