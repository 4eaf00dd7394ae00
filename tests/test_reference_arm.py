"""The reference arm of bench.py, as far as it goes without a GPU: the checkpoint it writes is one the unmodified
reference loads (its own ModelConfig and loader, on the CPU, in a process of its own), and the tokenizer file beside
it opens.  Skipped where the reference has not been put under baseline/_ref."""

import json
import os
import subprocess
import sys
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

TINY = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 64,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "vocab_size": 256,
        "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 128,
        "hidden_act": "silu", "torch_dtype": "bfloat16"}


def test_bench_refuses_more_than_one_gpu_and_names_every_size():
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"], capture_output=True, text=True)
    assert done.returncode == 2 and "one GPU" in done.stdout and len(done.stdout.strip().splitlines()) == 1


@pytest.mark.skipif(not os.path.isfile(os.path.join(REF, "lily", "engine.py")), reason="the reference is not under baseline/_ref")
def test_the_reference_loads_the_checkpoint_the_arm_writes():
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm
    with tempfile.TemporaryDirectory() as tmp:
        total = reference_arm.write_checkpoint(TINY, tmp, seed=3)
        index = json.load(open(os.path.join(tmp, "model.safetensors.index.json")))
        assert index["metadata"]["total_size"] == total and len(set(index["weight_map"].values())) == 2 + 2
        code = (
            "import sys, torch\n"
            f"sys.path.insert(0, {REF!r})\n"
            "from transformers import AutoTokenizer\n"
            "from lily.models.model_config import ModelConfig\n"
            "from lily.models.loader import get_model\n"
            f"mc = ModelConfig.from_pretrained({tmp!r}, dtype='bfloat16')\n"
            "model = get_model(mc, device='cpu', dtype=torch.bfloat16)\n"      # raises when a parameter is missing
            "n = sum(p.numel() for p in model.parameters())\n"
            f"tok = AutoTokenizer.from_pretrained({tmp!r})\n"
            "print(n, len(tok.encode('a a')))\n")
        env = dict(os.environ, LILY_DISABLE_CUDA_KERNELS="1", HF_HUB_OFFLINE="1", TRANSFORMERS_OFFLINE="1")
        done = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=600)
        assert done.returncode == 0, done.stderr[-2000:]
        params, tokens = done.stdout.split()[-2:]
        h, d, i, v = 64, 16, 128, 256
        per_layer = h * (4 + 2 * 2) * d + 4 * d * h + 3 * h * i + 2 * h + 2 * d
        assert int(params) == 2 * per_layer + 2 * v * h + h and int(tokens) == 2
