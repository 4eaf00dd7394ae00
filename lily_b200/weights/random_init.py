"""The random-weights mode: a model folder from a configuration and a seed.

Every tensor the architecture expects is drawn from its own generator, seeded by (seed, tensor
name), so a tensor's values do not depend on the order in which tensors are made or on which
other tensors exist: "normal" tensors are N(0, std), "gain" tensors 1 + N(0, gain_jitter),
"zeros" tensors 0.  ``write_random_model`` writes ``config.json`` and ``model.safetensors``;
``RandomSource`` hands the same tensors to the loader without a file (on the device when one is
given, which is how a model of several GB is made in seconds).

The reference has no such mode for this architecture; its tests of other architectures write
tiny random checkpoints the same way (tests/small_qwen35.py:1-5 in the reference).
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Optional, Tuple

import torch

from lily_b200.parts.base import BuildContext, TensorSpec
from lily_b200.weights.safetensors_io import write_safetensors

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _seed_for(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") & ((1 << 62) - 1)


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype, device="cpu", std: float = 0.02,
                  gain_jitter: float = 0.0) -> torch.Tensor:
    if spec.role == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    g = torch.Generator(device=device).manual_seed(_seed_for(seed, name))
    x = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
    if spec.init == "gain":
        x = 1.0 + x * gain_jitter
    else:
        x = x * std
    return x.to(dtype)


def expected_tensors(config: Any, architecture) -> Dict[str, TensorSpec]:
    """The tensors of the architecture's model, from its spec alone (no device, no kernels)."""
    from lily_b200.models.assembled import AssembledModel

    ctx = BuildContext(device=torch.device("cpu"), dtype=torch.float32, ops=None, max_position=1)
    return AssembledModel(architecture.build_spec(config), ctx).tensors()


class RandomSource:
    """Stands where a checkpoint stands for the loader."""

    def __init__(self, specs: Dict[str, TensorSpec], seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu",
                 std: float = 0.02, gain_jitter: float = 0.0):
        self.specs, self.seed, self.dtype, self.device = specs, seed, dtype, device
        self.std, self.gain_jitter = std, gain_jitter

    def entries(self) -> Dict[str, Tuple[torch.dtype, tuple]]:
        return {n: (torch.int32 if s.role == "table" else self.dtype, tuple(s.shape)) for n, s in self.specs.items()}

    def get(self, name: str) -> torch.Tensor:
        return random_tensor(name, self.specs[name], self.seed, self.dtype, self.device, self.std, self.gain_jitter)


def write_random_model(path: str, config_json: Dict[str, Any], seed: int, dtype: Optional[str] = None,
                       std: float = 0.02, gain_jitter: float = 0.0) -> str:
    """Writes ``path/config.json`` and ``path/model.safetensors`` for the architecture that
    ``config_json["architectures"]`` names.  ``dtype`` ("bfloat16" | "float32") defaults to the
    configuration's ``torch_dtype``."""
    from lily_b200.config.registry import resolve_architecture

    arch = resolve_architecture(config_json.get("architectures"))
    config = arch.config_from_dict(config_json, {}, architecture=arch.name)
    store = dtype or config_json.get("torch_dtype") or "bfloat16"
    if store not in _DTYPES:
        raise ValueError(f"random weights are written as bfloat16 or float32, not {store!r}")
    specs = expected_tensors(config, arch)
    src = RandomSource(specs, seed, _DTYPES[store], "cpu", std, gain_jitter)
    os.makedirs(path, exist_ok=True)
    cfg = dict(config_json)
    cfg["torch_dtype"] = store
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    entries = [(n, dt, shape) for n, (dt, shape) in src.entries().items()]
    write_safetensors(os.path.join(path, "model.safetensors"), entries, {"format": "pt", "seed": str(seed)},
                      produce=src.get)
    return path
