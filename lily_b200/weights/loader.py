"""Loading a model's tensors from safetensors by name.

The model says what it expects (``tensors()``: name -> shape and role); the files' headers say
what is there.  Names and shapes are compared before any data is read, and every problem is
reported at once in one ``WeightsError``: tensors the model needs and the files lack, tensors the
files hold and the model does not know, and tensors whose shape differs.

Kept dtypes: matrices are held in the compute dtype (bfloat16 stays bfloat16; a float32
checkpoint served in bfloat16 is cast, as lily/models/model_config.py:222-229 serves it);
gains and other vectors stored in 32-bit stay 32-bit; integer tables become int32.  With a
float32 compute dtype everything is float32.

Reference: lily/models/loader.py:24-33 (file discovery), :87-95 (iteration by name), :97-128
(missing parameters raise; unexpected ones are only logged there, and raised here).
"""

from __future__ import annotations

import logging
from typing import Callable, Dict, List, Tuple

import torch

from lily_b200.parts.base import TensorSpec
from lily_b200.weights.safetensors_io import SafetensorsFile, safetensors_files

logger = logging.getLogger(__name__)


class WeightsError(RuntimeError):
    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[Tuple[str, tuple, tuple]],
                 where: str):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = [f"checkpoint {where} does not fit the model:"]
        if missing:
            lines.append(f"  {len(missing)} missing tensor(s): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  {len(unexpected)} unexpected tensor(s): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  {len(wrong_shape)} tensor(s) of the wrong shape: " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong_shape))
        super().__init__("\n".join(lines))


def kept_dtype(spec: TensorSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if spec.role == "table":
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if spec.role == "vector" and stored in (torch.float32, torch.float64):
        return torch.float32
    return compute


class CheckpointSource:
    """``get(name)`` over the safetensors files of a model folder."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.files = [SafetensorsFile(p) for p in safetensors_files(model_dir)]
        self.where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name in f.entries:
                self.where[name] = f

    def entries(self) -> Dict[str, Tuple[torch.dtype, tuple]]:
        return {name: f.entries[name] for name, f in self.where.items()}

    def get(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)


def fits(spec: TensorSpec, stored: tuple) -> bool:
    """Whether a stored tensor of this shape serves: the expected shape, or, for a table that allows it, fewer rows."""
    want = tuple(spec.shape)
    if stored == want:
        return True
    return bool(spec.short_rows and len(stored) == len(want) and stored[1:] == want[1:] and 0 < stored[0] < want[0])


def check(expected: Dict[str, TensorSpec], present: Dict[str, Tuple[torch.dtype, tuple]],
          ignorable: Callable[[str], bool], where: str) -> None:
    missing = sorted(n for n in expected if n not in present)
    unexpected = sorted(n for n in present if n not in expected and not ignorable(n))
    wrong = sorted((n, tuple(present[n][1]), tuple(spec.shape)) for n, spec in expected.items()
                   if n in present and not fits(spec, tuple(present[n][1])))
    if missing or unexpected or wrong:
        raise WeightsError(missing, unexpected, wrong, where)


def load_model_weights(model, source, compute_dtype: torch.dtype, device) -> int:
    """Checks ``source`` against ``model.tensors()``, then lets the model pack its tensors.
    ``source`` has ``entries()`` and ``get(name)``.  Returns the bytes moved to the device."""
    expected = model.tensors()
    present = source.entries()
    check(expected, present, model.ignorable, getattr(source, "model_dir", "<generated>"))
    moved = 0

    def get(name: str) -> torch.Tensor:
        nonlocal moved
        t = source.get(name)
        want = kept_dtype(expected[name], t.dtype, compute_dtype)
        out = t.to(device=device, dtype=want)
        rows = expected[name].shape[0] if expected[name].shape else 0
        if out.dim() and out.shape[0] < rows:                       # a short vocabulary table: the rest is zero
            full = torch.zeros((rows, *out.shape[1:]), dtype=want, device=device)
            full[:out.shape[0]].copy_(out)
            out = full
        moved += out.numel() * out.element_size()
        return out

    model.load(get)
    return moved
