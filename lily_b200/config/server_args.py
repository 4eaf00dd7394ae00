"""Runtime arguments: every knob is a dataclass field with a matching ``--flag``.

Names, meanings and defaults are those of CodeMan62/lily's lily/server_args.py:17-174
for the fields this engine has (one GPU, no server, no quantization, no speculative
decoding); ``page_size`` is this engine's own (the reference's pool is token-granular,
lily/mem_cache/allocator.py:37-38).
"""

from __future__ import annotations

import argparse
import dataclasses
import typing
from dataclasses import dataclass
from typing import List, Optional


@dataclass
class ServerArgs:
    # Model
    model_path: str = ""
    dtype: str = "auto"                       # auto | bfloat16 | float32
    context_length: Optional[int] = None      # overrides max_position_embeddings

    # Memory
    mem_fraction_static: Optional[float] = None   # share of device memory for weights + KV pool
    max_total_tokens: Optional[int] = None        # KV pool size in tokens (rounded up to pages)
    max_running_requests: Optional[int] = None
    max_prefill_tokens: int = 16384
    chunked_prefill_size: int = 8192
    page_size: int = 64                           # tokens per KV page

    # Scheduling
    schedule_policy: str = "fcfs"
    disable_overlap_schedule: bool = False    # read each step's tokens before the next step is launched

    # CUDA graphs (decode steps)
    disable_cuda_graph: bool = False
    cuda_graph_max_bs: Optional[int] = None
    cuda_graph_bs: Optional[List[int]] = None

    log_level: str = "info"
    random_seed: Optional[int] = None
    device: str = "cuda"

    def __post_init__(self):
        if self.mem_fraction_static is not None and not (0 < self.mem_fraction_static < 1):
            raise ValueError("mem_fraction_static must be in (0, 1)")
        if self.schedule_policy not in ("fcfs",):
            raise ValueError(f"Unknown schedule policy {self.schedule_policy!r}")
        if self.dtype not in ("auto", "bfloat16", "float32"):
            raise ValueError(f"Unknown dtype {self.dtype!r}; this engine serves bfloat16 and float32")
        if self.page_size < 1 or self.page_size & (self.page_size - 1):
            raise ValueError("page_size must be a power of two")
        for name in ("max_prefill_tokens", "chunked_prefill_size"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be positive")
        for name in ("context_length", "max_total_tokens", "max_running_requests", "cuda_graph_max_bs"):
            v = getattr(self, name)
            if v is not None and v < 1:
                raise ValueError(f"{name} must be positive")

    # ---- command line: one --flag per field, its type read from the field's annotation ----
    # (the reference builds its flags from the fields as well, lily/server_args.py:145-174)

    @classmethod
    def _flag_kinds(cls):
        """(field name, scalar type, takes a list, default) for every field."""
        hints = typing.get_type_hints(cls)
        for f in dataclasses.fields(cls):
            kind, many = hints[f.name], False
            if typing.get_origin(kind) is typing.Union:                       # Optional[T]
                kind = next(a for a in typing.get_args(kind) if a is not type(None))
            if typing.get_origin(kind) in (list, typing.List):
                kind, many = typing.get_args(kind)[0], True
            yield f.name, kind, many, (None if f.default is dataclasses.MISSING else f.default)

    @classmethod
    def add_cli_args(cls, parser: argparse.ArgumentParser) -> None:
        for name, kind, many, default in cls._flag_kinds():
            flag = "--" + name.replace("_", "-")
            if kind is bool:
                parser.add_argument(flag, action="store_true", default=bool(default))
            else:
                parser.add_argument(flag, type=kind, default=default, **({"nargs": "+"} if many else {}))

    @classmethod
    def from_cli_args(cls, args: argparse.Namespace) -> "ServerArgs":
        given = vars(args)
        return cls(**{name: given[name] for name, *_ in cls._flag_kinds() if name in given})

    @classmethod
    def parse(cls, argv: Optional[List[str]] = None) -> "ServerArgs":
        parser = argparse.ArgumentParser("lily-b200")
        cls.add_cli_args(parser)
        return cls.from_cli_args(parser.parse_args(argv))
