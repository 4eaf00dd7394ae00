"""Runtime arguments: every knob is a dataclass field with a matching ``--flag``.

Names, meanings and defaults are those of CodeMan62/lily's lily/server_args.py:17-174
for the fields this engine has (one GPU, no server, no quantization, no speculative
decoding); ``page_size`` is this engine's own (the reference's pool is token-granular,
lily/mem_cache/allocator.py:37-38).
"""

from __future__ import annotations

import argparse
import dataclasses
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

    # ---- CLI binding (lily/server_args.py:145-174) ---------------------------

    @staticmethod
    def add_cli_args(parser: argparse.ArgumentParser) -> None:
        for f in dataclasses.fields(ServerArgs):
            flag = "--" + f.name.replace("_", "-")
            default = f.default if f.default is not dataclasses.MISSING else None
            if isinstance(default, bool):
                parser.add_argument(flag, action="store_true", default=default)
            elif f.name == "cuda_graph_bs":
                parser.add_argument(flag, type=int, nargs="+", default=default)
            elif isinstance(default, int) or f.type in ("Optional[int]", Optional[int]):
                parser.add_argument(flag, type=int, default=default)
            elif isinstance(default, float) or f.type in ("Optional[float]", Optional[float]):
                parser.add_argument(flag, type=float, default=default)
            else:
                parser.add_argument(flag, type=str, default=default)

    @classmethod
    def from_cli_args(cls, args: argparse.Namespace) -> "ServerArgs":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in vars(args).items() if k in names})

    @classmethod
    def parse(cls, argv: Optional[List[str]] = None) -> "ServerArgs":
        parser = argparse.ArgumentParser("lily-b200")
        cls.add_cli_args(parser)
        return cls.from_cli_args(parser.parse_args(argv))
