"""Where a decode step's time goes, measured inside the running engine.

``LILY_B200_PROFILE_BS=1,8`` arms the step function: the first all-decode step with that many
requests opens a window over the next ``LILY_B200_PROFILE_STEPS`` (default 20) such steps, and
when it closes a table goes to the log and, with ``LILY_B200_PROFILE_OUT=<folder>``, to
``<folder>/decode_step_bs<N>.txt``: for each kernel its launches per step and two times per step,
summed over every launch of the window (kernels inside replayed CUDA graphs included).  ``own`` is
the time from the end of whatever ran before it (or its own start, if later) to its own end: the
kernels of a step are launched so that one may start while its predecessor drains (programmatic
dependent launch), and a kernel that waits inside for its predecessor would otherwise be charged
for that wait; the ``own`` column adds up to the time the device was busy.  ``resident`` is the
plain start-to-end duration.  (The window opens at the second step of its batch size: the first
may capture a CUDA graph.)
The reference has the same switch for its server (lily/profiler.py:20-66, hooked at
lily/scheduler/scheduler.py:455-456).

The window is timed by the CUDA profiling interface underneath ``torch.profiler``: its per-kernel
durations are exact, while the steps themselves run a little slower than unprofiled ones, so the
table explains a step and a benchmark times it.
"""

from __future__ import annotations

import logging
import os
from collections import defaultdict
from typing import Dict, List, Optional, Tuple

import torch

logger = logging.getLogger(__name__)


class DecodeProfiler:
    def __init__(self, sizes: List[int], steps: int = 20, out_dir: Optional[str] = None):
        self.pending = set(sizes)
        self.steps = max(1, steps)
        self.out_dir = out_dir
        self.tables: Dict[int, str] = {}
        self._prof = None
        self._bs = self._n = 0
        self._elapsed = 0.0
        self._seen = set()

    @classmethod
    def from_env(cls) -> Optional["DecodeProfiler"]:
        spec = os.environ.get("LILY_B200_PROFILE_BS", "").strip()
        if not spec:
            return None
        return cls([int(x) for x in spec.split(",") if x.strip()], int(os.environ.get("LILY_B200_PROFILE_STEPS", "20")),
                   os.environ.get("LILY_B200_PROFILE_OUT") or None)

    def before_step(self, decode_requests: Optional[int]) -> None:
        """Called by the step function before every step; ``decode_requests`` is the batch size of an
        all-decode step and None for any other."""
        if self._prof is None:
            if decode_requests in self.pending and decode_requests not in self._seen:
                self._seen.add(decode_requests)         # this step may capture its graph: the next one opens the window
                return
            if decode_requests in self.pending:
                from torch.profiler import ProfilerActivity, profile
                self.pending.discard(decode_requests)
                self._bs, self._n = decode_requests, 0
                torch.cuda.synchronize()
                self._prof = profile(activities=[ProfilerActivity.CUDA])
                self._prof.__enter__()
            return
        self._n += 1
        if decode_requests == self._bs and self._n < self.steps:
            return
        self._close()

    def _close(self) -> None:
        torch.cuda.synchronize()
        self._prof.__exit__(None, None, None)
        table = self.table(self._kernel_times(), self._n, self._bs, elapsed=self._elapsed)
        self.tables[self._bs] = table
        logger.info("%s", table)
        if self.out_dir:
            os.makedirs(self.out_dir, exist_ok=True)
            with open(os.path.join(self.out_dir, f"decode_step_bs{self._bs}.txt"), "w") as f:
                f.write(table + "\n")
        self._prof = None

    def _kernel_times(self) -> List[Tuple[float, float, int, str]]:
        """(own microseconds, resident microseconds, launches, name) per kernel over the window."""
        spans = []
        for ev in self._prof.events():
            if ev.device_type.name == "CPU":
                continue
            start, end = float(ev.time_range.start), float(ev.time_range.end)
            if end > start:
                spans.append((start, end, ev.name))
        spans.sort()
        self._elapsed = (max(e for _, e, _ in spans) - spans[0][0]) if spans else 0.0
        own: Dict[str, float] = defaultdict(float)
        resident: Dict[str, float] = defaultdict(float)
        count: Dict[str, int] = defaultdict(int)
        busy_until = 0.0
        for start, end, name in spans:
            own[name] += max(0.0, end - max(start, busy_until))
            resident[name] += end - start
            count[name] += 1
            busy_until = max(busy_until, end)
        return sorted(((own[n], resident[n], count[n], n) for n in own), reverse=True)

    @staticmethod
    def table(items: List[Tuple[float, float, int, str]], steps: int, batch: int, rows: int = 40, elapsed: float = 0.0) -> str:
        whole = sum(t for t, _, _, _ in items) or 1.0
        idle = f" ({elapsed / steps:.1f} us a step from the first kernel's start to the last one's end)" if elapsed else ""
        lines = [f"decode step at batch {batch}: device time per step over {steps} steps{idle}",
                 f"{'own us':>9} {'%':>5} {'resident':>9} {'launches':>8}  kernel",
                 f"{whole / steps:9.1f} {100.0:5.1f} {sum(r for _, r, _, _ in items) / steps:9.1f} "
                 f"{sum(c for _, _, c, _ in items) / steps:8.1f}  all kernels"]
        lines += [f"{t / steps:9.1f} {100 * t / whole:5.1f} {r / steps:9.1f} {c / steps:8.1f}  {name[:100]}"
                  for t, r, c, name in items[:rows]]
        return "\n".join(lines)
