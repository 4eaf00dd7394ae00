"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

``ModelRunner`` owns the model, the cache manager and the scratch space.  ``step`` takes, for each
request in it, that request's next tokens (a portion of a prompt cut anywhere, or one decoded
token) and the places among them whose logits are wanted; it grows the requests' block tables,
runs only the tokens it is given as one batch against the cache that earlier steps left, and
returns float32 logits ``[wanted, vocab]`` in the order the entries and their ``want`` were given.
Generation (scheduler, engine), the command line and trace replay all drive this one function.

Takes the place of ``ModelRunner.forward(ForwardBatch)`` (lily/model_executor/model_runner.py:
292-304) together with the batch preparation of lily/scheduler/schedule_batch.py:184-237; pool
sizing follows model_runner.py:160-242.
"""

from __future__ import annotations

import logging
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from lily_b200.cache.kv_cache import KVCacheManager, OutOfPages, bytes_per_token, pool_pages_from_memory
from lily_b200.config.model_config import read_model_dir
from lily_b200.config.registry import resolve_architecture
from lily_b200.config.server_args import ServerArgs
from lily_b200.engine import check
from lily_b200.engine.batch import FUTURE, StepBatch, StepEntry, Workspace, build_step_batch, order_entries, rows_are_even
from lily_b200.engine.profiler import DecodeProfiler
from lily_b200.models.assembled import AssembledModel
from lily_b200.parts.base import BuildContext, ModelSpec
from lily_b200.weights.loader import CheckpointSource, load_model_weights

logger = logging.getLogger(__name__)

_DTYPES = {"auto": torch.bfloat16, "bfloat16": torch.bfloat16, "float32": torch.float32}


class _PinnedRing:
    """A few pinned int32 buffers used in turn for the per-step metadata copy; a buffer is
    reused only after the copy that read it has finished."""

    def __init__(self, count: int = 4, ints: int = 1 << 16):
        self.ints = ints
        self.buffers = [torch.empty(ints, dtype=torch.int32, pin_memory=True) for _ in range(count)]
        self.events: List[Optional[torch.cuda.Event]] = [None] * count
        self.next = 0

    def take(self, need: int):
        if need > self.ints:
            return None, -1
        i = self.next
        self.next = (i + 1) % len(self.buffers)
        if self.events[i] is not None:
            self.events[i].synchronize()
        return self.buffers[i], i

    def mark(self, i: int) -> None:
        if i >= 0:
            ev = torch.cuda.Event()
            ev.record()
            self.events[i] = ev


class _DecodeGraph:
    """One captured decode step for up to ``bucket`` requests of up to ``max_len`` positions, about equally long
    (``even``) or not; ``even_matters`` says whether some part planned by that.  Its metadata lives
    in one static int32 buffer that every replay overwrites; rows beyond the live requests point at slot 0 and
    page 0, which no request owns (lily/model_executor/cuda_graph_runner.py:53-65,153-186 pads
    the same way)."""

    def __init__(self, runner: "ModelRunner", bucket: int, max_len: int, even: bool = False):
        self.bucket = b = bucket
        self.max_len = max_len
        self.even = even
        self.widths = [runner.cache.max_pages_per_request for _ in runner.cache.groups]
        self.sizes = [b, b, b, b + 1, b, b, b, b] + [b * w for w in self.widths]
        total = sum(self.sizes)
        self.host = torch.zeros(total, dtype=torch.int32, pin_memory=True)
        self.static = torch.zeros(total, dtype=torch.int32, device=runner.device)
        self.copied: Optional[torch.cuda.Event] = None
        parts = torch.split(self.static, self.sizes)
        self.batch = StepBatch(
            num_tokens=b, num_requests=b, num_decode=b, token_ids=parts[0], positions=parts[1], token_req=parts[2],
            cu_seqlens=parts[3], prefix_lens=parts[4], seq_lens=parts[5], slots=parts[6], logit_rows=parts[7],
            block_tables=[parts[8 + i].view(b, w) for i, w in enumerate(self.widths)],
            h_new_lens=[1] * b, h_prefix_lens=[0] * b, h_slots=[0] * b, max_seq_len=max_len,
            max_decode_len=max_len,                     # the mixers plan for the longest sequence a replay may bring
            decode_even=even,
            workspace=Workspace(runner.device),         # scratch of its own: the graph holds its address
            future_tokens=runner.future_tokens)
        # views of the pinned copy, field by field; what never changes is written once, here
        self._np = self.host.numpy()
        offsets = [0]
        for n in self.sizes:
            offsets.append(offsets[-1] + n)
        field = lambda i: self._np[offsets[i]:offsets[i + 1]]
        self._tokens, self._positions, self._prefix, self._seq, self._slots = field(0), field(1), field(4), field(5), field(6)
        field(2)[:] = range(b)                                # token_req
        field(3)[:] = range(b + 1)                            # cu_seqlens
        field(7)[:] = range(b)                                # logit rows
        self._tables = [field(8 + i).reshape(b, w) for i, w in enumerate(self.widths)]
        self._rows: List[List[int]] = [[0] * b for _ in self.widths]       # the stamp of the table each row holds
        self.fill([], [], [[] for _ in self.widths], [], [[] for _ in self.widths])
        self.static.copy_(self.host)
        stream = torch.cuda.Stream(device=runner.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream), torch.no_grad():
            for _ in range(2):                      # sizes the workspace and sets kernel attributes
                runner.model.forward(self.batch, runner.cache)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        counter = runner.model.ctx.ops.launches
        before = counter["count"]
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.logits = runner.model.forward(self.batch, runner.cache)
        self.kernels = counter["count"] - before        # this package's kernels in one replay
        self._counter = counter
        self.even_matters = self.batch.even_asked

    def fill(self, tokens: Sequence[int], prefix: Sequence[int], tables, slots: Sequence[int], stamps) -> None:
        """Writes a decode batch (padded to the bucket) into the pinned host copy.  The short fields are written
        whole; of the block tables only the rows that changed since the last step (``stamps[g][r]`` is the cache
        manager's stamp of the table in row r: a request gains a page once every ``page_size`` steps)."""
        n = len(tokens)
        if self.copied is not None:
            self.copied.synchronize()                       # the copy that read the host buffer last has finished
        self._tokens[:n] = tokens
        self._tokens[n:] = 0
        self._positions[:n] = prefix
        self._positions[n:] = 0
        self._prefix[:] = self._positions
        self._seq[:] = self._positions
        self._seq += 1
        self._slots[:n] = slots
        self._slots[n:] = 0
        for view, held, group, stamp in zip(self._tables, self._rows, tables, stamps):
            for r in range(self.bucket):
                now = stamp[r] if r < n else 0
                if held[r] == now:
                    continue
                pages = group[r] if r < n else ()
                view[r, :len(pages)] = pages
                view[r, len(pages):] = 0
                held[r] = now

    def run(self, tokens, prefix, tables, slots, stamps) -> torch.Tensor:
        self.fill(tokens, prefix, tables, slots, stamps)
        self.static.copy_(self.host, non_blocking=True)
        self.copied = torch.cuda.Event()
        self.copied.record()
        self.graph.replay()
        self._counter["count"] += self.kernels
        return self.logits[:len(tokens)]


class ModelRunner:
    def __init__(self, spec: ModelSpec, source: Any, args: ServerArgs, ops: Any = None):
        if ops is None:
            from lily_b200.csrc import ops as _ops
            if not torch.cuda.is_available():
                raise RuntimeError("lily_b200 runs on a CUDA device (B200, sm_100a) and has no CPU path")
            _ops.library()                    # build / load now: a missing extension fails here, loudly
            ops = _ops
        self.args = args
        self.spec = spec
        self.device = torch.device(args.device)
        self.dtype = _DTYPES[args.dtype]
        self.context_len = int(args.context_length or spec.max_position)
        self.page_size = args.page_size
        if args.random_seed is not None:
            torch.manual_seed(args.random_seed)
        ctx = BuildContext(device=self.device, dtype=self.dtype, ops=ops, page_size=self.page_size,
                           max_position=self.context_len)
        t0 = time.time()
        self.model = AssembledModel(spec, ctx)
        moved = load_model_weights(self.model, source, self.dtype, self.device)
        self.weight_bytes = moved
        logger.info("loaded %s in %.1f s (%.2f GB on the device)", spec.architecture, time.time() - t0, moved / 1e9)

        groups = self.model.cache_groups
        if args.max_total_tokens is not None:
            pages = -(-args.max_total_tokens // self.page_size)
        else:
            if self.device.type == "cuda":
                torch.cuda.empty_cache()
                free, total = torch.cuda.mem_get_info(self.device)
            else:
                free = total = 1 << 30
            pages = pool_pages_from_memory(groups, self.dtype, self.page_size, free, total,
                                           args.mem_fraction_static or 0.85)
            if pages < 1:
                raise RuntimeError("no memory left for the KV cache; raise --mem-fraction-static or give "
                                   "--max-total-tokens")
        self.max_requests = int(args.max_running_requests or min(max(pages, 1), 256))
        self.cache = KVCacheManager(groups, self.model.state_needs, page_size=self.page_size, num_pages=pages,
                                    max_requests=self.max_requests, max_context=self.context_len, dtype=self.dtype,
                                    device=self.device)
        logger.info("KV cache: %d pages of %d tokens (%.2f GB), %d request slots", pages, self.page_size,
                    pages * self.page_size * bytes_per_token(groups, self.dtype) / 1e9, self.max_requests)
        self.workspace = Workspace(self.device)
        # the last token sampled for each request slot, on the device: a step may name it (FUTURE)
        # instead of a token id that the host has not read yet
        self.future_tokens = torch.zeros(self.max_requests + 1, dtype=torch.int32, device=self.device)
        self._last_rows: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None
        self.seq_lens: Dict[int, int] = {}
        self._ring = _PinnedRing() if self.device.type == "cuda" else None
        self.profiler = DecodeProfiler.from_env() if self.device.type == "cuda" else None
        self.steps_run = 0
        self.tokens_run = 0
        self.graph_steps = 0
        self._graphs: Dict[Tuple[int, int, bool], _DecodeGraph] = {}      # by (batch bucket, length class, rows even)
        self.use_graphs = self.device.type == "cuda" and not args.disable_cuda_graph and self.model.graph_safe
        max_bs = args.cuda_graph_max_bs or min(self.max_requests, 256)
        self.graph_buckets = sorted(set(args.cuda_graph_bs or
                                        [b for b in (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256) if b <= max_bs]
                                        + [max_bs]))
        # A mixer plans a captured step for the longest sequence a replay may bring, and the best plan for a long
        # sequence is a poor one for a short one (decode attention over 128 k keys wants many more key ranges than
        # over 4 k).  So graphs also come in classes of sequence length: 8 k positions, then doubling up to the
        # context length; a model with a context of 8 k or less has one class.
        self.length_classes = []
        bound = 8192
        while bound < self.context_len:
            self.length_classes.append(bound)
            bound *= 2
        self.length_classes.append(self.context_len)

    # ---- construction ---------------------------------------------------------------

    @classmethod
    def from_model_dir(cls, args: ServerArgs, ops: Any = None) -> "ModelRunner":
        cfg, gen = read_model_dir(args.model_path)
        arch = resolve_architecture(cfg.get("architectures"))
        config = arch.config_from_dict(cfg, gen, architecture=arch.name)
        return cls(arch.build_spec(config), CheckpointSource(args.model_path), args, ops)

    @classmethod
    def from_random(cls, config_json: Dict[str, Any], seed: int, args: ServerArgs, ops: Any = None,
                    std: float = 0.02, gain_jitter: float = 0.0) -> "ModelRunner":
        """A model with seeded random weights drawn on the device, without a file."""
        from lily_b200.weights.random_init import RandomSource, expected_tensors

        arch = resolve_architecture(config_json.get("architectures"))
        config = arch.config_from_dict(config_json, {}, architecture=arch.name)
        store = torch.float32 if args.dtype == "float32" else torch.bfloat16
        source = RandomSource(expected_tensors(config, arch), seed, store, args.device, std, gain_jitter)
        return cls(arch.build_spec(config), source, args, ops)

    # ---- requests --------------------------------------------------------------------

    def open_request(self) -> int:
        slot = self.cache.open_request()
        self.seq_lens[slot] = 0
        return slot

    def close_request(self, slot: int) -> None:
        self.cache.close_request(slot)
        del self.seq_lens[slot]

    def free_tokens(self) -> int:
        return self.cache.free_tokens()

    # ---- one step --------------------------------------------------------------------

    def prepare(self, entries: Sequence[StepEntry], logit_rows_in_given_order: bool = True) -> StepBatch:
        """Grows the block tables and packs the batch.  Raises ``OutOfPages`` before anything is
        changed when the pool cannot hold the step."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        vocab = self.spec.vocab_size
        seen = set()
        for e in entries:
            if e.slot not in self.seq_lens:
                raise KeyError(f"request slot {e.slot} is not open")
            if e.slot in seen:
                raise ValueError(f"request slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if len(e.tokens) == 0:
                raise ValueError("an entry brings at least one token")
            if not (len(e.tokens) == 1 and int(e.tokens[0]) == FUTURE) and any(not (0 <= int(t) < vocab) for t in e.tokens):
                raise ValueError(f"token id outside [0, {vocab})")
            if self.seq_lens[e.slot] + len(e.tokens) > self.context_len:
                raise ValueError(f"request would reach {self.seq_lens[e.slot] + len(e.tokens)} positions; "
                                 f"the context length is {self.context_len}")
        wants = [(e.slot, self.seq_lens[e.slot] + len(e.tokens)) for e in entries]
        if not self.cache.can_grow(wants):
            raise OutOfPages(f"step of {sum(len(e.tokens) for e in entries)} tokens does not fit: "
                             f"{self.cache.free_pages()} pages free")
        for slot, new_len in wants:
            self.cache.grow(slot, new_len)
        if check.ENABLED:
            check.check_entries(self, entries)
        order = order_entries(entries)
        ordered = [entries[i] for i in order]
        prefix = [self.seq_lens[e.slot] for e in ordered]
        offsets, run = {}, 0
        for i, e in zip(order, ordered):
            offsets[i] = run
            run += len(e.tokens)
        rows: List[int] = []
        for i, e in enumerate(entries):
            for w in e.want:
                if not (0 <= w < len(e.tokens)):
                    raise ValueError(f"wanted place {w} is outside the {len(e.tokens)} tokens of the entry")
                rows.append(offsets[i] + int(w))
        tables = [[self.cache.block_table(g, e.slot) for e in ordered] for g in range(len(self.cache.groups))]
        need = 3 * run + 4 * len(entries) + 1 + len(rows) + sum(
            len(entries) * max((len(t) for t in g), default=1) for g in tables) + 8
        pinned, ring_index = self._ring.take(need) if self._ring is not None else (None, -1)
        batch = build_step_batch(ordered, prefix, tables, self.device, workspace=self.workspace, pinned=pinned,
                                 logit_rows=rows)
        if self._ring is not None:
            self._ring.mark(ring_index)
        batch.future_tokens = self.future_tokens
        if check.ENABLED:
            check.check_batch(self, batch)
        return batch

    def store_future(self, tokens: torch.Tensor) -> None:
        """``tokens`` (int32, on the device) are what was sampled from the logits of the last step, row
        by row: each goes to its request's entry of ``future_tokens``, where a later step that names
        FUTURE for that request finds it."""
        if self._last_rows is None:
            raise RuntimeError("no step has run")
        rows, token_req, slots = self._last_rows
        self.model.ctx.ops.scatter_tokens(tokens, rows, token_req, slots, self.future_tokens)

    def _graph_bucket(self, entries: Sequence[StepEntry]) -> Optional[int]:
        if not self.use_graphs or len(entries) > self.graph_buckets[-1]:
            return None
        if any(len(e.tokens) != 1 or list(e.want) != [0] for e in entries):
            return None
        return next(b for b in self.graph_buckets if b >= len(entries))

    def _length_class(self, longest: int) -> int:
        return next((c for c in self.length_classes if c >= longest), self.length_classes[-1])

    def capture_decode_graphs(self, batch_sizes: Optional[Sequence[int]] = None,
                              max_len: Optional[int] = None) -> List[int]:
        """Captures the decode graphs for these batch sizes now (default: every bucket) instead of at the first step
        that needs each, and returns the buckets captured: for sequences of up to ``max_len`` positions, or, by
        default, for every class of sequence length the context allows (one, up to a context of 8 k positions); where
        a part plans by whether the rows are about equally long, for both kinds of batch.
        A capture runs the model three times on padded rows that belong to no request, so it needs no live request
        and disturbs none; a server that wants no pause at the first step of each batch size calls this once after
        loading (the reference captures all of its buckets when the runner is built:
        lily/model_executor/cuda_graph_runner.py:93,147-149)."""
        if not self.use_graphs:
            return []
        want = self.graph_buckets if batch_sizes is None else sorted(
            {next(b for b in self.graph_buckets if b >= n) for n in batch_sizes if 1 <= n <= self.graph_buckets[-1]})
        classes = self.length_classes if max_len is None else [self._length_class(max_len)]
        done = []
        for bucket in want:
            for cls in classes:
                for even in (False, True):
                    if (bucket, cls, even) not in self._graphs:
                        self._graph_for(bucket, cls, even)
                        if bucket not in done:
                            done.append(bucket)
        return done

    def _graph_for(self, bucket: int, cls: int, even: bool) -> _DecodeGraph:
        """The captured step for this bucket, length class and kind of batch; one capture serves both kinds when
        no part planned by the rows' evenness."""
        graph = self._graphs.get((bucket, cls, even))
        if graph is None:
            graph = self._graphs[(bucket, cls, even)] = _DecodeGraph(self, bucket, cls, even)
            if not graph.even_matters:
                self._graphs[(bucket, cls, not even)] = graph
        return graph

    def _decode_with_graph(self, entries: Sequence[StepEntry], bucket: int) -> torch.Tensor:
        """A step of one token per request, each wanting its logits, through a captured graph."""
        vocab = self.spec.vocab_size
        wants = []
        for e in entries:
            if e.slot not in self.seq_lens:
                raise KeyError(f"request slot {e.slot} is not open")
            if int(e.tokens[0]) != FUTURE and not (0 <= int(e.tokens[0]) < vocab):
                raise ValueError(f"token id outside [0, {vocab})")
            if self.seq_lens[e.slot] + 1 > self.context_len:
                raise ValueError(f"request would pass the context length {self.context_len}")
            wants.append((e.slot, self.seq_lens[e.slot] + 1))
        if len({e.slot for e in entries}) != len(entries):
            raise ValueError("a request slot appears twice in one step")
        if not self.cache.can_grow(wants):
            raise OutOfPages(f"decode step of {len(entries)} tokens does not fit: {self.cache.free_pages()} pages free")
        for slot, new_len in wants:
            self.cache.grow(slot, new_len)
        if check.ENABLED:
            check.check_entries(self, entries)
        graph = self._graph_for(bucket, self._length_class(max(n for _, n in wants)), rows_are_even([n for _, n in wants]))
        groups = range(len(self.cache.groups))
        tables = [[self.cache.block_table(g, e.slot) for e in entries] for g in groups]
        stamps = [[self.cache.table_stamp(g, e.slot) for e in entries] for g in groups]
        self.graph_steps += 1
        self._last_rows = (graph.batch.logit_rows, graph.batch.token_req, graph.batch.slots)
        if check.ENABLED:
            graph.fill([e.wire_tokens[0] for e in entries], [self.seq_lens[e.slot] for e in entries], tables,
                       [e.slot for e in entries], stamps)
            check.check_graph_fill(self, graph, len(entries))
        return graph.run([e.wire_tokens[0] for e in entries], [self.seq_lens[e.slot] for e in entries], tables,
                         [e.slot for e in entries], stamps)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs one step and returns float32 logits ``[sum(len(e.want)), vocab]`` on the device.
        (A step replayed from a graph returns a view of the graph's output, valid until the next
        step of the same batch bucket.)"""
        if self.profiler is not None:
            self.profiler.before_step(len(entries) if all(len(e.tokens) == 1 for e in entries) else None)
        bucket = self._graph_bucket(entries)
        if bucket is not None:
            logits = self._decode_with_graph(entries, bucket)
            batch = None
        else:
            batch = self.prepare(entries)
            self._last_rows = (batch.logit_rows, batch.token_req, batch.slots)
            with torch.no_grad():
                logits = self.model.forward(batch, self.cache)
        for e in entries:
            self.seq_lens[e.slot] += len(e.tokens)
            self.cache.advance(e.slot, self.seq_lens[e.slot])
        self.steps_run += 1
        self.tokens_run += sum(len(e.tokens) for e in entries)
        return logits
