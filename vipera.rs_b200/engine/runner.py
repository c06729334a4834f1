"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

One step runs only the tokens it is given, as one flattened batch, against the cache that
earlier steps left: portions of prompts beside single decode tokens, cut anywhere.  The
reference's seam has the same shape — ``logits_batch(BatchContext{kv, entries})`` with an
entry = (tokens, new_tokens, first_position, block_table) (crates/vipera-runtime/src/
pipeline.rs:139-152, 219-229) — but its CPU backend runs every entry of a mixed batch alone
(crates/vipera-backend-cpu/src/model.rs:796-827); here all entries share every product.

Host-side checks before any launch follow model.rs:890-927, 957-964: token ids inside the
vocabulary, positions inside the model's reach, block tables that cover every position.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import gc
import os
import weakref

import numpy as np
import torch

from ..errors import InternalError, InvalidArgumentError
from ..parts.base import StepContext, Workspace


@dataclass
class StepInput:
    """One step on the host side.  ``requests[i]`` is open in the cache manager with pages
    reserved for positions ``pos0[i] .. pos0[i] + counts[i] - 1``."""

    requests: Sequence[int]
    tokens: np.ndarray          # int32, entry after entry
    counts: Sequence[int]
    pos0: Sequence[int]
    fresh: Sequence[int]
    logit_rows: np.ndarray      # int32 indices into tokens


def _round_up_pow2(value: int, least: int = 8) -> int:
    out = least
    while out < value:
        out *= 2
    return out


def _width_bucket(pages: int) -> int:
    """The width a decode graph's block tables are rounded up to: a power of two up to 128
    pages, eighths of an octave beyond (the cut of the keys for the split-key attention is
    chosen for the graph's width, so a width far above the longest history cuts badly)."""
    width = _round_up_pow2(pages)
    if width <= 128:
        return width
    step = width // 16
    return -(-pages // step) * step


# Token counts a captured step is padded to.  Steps under a token budget are mostly full, so the
# steps that matter hit a bucket exactly; in between at most a third of a step is padding.
_TOKEN_BUCKETS = (8, 16, 32, 64, 96, 128, 192, 256, 384, 512, 768, 1024, 1536, 2048, 3072, 4096, 6144, 8192)


def _capture(forward):
    """Capture `forward()` (kernel launches on the current stream) in a CUDA graph; returns the
    graph and what `forward` returned.  The collector is held off meanwhile: it may run in any
    thread at any allocation, and an object it finalises there (an old graph, a pool) can make
    a CUDA call that is not allowed while a stream is capturing, which spoils the capture.  For
    the same reason only this thread's calls count as part of the capture."""
    graph = torch.cuda.CUDAGraph()
    collecting = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            result = forward()
    finally:
        if collecting:
            gc.enable()
    return graph, result


def _token_bucket(tokens: int) -> Optional[int]:
    for bucket in _TOKEN_BUCKETS:
        if tokens <= bucket:
            return bucket
    return None


class ModelRunner:
    """Owns the workspace and the staging buffers; turns a StepInput into device tensors,
    runs the model, and returns the logits tensor (device, float32, [rows, vocab])."""

    def __init__(self, model, pools, *, max_model_len: int):
        if not torch.cuda.is_available():
            raise InternalError("no CUDA device: this engine has no CPU path")
        self.model = model
        self.pools = pools
        self.manager = pools.manager
        self.device = model.device
        self.max_model_len = int(max_model_len)
        prepare = getattr(model, "prepare", None)
        if prepare is not None:
            prepare(self.max_model_len)
        self.workspace = Workspace(self.device)
        self._staging_host: Optional[torch.Tensor] = None
        self._staging_dev: Optional[torch.Tensor] = None
        self._copy_done = torch.cuda.Event()
        self._copy_pending = False
        self.steps_run = 0
        self.decode_graphs = True
        # Steps that bring portions of prompts replay captured graphs too (padded to a size
        # class); VIPERA_STEP_GRAPHS=0 launches them kernel by kernel.
        self.step_graphs = os.environ.get("VIPERA_STEP_GRAPHS", "1") != "0"
        self._graph_safe = None  # asked of the model once
        self.max_graph_entries = 256
        self.max_kept_graphs = 256
        self._graphs = {}
        self._step_graphs = {}
        self.graph_replays = 0   # steps that replayed a captured graph ...
        self.eager_steps = 0     # ... and steps launched kernel by kernel
        self.graph_captures = 0  # graphs captured (a buffer that grows makes the graphs before it stale)
        self._page_sizes = [self.manager.group(g)[0] for g in range(self.manager.num_groups)]

    # ------------------------------------------------------------------------------
    def _staging(self, count: int):
        if self._staging_host is None or self._staging_host.numel() < count:
            size = max(count, 1 << 16)
            self._staging_host = torch.empty(size, dtype=torch.int32, pin_memory=True)
            self._staging_dev = torch.empty(size, dtype=torch.int32, device=self.device)
        return self._staging_host, self._staging_dev

    def validate(self, step: StepInput) -> None:
        tokens = step.tokens
        total = int(sum(step.counts))
        if total != tokens.shape[0] or total == 0:
            raise InvalidArgumentError("a step needs at least one token and counts that add up to its tokens")
        if len(step.requests) != len(step.counts) or len(step.pos0) != len(step.counts):
            raise InvalidArgumentError("requests, counts and first positions must have one item per entry")
        if min(step.counts) < 1:
            raise InvalidArgumentError("every entry of a step needs at least one token")
        vocab = self.model.spec.vocab_size
        if int(tokens.min()) < 0 or int(tokens.max()) >= vocab:
            raise InvalidArgumentError(f"token id outside the vocabulary of {vocab}")
        for request, count, first in zip(step.requests, step.counts, step.pos0):
            if first < 0 or first + count > self.max_model_len:
                raise InvalidArgumentError(
                    f"request {request}: positions {first}..{first + count - 1} exceed the limit of "
                    f"{self.max_model_len}")
        if step.logit_rows.size and (int(step.logit_rows.min()) < 0 or int(step.logit_rows.max()) >= total):
            raise InvalidArgumentError("a wanted row lies outside the step's tokens")

    def _host_arrays(self, step: StepInput, widths=None):
        """The step's description as host arrays, checked: per token (positions, entry), per
        entry (starts, first position, state slot, fresh), wanted rows, and per group the block
        tables, as wide as `widths` says or as the longest request needs."""
        self.validate(step)
        counts = np.asarray(step.counts, dtype=np.int32)
        pos0 = np.asarray(step.pos0, dtype=np.int32)
        entries = counts.shape[0]
        total = int(counts.sum())
        starts = np.zeros(entries + 1, dtype=np.int32)
        np.cumsum(counts, out=starts[1:])
        token_entry = np.repeat(np.arange(entries, dtype=np.int32), counts)
        positions = np.arange(total, dtype=np.int32) - np.repeat(starts[:-1] - pos0, counts)
        rows = np.asarray(step.logit_rows, dtype=np.int32)
        max_len = int((pos0 + counts).max())
        tables = []
        for g in range(self.manager.num_groups):
            page_size = self._page_sizes[g]
            width = widths[g] if widths is not None else _round_up_pow2((max_len + page_size - 1) // page_size)
            table = self.manager.tables(list(step.requests), g, width)
            # Every position of the step must have its page.
            last_page = (pos0 + counts - 1) // page_size
            if (table[np.arange(entries), last_page] < 0).any():
                raise InvalidArgumentError("a request of the step has no page reserved for its last position")
            tables.append(table)
        slots = np.asarray([self.manager.state_slot(r) for r in step.requests], dtype=np.int32)
        fresh = np.asarray(step.fresh, dtype=np.int32)
        return counts, pos0, starts, token_entry, positions, rows, tables, slots, fresh, max_len

    def build_context(self, step: StepInput, dtype: torch.dtype) -> StepContext:
        counts, pos0, starts, token_entry, positions, rows, tables, slots, fresh, max_len = self._host_arrays(step)
        entries, total = counts.shape[0], int(starts[-1])
        pieces = [step.tokens.astype(np.int32, copy=False), positions, token_entry, starts, pos0, slots, fresh, rows]
        pieces += [t.reshape(-1) for t in tables]
        sizes = [p.shape[0] for p in pieces]
        host, dev = self._staging(sum(sizes))
        if self._copy_pending:
            self._copy_done.synchronize()
        view = host.numpy()
        offsets, cursor = [], 0
        for piece, size in zip(pieces, sizes):
            view[cursor:cursor + size] = piece
            offsets.append(cursor)
            cursor += size
        dev[:cursor].copy_(host[:cursor], non_blocking=True)
        self._copy_done.record()
        self._copy_pending = True

        def part(index):
            return dev[offsets[index]:offsets[index] + sizes[index]]

        block_tables = [part(8 + g).view(entries, tables[g].shape[1]) for g in range(len(tables))]
        return StepContext(
            num_tokens=total, num_entries=entries, tokens=part(0), positions=part(1), token_entry=part(2),
            entry_starts=part(3), entry_pos0=part(4), state_slots=part(5), fresh=part(6),
            block_tables=block_tables, logit_rows=part(7) if rows.size else None, num_logit_rows=int(rows.size),
            host_counts=[int(c) for c in counts], host_pos0=[int(p) for p in pos0],
            max_count=int(counts.max()), max_kv_len=max_len, all_single=bool((counts == 1).all()),
            any_single=bool((counts == 1).any()), dtype=self.model.dtype, workspace=self.workspace,
            logits_all_rows=bool(rows.size == total and np.array_equal(rows, np.arange(total))))

    def forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """The model's forward pass for a prepared step."""
        return self.model.forward(ctx, self.pools.views)

    def run(self, step: StepInput) -> Optional[torch.Tensor]:
        """Run one step.  A step in which every entry brings one token and wants its logits
        (a decode step) is replayed from a captured CUDA graph of its size class; every other
        step is launched kernel by kernel."""
        self.steps_run += 1
        entries = len(step.counts)
        if self._graph_safe is None:
            self._graph_safe = bool(self.model.graph_safe)
        if (self.decode_graphs and self._graph_safe and 0 < entries <= self.max_graph_entries
                and len(step.tokens) == entries and len(step.logit_rows) == entries):
            logits = self._run_graph(step)
            if logits is not None:
                self.graph_replays += 1
                return logits
        if self.step_graphs and self._graph_safe and entries < self.max_graph_entries:
            graph = self._step_graph_for(step)
            if graph is not None:
                self.graph_replays += 1
                return graph.run(step)
        self.eager_steps += 1
        ctx = self.build_context(step, self.model.dtype)
        return self.forward(ctx)

    def _step_graph_for(self, step: StepInput):
        """The captured graph of the step's size class (made at the first step of the class), or
        None where the step is larger than any class."""
        total = len(step.tokens)
        bucket = _token_bucket(total)
        if bucket is None:
            return None
        entries = len(step.counts) + (1 if total < bucket else 0)   # padding tokens form an entry of their own
        entry_bucket = _round_up_pow2(entries, 2)
        rows = len(step.logit_rows)
        row_bucket = min(_round_up_pow2(rows, 1), bucket) if rows else 0
        longest = int(max(first + count for first, count in zip(step.pos0, step.counts)))
        widths = tuple(_round_up_pow2(max(-(-longest // page_size), -(-bucket // page_size)))
                       for page_size in self._page_sizes)
        # whether the split-key attention runs beside the flash kernel is part of the class: some
        # entry (the padding entry included) brings exactly one token
        any_single = 1 in step.counts or bucket - total == 1
        key = (bucket, entry_bucket, row_bucket, widths, any_single)
        graph = self._step_graphs.get(key)
        if graph is not None and graph.stale():
            graph = None
        if graph is None:
            if len(self._step_graphs) >= self.max_kept_graphs:
                self._step_graphs.pop(next(iter(self._step_graphs)))
            graph = self._step_graphs[key] = _StepGraph(self, bucket, entry_bucket, row_bucket, widths, any_single)
        return graph

    # ------------------------------------------------------------------------------
    # decode steps through CUDA graphs
    # ------------------------------------------------------------------------------
    def _run_graph(self, step: StepInput) -> Optional[torch.Tensor]:
        """The step through the graph of its size class, or None when it turns out not to be
        a plain decode step (the native routine that fills the graph's inputs checks the step)."""
        entries = len(step.counts)
        bucket = _round_up_pow2(entries, 1)
        last = int(max(step.pos0))
        widths = []
        for g, page_size in enumerate(self._page_sizes):
            widths.append(_width_bucket((last + page_size) // page_size))
        key = (bucket, tuple(widths))
        graph = self._graphs.get(key)
        if graph is not None and graph.stale():
            graph = None
        if graph is None:
            graph = _DecodeGraph(self, bucket, widths)
            if graph.fill(step) < 0:
                return None
            self._graphs.pop(key, None)
            if len(self._graphs) >= self.max_kept_graphs:   # the oldest goes (widths come in eighths of an octave)
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = graph
            graph.capture()
        elif graph.fill(step) < 0:
            return None
        return graph.replay(entries)


    def run_ahead(self, requests: Sequence[int], pos0: np.ndarray, token_source: torch.Tensor) -> Optional[torch.Tensor]:
        """Launch the decode step of `requests` at positions `pos0` whose input tokens are the
        first len(requests) of `token_source` (device, int32: what the step before draws), or
        return None when no captured graph serves it yet.  The pages of the positions must be
        reserved.  Nothing waits: the step before may still be running."""
        entries = len(requests)
        if not (self.decode_graphs and self._graph_safe and 0 < entries <= self.max_graph_entries):
            return None
        bucket = _round_up_pow2(entries, 1)
        last = int(pos0.max())
        widths = tuple(_width_bucket((last + page_size) // page_size) for page_size in self._page_sizes)
        graph = self._graphs.get((bucket, widths))
        if graph is None or graph.stale():
            return None
        self.steps_run += 1
        graph.fill_ahead(requests, pos0, token_source)
        return graph.replay(entries)


class _DecodeGraph:
    """One captured decode step for `bucket` entries and block tables of the given widths.
    Steps with fewer entries are padded with copies of their first entry, which computes and
    stores the same values twice."""

    def __init__(self, runner: ModelRunner, bucket: int, widths):
        self._runner = weakref.ref(runner)   # the runner owns its graphs, not the other way round
        self.bucket = bucket
        self.widths = [int(w) for w in widths]
        b = bucket
        self.sizes = [b, b, b, b + 1, b, b, b, b] + [b * w for w in self.widths]
        self.offsets = np.concatenate([[0], np.cumsum(self.sizes)]).astype(np.int64)
        total = int(self.offsets[-1])
        self.host = torch.empty(total, dtype=torch.int32, pin_memory=True)
        self.dev = torch.empty(total, dtype=torch.int32, device=runner.device)
        # the parts that are the same in every step: each token is its own entry and wants its logits
        view, o = self.host.numpy(), self.offsets
        view[int(o[2]):int(o[3])] = np.arange(b, dtype=np.int32)
        view[int(o[3]):int(o[4])] = np.arange(b + 1, dtype=np.int32)
        view[int(o[7]):int(o[8])] = np.arange(b, dtype=np.int32)
        self.host_address = self.host.data_ptr()
        self.vocab = int(runner.model.spec.vocab_size)
        self.copy_done = torch.cuda.Event()
        self.pending = False
        self.graph = None
        self.logits = None
        self.generations = None
        self._plain = {}  # per entry count: the constant arrays of a step launched ahead

    @property
    def runner(self) -> "ModelRunner":
        return self._runner()

    def stale(self) -> bool:
        from ..kernels import ops

        return self.generations != (self.runner.workspace.generation, ops.buffer_generation)

    def _part(self, index):
        return self.dev[int(self.offsets[index]):int(self.offsets[index + 1])]

    def fill(self, step: StepInput) -> int:
        """The step's inputs into the staging buffer and on their way to the device; -1 (and
        nothing copied) when the step is not a plain decode step."""
        runner = self.runner
        if self.pending:
            self.copy_done.synchronize()
            self.pending = False
        n = runner.manager.fill_decode(step.requests, step.tokens, step.counts, step.pos0, step.fresh, step.logit_rows,
                                       self.host_address, self.bucket, self.widths, self.vocab, runner.max_model_len)
        if n < 0:
            return n
        self.dev.copy_(self.host, non_blocking=True)
        self.copy_done.record()
        self.pending = True
        return n

    def fill_ahead(self, requests: Sequence[int], pos0: np.ndarray, token_source: torch.Tensor) -> None:
        """As fill(), for a step whose tokens are still being drawn on the device: everything
        but the tokens comes from the host, then the tokens are fed from `token_source`."""
        from ..kernels import ops

        runner = self.runner
        n = len(requests)
        if self.pending:
            self.copy_done.synchronize()
            self.pending = False
        plain = self._plain.get(n)
        if plain is None:
            plain = self._plain[n] = (np.zeros(n, dtype=np.int32), np.ones(n, dtype=np.int32), np.arange(n, dtype=np.int32))
        zeros, ones, rows = plain
        runner.manager.fill_decode(requests, zeros, ones, pos0, zeros, rows, self.host_address, self.bucket, self.widths,
                                   self.vocab, runner.max_model_len)
        self.dev.copy_(self.host, non_blocking=True)
        self.copy_done.record()
        self.pending = True
        ops.feed_tokens(token_source, self._part(0), n)

    def _context(self) -> StepContext:
        runner, b = self.runner, self.bucket
        tables = [self._part(8 + g).view(b, w) for g, w in enumerate(self.widths)]
        return StepContext(
            num_tokens=b, num_entries=b, tokens=self._part(0), positions=self._part(1),
            token_entry=self._part(2), entry_starts=self._part(3), entry_pos0=self._part(4),
            state_slots=self._part(5), fresh=self._part(6), block_tables=tables, logit_rows=self._part(7),
            num_logit_rows=b, host_counts=[1] * b, host_pos0=[0] * b, max_count=1,
            max_kv_len=min(w * runner.manager.group(g)[0] for g, w in enumerate(self.widths)) if self.widths else 0,
            all_single=True, any_single=True, dtype=runner.model.dtype, workspace=runner.workspace,
            logits_all_rows=True, extras={"graph": True})

    def capture(self) -> None:
        """Capture the step whose inputs `fill` has just put on their way."""
        from ..kernels import ops

        runner = self.runner
        ctx = self._context()
        # Once outside a graph: buffers get their final sizes, kernels are loaded.  The step's
        # own keys and values are written here and again, identically, by the replay.
        runner.forward(ctx)
        torch.cuda.current_stream().synchronize()
        before = ops.launches
        self.graph, self.logits = _capture(lambda: runner.forward(ctx))
        self.kernels = ops.launches - before
        ops.launches = before
        self.generations = (runner.workspace.generation, ops.buffer_generation)
        runner.graph_captures += 1

    def replay(self, entries: int) -> torch.Tensor:
        from ..kernels import ops

        self.graph.replay()
        ops.launches += self.kernels
        return self.logits if entries == self.bucket else self.logits[:entries]


class _StepGraph:
    """One captured step of any make-up: `tokens` tokens in `entries` entries, `rows` wanted
    rows, block tables of the given widths.  A step of the class that is smaller is padded:
    the spare tokens form one more entry that starts at position 0 and whose block table names
    only the group's scratch page (a page no request ever holds), so what they compute lands
    nowhere; entries beyond that bring no tokens; spare wanted rows repeat the first."""

    def __init__(self, runner: ModelRunner, tokens: int, entries: int, rows: int, widths, any_single: bool):
        self._runner = weakref.ref(runner)   # the runner owns its graphs, not the other way round
        self.tokens, self.entries, self.rows = int(tokens), int(entries), int(rows)
        self.any_single = bool(any_single)
        self.widths = [int(w) for w in widths]
        t, e = self.tokens, self.entries
        self.sizes = [t, t, t, e + 1, e, e, e, max(self.rows, 1)] + [e * w for w in self.widths]
        self.offsets = np.concatenate([[0], np.cumsum(self.sizes)]).astype(np.int64)
        total = int(self.offsets[-1])
        self.host = torch.empty(total, dtype=torch.int32, pin_memory=True)
        self.dev = torch.empty(total, dtype=torch.int32, device=runner.device)
        self.copy_done = torch.cuda.Event()
        self.pending = False
        self.graph = None
        self.logits = None
        self.generations = None
        self.kernels = 0

    @property
    def runner(self) -> "ModelRunner":
        return self._runner()

    def stale(self) -> bool:
        from ..kernels import ops

        return self.graph is not None and self.generations != (self.runner.workspace.generation, ops.buffer_generation)

    def _part(self, index):
        return self.dev[int(self.offsets[index]):int(self.offsets[index + 1])]

    def _host_part(self, index):
        return self.host.numpy()[int(self.offsets[index]):int(self.offsets[index + 1])]

    def fill(self, step: StepInput) -> int:
        """The step's inputs, padded to the class, into the staging buffer and on their way to
        the device; returns the number of wanted rows."""
        runner = self.runner
        counts, pos0, starts, token_entry, positions, rows, tables, slots, fresh, _ = runner._host_arrays(
            step, self.widths)
        own_tokens, own_entries = int(starts[-1]), counts.shape[0]
        if self.pending:
            self.copy_done.synchronize()
            self.pending = False
        t, e = self.tokens, self.entries
        spare = t - own_tokens
        part = self._host_part
        tokens_h, positions_h, entry_h = part(0), part(1), part(2)
        tokens_h[:own_tokens] = step.tokens
        positions_h[:own_tokens] = positions
        entry_h[:own_tokens] = token_entry
        if spare:
            tokens_h[own_tokens:] = 0
            positions_h[own_tokens:] = np.arange(spare, dtype=np.int32)
            entry_h[own_tokens:] = own_entries
        starts_h = part(3)
        starts_h[:own_entries + 1] = starts
        starts_h[own_entries + 1:] = t          # the padding entry ends the step; the rest bring nothing
        for index, values in ((4, pos0), (5, slots), (6, fresh)):
            target = part(index)
            target[:own_entries] = values
            target[own_entries:] = 0
        rows_h = part(7)
        if self.rows:
            rows_h[:rows.size] = rows
            rows_h[rows.size:] = rows[0]
        for g, table in enumerate(tables):
            target = part(8 + g).reshape(e, self.widths[g])
            target[:own_entries] = table
            target[own_entries:] = runner.pools.scratch_pages[g]
        self.dev.copy_(self.host, non_blocking=True)
        self.copy_done.record()
        self.pending = True
        return int(rows.size)

    def _context(self) -> StepContext:
        runner, t, e = self.runner, self.tokens, self.entries
        tables = [self._part(8 + g).view(e, w) for g, w in enumerate(self.widths)]
        return StepContext(
            num_tokens=t, num_entries=e, tokens=self._part(0), positions=self._part(1), token_entry=self._part(2),
            entry_starts=self._part(3), entry_pos0=self._part(4), state_slots=self._part(5), fresh=self._part(6),
            block_tables=tables, logit_rows=self._part(7) if self.rows else None, num_logit_rows=self.rows,
            host_counts=[], host_pos0=[], max_count=t,
            max_kv_len=min(w * runner._page_sizes[g] for g, w in enumerate(self.widths)) if self.widths else 0,
            all_single=False, any_single=self.any_single, dtype=runner.model.dtype, workspace=runner.workspace,
            logits_all_rows=False, extras={"graph": True})

    def run(self, step: StepInput) -> Optional[torch.Tensor]:
        from ..kernels import ops

        rows = self.fill(step)
        runner = self.runner
        if self.graph is None or self.stale():
            ctx = self._context()
            # Once outside a graph: buffers get their final sizes, kernels are loaded.  The keys
            # and values of the step are written here and again, identically, by the replay.
            runner.forward(ctx)
            torch.cuda.current_stream().synchronize()
            before = ops.launches
            self.graph, self.logits = _capture(lambda: runner.forward(ctx))
            self.kernels = ops.launches - before
            ops.launches = before
            self.generations = (runner.workspace.generation, ops.buffer_generation)
            runner.graph_captures += 1
        self.graph.replay()
        ops.launches += self.kernels
        if self.logits is None:
            return None
        return self.logits if rows == self.rows else self.logits[:rows]
