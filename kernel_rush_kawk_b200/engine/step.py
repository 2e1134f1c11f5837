"""The step function: one batch of sequences, their next tokens, from the cache.

``Stepper.step(entries)`` takes, for each live sequence, the tokens it brings
now (a whole prompt, a piece of one, or a single token) and the places among
them whose logits are wanted. It runs exactly those tokens as one packed batch
(no padding rows exist), each sequence continuing at its own cached length, and
returns float32 logits ``[wanted, vocab]`` in the order of the entries and of
their ``want`` lists.

The reference has two step functions, ``Plan.prefill`` (equal lengths, from
position 0, last-position logits) and ``Plan.decode`` (one token each), and a
third for R rows at ``pos[b]`` (``VerifyPlan.verify``): engine/model.py:284-318,
354-365 of willzeng274/kernel-rush-kawk. Here one function covers all three.

A step that is too large for one pass (more rows than ``max_step_rows``, or more
tokens of one sequence than a window group's ring allows) is cut into passes;
since a pass may start anywhere in a sequence, the cut changes nothing but
rounding. A step in which every sequence brings one token runs from a captured
CUDA graph when the model's parts allow it. The tensor such a step returns is the
captured step's own output buffer: the next single-token step of the same batch
size overwrites it, so a caller that keeps logits across steps copies them.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.store import SequenceCache


@dataclass
class StepEntry:
    slot: int
    tokens: list
    want: list = field(default_factory=list)


class BatchMeta:
    """Device-side description of one pass. All arrays are int32 views of one
    buffer that a single host-to-device copy fills.

    tokens[r], row_seq[r] (which sequence of the pass row r belongs to), row_pos[r]
    (its position in the sequence); seq_slot[s], seq_start[s] (cached length before
    the pass), seq_qlen[s], cu_q[s] (first row of sequence s; cu_q[n_seqs] = rows);
    want[w] (rows whose logits are asked for)."""

    FIELDS = ("tokens", "row_seq", "row_pos", "seq_slot", "seq_start", "seq_qlen", "cu_q", "want")

    def __init__(self, n_rows: int, n_seqs: int, n_want: int, device):
        self.n_rows, self.n_seqs, self.n_want = n_rows, n_seqs, n_want
        sizes = (n_rows, n_rows, n_rows, n_seqs, n_seqs, n_seqs, n_seqs + 1, n_want)
        # every array starts on a 16-byte boundary
        offsets, total = [], 0
        for s in sizes:
            offsets.append(total)
            total += -(-s // 4) * 4
        self.total = max(total, 4)
        self.offsets, self.sizes = offsets, sizes
        self.buffer = torch.zeros(self.total, dtype=torch.int32, device=device)
        self.host = torch.zeros(self.total, dtype=torch.int32, pin_memory=self.buffer.is_cuda)
        self.host_np = self.host.numpy()
        self._host_views = {name: self.host_np[off:off + size] for name, off, size in zip(self.FIELDS, offsets, sizes)}
        self._single_token_shape = False  # the pinned buffer holds the constant arrays of a one-token-each pass
        for name, off, size in zip(self.FIELDS, offsets, sizes):
            setattr(self, name, self.buffer[off:off + size])
        self.copied = torch.cuda.Event() if self.buffer.is_cuda else None
        # host-side facts, valid for the pass being built
        self.max_q_len = 1
        self.max_kv_len = 1
        self.is_decode = False
        self.want_all = False  # the wanted rows are all rows, in order
        self.slots: list[int] = []
        self.starts: list[int] = []
        self.q_lens: list[int] = []

    def host_field(self, name: str) -> np.ndarray:
        return self._host_views[name]

    def fill(self, slots, starts, token_lists, want_rows) -> None:
        """Write one pass into the pinned buffer and start its copy to the device."""
        if self.copied is not None:
            self.copied.synchronize()  # the previous copy out of this pinned buffer is over
        q_lens = [len(t) for t in token_lists]
        view = self._host_views
        if self.n_rows == self.n_seqs:
            # one token each (this buffer's shape admits nothing else): row r is sequence r, and only the
            # tokens, positions and slots change from step to step
            if not self._single_token_shape:
                n = self.n_seqs
                view["row_seq"][:] = np.arange(n, dtype=np.int32)
                view["seq_qlen"][:] = 1
                view["cu_q"][:] = np.arange(n + 1, dtype=np.int32)
                self._single_token_shape = True
            view["tokens"][:] = [t[0] for t in token_lists]
            view["row_pos"][:] = starts
        else:
            cu = np.zeros(len(q_lens) + 1, dtype=np.int32)
            np.cumsum(q_lens, out=cu[1:])
            view["tokens"][:] = np.concatenate([np.asarray(t, dtype=np.int32) for t in token_lists])
            view["row_seq"][:] = np.repeat(np.arange(len(q_lens), dtype=np.int32), q_lens)
            view["row_pos"][:] = np.concatenate([np.arange(s, s + n, dtype=np.int32) for s, n in zip(starts, q_lens)])
            view["seq_qlen"][:] = q_lens
            view["cu_q"][:] = cu
        view["seq_slot"][:] = slots
        view["seq_start"][:] = starts
        view["want"][:] = want_rows
        self.upload()
        self.max_q_len = max(q_lens)
        self.max_kv_len = max(s + n for s, n in zip(starts, q_lens))
        self.is_decode = self.max_q_len == 1
        self.want_all = list(want_rows) == list(range(self.n_rows))
        self.slots, self.starts, self.q_lens = list(slots), list(starts), q_lens

    uploaded = 0  # bytes of batch descriptions copied to the device so far, all instances together

    def upload(self) -> None:
        BatchMeta.uploaded += self.total * 4
        self.buffer.copy_(self.host, non_blocking=True)
        if self.copied is not None:
            self.copied.record()

    @property
    def bytes(self) -> int:
        return self.total * 4


class StepContext:
    def __init__(self, ops, batch: BatchMeta, cache: SequenceCache):
        self.ops = ops
        self.batch = batch
        self.cache = cache

    def cache_view(self, run: int):
        return self.cache.view(run)


class _DecodeGraph:
    def __init__(self, graph, meta: BatchMeta, logits: torch.Tensor):
        self.graph, self.meta, self.logits = graph, meta, logits


class DecodeRun:
    """Single-token steps of a fixed set of sequences, queued ahead of the host.

    ``launch`` queues one step: page reservation, the captured step, the selection kernel, which
    also writes the chosen tokens and the positions of the next step into the step's batch
    description on the device, and a copy of the tokens (and of the kernels' error word) into a
    ring of pinned rows, fenced by an event. ``collect`` waits for the oldest queued step and
    returns its tokens. At most ``depth`` steps are queued. The reference's ``GraphPlan.run``
    works the same way (engine/engine.py:81-83,458-469 of willzeng274/kernel-rush-kawk)."""

    def __init__(self, stepper, slots, tokens, sampling, requests, first_step: int, depth: int):
        self.stepper, self.slots, self.sampling = stepper, slots, sampling
        self.depth = max(1, depth)
        n = self.n = len(slots)
        cache, dev = stepper.cache, stepper.device
        starts = [cache.length[s] for s in slots]
        for s, start in zip(slots, starts):
            cache.reserve(s, start + 1)
        cache.sync()
        token_lists = [[t] for t in tokens]
        self.graph = stepper._graphs.get(n) or stepper._capture(n, slots, starts, token_lists)
        self.graph.meta.fill(slots, starts, token_lists, list(range(n)))
        stepper.h2d_bytes = self.graph.meta.bytes
        ring = stepper._run_rings.get((n, self.depth))
        if ring is None:
            if len(stepper._run_rings) > 64:
                stepper._run_rings.clear()
            ring = stepper._run_rings[(n, self.depth)] = (
                torch.empty((self.depth, n), dtype=torch.int32, device=dev),
                torch.empty((self.depth, n + 1), dtype=torch.int32, pin_memory=True),
                [torch.cuda.Event() for _ in range(self.depth)])
        self.device_tokens, self.host_tokens, self.events = ring
        self.requests = torch.tensor(requests, dtype=torch.int32).to(dev)
        self.step = first_step
        self.launched = self.collected = 0

    @property
    def in_flight(self) -> int:
        return self.launched - self.collected

    def launch(self) -> None:
        if self.in_flight >= self.depth:
            raise RuntimeError(f"{self.depth} steps are queued already; collect one first")
        st, cache, n = self.stepper, self.stepper.cache, self.n
        if self.launched:  # the first step's pages were reserved with the batch description
            for s in self.slots:
                cache.reserve(s, cache.length[s] + 1)
            cache.sync()
        k = self.launched % self.depth
        self.graph.graph.replay()
        st.ops.select_tokens(self.graph.logits, float(self.sampling.temperature), int(self.sampling.seed), self.requests,
                             self.step + self.launched, feed=self.graph.meta, out=self.device_tokens[k])
        self.host_tokens[k, :n].copy_(self.device_tokens[k], non_blocking=True)
        self.host_tokens[k, n:].copy_(st.ops.error, non_blocking=True)
        self.events[k].record()
        for s in self.slots:
            cache.advance(s, 1)
        st.passes += 1
        self.launched += 1

    def collect(self) -> list:
        if self.in_flight == 0:
            raise RuntimeError("no step is queued")
        k = self.collected % self.depth
        self.events[k].synchronize()
        row = self.host_tokens[k].tolist()
        self.collected += 1
        if row[-1]:
            self.stepper.ops.check()  # raises with the flag's meaning and clears the word
        return row[:-1]


class Stepper:
    def __init__(self, model, cache: SequenceCache, ops, max_step_rows: int = 16384, use_graphs: bool = True):
        self.model = model
        self.cache = cache
        self.ops = ops
        self.max_step_rows = int(max_step_rows)
        self.device = cache.device
        self.use_graphs = bool(use_graphs) and self.device.type == "cuda" and model.graph_safe
        self.vocab = model.plan.vocab_size
        self._graphs: dict[int, _DecodeGraph] = {}
        self._metas: dict[tuple, list] = {}
        self.graph_launches: dict[int, int] = {}  # kernels of this package inside each captured step
        self.h2d_bytes = 0  # bytes of the last step's host-to-device copies
        self.passes = 0
        self._run_rings: dict = {}  # (sequences, depth) -> token ring of a DecodeRun, reused by later runs

    def h2d_total(self) -> int:
        """Bytes copied from the host to the device for steps so far: batch descriptions and page-table rows."""
        return BatchMeta.uploaded + self.cache.h2d_bytes

    # ------------------------------------------------------------------
    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        if not entries:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=self.device)
        self._validate(entries)
        per_seq = min(self.max_step_rows, self.cache.per_sequence_step_limit() or self.max_step_rows)
        done = [0] * len(entries)
        pieces, order = [], []
        self.h2d_bytes = 0
        many = any(len(e.tokens) > 1 for e in entries)
        while True:
            rows_left = self.max_step_rows
            chosen = []
            for i, e in enumerate(entries):
                left = len(e.tokens) - done[i]
                if left <= 0 or rows_left <= 0:
                    continue
                n = min(left, per_seq, rows_left)
                chosen.append((i, done[i], n))
                rows_left -= n
            if not chosen:
                break
            logits, which = self._pass(entries, chosen)
            if which:
                pieces.append(logits)
                order.extend(which)
            for i, _, n in chosen:
                done[i] += n
        if many and hasattr(self.ops, "check"):
            self.ops.check()  # a multi-token step ends with a look at the kernels' error word
        wanted = [(i, w) for i, e in enumerate(entries) for w in e.want]
        if not wanted:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=self.device)
        out = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=0)
        if order != wanted:
            place = {key: r for r, key in enumerate(order)}
            idx = torch.as_tensor([place[key] for key in wanted], dtype=torch.int64, device=self.device)
            out = out.index_select(0, idx)
        return out

    # ------------------------------------------------------------------
    def _validate(self, entries) -> None:
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise ValueError(f"cache slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not self.cache.slots.is_held(e.slot):
                raise ValueError(f"cache slot {e.slot} is not held")
            if len(e.tokens) == 0:
                raise ValueError("a step entry brings no tokens")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= self.vocab:
                raise ValueError(f"token id {lo if lo < 0 else hi} lies outside the vocabulary of {self.vocab}")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"wanted place {w} lies outside the {len(e.tokens)} tokens of its entry")

    def _meta(self, n_rows: int, n_seqs: int, n_want: int) -> BatchMeta:
        """Two buffers per shape, used in turn, so that a pass can be prepared while
        the previous one of the same shape still runs."""
        key = (n_rows, n_seqs, n_want)
        ring = self._metas.get(key)
        if ring is None:
            if len(self._metas) > 64:
                self._metas.clear()
            ring = self._metas[key] = [0, [BatchMeta(n_rows, n_seqs, n_want, self.device) for _ in range(2)]]
        ring[0] ^= 1
        return ring[1][ring[0]]

    def _pass(self, entries, chosen):
        cache = self.cache
        slots, starts, token_lists, want_rows, which = [], [], [], [], []
        row = 0
        for i, first, n in chosen:
            e = entries[i]
            start = cache.length[e.slot]
            cache.reserve(e.slot, start + n)
            slots.append(e.slot)
            starts.append(start)
            token_lists.append(e.tokens[first:first + n])
            for w in e.want:
                if first <= w < first + n:
                    want_rows.append(row + w - first)
                    which.append((i, w))
            row += n
        cache.sync()
        n_rows, n_seqs = row, len(chosen)
        decode = all(n == 1 for _, _, n in chosen)
        if decode and self.use_graphs:
            logits = self._replay(slots, starts, token_lists, want_rows, n_seqs)
        else:
            meta = self._meta(n_rows, n_seqs, len(want_rows))
            meta.fill(slots, starts, token_lists, want_rows)
            self.h2d_bytes += meta.bytes
            ctx = StepContext(self.ops, meta, cache)
            logits = self.model.forward(ctx, meta.want) if want_rows else self._forward_no_logits(ctx)
        for (i, _, n), slot in zip(chosen, slots):
            cache.advance(slot, n)
        self.passes += 1
        return logits, which

    def _forward_no_logits(self, ctx):
        """A pass whose logits nobody wants still has to fill the cache. The last row's
        logits are computed and dropped, which keeps one code path."""
        last = ctx.batch.row_seq[:0]  # empty int32 tensor on the device
        self.model.forward(ctx, last)
        return None

    # -- decode from a captured graph ------------------------------------------
    def _replay(self, slots, starts, token_lists, want_rows, n: int):
        g = self._graphs.get(n)
        if g is None:
            g = self._capture(n, slots, starts, token_lists)
        g.meta.fill(slots, starts, token_lists, list(range(n)))
        self.h2d_bytes += g.meta.bytes
        g.graph.replay()
        if len(want_rows) == n:
            return g.logits
        if not want_rows:
            return None
        idx = torch.as_tensor(want_rows, dtype=torch.int64, device=self.device)
        return g.logits.index_select(0, idx)

    def decode_on_device(self, slots, tokens, n_steps: int, temperature: float = 0.0, seed: int = 0,
                         requests=None, first_step: int = 0) -> torch.Tensor:
        """``n_steps`` single-token steps without a host round trip: the selection kernel
        writes each step's tokens into the next step's batch description. Returns the
        chosen tokens, int32 [n_steps, sequences], on the device. Pages for all steps
        are reserved before the first one."""
        n = len(slots)
        cache = self.cache
        starts = [cache.length[s] for s in slots]
        for s in slots:
            cache.reserve(s, cache.length[s] + n_steps)
        cache.sync()
        token_lists = [[int(t)] for t in tokens]
        if self.use_graphs:
            g = self._graphs.get(n) or self._capture(n, slots, starts, token_lists)
            meta = g.meta
        else:
            g, meta = None, self._meta(n, n, n)
        meta.fill(slots, starts, token_lists, list(range(n)))
        self.h2d_bytes = meta.bytes
        req = torch.tensor(list(requests) if requests is not None else list(range(n)), dtype=torch.int32).to(self.device)
        out = torch.empty((n_steps, n), dtype=torch.int32, device=self.device)
        ctx = StepContext(self.ops, meta, cache)
        for t in range(n_steps):
            if g is not None:
                g.graph.replay()
                logits = g.logits
            else:
                logits = self.model.forward(ctx, meta.want)
            self.ops.select_tokens(logits, temperature, seed, req, first_step + t, feed=meta, out=out[t])
        for s in slots:
            cache.advance(s, n_steps)
        self.passes += n_steps
        return out

    def open_decode_run(self, slots, tokens, sampling, requests, first_step: int, depth: int = 3):
        """A ``DecodeRun`` over these sequences, or None where single-token steps cannot be queued
        ahead of the host (no captured graph: graphs are off, or a part reads the step on the host)."""
        if not self.use_graphs or not slots:
            return None
        return DecodeRun(self, list(slots), [int(t) for t in tokens], sampling, list(requests), int(first_step), int(depth))

    def _capture(self, n: int, slots, starts, token_lists) -> _DecodeGraph:
        meta = BatchMeta(n, n, n, self.device)
        meta.fill(slots, starts, token_lists, list(range(n)))
        ctx = StepContext(self.ops, meta, self.cache)
        # Run once outside a capture: everything that allocates or initialises lazily
        # does so now. The pass writes this step's keys and values; the replay of the
        # captured step writes the same values to the same places again. Fixed-size
        # state is not like that (a second update is a different state), so the
        # sequences' state is put back as it was before the trial run.
        saved = self.cache.save_state(slots)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self.model.forward(ctx, meta.want)
        torch.cuda.current_stream(self.device).wait_stream(side)
        self.cache.restore_state(slots, saved)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        before = getattr(self.ops, "launches", 0)
        with torch.cuda.graph(graph):
            logits = self.model.forward(ctx, meta.want)
        self.graph_launches[n] = getattr(self.ops, "launches", 0) - before
        g = self._graphs[n] = _DecodeGraph(graph, meta, logits)
        return g
