"""The step function: run the tokens a step brings, as one packed batch, from the cache, and
return logits at the wanted places.

A step is a list of (slot, tokens) entries.  The sequences of a step start together (each
brings its whole prompt, lengths unequal) or go on by one token each; the function itself takes
any mix of lengths, so a long prompt can also be fed in pieces.  Rows are packed without
padding; each row carries (sequence, absolute position) and attends only to keys of its own
sequence at positions <= its own (internal/qwen3lm/evaluator.go:582-602 packs unequal sequences
the same way, with per-row start/position; gpu_darwin.go:1578-1593).  Everything is validated
before the cache is touched, so a refused step leaves every sequence as it was
(internal/qwen3lm/decode_batch.go:80-128).  Very large steps are cut into row chunks
(gpu_darwin.go:1471-1487 loops long prompts pass by pass); a chunk boundary changes no result
beyond rounding because later rows read earlier keys from the cache.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import Cache, CacheError
from .model import Model


class StepError(ValueError):
    pass


@dataclass
class StepBatch:
    """Device-side description of the rows of one (chunk of a) step."""
    rows: int
    nseq: int
    max_q_len: int
    max_kv_len: int
    ids: torch.Tensor          # [rows] int32 token ids
    row_pos: torch.Tensor      # [rows] absolute position of each row in its sequence
    row_seq: torch.Tensor      # [rows] index of the row's sequence within this batch
    seq_slot: torch.Tensor     # [nseq] cache slot
    seq_q_start: torch.Tensor  # [nseq] first packed row
    seq_q_len: torch.Tensor    # [nseq] rows in this batch
    seq_kv_len: torch.Tensor   # [nseq] keys visible to the sequence's last row (= its length after them)
    device: torch.device = None
    sm_count: int = 148
    # launch plans of the step's mixers, by the mixer's identity (``Mixer.plan``); a mixer that is
    # not listed is asked when it first runs
    plans: Dict[int, object] = field(default_factory=dict)
    _workspaces: Dict[object, torch.Tensor] = field(default_factory=dict)

    def plan_for(self, part):
        """The launch plan of ``part`` for this step (asked once per step and part)."""
        key = id(part)
        if key not in self.plans:
            self.plans[key] = part.plan(self.nseq, self.max_q_len, self.max_kv_len, self.sm_count)
        return self.plans[key]

    def workspace(self, key, numel: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """Scratch memory of this step: parts that ask with the same ``key`` share one buffer (they run
        one after the other on the stream), and a captured step keeps its buffers for its replays."""
        t = self._workspaces.get(key)
        if t is None or t.numel() < numel or t.dtype != dtype:
            t = self._workspaces[key] = torch.empty(numel, dtype=dtype, device=self.device)
        return t


class HostStager:
    """Pinned host buffers for the per-step upload of row metadata.  A small ring, each buffer
    guarded by an event recorded after its copy, so the host may run ahead of the device without
    overwriting a buffer whose copy has not happened yet."""

    def __init__(self, device, ring: int = 4):
        self.device = torch.device(device)
        self.ring = ring
        self.bufs: List[Optional[torch.Tensor]] = [None] * ring
        self.events: List[Optional[torch.cuda.Event]] = [None] * ring
        self.at = 0
        self.bytes_uploaded = 0

    def upload(self, n: int, fill) -> torch.Tensor:
        """A device int32 tensor of ``n`` elements whose contents ``fill(numpy_view)`` writes."""
        dev = torch.empty(n, dtype=torch.int32, device=self.device)
        self.upload_into(dev, fill)
        return dev

    def upload_into(self, dev: torch.Tensor, fill) -> None:
        """Fill the device int32 tensor ``dev`` with what ``fill(numpy_view)`` writes."""
        n = dev.numel()
        i = self.at
        self.at = (self.at + 1) % self.ring
        if self.events[i] is not None:
            self.events[i].synchronize()
        if self.bufs[i] is None or self.bufs[i].numel() < n:
            self.bufs[i] = torch.empty(max(1024, 2 * n), dtype=torch.int32).pin_memory()
        host = self.bufs[i][:n]
        fill(host.numpy())
        dev.copy_(host, non_blocking=True)
        if self.events[i] is None:
            self.events[i] = torch.cuda.Event()
        self.events[i].record()
        self.bytes_uploaded += 4 * n


class TokenFetch:
    """Tokens on their way from the device to the host: a pinned buffer and the event of its copy."""

    def __init__(self, host: torch.Tensor, event: torch.cuda.Event):
        self.host = host
        self.event = event

    def wait(self) -> List[int]:
        self.event.synchronize()
        return self.host.tolist()


def build_batch(pieces: Sequence[Tuple[int, Sequence[int], int]], device, sm_count: int = 148,
                want_rows: Optional[Sequence[int]] = None,
                stager: Optional[HostStager] = None) -> Tuple[StepBatch, Optional[torch.Tensor]]:
    """``pieces[i] = (slot, tokens, first_position)``: one device upload for all row metadata."""
    nseq = len(pieces)
    rows = sum(len(t) for _, t, _ in pieces)
    nw = 0 if want_rows is None else len(want_rows)
    total = 3 * rows + 4 * nseq + nw
    state = {}

    def fill(buf):
        state["max"] = _fill_batch(buf, pieces, rows, nseq, nw, want_rows)
    if stager is not None:
        dev = stager.upload(total, fill)
    else:
        host = np.empty(total, dtype=np.int32)
        fill(host)
        dev = torch.from_numpy(host).to(device)
    max_q, max_kv = state["max"]
    o = 3 * rows
    o2 = o + 4 * nseq
    batch = StepBatch(rows=rows, nseq=nseq, max_q_len=max_q, max_kv_len=max_kv, ids=dev[:rows],
                      row_pos=dev[rows:2 * rows], row_seq=dev[2 * rows:3 * rows],
                      seq_slot=dev[o:o + nseq], seq_q_start=dev[o + nseq:o + 2 * nseq],
                      seq_q_len=dev[o + 2 * nseq:o + 3 * nseq], seq_kv_len=dev[o + 3 * nseq:o2],
                      device=torch.device(device), sm_count=sm_count)
    return batch, (dev[o2:] if nw else None)


def _fill_batch(buf, pieces, rows, nseq, nw, want_rows):
    ids, row_pos, row_seq = buf[:rows], buf[rows:2 * rows], buf[2 * rows:3 * rows]
    o = 3 * rows
    seq_slot, q_start, q_len, kv_len = (buf[o + i * nseq:o + (i + 1) * nseq] for i in range(4))
    r = 0
    max_q = max_kv = 0
    for i, (slot, toks, first) in enumerate(pieces):
        n = len(toks)
        ids[r:r + n] = toks
        row_pos[r:r + n] = np.arange(first, first + n, dtype=np.int32)
        row_seq[r:r + n] = i
        seq_slot[i], q_start[i], q_len[i], kv_len[i] = slot, r, n, first + n
        max_q, max_kv = max(max_q, n), max(max_kv, first + n)
        r += n
    if nw:
        buf[o + 4 * nseq:] = want_rows
    return max_q, max_kv


class Engine:
    """A model, its cache and the step function over them."""

    def __init__(self, model: Model, max_tokens: int, max_slots: Optional[int] = None,
                 max_seq_tokens: Optional[int] = None, max_rows_per_pass: int = 16384, use_graphs: bool = True,
                 max_graph_batch: int = 128):
        self.model = model
        self.device = model.rt.device
        self.cache: Cache = model.new_cache(max_tokens, max_slots, max_seq_tokens)
        self.capacity = min(self.cache.max_pages_per_seq * 64, int(model.spec.max_positions))
        self.max_rows_per_pass = max_rows_per_pass
        self.vocab = model.spec.vocab
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.stager = HostStager(self.device)
        self.cache.attach(model.rt.ops, self.stager)
        self._fetch_bufs: List[Optional[torch.Tensor]] = [None] * 4
        self._fetch_at = 0
        self.passes = 0
        self.graphs = None
        if use_graphs and model.capturable:
            from .graphs import DecodeGraphs
            self.graphs = DecodeGraphs(self, max_graph_batch)

    # ---- slots ---------------------------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.alloc_slot()

    def end_sequence(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def truncate(self, slot: int, n: int) -> None:
        """Forget everything after the first ``n`` tokens of the sequence in ``slot``: the next step
        goes on from position ``n`` (internal/qwen3lm/evaluator.go:185-226 keeps a prefix of its
        key/value store the same way; a chat session that branches, or whose last reply was cut
        short, lives on it).  Refused for a model whose mixers keep fixed-size state, which has no
        positions to cut at: use ``checkpoint`` / ``restore``."""
        try:
            self.cache.truncate(slot, n)
        except CacheError as e:
            raise StepError(str(e)) from None

    def checkpoint(self, slot: int):
        """A mark of the sequence as it is (its length and a copy of its fixed-size state) for ``restore``."""
        try:
            return self.cache.snapshot(slot)
        except CacheError as e:
            raise StepError(str(e)) from None

    def restore(self, slot: int, mark) -> None:
        """Go back to a mark taken of this sequence earlier: works for every kind of mixer."""
        try:
            self.cache.restore(slot, mark)
        except CacheError as e:
            raise StepError(str(e)) from None

    def check_kernels(self) -> None:
        """Raise if a kernel recorded that it gave up waiting on a barrier (synchronises)."""
        ops = self.model.rt.ops
        code = ops.tc5_status()
        if code:
            raise RuntimeError(f"a tcgen05 kernel gave up waiting on a barrier (role {code}); results are not valid")
        if ops.is_checked_build():
            found = ops.checked_status()
            if found is not None:
                where, what, value, bound, count = found
                raise RuntimeError(f"a kernel ({where}) met {what}: {value} against a bound of {bound} ({count} in all); "
                                   f"the accesses were skipped, results are not valid")

    def room(self) -> int:
        """Free pages of 64 tokens."""
        return self.cache.pages.available()

    # ---- the step ------------------------------------------------------------------------
    def validate(self, entries: Sequence[Tuple[int, Sequence[int]]], want: Optional[Sequence[Sequence[int]]]):
        if not entries:
            raise StepError("a step without entries")
        if want is not None and len(want) != len(entries):
            raise StepError(f"{len(want)} want lists for {len(entries)} entries")
        seen = set()
        for i, (slot, toks) in enumerate(entries):
            if slot in seen:
                raise StepError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            try:
                have = self.cache.length(slot)
            except CacheError as e:
                raise StepError(str(e)) from None
            if len(toks) == 0:
                raise StepError(f"entry {i} (slot {slot}) brings no tokens")
            if have + len(toks) > self.capacity:
                raise StepError(f"entry {i} (slot {slot}): {have} + {len(toks)} tokens exceed the per-sequence "
                                f"capacity {self.capacity}")
            ids = np.asarray(toks)
            if ids.ndim != 1 or ids.dtype.kind not in "iu":
                raise StepError(f"entry {i} (slot {slot}): tokens must be a flat sequence of integers")
            if int(ids.min()) < 0 or int(ids.max()) >= self.vocab:
                t = int(ids[(ids < 0) | (ids >= self.vocab)][0])
                raise StepError(f"entry {i} (slot {slot}): token id {t} is outside [0, {self.vocab})")
            if want is not None:
                for w in want[i]:
                    if not 0 <= int(w) < len(toks):
                        raise StepError(f"entry {i} (slot {slot}): wanted place {w} is outside its {len(toks)} tokens")

    # ``step(..., borrow=True)`` may return the output buffer of a replayed graph (see ``step``)
    lends_logits = True

    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Optional[Sequence[Sequence[int]]] = None, borrow: bool = False) -> Optional[torch.Tensor]:
        """Run ``entries = [(slot, tokens), ...]``; return fp32 logits [sum(len(w) for w in want), vocab]
        in the order of the entries and of each want list.  ``want=None`` asks for the last place
        of every entry.

        The tensor returned is the caller's to keep.  With ``borrow`` it may instead be the output
        buffer of a replayed CUDA graph, which the next step of the same shape overwrites: for a
        caller that consumes the logits before it steps again (the generation loop), this saves a
        copy."""
        self.validate(entries, want)
        if want is None:
            want = [[len(toks) - 1] for _, toks in entries]
        grow = [(slot, self.cache.length(slot) + len(toks)) for slot, toks in entries]
        self.cache.reserve(grow)  # raises CacheFull without changing anything

        # packed row index of every wanted place, in output order
        starts, r = [], 0
        for _, toks in entries:
            starts.append(r)
            r += len(toks)
        total_rows = r
        want_rows = [starts[i] + int(w) for i in range(len(entries)) for w in want[i]]

        single = total_rows == len(entries)
        if (single and self.graphs is not None and total_rows <= self.graphs.max_batch
                and want_rows == list(range(total_rows))):
            logits = self._graph_pass(entries)
            if not borrow:
                logits = logits.clone()
        elif total_rows <= self.max_rows_per_pass:
            pieces = [(slot, list(toks), self.cache.length(slot)) for slot, toks in entries]
            logits = self._pass(pieces, want_rows)
        else:
            logits = self._chunked(entries, starts, want_rows)
        self.cache.commit(grow)
        return logits

    def step_from(self, slots: Sequence[int], source: torch.Tensor, positions: Sequence[int],
                  borrow: bool = False) -> torch.Tensor:
        """One token each: sequence ``slots[i]`` goes on by ``source[positions[i]]``, where ``source``
        is a device int32 tensor (what the sampler left for the step before).  The host need not
        have read the tokens, so this step can be enqueued while the last one still runs.  Returns
        fp32 logits [len(slots), vocab]; ``borrow`` as for ``step``."""
        if source.dtype != torch.int32 or source.dim() != 1 or source.device != self.device:
            raise StepError("step_from: the token source must be a 1-d int32 tensor on the engine's device")
        if len(slots) != len(positions) or not slots:
            raise StepError(f"step_from: {len(slots)} slots, {len(positions)} positions")
        for p in positions:
            if not 0 <= int(p) < source.numel():
                raise StepError(f"step_from: position {p} is outside the source of {source.numel()} tokens")
        # the positions stand where token ids would; validation of ids is the sampler's guarantee
        entries = [(slot, [0]) for slot in slots]
        self.validate(entries, None)
        entries = [(slot, [int(p)]) for slot, p in zip(slots, positions)]
        grow = [(slot, self.cache.length(slot) + 1) for slot in slots]
        self.cache.reserve(grow)
        n = len(entries)
        if self.graphs is not None and n <= self.graphs.max_batch:
            logits = self._graph_pass(entries, source)
            if not borrow:
                logits = logits.clone()
        elif n <= self.max_rows_per_pass:
            pieces = [(slot, toks, self.cache.length(slot)) for slot, toks in entries]
            logits = self._pass(pieces, list(range(n)), source)
        else:
            raise StepError(f"step_from: {n} sequences exceed one pass of {self.max_rows_per_pass} rows")
        self.cache.commit(grow)
        return logits

    def fetch_tokens(self, tokens: torch.Tensor) -> TokenFetch:
        """Start copying a device int32 tensor of tokens to pinned host memory; ``wait()`` on the
        result gives them as a list once the copy has happened."""
        n = tokens.numel()
        i = self._fetch_at
        self._fetch_at = (i + 1) % len(self._fetch_bufs)
        if self._fetch_bufs[i] is None or self._fetch_bufs[i].numel() < n:
            self._fetch_bufs[i] = torch.empty(max(256, 2 * n), dtype=torch.int32).pin_memory()
        host = self._fetch_bufs[i][:n]
        host.copy_(tokens, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return TokenFetch(host, ev)

    def _pass(self, pieces, want_rows: Sequence[int], source: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        batch, want_dev = build_batch(pieces, self.device, self.sm_count, want_rows if want_rows else None,
                                      self.stager)
        if source is not None:
            self.model.rt.ops.gather_tokens(batch.ids, source)
        self.passes += 1
        return self.model.forward(batch, self.cache, want_dev)

    def _graph_pass(self, entries, source: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token each, every row wanted: replay the captured step.  Steps are captured at a few
        batch sizes only (every size up to 8, then 12, 16, 24, ... 128): a batch between two of them
        is filled up with rows that read and write the cache's spare slot and whose logits nobody
        sees, so that a batch which shrinks one sequence at a time does not capture a graph at every
        size."""
        n = len(entries)
        firsts = [self.cache.length(slot) for slot, _ in entries]
        g = self.graphs.get(n, max(firsts) + 1)
        if g.logits is None:
            # the capture runs the step's kernels on the graph's own input buffer: fill it first
            self._fill_graph_meta(g, entries, firsts)
            if source is not None:
                self.model.rt.ops.gather_tokens(g.meta[:n], source)
            torch.cuda.synchronize()
            g.capture()
        self._fill_graph_meta(g, entries, firsts)
        if source is not None:
            self.model.rt.ops.gather_tokens(g.meta[:n], source)  # the ids section held positions
        self.passes += 1
        return g.replay()[:n]

    def _fill_graph_meta(self, g, entries, firsts) -> None:
        n, nb = len(entries), g.nseq
        spare = self.cache.spare_slot

        def fill(buf):
            for i, ((slot, toks), first) in enumerate(zip(entries, firsts)):
                buf[i] = toks[0]
                buf[nb + i] = first
                buf[3 * nb + i] = slot
                buf[6 * nb + i] = first + 1
            for i in range(n, nb):      # filler rows: token 0 at places of their own in the spare page
                buf[i] = 0
                buf[nb + i] = (i - n) % 64
                buf[3 * nb + i] = spare
                buf[6 * nb + i] = (i - n) % 64 + 1
            for i in range(nb):
                buf[2 * nb + i] = i
                buf[4 * nb + i] = i
                buf[5 * nb + i] = 1
                buf[7 * nb + i] = i
        self.stager.upload_into(g.meta, fill)

    def _chunked(self, entries, starts, want_rows) -> Optional[torch.Tensor]:
        """Cut the packed rows into passes of at most ``max_rows_per_pass`` rows."""
        order: Dict[int, List[int]] = {}
        for k, row in enumerate(want_rows):
            order.setdefault(row, []).append(k)
        n_want = len(want_rows)
        result = None
        if n_want:
            result = torch.empty((n_want, self.vocab), dtype=torch.float32, device=self.device)
        lo = 0
        total = starts[-1] + len(entries[-1][1])
        while lo < total:
            hi = min(total, lo + self.max_rows_per_pass)
            pieces = []
            for i, (slot, toks) in enumerate(entries):
                a, b = max(lo, starts[i]), min(hi, starts[i] + len(toks))
                if a < b:
                    pieces.append((slot, list(toks[a - starts[i]:b - starts[i]]), self.cache.length(slot) + a - starts[i]))
            local = sorted({row for row in want_rows if lo <= row < hi})
            logits = self._pass(pieces, [row - lo for row in local])
            ks = [k for row in local for k in order[row]]
            if ks:
                js = [j for j, row in enumerate(local) for _ in order[row]]
                result.index_copy_(0, torch.tensor(ks, dtype=torch.int64, device=self.device),
                                   logits.index_select(0, torch.tensor(js, dtype=torch.int64, device=self.device)))
            lo = hi
        return result
