"""The cache: a slot for each live sequence, paged keys and values for each run of a layer, and
per-sequence state of fixed size beside them.

Unit of storage.  Keys and values live in pages of 64 tokens.  A sequence holds
ceil(length / 64) pages; ``max_tokens`` (each sequence's count rounded up to 64) sizes the pool.
Within a page the layout is [kv_head][64][head_dim], so one head's 64 keys are one contiguous
block.  A block table [slot][logical page] -> physical page, mirrored on the device, is shared
by every group: page p of a sequence is physical page table[slot][p] in every plane.

Groups.  Runs of layers are grouped by what they need: (kv_heads, head_dim, window) for
key/value planes, (shape, dtype) for fixed-size state.  Each group has storage of its own; a run
is given the plane with its ordinal inside its group (the reference indexes KV planes the same
way, by a layer's place among layers of its kind: internal/qwen3lm/gpu_darwin.go:51-55, 270-277,
831, and keeps per-sequence state beside K/V: gpu_darwin.go:800-808).  A run that reads another
run's cache gets that run's plane, read-only.

Slots.  ``alloc_slot`` hands out a free slot with length 0 and zeroed state; ``free_slot``
returns its pages and the slot; both are reused.  A page is cleared, in every key/value plane,
when it is handed to a sequence: the attention kernels mask what lies beyond a sequence's length
but the tensor-core ones still multiply whole pages of values by probabilities of zero, and zero
times an Inf or NaN that an earlier sequence left behind would not be zero.  So what a sequence
can ever see in its pages is zeros or its own values (after a ``truncate``, its own old ones).
Every mutation is checked first, so a refused call leaves the cache as it was
(internal/qwen3lm/decode_batch.go:80-128 validates before mutating).

A step's new pages reach the device as one list of (slot, logical page, physical page) triples:
with kernels and an upload ring attached (``attach``, the engine does so) one pinned asynchronous
copy and two small kernels write the block table and clear the pages, in stream order and without
making the host wait; without them (tests on the CPU) torch indexing does the same.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import KVRequest, StateRequest

PAGE = 64


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    pass


def pages_for(tokens: int) -> int:
    return (tokens + PAGE - 1) // PAGE


class FreeList:
    """Integers 0..n-1, each either free or held; refuses to hand one out twice or take one back twice."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free = list(range(n - 1, -1, -1))  # pop() gives the lowest first
        self._held = [False] * n

    def available(self) -> int:
        return len(self._free)

    def held(self) -> int:
        return self.n - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def give(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheError(f"{self.what} {i} does not exist (there are {self.n})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is freed twice or was never handed out")
        self._held[i] = False
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def check(self) -> None:
        """No item lost or duplicated."""
        if len(set(self._free)) != len(self._free):
            raise CacheError(f"a {self.what} is on the free list twice")
        for i in self._free:
            if self._held[i]:
                raise CacheError(f"{self.what} {i} is both free and held")
        if sum(self._held) + len(self._free) != self.n:
            raise CacheError(f"a {self.what} was lost")


@dataclass
class KVView:
    """What a mixer run sees of its key/value plane."""
    k: torch.Tensor            # [n_pages, kv_heads, 64, head_dim]
    v: torch.Tensor
    block_table: torch.Tensor  # [max_slots, max_pages_per_seq] int32
    writable: bool
    window: int


@dataclass
class StateView:
    state: torch.Tensor        # [max_slots, *shape]
    writable: bool


@dataclass
class CacheMark:
    """What ``Cache.snapshot`` returns: a length and the state of that moment."""
    slot: int
    length: int
    state: Dict[object, torch.Tensor]


class Cache:
    def __init__(self, requests: Sequence[Tuple[object, Optional[int]]], max_tokens: int, device,
                 dtype: torch.dtype, max_slots: Optional[int] = None, max_seq_tokens: Optional[int] = None):
        """``requests[pos] = (KVRequest | StateRequest | None, cache_of)`` for each schedule position."""
        if max_tokens <= 0:
            raise CacheError(f"cache of {max_tokens} tokens")
        self.device = torch.device(device)
        self.dtype = dtype
        self.n_pages = pages_for(max_tokens)
        self.max_pages_per_seq = self.n_pages if max_seq_tokens is None else min(self.n_pages, pages_for(max_seq_tokens))
        if max_slots is None:
            max_slots = min(self.n_pages, 1024)
            while max_slots > 1 and max_slots * self.max_pages_per_seq > (64 << 20):
                max_slots //= 2
        self.max_slots = max_slots
        self.pages = FreeList(self.n_pages, "page")
        self.slots = FreeList(self.max_slots, "slot")
        self._length = [0] * self.max_slots
        self._pages_of: List[List[int]] = [[] for _ in range(self.max_slots)]
        # One slot and one page beyond the pools belong to nobody: rows that only fill a step up to a
        # captured size read and write there (``spare_slot``, whose first page is ``spare_page``).
        self.spare_slot, self.spare_page = self.max_slots, self.n_pages
        self.block_table = torch.zeros((self.max_slots + 1, self.max_pages_per_seq), dtype=torch.int32, device=self.device)
        self.block_table[self.spare_slot, 0] = self.spare_page

        # groups
        self._kv_groups: Dict[Tuple[int, int, int], List[int]] = {}
        self._state_groups: Dict[Tuple[Tuple[int, ...], torch.dtype], List[int]] = {}
        self._plane: Dict[int, Tuple[str, object, int]] = {}
        self._cache_of: Dict[int, Optional[int]] = {}
        for pos, (req, cache_of) in enumerate(requests):
            self._cache_of[pos] = cache_of
            if cache_of is not None or req is None:
                continue
            if isinstance(req, KVRequest):
                key = (req.kv_heads, req.head_dim, req.window)
                planes = self._kv_groups.setdefault(key, [])
                self._plane[pos] = ("kv", key, len(planes))
                planes.append(pos)
            elif isinstance(req, StateRequest):
                key = (tuple(req.shape), req.dtype)
                planes = self._state_groups.setdefault(key, [])
                self._plane[pos] = ("state", key, len(planes))
                planes.append(pos)
            else:
                raise CacheError(f"schedule position {pos}: unknown cache request {req!r}")
        for pos, cache_of in self._cache_of.items():
            if cache_of is not None and cache_of not in self._plane:
                raise CacheError(f"schedule position {pos} reads the cache of position {cache_of}, which has none")
        self._k: Dict[Tuple[int, int, int], torch.Tensor] = {}
        self._v: Dict[Tuple[int, int, int], torch.Tensor] = {}
        for key, planes in self._kv_groups.items():
            kvh, d, _w = key
            shape = (len(planes), self.n_pages + 1, kvh, PAGE, d)
            self._k[key] = torch.zeros(shape, dtype=dtype, device=self.device)
            self._v[key] = torch.zeros(shape, dtype=dtype, device=self.device)
        self._state: Dict[Tuple[Tuple[int, ...], torch.dtype], torch.Tensor] = {}
        for key, planes in self._state_groups.items():
            shape, sdtype = key
            self._state[key] = torch.zeros((len(planes), self.max_slots + 1) + tuple(shape), dtype=sdtype, device=self.device)
        self._ops = None
        self._stager = None

    def attach(self, ops, stager) -> None:
        """Use the kernel library (``block_table_set``, ``zero_pages``) and a pinned upload ring
        (``upload(n, fill) -> device int32 tensor``) for the pages a step hands out."""
        self._ops, self._stager = ops, stager

    # ---- description -------------------------------------------------------------------
    def groups(self) -> List[dict]:
        out = []
        for (kvh, d, w), planes in self._kv_groups.items():
            out.append({"kind": "kv", "kv_heads": kvh, "head_dim": d, "window": w, "planes": list(planes),
                        "bytes_per_token": 2 * len(planes) * kvh * d * torch.empty((), dtype=self.dtype).element_size()})
        for (shape, sdtype), planes in self._state_groups.items():
            out.append({"kind": "state", "shape": shape, "dtype": str(sdtype), "planes": list(planes)})
        return out

    def bytes_per_token(self) -> int:
        return sum(g["bytes_per_token"] for g in self.groups() if g["kind"] == "kv")

    def view(self, pos: int):
        """The cache view of schedule position ``pos`` (None if it asked for nothing)."""
        src = self._cache_of.get(pos)
        writable = src is None
        at = pos if src is None else src
        if at not in self._plane:
            return None
        kind, key, ordinal = self._plane[at]
        if kind == "kv":
            return KVView(self._k[key][ordinal], self._v[key][ordinal], self.block_table, writable, key[2])
        return StateView(self._state[key][ordinal], writable)

    # ---- slots -------------------------------------------------------------------------
    def alloc_slot(self) -> int:
        slot = self.slots.take()
        self._length[slot] = 0
        self._pages_of[slot] = []
        for t in self._state.values():
            t[:, slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is freed twice or was never handed out")
        for p in self._pages_of[slot]:
            self.pages.give(p)
        self._pages_of[slot] = []
        self._length[slot] = 0
        self.slots.give(slot)

    def length(self, slot: int) -> int:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not live")
        return self._length[slot]

    def live_slots(self) -> List[int]:
        return [s for s in range(self.max_slots) if self.slots.is_held(s)]

    def tokens_held(self) -> int:
        """Tokens the live sequences hold, each rounded up to a page."""
        return PAGE * self.pages.held()

    # ---- growth ------------------------------------------------------------------------
    def reserve(self, grow: Sequence[Tuple[int, int]]) -> None:
        """Make room for ``grow = [(slot, new_length), ...]`` or change nothing.

        Pages are taken and the block table is updated (host mirror and device); lengths move
        only with ``commit``.
        """
        need_total = 0
        seen = set()
        for slot, new_len in grow:
            if not self.slots.is_held(slot):
                raise CacheError(f"slot {slot} is not live")
            if slot in seen:
                raise CacheError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if new_len < self._length[slot]:
                raise CacheError(f"slot {slot}: new length {new_len} is below its length {self._length[slot]}")
            want = pages_for(new_len)
            if want > self.max_pages_per_seq:
                raise CacheFull(f"slot {slot}: {new_len} tokens exceed the per-sequence limit of "
                                f"{self.max_pages_per_seq * PAGE}")
            need_total += max(0, want - len(self._pages_of[slot]))
        if need_total > self.pages.available():
            raise CacheFull(f"the step needs {need_total} more pages of {PAGE} tokens and {self.pages.available()} "
                            f"of {self.n_pages} are free")
        triples: List[int] = []
        for slot, new_len in grow:
            have = len(self._pages_of[slot])
            want = pages_for(new_len)
            for lp in range(have, want):
                page = self.pages.take()
                self._pages_of[slot].append(page)
                triples += (slot, lp, page)
        if triples:
            self._hand_out(triples)

    def _hand_out(self, triples: List[int]) -> None:
        """Write the block table entries of the (slot, logical, physical) triples and clear their pages."""
        n = len(triples) // 3
        if self._ops is not None and self._stager is not None:
            def fill(buf):
                buf[:] = triples
            dev = self._stager.upload(3 * n, fill)
            self._ops.block_table_set(self.block_table, dev, n)
            for key in self._k:
                self._ops.zero_pages(self._k[key], dev, n)
                self._ops.zero_pages(self._v[key], dev, n)
            return
        t = torch.tensor(triples, dtype=torch.int64).view(n, 3).to(self.device)
        self.block_table[t[:, 0], t[:, 1]] = t[:, 2].to(torch.int32)
        for key in self._k:
            self._k[key][:, t[:, 2]] = 0
            self._v[key][:, t[:, 2]] = 0

    def commit(self, grow: Sequence[Tuple[int, int]]) -> None:
        for slot, new_len in grow:
            self._length[slot] = new_len

    def truncate(self, slot: int, n: int) -> None:
        """Forget everything after the first ``n`` tokens of a sequence.  Only key/value planes can
        be cut at any position; a model with fixed-size state goes back to a ``snapshot`` instead.
        The pages past the cut go back to the pool; the kept last page still holds the sequence's
        old keys and values beyond ``n``, which are overwritten before anything can attend to them."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not live")
        if not 0 <= n <= self._length[slot]:
            raise CacheError(f"slot {slot}: cannot truncate {self._length[slot]} tokens to {n}")
        if self._state and n != self._length[slot]:
            raise CacheError("a cache with per-sequence state cannot be truncated")
        keep = pages_for(n)
        while len(self._pages_of[slot]) > keep:
            self.pages.give(self._pages_of[slot].pop())
        self._length[slot] = n

    def snapshot(self, slot: int) -> "CacheMark":
        """A mark of the sequence as it is: its length and a copy of its fixed-size state.  Keys and
        values are not copied (what lies below the mark's length stays where it is as the sequence
        grows), so a mark is only good for going back, while the sequence lives."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not live")
        return CacheMark(slot, self._length[slot], {key: t[:, slot].clone() for key, t in self._state.items()})

    def restore(self, slot: int, mark: "CacheMark") -> None:
        """Go back to ``mark``: forget the keys and values after its length and put its state back.
        This is how a sequence with fixed-size state is rewound (``truncate`` cannot: a state has no
        positions to cut at)."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not live")
        if mark.slot != slot:
            raise CacheError(f"the mark was taken of slot {mark.slot}, not of slot {slot}")
        if mark.length > self._length[slot]:
            raise CacheError(f"slot {slot}: the mark lies at {mark.length} tokens, beyond its {self._length[slot]}")
        keep = pages_for(mark.length)
        while len(self._pages_of[slot]) > keep:
            self.pages.give(self._pages_of[slot].pop())
        self._length[slot] = mark.length
        for key, saved in mark.state.items():
            self._state[key][:, slot].copy_(saved)

    def check(self) -> None:
        """Invariants: no slot or page lost, held twice, or held by a dead slot."""
        self.pages.check()
        self.slots.check()
        owned: Dict[int, int] = {}
        for slot in range(self.max_slots):
            if not self.slots.is_held(slot):
                if self._pages_of[slot]:
                    raise CacheError(f"free slot {slot} still owns pages")
                continue
            if len(self._pages_of[slot]) < pages_for(self._length[slot]):
                raise CacheError(f"slot {slot} has fewer pages than its length needs")
            for p in self._pages_of[slot]:
                if p in owned:
                    raise CacheError(f"page {p} is held by slots {owned[p]} and {slot}")
                if not self.pages.is_held(p):
                    raise CacheError(f"page {p} of slot {slot} is on the free list")
                owned[p] = slot
        if len(owned) != self.pages.held():
            raise CacheError("a page is held by no slot")
