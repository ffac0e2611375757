"""What every part must offer, and the small value types parts exchange with the rest.

A *part* is one of: mixer, feed-forward, norm, position encoding, block.  A part class has

* ``declare(spec, prefix) -> [TensorDecl]`` (classmethod): the tensors it resolves, by full name,
  with shape and role.  The loader and the random-weights writer work from these declarations
  alone, so they never need to know a model.
* ``__init__(spec, prefix, tensors, runtime)``: ``tensors`` maps each declared name to a device
  tensor already in the dtype the loader's rules give it.
* its forward method (see each category below).

A mixer additionally says what it needs from the cache, per sequence:
``cache_request(spec) -> KVRequest | StateRequest | None`` (classmethod).

No part receives the model or its configuration: sizes and constants arrive in the part's own
spec.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part reads from the checkpoint.

    role: "matrix" (projection, [out, in]), "embedding" ([vocab, hidden]), "norm" (a scale
    vector; initialised near 1), "vector" (initialised near 0), "table" (integers).
    ``optional``: absence is not an error (the tied head).
    """
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


@dataclass(frozen=True)
class KVRequest:
    """Per token, per sequence: keys and values of ``kv_heads`` x ``head_dim``.
    window = 0: every key is kept; w > 0: only the last w keys are ever read."""
    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateRequest:
    """Per sequence, fixed size: a tensor of ``shape`` and ``dtype``, zero when a sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class RowStats:
    """What travels between parts instead of a pending addend when the residual is already complete
    and its statistics are known: ``partials[row, :count]`` are partial sums of squares of row
    ``row`` of the residual, written by whichever kernel last changed it (a product that added its
    output into the residual, or the embedding).  If that kernel was told which norm comes next,
    ``prescaled`` holds bf16(residual * that norm's weight), the norm's output but for each row's
    factor, and ``prescaled_for`` is that norm.  A part that can apply the factor in its own first
    product (``folds_norm``) then needs no norm kernel; every other part ignores all this and
    runs its norm as usual."""
    partials: torch.Tensor                      # float32 [>= rows, capacity]
    count: int
    prescaled: Optional[torch.Tensor] = None    # bfloat16 [rows, width]
    prescaled_for: Optional[object] = None


FOLD_ROWS = 64   # rows the buffers for ``RowStats`` hold; the kernels refuse more rows than their buffers have


def fold_buffers(batch, which: int, width: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """One of the step's two pairs of buffers for ``RowStats`` (they alternate: a product reads one
    pair while the next product that changes the residual writes the other): statistics, float32
    [64, capacity] with room for the partial sums a producing kernel leaves of a residual ``width``
    wide (``ops.fold_capacity``), and prescaled rows, bfloat16 [64, width]."""
    capacity = max(8, (width + 15) // 16)
    stats = batch.workspace(("row statistics", which & 1, capacity), FOLD_ROWS * capacity).view(FOLD_ROWS, capacity)
    rows = batch.workspace(("prescaled rows", which & 1, width), FOLD_ROWS * width, torch.bfloat16).view(FOLD_ROWS, width)
    return stats, rows


def other_fold_buffers(batch, stats: RowStats, width: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """The pair of buffers ``stats`` did not come in: nothing reads it any more."""
    pair = fold_buffers(batch, 0, width)
    if pair[0].data_ptr() == stats.partials.data_ptr():
        pair = fold_buffers(batch, 1, width)
    return pair


def fold_weight(norm, width: int) -> Optional[torch.Tensor]:
    """The weight of ``norm`` if a producing kernel can prescale rows of ``width`` for it, else None."""
    fold = norm.rms_fold() if norm is not None and hasattr(norm, "rms_fold") else None
    if fold is None or fold[0].numel() != width:
        return None
    return fold[0]


@dataclass
class Runtime:
    """What parts need to run: the device, the activation dtype of this model instance
    (torch.float32 for the true 32-bit path, torch.bfloat16 for the serving path) and the
    kernel library."""
    device: torch.device
    act_dtype: torch.dtype
    ops: object

    @property
    def is_fp32(self) -> bool:
        return self.act_dtype == torch.float32


class Part:
    category = ""
    # True if forward only enqueues work on the current CUDA stream (no host reads of device data,
    # no fresh host-side state): such a part may be captured into a CUDA graph.  The default is the
    # safe one; the engine replays single-token steps from graphs only if every part says True.
    capturable = False

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        return []


class Norm(Part):
    """forward(h, out, delta=None, rows=None): if ``delta`` is given, h += delta first (both fp32,
    in place); then out = norm(h) in the activation dtype.  With ``rows`` (int32 row indices) the
    sum h[rows] + delta[rows] is normalised into out[i] and h is left untouched."""
    category = "norm"

    def rms_fold(self):
        """(weight, eps) if this norm is y = x / sqrt(mean(x^2) + eps) * weight with a float32 weight
        vector, so that a product's kernel may apply it from the residual's ``RowStats``; else None."""
        return None


class PositionEncoding(Part):
    """Owned by a mixer.  ``prepare(capacity)`` makes whatever tables positions < capacity need."""
    category = "position"

    def prepare(self, capacity: int) -> None:
        pass


class Mixer(Part):
    """forward(batch, x, out, cache): x is [rows, hidden] in the activation dtype, out is
    [rows, hidden] fp32 (added to the residual by the block).  ``cache`` is this run's view of
    the cache (a KV plane or a state tensor, or None) and ``cache.writable`` says whether this
    run stores into it."""
    category = "mixer"

    @classmethod
    def cache_request(cls, spec):
        return None

    def prepare(self, capacity: int) -> None:
        pass

    def plan(self, nseq: int, max_q_len: int, max_kv_len: int, sm_count: int):
        """How this mixer will launch a step of ``nseq`` sequences that bring at most ``max_q_len``
        rows each and see at most ``max_kv_len`` keys: any hashable value, or None if the launch
        does not depend on these numbers.  The engine does not look inside: it asks once per step,
        hands the answer back through ``batch.plan_for(self)``, and keys its captured steps on the
        answers of all mixers, so a step is replayed only with the launch shape it was captured
        with.  Scratch memory that the plan calls for comes from ``batch.workspace(key, n)``."""
        return None

    def folds_norm(self, rows: int, norm) -> bool:
        """True if, for a step of ``rows`` rows, ``forward_folded(batch, h, stats, norm, cache,
        next_norm)`` can run: the part then takes its activations from ``stats.prescaled`` (made for
        ``norm``), applies the rows' factors from the statistics in its first product, adds its
        output into the float32 residual ``h`` in its last product and returns the new ``RowStats``,
        prescaled for ``next_norm`` if that is given and can be.  Only offered where it is faster
        (single-token steps of up to 64 rows); the default is False."""
        return False

    def adds_in_place(self, rows: int) -> bool:
        """True if, for a step of ``rows`` rows, ``forward_into(batch, x, h, cache)`` is the faster
        way: the part then adds its output to the fp32 residual ``h`` itself (in the epilogue of its
        last product) and the block has no addend to hand on.  The sum must be the one a separate
        fp32 add would give.  The default is False: ``forward`` into a buffer of its own."""
        return False


class FeedForward(Part):
    """forward(batch, x, out): x [rows, hidden] activation dtype -> out [rows, hidden] fp32.
    Optionally ``adds_in_place(rows)`` / ``forward_into(batch, x, h)`` as for a mixer."""
    category = "feed_forward"

    def folds_norm(self, rows: int, norm) -> bool:
        """As for a mixer: ``forward_folded(batch, h, stats, norm, next_norm) -> RowStats``."""
        return False

    def adds_in_place(self, rows: int) -> bool:
        return False
