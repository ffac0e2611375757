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

    def adds_in_place(self, rows: int) -> bool:
        return False
