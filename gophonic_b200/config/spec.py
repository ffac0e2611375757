"""Architecture-neutral description of a decoder: what the parts are and how they are arranged.

A model is data: an embedding, a list of layers, a schedule that says in which order the layers
run (and whose cache each run uses), a final norm and a head.  Every layer names its parts by
*kind* and carries the sizes and constants of each part; nothing here knows which architecture it
describes.  An architecture (see ``gophonic_b200.registry``) is a function from its own typed
configuration to a ``ModelSpec``.

The reference keeps the same information in one flat ``modelConfig`` with per-layer flags
(internal/qwen3lm/weights.go:108-127, the ``linear []bool`` per-layer kind list at :122); here it
is split per part so that a new mixer or feed-forward is a new spec class, not a new field on a
shared struct.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple


@dataclass(frozen=True)
class RMSNormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * weight  (internal/qwen3lm/ops.go:251-254)."""
    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RotarySpec:
    """Rotate-half rotary embedding over the first ``rotary_dim`` elements of each head.

    inv_freq_i = theta^(-2i/rotary_dim) (internal/qwen3lm/weights.go:681-688); element i pairs with
    i + rotary_dim/2 (internal/qwen3lm/kernels_scalar.go:73-80).
    """
    head_dim: int
    rotary_dim: int
    theta: float
    kind: str = "rope"


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding inside the mixer."""
    head_dim: int
    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query causal attention (internal/qwen3lm/ops.go:231-293).

    ``qk_norm`` is the per-head norm applied to q and k before the position encoding, or None.
    ``window`` = 0 attends to every earlier key; w > 0 only to the last w keys (itself included).
    """
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    scale: float
    position: object
    qk_norm: Optional[RMSNormSpec] = None
    window: int = 0
    kind: str = "attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    """down(silu(gate(x)) * up(x))  (internal/qwen3lm/ops.go:442-461)."""
    hidden: int
    intermediate: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class LayerSpec:
    """One layer of the pre-norm arrangement: the block kind and the four parts it arranges.

    ``prefix`` is the tensor-name prefix of the layer ("model.layers.3."); each part resolves its
    tensors under the sub-prefix named here (the defaults are the names Qwen3 checkpoints use).

    The model, the loader and the cache read only two fields of a layer's spec, ``block`` and
    ``prefix``; everything else is between the spec and the block class registered under that
    kind (``declare``, ``cache_request``, ``mixers``, ``prepare``, ``weight_bytes``, ``forward``).
    A block with another arrangement (one shared norm, norms after the parts, two mixers) brings a
    spec class of its own with those two fields.
    """
    prefix: str
    mixer: object
    feed_forward: object
    mixer_norm: object
    feed_forward_norm: object
    block: str = "prenorm"
    mixer_prefix: str = "self_attn."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    feed_forward_norm_prefix: str = "post_attention_layernorm."


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    ``layer`` indexes ``ModelSpec.layers``; a layer may appear in several entries (its weights are
    then used more than once, each run with a cache plane of its own).  ``cache_of`` names the
    schedule position whose cache plane this run reads instead of writing one of its own
    (None: own plane).
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class EmbeddingSpec:
    name: str
    vocab: int
    hidden: int


@dataclass(frozen=True)
class HeadSpec:
    """Output projection hidden -> vocab.  If the checkpoint has no tensor ``name`` the head is
    tied to ``tied_to`` (qwen3/chat.go:55-65 decides by tensor presence, never by a flag)."""
    name: str
    vocab: int
    hidden: int
    tied_to: Optional[str] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden: int
    vocab: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: object
    final_norm_name: str
    head: HeadSpec

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("model spec: no layers")
        if not self.schedule:
            raise ValueError("model spec: empty schedule")
        for pos, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"model spec: schedule[{pos}] names layer {e.layer}, "
                                 f"there are {len(self.layers)}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < pos:
                    raise ValueError(f"model spec: schedule[{pos}] reads the cache of position "
                                     f"{e.cache_of}, which does not run before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"model spec: schedule[{pos}] reads the cache of position "
                                     f"{e.cache_of}, which has no cache of its own")


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(layer=i) for i in range(n_layers))
