"""The list of tensors a model resolves, gathered from its parts' declarations."""
from __future__ import annotations

from typing import List

from .. import registry
from ..parts.base import TensorDecl


def declare_model(spec) -> List[TensorDecl]:
    """Every tensor of ``spec`` by checkpoint name: embedding, each layer's parts (each layer once,
    however often the schedule runs it), final norm, and the head (optional when it can be tied)."""
    from .. import parts  # noqa: F401  (registers the built-in parts)
    decls: List[TensorDecl] = [TensorDecl(spec.embedding.name, (spec.embedding.vocab, spec.embedding.hidden),
                                          role="embedding")]
    for layer in spec.layers:
        decls += registry.part_class("block", layer.block).declare(layer)
    norm_name = spec.final_norm_name
    if not norm_name.endswith("weight"):
        raise ValueError(f"final norm tensor name '{norm_name}' must end in 'weight'")
    decls += registry.part_class("norm", spec.final_norm.kind).declare(spec.final_norm, norm_name[:-len("weight")])
    decls.append(TensorDecl(spec.head.name, (spec.head.vocab, spec.head.hidden), role="matrix",
                            optional=spec.head.tied_to is not None))
    seen = set()
    for d in decls:
        if d.name in seen:
            raise ValueError(f"tensor '{d.name}' is declared twice")
        seen.add(d.name)
    return decls
