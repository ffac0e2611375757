"""Registries: part kinds -> part classes, and architecture names -> typed configurations.

One table maps an architecture's name (``config.json``'s ``architectures[0]``, with ``model_type``
as a fallback) to its configuration class; the class turns the file's keys into a ``ModelSpec``.
A second set of tables maps the *kind* string carried by each part spec to the class that runs
it.  Adding a mixer, feed-forward, norm, position encoding, block arrangement or a whole
architecture is one ``register_*`` call from any module; nothing in the package has to change.

The reference dispatches on the checkpoint in the same two steps: ``IsModelDir`` reads
``config.json.model_type`` (qwen3/model.go:110-129) and ``TextConfig.model()`` switches on it
(internal/qwen3lm/weights.go:647-665).
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, List, Optional, Type

PART_CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block")

_parts: Dict[str, Dict[str, type]] = {c: {} for c in PART_CATEGORIES}
_architectures: Dict[str, type] = {}
_model_types: Dict[str, str] = {}


class RegistryError(KeyError):
    def __str__(self) -> str:  # KeyError quotes its message; keep it readable
        return self.args[0] if self.args else ""


def register_part(category: str, kind: str, cls: type) -> None:
    """Make ``cls`` the implementation of part ``kind`` in ``category``.

    Registering a kind again replaces it (later wins, as gophonic.Register does for formats:
    gophonic.go:176-186)."""
    if category not in _parts:
        raise RegistryError(f"unknown part category '{category}'; categories are {PART_CATEGORIES}")
    _parts[category][kind] = cls


def part_class(category: str, kind: str) -> type:
    try:
        return _parts[category][kind]
    except KeyError:
        known = sorted(_parts.get(category, {}))
        raise RegistryError(f"no {category} part of kind '{kind}' is registered; known: {known}") from None


def register_mixer(kind: str, cls: type) -> None:
    register_part("mixer", kind, cls)


def register_feed_forward(kind: str, cls: type) -> None:
    register_part("feed_forward", kind, cls)


def register_norm(kind: str, cls: type) -> None:
    register_part("norm", kind, cls)


def register_position(kind: str, cls: type) -> None:
    register_part("position", kind, cls)


def register_block(kind: str, cls: type) -> None:
    register_part("block", kind, cls)


def register_architecture(name: str, config_cls: type, model_type: Optional[str] = None) -> None:
    """``config_cls`` must offer ``from_dict(dict)``, ``to_dict()`` and ``model_spec()``."""
    for attr in ("from_dict", "to_dict", "model_spec"):
        if not hasattr(config_cls, attr):
            raise TypeError(f"architecture '{name}': configuration class lacks '{attr}'")
    _architectures[name] = config_cls
    if model_type:
        _model_types[model_type] = name


def architectures() -> List[str]:
    return sorted(_architectures)


def architecture_of(config: Dict[str, Any]) -> str:
    """The registered architecture name a parsed config.json selects."""
    archs = config.get("architectures")
    if isinstance(archs, list) and archs and archs[0] in _architectures:
        return archs[0]
    mt = config.get("model_type")
    if mt in _model_types:
        return _model_types[mt]
    named = archs[0] if isinstance(archs, list) and archs else mt
    raise RegistryError(f"no architecture registered for '{named}'; registered: {architectures()}")


def config_class(name: str) -> type:
    try:
        return _architectures[name]
    except KeyError:
        raise RegistryError(f"no architecture registered for '{name}'; registered: {architectures()}") from None


def read_config(model_dir: str):
    """Parse ``model_dir/config.json`` with the configuration class its architecture selects."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r") as f:
            raw = json.load(f)
    except OSError as e:
        raise FileNotFoundError(f"cannot read {path}: {e}") from e
    if not isinstance(raw, dict):
        raise ValueError(f"{path}: not a JSON object")
    return config_class(architecture_of(raw)).from_dict(raw)


def _register_builtin() -> None:
    from .config.qwen3 import Qwen3Config
    register_architecture("Qwen3ForCausalLM", Qwen3Config, model_type="qwen3")


_register_builtin()
