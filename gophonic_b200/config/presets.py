"""Named configurations for the random-weights mode: each is a ``config.json`` kept as a file beside
this module (the two tiny test shapes and the layer sizes of Qwen3-1.7B, 8B and 32B), read through
the same registry and configuration class as a checkpoint's own file, so no size stands in code."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "presets")


def preset_names() -> List[str]:
    return sorted(n[:-5] for n in os.listdir(_DIR) if n.endswith(".json"))


def preset(name: str) -> Dict[str, Any]:
    """The parsed config.json of the named configuration."""
    path = os.path.join(_DIR, name + ".json")
    if os.sep in name or not os.path.exists(path):
        raise KeyError(f"no configuration named '{name}'; there are {', '.join(preset_names())}")
    with open(path) as f:
        return json.load(f)
