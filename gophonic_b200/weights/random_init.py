"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed, in the checkpoint's real layout, so that it is read back through the
ordinary loader (internal/qwen3lm/lmtest/lmtest.go:59-133 writes its test snapshots the same way).

Every tensor has a generator of its own, seeded by (seed, tensor name): the values of a tensor do
not depend on which other tensors exist or in which order they are written.  Matrices and the
embedding are N(0, std); norm scale vectors are 1 + N(0, norm_std).
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass
from typing import Dict, Optional, Sequence

import numpy as np
import torch

from ..parts.base import TensorDecl
from .declare import declare_model
from .safetensors_io import float32_to_bf16_bits, write_safetensors


@dataclass(frozen=True)
class InitScales:
    matrix: float = 0.02
    embedding: float = 0.02
    head: float = 0.02
    norm: float = 0.02


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little")


def _std_and_mean(d: TensorDecl, scales: InitScales, head_name: Optional[str]):
    if d.role == "norm":
        return scales.norm, 1.0
    if d.role == "embedding":
        return scales.embedding, 0.0
    if head_name is not None and d.name == head_name:
        return scales.head, 0.0
    return scales.matrix, 0.0


def random_tensor(d: TensorDecl, seed: int, scales: InitScales, head_name: Optional[str] = None) -> np.ndarray:
    """fp32 values of one declared tensor."""
    std, mean = _std_and_mean(d, scales, head_name)
    rng = np.random.Generator(np.random.PCG64(_tensor_seed(seed, d.name)))
    n = int(np.prod(d.shape))
    out = np.empty(n, dtype=np.float32)
    chunk = 1 << 24
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        out[lo:hi] = rng.standard_normal(hi - lo, dtype=np.float32) * np.float32(std) + np.float32(mean)
    return out.reshape(d.shape)


def write_random_model(config, seed: int, out_dir: str, weight_dtype: str = "bfloat16",
                       scales: InitScales = InitScales(), tied: Optional[bool] = None) -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors`` for ``config``.

    ``weight_dtype``: "bfloat16" (values rounded to nearest even) or "float32".  ``tied`` = True
    leaves the head out so it is tied to the embedding; default: the configuration's
    ``tie_word_embeddings`` if it has one.
    """
    if weight_dtype not in ("bfloat16", "float32"):
        raise ValueError(f"weight dtype '{weight_dtype}' must be bfloat16 or float32")
    spec = config.model_spec()
    if tied is None:
        tied = bool(getattr(config, "tie_word_embeddings", False))
    os.makedirs(out_dir, exist_ok=True)
    tensors = {}
    for d in declare_model(spec):
        if d.name == spec.head.name and tied:
            if spec.head.tied_to is None:
                raise ValueError("this architecture's head cannot be tied")
            continue
        if d.role == "table":
            raise ValueError(f"random weights: no rule for the integer table {d.name}")
        vals = random_tensor(d, seed, scales, spec.head.name)
        if weight_dtype == "bfloat16":
            tensors[d.name] = ("BF16", d.shape, float32_to_bf16_bits(vals).reshape(-1))
        else:
            tensors[d.name] = ("F32", d.shape, vals.reshape(-1))
    cfg = config.to_dict()
    cfg["torch_dtype"] = weight_dtype
    if "tie_word_embeddings" in cfg:
        cfg["tie_word_embeddings"] = bool(tied)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors)
    return out_dir


def random_tensors_on_device(spec, seed: int, mode: str, device, scales: InitScales = InitScales(),
                             tied: bool = False) -> Dict[str, torch.Tensor]:
    """Seeded random tensors made on the device, for models too large to pass through a file in
    a benchmark's time.  The values differ from ``write_random_model``'s (another generator); the
    distributions are the same."""
    from .loader import place
    out: Dict[str, torch.Tensor] = {}
    for d in declare_model(spec):
        if d.name == spec.head.name and tied:
            continue
        std, mean = _std_and_mean(d, scales, spec.head.name)
        g = torch.Generator(device=device)
        g.manual_seed(_tensor_seed(seed, d.name) & 0x7FFFFFFFFFFFFFFF)
        stored = "BF16"
        if mode == "float32" or d.role == "norm":
            t = torch.empty(d.shape, dtype=torch.float32, device=device).normal_(mean, std, generator=g)
            t = t.to(torch.bfloat16).to(torch.float32)  # values a bfloat16 checkpoint could hold
        else:
            t = torch.empty(d.shape, dtype=torch.bfloat16, device=device).normal_(mean, std, generator=g)
        out[d.name] = place(t, stored, d.role, mode, device)
    return out
