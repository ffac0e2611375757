"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed, in the checkpoint's real layout, so that it is read back through the
ordinary loader (internal/qwen3lm/lmtest/lmtest.go:59-133 writes its test snapshots the same way),
or make the same tensors directly on the device for sizes too large to pass through a file.

One fill serves both.  Every tensor has a key of its own, a digest of (seed, tensor name), and
element i of the tensor is a function of (key, i) alone: two splitmix64 words, the sum of their
eight 16-bit fields (a sum of eight uniform integers: mean and variance of the normal law, tails
to 4.9 deviations), centred, multiplied by one fp32 constant and shifted by the mean.  Only
integer arithmetic, one fp32 multiplication and one fp32 addition are involved, so numpy here and
the CUDA kernel (``csrc/cache_fill.cu``) give the same bits; a tensor's values do not depend on
which other tensors exist, on the order of writing or on how the work is cut.  Matrices and the
embedding are centred on 0 with deviation std; norm scale vectors on 1.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import json
import math
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


_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_CHUNK = 1 << 22


def fill_constant(std: float) -> np.float32:
    """The fp32 factor that gives the centred sum of eight 16-bit uniforms the deviation ``std``."""
    return np.float32(float(std) / math.sqrt(2.0 * (2.0 ** 32 - 1.0) / 3.0))


def _fill_chunk(key: int, lo: int, hi: int, c: np.float32, mean: np.float32, out: np.ndarray) -> None:
    """out[:] = elements lo..hi-1 of the fill with ``key``."""
    n = hi - lo
    with np.errstate(over="ignore"):
        x = np.arange(2 * lo + 1, 2 * hi + 1, dtype=np.uint64)   # word index + 1, two words an element
        x *= _GAMMA
        x += np.uint64(key)
        t = x >> np.uint64(30)
        x ^= t
        x *= np.uint64(0xBF58476D1CE4E5B9)
        np.right_shift(x, np.uint64(27), out=t)
        x ^= t
        x *= np.uint64(0x94D049BB133111EB)
        np.right_shift(x, np.uint64(31), out=t)
        x ^= t
    fields = x.view(np.uint16).reshape(n, 8)
    total = fields[:, 0].astype(np.int32)
    for j in range(1, 8):
        total += fields[:, j]
    total -= 262140
    np.multiply(total.astype(np.float32), c, out=out)
    out += mean


def counter_fill(key: int, n: int, std: float, mean: float) -> np.ndarray:
    """fp32 values of the ``n`` elements of the tensor with fill key ``key``."""
    out = np.empty(n, dtype=np.float32)
    c, m = fill_constant(std), np.float32(mean)
    spans = [(lo, min(n, lo + _CHUNK)) for lo in range(0, n, _CHUNK)]
    if len(spans) <= 1:
        for lo, hi in spans:
            _fill_chunk(key, lo, hi, c, m, out[lo:hi])
        return out
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(spans), os.cpu_count() or 1, 16)) as ex:
        list(ex.map(lambda span: _fill_chunk(key, span[0], span[1], c, m, out[span[0]:span[1]]), spans))
    return out


def random_tensor(d: TensorDecl, seed: int, scales: InitScales, head_name: Optional[str] = None) -> np.ndarray:
    """fp32 values of one declared tensor."""
    std, mean = _std_and_mean(d, scales, head_name)
    return counter_fill(_tensor_seed(seed, d.name), int(np.prod(d.shape)), std, mean).reshape(d.shape)


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
                             tied: bool = False, ops=None) -> Dict[str, torch.Tensor]:
    """The tensors ``write_random_model`` would write with bfloat16 weights and the loader would then
    place, made on the device by the fill kernel: the same bits, without the file."""
    from .loader import place
    if ops is None:
        from .. import ops
    out: Dict[str, torch.Tensor] = {}
    for d in declare_model(spec):
        if d.name == spec.head.name and tied:
            continue
        if d.role == "table":
            raise ValueError(f"random weights: no rule for the integer table {d.name}")
        std, mean = _std_and_mean(d, scales, spec.head.name)
        t = torch.empty(d.shape, dtype=torch.bfloat16, device=device)   # what a BF16 checkpoint stores
        ops.random_fill(t, _tensor_seed(seed, d.name), float(fill_constant(std)), float(mean))
        out[d.name] = place(t, "BF16", d.role, mode, device)
    return out
