"""Loading weights by tensor name.

The loader works from tensor declarations alone (name, shape, role) and reports every problem of
a checkpoint in one error: tensors that are missing, tensors of the wrong shape or an unusable
dtype, and, beside them, the tensors nobody declared, since an unexpected name next to a missing
one is usually the same tensor misnamed (internal/safetensors/safetensors.go:143-165 checks one
tensor at a time; internal/qwen3lm/weights.go:325-351 is the table of names it asks for).  A
checkpoint that only carries tensors beyond the declared ones is loaded: tensors are resolved by
name and the rest is left alone, as the reference does (weights.go:291-351); the extra names are
reported in a warning, or in the error when ``strict`` is asked for.

Storage rule.  In ``bfloat16`` mode a tensor stays as the checkpoint stores it: BF16 stays
bfloat16 and a tensor stored in 32-bit stays float32; an F16 tensor is widened to float32, which
changes no value (rounding it to bfloat16 would), and its products then run on the 32-bit kernel.
In ``float32`` mode every floating tensor is widened to float32, exactly (a bfloat16 value is its
bits << 16: internal/q8gemm/packed.go:178-179).  Scale vectors of norms are widened to float32
in both modes, which changes no value.  Integer tables become int32.  Non-finite values in norm
vectors are rejected (internal/safetensors/safetensors.go:219-254).
"""
from __future__ import annotations

import warnings
from typing import Dict, Iterable, List, Mapping, Sequence

import numpy as np
import torch

from ..parts.base import TensorDecl
from .safetensors_io import Checkpoint, CheckpointError

MODES = ("bfloat16", "float32")


class WeightsError(ValueError):
    """One error for everything that is wrong with a checkpoint."""

    def __init__(self, model_dir: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[str], wrong_dtype: Sequence[str]):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = [f"checkpoint {model_dir} does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  unusable dtypes ({len(self.wrong_dtype)}): " + "; ".join(self.wrong_dtype))
        super().__init__("\n".join(lines))


_FLOAT = ("BF16", "F16", "F32")
_INT = ("I64", "I32", "I16", "I8", "U8")


def check(ckpt: Checkpoint, decls: Sequence[TensorDecl], strict: bool = False) -> List[str]:
    """Raise one ``WeightsError`` if a declared tensor is missing, misshaped or of an unusable dtype
    (or, with ``strict``, if the checkpoint holds a tensor nobody declared); return the undeclared
    names otherwise."""
    declared = {d.name: d for d in decls}
    missing = [d.name for d in decls if not d.optional and not ckpt.has(d.name)]
    unexpected = [n for n in ckpt.names() if n not in declared]
    wrong_shape, wrong_dtype = [], []
    for d in decls:
        e = ckpt.tensors.get(d.name)
        if e is None:
            continue
        if tuple(e.shape) != tuple(d.shape):
            wrong_shape.append(f"{d.name} has shape {list(e.shape)}, want {list(d.shape)}")
        ok = _INT if d.role == "table" else _FLOAT
        if e.dtype not in ok:
            wrong_dtype.append(f"{d.name} is {e.dtype}, want one of {'/'.join(ok)}")
    if missing or wrong_shape or wrong_dtype or (strict and unexpected):
        raise WeightsError(ckpt.dir, missing, unexpected, wrong_shape, wrong_dtype)
    return unexpected


def _to_torch(arr: np.ndarray, dtype: str) -> torch.Tensor:
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        if dtype == "BF16":
            return torch.from_numpy(arr.view(np.int16)).view(torch.bfloat16)
        return torch.from_numpy(arr)


def place(t: torch.Tensor, stored: str, role: str, mode: str, device) -> torch.Tensor:
    """Apply the storage rule to one tensor and move it to ``device``."""
    if mode not in MODES:
        raise ValueError(f"dtype mode '{mode}' is not one of {MODES}")
    if role == "table":
        return t.to(device=device, dtype=torch.int32)
    t = t.to(device)
    if role in ("norm",) or mode == "float32":
        return t.to(torch.float32)
    if stored == "F32":
        return t
    if stored == "F16":
        return t.to(torch.float32)
    return t.to(torch.bfloat16)


def load_tensors(model_dir: str, decls: Sequence[TensorDecl], mode: str, device, strict: bool = False) -> Dict[str, torch.Tensor]:
    """Read every declared tensor that the checkpoint holds; raise one WeightsError otherwise."""
    out: Dict[str, torch.Tensor] = {}
    with Checkpoint(model_dir) as ckpt:
        extra = check(ckpt, decls, strict)
        if extra:
            shown = ", ".join(extra[:8]) + (f", ... ({len(extra)} in all)" if len(extra) > 8 else "")
            warnings.warn(f"checkpoint {model_dir}: tensors the model does not use are left alone: {shown}")
        for d in decls:
            if not ckpt.has(d.name):
                continue
            e = ckpt.tensors[d.name]
            arr = ckpt.read(d.name)
            if d.role == "norm":
                vals = arr if e.dtype != "BF16" else (arr.astype(np.uint32) << np.uint32(16)).view(np.float32)
                if not np.all(np.isfinite(vals)):
                    raise CheckpointError(f"{d.name} holds a non-finite value")
            out[d.name] = place(_to_torch(arr, e.dtype), e.dtype, d.role, mode, device)
    return out
