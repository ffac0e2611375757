"""Position encodings owned by a mixer.

``RotaryEmbedding``: rotate-half rotary embedding over the first ``rotary_dim`` elements of a head.
inv_freq_i = theta^(-2i/rotary_dim) and the angles pos * inv_freq_i are computed in float64, their
cosines and sines rounded to fp32 tables (internal/qwen3lm/weights.go:681-688;
internal/qwen3lm/evaluator.go:847-858).  The tables are consumed by the fused
norm + rotation + cache-write kernel; this part only owns them.

``NoPosition``: nothing is applied.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from .base import PositionEncoding, Runtime


class RotaryEmbedding(PositionEncoding):
    def __init__(self, spec, prefix, tensors, runtime: Runtime):
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim:
            raise ValueError(f"rotary width {spec.rotary_dim} must be even and in (0, head_dim={spec.head_dim}]")
        self.spec = spec
        self.rt = runtime
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None
        self.capacity = 0

    def prepare(self, capacity: int) -> None:
        if capacity <= self.capacity:
            return
        rot = self.spec.rotary_dim
        i = np.arange(rot // 2, dtype=np.float64)
        inv_freq = 1.0 / np.power(float(self.spec.theta), 2.0 * i / float(rot))
        ang = np.arange(capacity, dtype=np.float64)[:, None] * inv_freq[None, :]
        self.cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(self.rt.device)
        self.sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(self.rt.device)
        self.capacity = capacity

    def kernel_args(self) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], int]:
        return self.cos, self.sin, self.spec.rotary_dim


class NoPosition(PositionEncoding):
    def __init__(self, spec, prefix, tensors, runtime: Runtime):
        self.spec = spec
        self.capacity = 1 << 62

    def kernel_args(self):
        return None, None, 0
