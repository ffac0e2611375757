"""RMSNorm part: y = x * (1 / sqrt(mean(x^2) + eps)) * weight, plain weight (not 1 + w)
(internal/qwen3lm/ops.go:251-254; kernels_scalar.go:15-35).  Statistics are fp32; the weight is
held in fp32 (an exact widening of a bfloat16 checkpoint vector)."""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .base import Norm, Runtime, TensorDecl


class RMSNorm(Norm):
    capturable = True

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        return [TensorDecl(prefix + "weight", (spec.size,), role="norm")]

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.weight = tensors[prefix + "weight"].to(torch.float32).contiguous()
        self.eps = float(spec.eps)

    def rms_fold(self):
        return self.weight, self.eps

    def forward(self, h: torch.Tensor, out: torch.Tensor, delta: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> None:
        self.rt.ops.add_rmsnorm(h, delta, self.weight, self.eps, out, rows)
