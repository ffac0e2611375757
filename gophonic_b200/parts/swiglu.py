"""SwiGLU feed-forward: out = down(silu(gate(x)) * up(x))  (internal/qwen3lm/evaluator.go:679-682;
ops.go:442-461).  gate and up are kept as one [2I, H] matrix so x is read once
(internal/qwen3lm/evaluator.go:680 projects both in one dispatch)."""
from __future__ import annotations

from typing import List, Mapping

import torch

from .base import FeedForward, RowStats, Runtime, TensorDecl, fold_weight, other_fold_buffers


class SwiGLU(FeedForward):
    capturable = True

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        return [TensorDecl(prefix + "gate_proj.weight", (spec.intermediate, spec.hidden)),
                TensorDecl(prefix + "up_proj.weight", (spec.intermediate, spec.hidden)),
                TensorDecl(prefix + "down_proj.weight", (spec.hidden, spec.intermediate))]

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        gate, up = tensors[prefix + "gate_proj.weight"], tensors[prefix + "up_proj.weight"]
        if gate.dtype != up.dtype:
            raise ValueError(f"{prefix}: gate_proj is {gate.dtype} and up_proj is {up.dtype}; they must agree")
        # bfloat16 weights whose width allows it are kept with gate and up rows alternating in blocks
        # of eight, so the few-row kernel can apply the activation in its epilogue
        # (internal/qwen3lm/gpu_darwin.go:406-417 interleaves gate/up rows for the same reason)
        inter, hidden = spec.intermediate, spec.hidden
        self.interleaved = gate.dtype == torch.bfloat16 and inter % 8 == 0
        if self.interleaved:
            self.gate_up = torch.stack([gate.view(inter // 8, 8, hidden), up.view(inter // 8, 8, hidden)], dim=1) \
                .reshape(2 * inter, hidden).contiguous()
        else:
            self.gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.down = tensors[prefix + "down_proj.weight"].contiguous()

    def weight_bytes(self) -> int:
        return self.gate_up.numel() * self.gate_up.element_size() + self.down.numel() * self.down.element_size()

    def forward(self, batch, x: torch.Tensor, out: torch.Tensor) -> None:
        self.rt.ops.gemm(self._activation(x), self.down, out)

    def adds_in_place(self, rows: int) -> bool:
        ops = self.rt.ops
        return (self.down.dtype == torch.bfloat16 and self.rt.act_dtype == torch.bfloat16 and self.spec.intermediate % 8 == 0 and self.spec.hidden % 4 == 0
                and ops.gemm_algo(rows, self.spec.hidden, self.spec.intermediate) == "tc5_pair")

    def forward_into(self, batch, x: torch.Tensor, h: torch.Tensor) -> None:
        self.rt.ops.gemm_add(self._activation(x), self.down, h)

    def folds_norm(self, rows: int, norm) -> bool:
        """Steps of up to 64 rows in bfloat16, gate and up interleaved: the gate/up
        product applies the rows' norm factors from the residual's statistics, the down projection
        adds into the residual."""
        ops = self.rt.ops
        return (rows <= ops.FOLD_ROWS and self.interleaved and self.rt.act_dtype == torch.bfloat16 and self.down.dtype == torch.bfloat16
                and norm.rms_fold() is not None and self.spec.hidden % 8 == 0 and self.spec.intermediate % 8 == 0
                and self.gate_up.data_ptr() % 16 == 0 and self.down.data_ptr() % 16 == 0)

    def forward_folded(self, batch, h: torch.Tensor, stats: RowStats, norm, next_norm=None) -> RowStats:
        ops = self.rt.ops
        rows = h.shape[0]
        _, eps = norm.rms_fold()
        act = torch.empty((rows, self.spec.intermediate), dtype=self.rt.act_dtype, device=h.device)
        made_by = ops.gemm_scaled(stats.prescaled, eps, stats.partials, stats.count, self.gate_up, act, swiglu=True)
        out_stats, out_rows = other_fold_buffers(batch, stats, self.spec.hidden)
        weight = fold_weight(next_norm, self.spec.hidden)
        count = ops.gemm_residual(act, self.down, h, out_stats, weight, out_rows[:rows] if weight is not None else None, behind=made_by)
        return RowStats(out_stats, count, out_rows[:rows] if weight is not None else None, next_norm if weight is not None else None)

    def _activation(self, x: torch.Tensor) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T): [rows, intermediate] in the activation dtype."""
        ops = self.rt.ops
        rows = x.shape[0]
        act = torch.empty((rows, self.spec.intermediate), dtype=x.dtype, device=x.device)
        if self.interleaved and ops.gemm_swiglu_accepts(x, self.gate_up):
            ops.gemm_swiglu(x, self.gate_up, act)
        else:
            gu = torch.empty((rows, 2 * self.spec.intermediate), dtype=x.dtype, device=x.device)
            ops.gemm(x, self.gate_up, gu)
            ops.swiglu(gu, act, self.interleaved)
        return act
