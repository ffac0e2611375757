"""Block arrangements: how a layer's mixer, feed-forward and norms are wired around the residual.

``PreNormBlock``: h += mixer(norm_m(h)); h += ffn(norm_f(h)).  A part's output is either added to
the residual by the part itself, in the epilogue of its last product (prompt-sized steps of the
built-in parts: ``adds_in_place``), or it is not added at once: it is handed on as a pending
addend and added by whatever norms the residual next (the layer's second norm, the next block's
first norm, or the final norm), in the same kernel that takes the statistics
(internal/qwen3lm/evaluator.go:641-647, 678-682; ops.go:94-108 does the same).  In single-token
steps of up to 64 rows the built-in parts go one step further (``folds_norm``): the part's last
product adds into the residual, leaves the rows' sums of squares behind and writes the rows
already multiplied by the next norm's weight (``RowStats``), and the next part's first product
multiplies its finished sums by the rows' factors, so no norm kernel runs at all
(internal/qwen3lm/gpu.metal:70-162 folds its norms in the same spirit).  The residual h stays
fp32 throughout.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .. import registry
from .base import Part, RowStats, Runtime, TensorDecl


class PreNormBlock(Part):
    category = "block"

    @classmethod
    def declare(cls, layer, prefix: str = "") -> List[TensorDecl]:
        p = layer.prefix
        decls: List[TensorDecl] = []
        decls += registry.part_class("norm", layer.mixer_norm.kind).declare(layer.mixer_norm, p + layer.mixer_norm_prefix)
        decls += registry.part_class("mixer", layer.mixer.kind).declare(layer.mixer, p + layer.mixer_prefix)
        decls += registry.part_class("norm", layer.feed_forward_norm.kind).declare(
            layer.feed_forward_norm, p + layer.feed_forward_norm_prefix)
        decls += registry.part_class("feed_forward", layer.feed_forward.kind).declare(
            layer.feed_forward, p + layer.feed_forward_prefix)
        return decls

    def __init__(self, layer, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        p = layer.prefix
        self.layer = layer
        self.rt = runtime
        self.mixer_norm = registry.part_class("norm", layer.mixer_norm.kind)(
            layer.mixer_norm, p + layer.mixer_norm_prefix, tensors, runtime)
        self.mixer = registry.part_class("mixer", layer.mixer.kind)(
            layer.mixer, p + layer.mixer_prefix, tensors, runtime)
        self.feed_forward_norm = registry.part_class("norm", layer.feed_forward_norm.kind)(
            layer.feed_forward_norm, p + layer.feed_forward_norm_prefix, tensors, runtime)
        self.feed_forward = registry.part_class("feed_forward", layer.feed_forward.kind)(
            layer.feed_forward, p + layer.feed_forward_prefix, tensors, runtime)
        self._native = None       # the library's record of this layer, if it can issue the layer itself
        self._native_tables = None

    def _native_layer(self):
        """The layer as the library's one-call issue takes it, if mixer, feed-forward and norms are
        exactly the built-in attention, SwiGLU and RMSNorm (a subclass may have changed what they
        compute); None otherwise."""
        from .attention import Attention
        from .norm import RMSNorm
        from .rope import NoPosition, RotaryEmbedding
        from .swiglu import SwiGLU
        m, f = self.mixer, self.feed_forward
        if not (type(m) is Attention and type(f) is SwiGLU and type(self.mixer_norm) is RMSNorm
                and type(self.feed_forward_norm) is RMSNorm and type(m.position) in (RotaryEmbedding, NoPosition)):
            return None
        ops = self.rt.ops
        cos, sin, rot = m.position.kernel_args()
        tables = (None if cos is None else cos.data_ptr(), None if sin is None else sin.data_ptr())
        if self._native is not None and tables == self._native_tables:
            return self._native
        code = {torch.float32: ops.F32, torch.bfloat16: ops.BF16}
        ptr = lambda t: 0 if t is None else t.data_ptr()
        s = m.spec
        self._native = ops.PrenormLayer(
            s.hidden, s.heads, s.kv_heads, s.head_dim, f.spec.intermediate, self.mixer_norm.eps, self.feed_forward_norm.eps,
            m.eps, float(s.scale), int(s.window), rot, 0 if cos is None else cos.shape[0], code[self.rt.act_dtype],
            1 if f.interleaved else 0, ptr(self.mixer_norm.weight), ptr(self.feed_forward_norm.weight),
            ptr(m.qkv), code[m.qkv.dtype], ptr(m.o), code[m.o.dtype], ptr(f.gate_up), code[f.gate_up.dtype],
            ptr(f.down), code[f.down.dtype], ptr(m.q_norm), ptr(m.k_norm), ptr(cos), ptr(sin))
        self._native_tables = tables
        return self._native

    # What a model asks of a block, whatever its arrangement: the cache its runs need, tables for a
    # capacity, its mixers' launch plans, the weight bytes of one run, and whether it can be captured.
    @classmethod
    def cache_request(cls, layer):
        return registry.part_class("mixer", layer.mixer.kind).cache_request(layer.mixer)

    def prepare(self, capacity: int) -> None:
        self.mixer.prepare(capacity)

    def mixers(self) -> List[Part]:
        return [self.mixer]

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.mixer, self.feed_forward) if hasattr(p, "weight_bytes"))

    @property
    def capturable(self) -> bool:
        return all(p.capturable for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward))

    def first_norm(self):
        """The norm that reads the residual first: whoever changes the residual ahead of this block
        may prepare its rows for it."""
        return self.mixer_norm

    def wants_stats(self, rows: int) -> bool:
        """Whether the block's first part would apply its norm's row factors itself if the residual
        came with ``RowStats`` prescaled for ``first_norm()``."""
        return self.mixer.folds_norm(rows, self.mixer_norm)

    def forward(self, batch, h: torch.Tensor, pending, cache, next_norm=None):
        """Runs the layer on residual ``h`` (fp32, updated in place).  ``pending`` says what is still
        owed to the residual: a float32 tensor that has yet to be added, ``RowStats`` (nothing owed,
        the rows' sums of squares are known and the rows may be prescaled for a norm), or None
        (nothing owed, nothing known).  ``next_norm`` is the norm that will read the residual after
        this layer, if the caller knows it.  Returns what is owed for the layer after."""
        rows, hidden = h.shape
        act = self.rt.act_dtype
        x = None
        folds = (isinstance(pending, RowStats) and pending.prescaled_for is self.mixer_norm
                 and self.mixer.folds_norm(rows, self.mixer_norm))
        native = None if folds or cache is None else self._native_layer()
        if native is not None:
            # the whole layer from one call into the library: the same kernels in the same order
            ops = self.rt.ops
            work = batch.workspace(("prenorm layer", ops.prenorm_layer_workspace(native, rows)),
                                   ops.prenorm_layer_workspace(native, rows), torch.uint8)
            splits, scratch = self.mixer.key_splits(batch)
            return ops.prenorm_layer_forward(native, batch, cache, h, pending if isinstance(pending, torch.Tensor) else None,
                                             work, splits, scratch)
        if folds:
            pending = self.mixer.forward_folded(batch, h, pending, self.mixer_norm, cache, self.feed_forward_norm)
        else:
            x = torch.empty((rows, hidden), dtype=act, device=h.device)
            self.mixer_norm.forward(h, x, pending if isinstance(pending, torch.Tensor) else None)
            if self.mixer.adds_in_place(rows):
                self.mixer.forward_into(batch, x, h, cache)   # h += mixer(x) in the mixer's own last kernel
                pending = None
            else:
                pending = torch.empty((rows, hidden), dtype=torch.float32, device=h.device)
                self.mixer.forward(batch, x, pending, cache)
        if (isinstance(pending, RowStats) and pending.prescaled_for is self.feed_forward_norm
                and self.feed_forward.folds_norm(rows, self.feed_forward_norm)):
            return self.feed_forward.forward_folded(batch, h, pending, self.feed_forward_norm, next_norm)
        if x is None:
            x = torch.empty((rows, hidden), dtype=act, device=h.device)
        self.feed_forward_norm.forward(h, x, pending if isinstance(pending, torch.Tensor) else None)
        if self.feed_forward.adds_in_place(rows):
            self.feed_forward.forward_into(batch, x, h)
            return None
        out = torch.empty((rows, hidden), dtype=torch.float32, device=h.device)
        self.feed_forward.forward(batch, x, out)
        return out
