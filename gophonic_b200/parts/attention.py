"""Grouped-query causal attention over the paged cache.

Per row: q, k, v = x Wq^T, x Wk^T, x Wv^T in one product (internal/qwen3lm/evaluator.go:648);
optional per-head RMSNorm of q and k, then the position encoding, k and v stored at the row's
position (internal/qwen3lm/ops.go:231-248; gpu.metal:1032-1055); scores (q.k) * scale over the
keys j <= i of the same sequence, within the window if there is one; streaming softmax in fp32;
out = ctx Wo^T (internal/qwen3lm/ops.go:259-293; evaluator.go:678).  Head h reads kv head
h // (heads / kv_heads).

The part knows sizes and constants only through its spec.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .. import registry
from .base import KVRequest, Mixer, RowStats, Runtime, TensorDecl, fold_weight, other_fold_buffers


def choose_splits(units: int, max_kv_len: int, sm_count: int = 148, page_bytes: int = 32768) -> int:
    """How many pieces single-token attention cuts each sequence's keys into.  ``units`` =
    (sequence, kv head) pairs, each one CTA per piece; ``page_bytes`` = keys and values of one kv
    head for one page of 64 tokens.

    The choice minimises a small model of the kernel's time that was fitted to measurements at 1
    to 64 sequences of 4096 keys: two CTAs fit on an SM and run in waves; a wave takes the longer
    of its bytes at the memory bandwidth and of one CTA's own pace (a little over a microsecond a page),
    so a thin last wave costs as much as a full one unless its CTAs are short; cutting the keys
    costs the merge kernel and the traffic of the partial results.  A piece keeps at least 256
    keys.
    """
    units = max(1, units)
    pages = max(1, (max_kv_len + 63) // 64)
    most = max(1, min(32, max_kv_len // 256))
    slots = 2 * sm_count
    bytes_per_us = 6.0e6
    page_us = 0.575 + 0.575 * page_bytes / 32768.0
    if 4 * units > 9 * slots:
        # more than two and a quarter waves uncut: the CTAs no longer run in step and a thin last
        # wave costs little (112 sequences x 8 kv heads ran 2 % faster uncut than in 4 or 8 pieces)
        return 1
    best, best_t = 1, None
    for s in range(1, most + 1):
        p = (pages + s - 1) // s
        ctas = units * s
        full, rest = divmod(ctas, slots)
        pace = p * page_us + 3.0
        t = full * max(slots * p * page_bytes / bytes_per_us, pace)
        if rest:
            t += max(rest * p * page_bytes / bytes_per_us, pace)
        if s > 1:
            # the merge kernel, and the partial results (about four heads a unit, 130 floats each)
            # written and read back
            t += 5.0 + 0.15 * s + units * s * 4 * 1040 / 3.0e6
        if best_t is None or t < 0.99 * best_t:
            best, best_t = s, t
    return best


class Attention(Mixer):
    capturable = True

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        qd, kvd = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim
        decls = [TensorDecl(prefix + "q_proj.weight", (qd, spec.hidden)),
                 TensorDecl(prefix + "k_proj.weight", (kvd, spec.hidden)),
                 TensorDecl(prefix + "v_proj.weight", (kvd, spec.hidden)),
                 TensorDecl(prefix + "o_proj.weight", (spec.hidden, qd))]
        if spec.qk_norm is not None:
            decls += [TensorDecl(prefix + "q_norm.weight", (spec.head_dim,), role="norm"),
                      TensorDecl(prefix + "k_norm.weight", (spec.head_dim,), role="norm")]
        return decls

    @classmethod
    def cache_request(cls, spec):
        return KVRequest(kv_heads=spec.kv_heads, head_dim=spec.head_dim, window=spec.window)

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"{prefix}: {spec.heads} heads are not a multiple of {spec.kv_heads} kv heads")
        self.spec = spec
        self.rt = runtime
        q, k, v = (tensors[prefix + n] for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight"))
        if not (q.dtype == k.dtype == v.dtype):
            raise ValueError(f"{prefix}: q/k/v projections are stored as {q.dtype}/{k.dtype}/{v.dtype}; they must agree")
        self.qkv = torch.cat([q, k, v], dim=0).contiguous()
        self.o = tensors[prefix + "o_proj.weight"].contiguous()
        self.q_norm = self.k_norm = None
        self.eps = 0.0
        if spec.qk_norm is not None:
            self.q_norm = tensors[prefix + "q_norm.weight"].to(torch.float32).contiguous()
            self.k_norm = tensors[prefix + "k_norm.weight"].to(torch.float32).contiguous()
            self.eps = float(spec.qk_norm.eps)
        pos_cls = registry.part_class("position", spec.position.kind)
        self.position = pos_cls(spec.position, prefix, tensors, runtime)
        self.q_dim = spec.heads * spec.head_dim
        self.kv_dim = spec.kv_heads * spec.head_dim

    def weight_bytes(self) -> int:
        return self.qkv.numel() * self.qkv.element_size() + self.o.numel() * self.o.element_size()

    def prepare(self, capacity: int) -> None:
        self.position.prepare(capacity)

    def plan(self, nseq: int, max_q_len: int, max_kv_len: int, sm_count: int):
        """Into how many pieces the keys of each sequence are cut: only single-token steps cut them
        (few sequences with long contexts would otherwise leave most SMs idle)."""
        if max_q_len != 1:
            return 1
        elem = 4 if self.rt.is_fp32 else 2
        page_bytes = 2 * 64 * self.spec.head_dim * elem     # keys and values of one kv head for one page
        return choose_splits(nseq * self.spec.kv_heads, max_kv_len, sm_count, page_bytes)

    def forward(self, batch, x: torch.Tensor, out: torch.Tensor, cache) -> None:
        self.rt.ops.gemm(self._context(batch, x, cache), self.o, out)

    def adds_in_place(self, rows: int) -> bool:
        ops = self.rt.ops
        return (self.o.dtype == torch.bfloat16 and self.rt.act_dtype == torch.bfloat16 and self.q_dim % 8 == 0 and self.spec.hidden % 4 == 0
                and ops.gemm_algo(rows, self.spec.hidden, self.q_dim) == "tc5_pair")

    def forward_into(self, batch, x: torch.Tensor, h: torch.Tensor, cache) -> None:
        self.rt.ops.gemm_add(self._context(batch, x, cache), self.o, h)

    def folds_norm(self, rows: int, norm) -> bool:
        """Steps of up to 64 rows in bfloat16: the q/k/v product applies the rows'
        norm factors from the residual's statistics and the output projection adds into the residual."""
        ops = self.rt.ops
        return (rows <= ops.FOLD_ROWS and self.rt.act_dtype == torch.bfloat16 and self.qkv.dtype == torch.bfloat16
                and self.o.dtype == torch.bfloat16 and norm.rms_fold() is not None and self.spec.hidden % 8 == 0
                and self.q_dim % 8 == 0 and self.qkv.data_ptr() % 16 == 0
                and self.o.data_ptr() % 16 == 0)

    def forward_folded(self, batch, h: torch.Tensor, stats: RowStats, norm, cache, next_norm=None) -> RowStats:
        ops = self.rt.ops
        rows = h.shape[0]
        _, eps = norm.rms_fold()
        qkv = torch.empty((rows, self.q_dim + 2 * self.kv_dim), dtype=self.rt.act_dtype, device=h.device)
        ops.gemm_scaled(stats.prescaled, eps, stats.partials, stats.count, self.qkv, qkv)
        ctx = self._attend(batch, qkv, cache)
        out_stats, out_rows = other_fold_buffers(batch, stats, self.spec.hidden)
        weight = fold_weight(next_norm, self.spec.hidden)
        count = ops.gemm_residual(ctx, self.o, h, out_stats, weight, out_rows[:rows] if weight is not None else None)
        return RowStats(out_stats, count, out_rows[:rows] if weight is not None else None, next_norm if weight is not None else None)

    def key_splits(self, batch):
        """(pieces the keys are cut into for this step, scratch for their partial results or None)."""
        s = self.spec
        splits = int(batch.plan_for(self) or 1)
        if splits <= 1:
            return 1, None
        return splits, batch.workspace(("attention key splits", s.heads, s.head_dim, splits),
                                       self.rt.ops.attention_scratch_floats(batch.nseq, s.heads, s.head_dim, splits))

    def _context(self, batch, x: torch.Tensor, cache) -> torch.Tensor:
        """Everything up to the output projection: [rows, heads * head_dim] in the activation dtype."""
        rows = x.shape[0]
        qkv = torch.empty((rows, self.q_dim + 2 * self.kv_dim), dtype=x.dtype, device=x.device)
        self.rt.ops.gemm(x, self.qkv, qkv)
        return self._attend(batch, qkv, cache)

    def _attend(self, batch, qkv: torch.Tensor, cache) -> torch.Tensor:
        """q/k norm, position encoding, cache write and attention on the rows of ``qkv``."""
        ops, s = self.rt.ops, self.spec
        rows = qkv.shape[0]
        x = qkv
        if cache is None:
            raise ValueError("attention needs a key/value cache plane")
        if cache.k.dtype != x.dtype:
            raise ValueError(f"attention: cache holds {cache.k.dtype}, activations are {x.dtype}")
        cos, sin, rot = self.position.kernel_args()
        rope_args = (s.heads, s.kv_heads, s.head_dim, self.q_norm, self.k_norm, self.eps, cos, sin, rot, batch.row_pos,
                     batch.row_seq, batch.seq_slot, cache.block_table, cache.k, cache.v, cache.writable)
        ctx = torch.empty((rows, self.q_dim), dtype=x.dtype, device=x.device)
        splits, scratch = self.key_splits(batch)
        attn_args = (cache.k, cache.v, cache.block_table, batch.seq_slot, batch.seq_q_start, batch.seq_q_len, batch.seq_kv_len,
                     batch.nseq, batch.max_q_len, s.heads, s.kv_heads, s.head_dim, float(s.scale), int(s.window), splits, scratch)
        if ops.attention_decode_rope_accepts(x.dtype, s.head_dim, rot, batch.max_q_len):
            # single tokens: the attention kernel norms and rotates its queries and places the token's key and value itself
            ops.attention_decode_rope(qkv, ctx, rope_args, attn_args)
        else:
            ops.qk_norm_rope_kv_write(qkv, *rope_args)
            ops.attention(qkv[:, :self.q_dim], ctx, *attn_args)
        return ctx
