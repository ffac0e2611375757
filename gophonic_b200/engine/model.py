"""A decoder assembled from a ``ModelSpec``: embedding, blocks run in schedule order, final norm,
head.  The class knows no architecture: everything it runs was chosen by the spec through the
part registries.

Forward pass of one step, as the reference orders it (internal/qwen3lm/evaluator.go:594-599 embed,
638-683 layers, 685-709 final add + norm, 357-381 head): rows are packed (no padding), the
residual is fp32, and only the rows whose logits are wanted reach the final norm and the head
(evaluator.go:669-677 prunes to the wanted rows the same way).
"""
from __future__ import annotations

import inspect
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from .. import registry
from ..cache import Cache
from ..parts.base import RowStats, Runtime, fold_buffers, fold_weight
from ..weights import InitScales, declare_model, load_tensors, random_tensors_on_device

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def dtype_mode(name) -> str:
    if isinstance(name, torch.dtype):
        name = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(name, str(name))
    if name not in _DTYPES:
        raise ValueError(f"dtype '{name}' is not one of bfloat16, float32")
    return "bfloat16" if _DTYPES[name] == torch.bfloat16 else "float32"


def make_runtime(mode: str, device) -> Runtime:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(f"the engine runs on CUDA devices only (asked for '{device}'); there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; the engine has no CPU path")
    from .. import ops  # builds / loads the kernel library, or raises
    ops.use_device(device.index if device.index is not None else torch.cuda.current_device())
    return Runtime(device=device, act_dtype=_DTYPES[mode], ops=ops)


class Model:
    def __init__(self, spec, tensors: Mapping[str, torch.Tensor], runtime: Runtime, config=None):
        from .. import parts  # noqa: F401  (registers the built-in parts)
        spec.validate()
        self.spec = spec
        self.config = config
        self.rt = runtime
        self.embedding = tensors[spec.embedding.name]
        self.blocks = [registry.part_class("block", layer.block)(layer, layer.prefix, tensors, runtime)
                       for layer in spec.layers]
        # a block arrangement may take the norm that follows it (to prepare the residual's rows for it)
        self._takes_next_norm = ["next_norm" in inspect.signature(b.forward).parameters for b in self.blocks]
        norm_prefix = spec.final_norm_name[:-len("weight")]
        self.final_norm = registry.part_class("norm", spec.final_norm.kind)(spec.final_norm, norm_prefix, tensors, runtime)
        if spec.head.name in tensors:
            self.head = tensors[spec.head.name]
            self.tied = False
        elif spec.head.tied_to is not None and spec.head.tied_to in tensors:
            self.head = tensors[spec.head.tied_to]  # the same storage, no second copy
            self.tied = True
        else:
            raise ValueError(f"no head tensor '{spec.head.name}' and nothing to tie it to")
        if tuple(self.head.shape) != (spec.head.vocab, spec.head.hidden):
            raise ValueError(f"head has shape {tuple(self.head.shape)}, want {(spec.head.vocab, spec.head.hidden)}")

    # ---- construction --------------------------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir: str, dtype="bfloat16", device="cuda:0") -> "Model":
        mode = dtype_mode(dtype)
        config = registry.read_config(model_dir)
        spec = config.model_spec()
        rt = make_runtime(mode, device)
        tensors = load_tensors(model_dir, declare_model(spec), mode, rt.device)
        return cls(spec, tensors, rt, config)

    @classmethod
    def from_random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0",
                    scales: InitScales = InitScales()) -> "Model":
        """Random weights made on the device (for sizes too large to pass through a file): the tensors
        ``write_random_model`` writes for the same configuration and seed, bit for bit."""
        mode = dtype_mode(dtype)
        spec = config.model_spec()
        rt = make_runtime(mode, device)
        tied = bool(getattr(config, "tie_word_embeddings", False))
        tensors = random_tensors_on_device(spec, seed, mode, rt.device, scales, tied=tied, ops=rt.ops)
        return cls(spec, tensors, rt, config)

    # ---- description ---------------------------------------------------------------------
    def cache_requests(self) -> List[Tuple[object, Optional[int]]]:
        out = []
        for entry in self.spec.schedule:
            layer = self.spec.layers[entry.layer]
            out.append((registry.part_class("block", layer.block).cache_request(layer), entry.cache_of))
        return out

    def step_plans(self, nseq: int, max_q_len: int, max_kv_len: int, sm_count: int) -> Tuple:
        """The launch plans of every mixer for a step of this shape, block by block: a hashable value
        the engine keys its captured steps on without looking inside."""
        return tuple(m.plan(nseq, max_q_len, max_kv_len, sm_count) for b in self.blocks for m in b.mixers())

    def bind_plans(self, plans: Sequence) -> Dict[int, object]:
        """``step_plans``' answer in the form ``StepBatch.plans`` takes: by mixer."""
        mixers = [m for b in self.blocks for m in b.mixers()]
        return {id(m): p for m, p in zip(mixers, plans)}

    def new_cache(self, max_tokens: int, max_slots: Optional[int] = None,
                  max_seq_tokens: Optional[int] = None) -> Cache:
        limit = int(self.spec.max_positions)
        max_seq_tokens = limit if max_seq_tokens is None else min(limit, int(max_seq_tokens))
        cache = Cache(self.cache_requests(), max_tokens, self.rt.device, self.rt.act_dtype, max_slots, max_seq_tokens)
        capacity = cache.max_pages_per_seq * 64
        for b in self.blocks:
            b.prepare(capacity)
        return cache

    @property
    def capturable(self) -> bool:
        """Whether every part only enqueues stream work, so a step can be captured in a CUDA graph."""
        return all(b.capturable for b in self.blocks) and self.final_norm.capturable

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a step reads once: every layer run's matrices and the head."""
        total = self.head.numel() * self.head.element_size()
        for entry in self.spec.schedule:
            total += self.blocks[entry.layer].weight_bytes()
        return total

    # ---- forward -------------------------------------------------------------------------
    def forward(self, batch, cache: Cache, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the rows of ``batch`` through every scheduled layer; return fp32 logits
        [len(want_rows), vocab] for the wanted packed rows (None if none are wanted)."""
        ops = self.rt.ops
        rows = batch.rows
        h = torch.empty((rows, self.spec.hidden), dtype=torch.float32, device=self.rt.device)
        # What is still owed to the residual travels from block to block: an addend not yet added, the
        # rows' statistics (``RowStats``) where the last kernel left them, or nothing.
        pending = None
        schedule = self.spec.schedule
        first = self.blocks[schedule[0].layer]
        weight = None
        # Single-token steps, which are replayed from graphs, fold their norms into the products around
        # them.  A short prompt is issued live, where a layer from one call into the library (two norm
        # kernels included) takes the host less time than the folded path's calls part by part take it
        # (8B sizes, 16 / 64 rows: 133 / 147 us a layer against 185 / 161).
        if batch.max_q_len == 1 and rows <= ops.FOLD_ROWS and hasattr(first, "wants_stats") and first.wants_stats(rows):
            weight = fold_weight(first.first_norm(), self.spec.hidden)
        if weight is not None:
            stats, prescaled = fold_buffers(batch, 0, self.spec.hidden)
            ops.embed_gather(self.embedding, batch.ids, h, stats, weight, prescaled[:rows])
            pending = RowStats(stats, 1, prescaled[:rows], first.first_norm())
        else:
            ops.embed_gather(self.embedding, batch.ids, h)
        for pos, entry in enumerate(schedule):
            block = self.blocks[entry.layer]
            if self._takes_next_norm[entry.layer]:
                after = self.blocks[schedule[pos + 1].layer] if pos + 1 < len(schedule) else None
                next_norm = self.final_norm if after is None else (after.first_norm() if hasattr(after, "first_norm") else None)
                pending = block.forward(batch, h, pending, cache.view(pos), next_norm=next_norm)
            else:
                pending = block.forward(batch, h, pending, cache.view(pos))
        delta = pending if isinstance(pending, torch.Tensor) else None
        if want_rows is None or want_rows.numel() == 0:
            return None
        n = want_rows.numel()
        x = torch.empty((n, self.spec.hidden), dtype=self.rt.act_dtype, device=self.rt.device)
        self.final_norm.forward(h, x, delta, rows=want_rows)
        logits = torch.empty((n, self.spec.vocab), dtype=torch.float32, device=self.rt.device)
        ops.gemm(x, self.head, logits)
        return logits
