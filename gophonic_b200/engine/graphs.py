"""CUDA graphs of the single-token step.

A decode step launches some ten small kernels a layer; issued one by one from Python they cost
more host time than the GPU needs to run them.  The step's kernels are therefore captured once
per (batch size, key splits) into a CUDA graph and replayed: the host uploads the step's row
metadata into the graph's fixed input buffer and launches one graph.  The kernels, their order
and their arguments are those of the eager path (the reference keeps a decode run in one
submission for the same reason: internal/qwen3lm/gpu_darwin.go:1596-1622, 1910-2004), so a
replayed step gives the eager step's logits bit for bit.
"""
from __future__ import annotations

import gc
import weakref
from typing import Dict, Optional, Tuple

import torch

from .step import StepBatch, choose_splits


class DecodeGraph:
    def __init__(self, engine, nseq: int, splits: int, pool):
        # the engine owns its graphs; a strong reference back would make a cycle, and an engine
        # dropped by its user would then be freed by the collector at some later time, perhaps in
        # the middle of another engine's capture, where freeing device memory is an error
        self._engine = weakref.ref(engine)
        self.nseq = nseq
        dev = engine.device
        # ids | row_pos | row_seq | seq_slot | q_start | q_len | kv_len | want rows
        self.meta = torch.zeros(8 * nseq, dtype=torch.int32, device=dev)
        n = nseq
        m = self.meta
        self.batch = StepBatch(rows=n, nseq=n, max_q_len=1, max_kv_len=0, ids=m[:n], row_pos=m[n:2 * n],
                               row_seq=m[2 * n:3 * n], seq_slot=m[3 * n:4 * n], seq_q_start=m[4 * n:5 * n],
                               seq_q_len=m[5 * n:6 * n], seq_kv_len=m[6 * n:7 * n], device=dev,
                               sm_count=engine.sm_count, fixed_splits=splits)
        self.want = m[7 * n:8 * n]
        self.logits: Optional[torch.Tensor] = None
        self.graph = torch.cuda.CUDAGraph()
        self.pool = pool
        self.kernels = 0

    @property
    def engine(self):
        return self._engine()

    def capture(self) -> None:
        eng = self.engine
        ops = eng.model.rt.ops
        # one eager run first: kernels configure themselves (shared-memory limits) outside capture
        eng.model.forward(self.batch, eng.cache, self.want)
        torch.cuda.synchronize()
        before = ops.launches
        # Nothing may be freed on the device while the stream captures: collect what is garbage
        # now, and keep the collector from running until the capture has ended.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph, pool=self.pool):
                self.logits = eng.model.forward(self.batch, eng.cache, self.want)
        finally:
            if collecting:
                gc.enable()
        self.kernels = ops.launches - before
        ops.launches = before  # captured, not run

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        self.engine.model.rt.ops.launches += self.kernels
        return self.logits


class DecodeGraphs:
    def __init__(self, engine, max_batch: int = 64):
        self._engine = weakref.ref(engine)
        self.max_batch = max_batch
        self.graphs: Dict[Tuple[int, int], DecodeGraph] = {}
        self.pool = None

    @property
    def engine(self):
        return self._engine()

    def get(self, nseq: int, max_kv_len: int, kv_heads_hint: int, page_bytes_hint: int = 32768) -> DecodeGraph:
        splits = choose_splits(nseq * kv_heads_hint, max_kv_len, self.engine.sm_count, page_bytes_hint)
        key = (nseq, splits)
        g = self.graphs.get(key)
        if g is None:
            if self.pool is None:
                self.pool = torch.cuda.graph_pool_handle()
            g = DecodeGraph(self.engine, nseq, splits, self.pool)
            self.graphs[key] = g
        return g
