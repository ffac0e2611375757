"""CUDA graphs of the single-token step.

A decode step launches some ten small kernels a layer; issued one by one from Python they cost
more host time than the GPU needs to run them.  The step's kernels are therefore captured once
per (batch size, launch plans of the mixers) into a CUDA graph and replayed: the host uploads the step's row
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

from .step import StepBatch


class DecodeGraph:
    def __init__(self, engine, nseq: int, plans, pool):
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
                               sm_count=engine.sm_count, plans=engine.model.bind_plans(plans))
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


def captured_size(nseq: int) -> int:
    """The batch size a step of ``nseq`` sequences is captured and replayed at: itself up to 8, then
    the next of 12, 16, 24, 32, 48, 64, 96, 128, ... (filler rows cost a decode step next to nothing:
    its products read the same weights and run on the same kernels within such a range)."""
    if nseq <= 8:
        return nseq
    size = 8
    while True:
        for cand in (size + size // 2, 2 * size):
            if nseq <= cand:
                return cand
        size *= 2


class DecodeGraphs:
    def __init__(self, engine, max_batch: int = 64, max_graphs: int = 48):
        self._engine = weakref.ref(engine)
        self.max_batch = max_batch
        self.max_graphs = max_graphs
        self.graphs: Dict[Tuple[int, Tuple], DecodeGraph] = {}   # in order of last use
        self.pool = None

    @property
    def engine(self):
        return self._engine()

    def get(self, nseq: int, max_kv_len: int) -> DecodeGraph:
        """The captured step that serves ``nseq`` sequences which see at most ``max_kv_len`` keys: one
        graph per captured batch size and per answer of the model's mixers to ``plan`` (whatever
        those answers are).  At most ``max_graphs`` graphs are kept; the one unused longest goes."""
        eng = self.engine
        size = min(captured_size(nseq), max(self.max_batch, nseq))
        plans = eng.model.step_plans(size, 1, max_kv_len, eng.sm_count)
        key = (size, plans)
        g = self.graphs.pop(key, None)
        if g is None:
            if self.pool is None:
                self.pool = torch.cuda.graph_pool_handle()
            while len(self.graphs) >= self.max_graphs:
                self.graphs.pop(next(iter(self.graphs)))
            g = DecodeGraph(eng, size, plans, self.pool)
        self.graphs[key] = g
        return g
