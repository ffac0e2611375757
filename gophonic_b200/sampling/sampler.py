"""Token selection for a batch of live sequences, on the device.

Every sequence has options of its own, a seed of its own and a draw counter (the number of
tokens it has drawn so far); the token it draws is a function of its logits and these alone, so
it does not depend on which other sequences share the batch
(internal/qwen3lm/decode.go:23-32: "step i draws with Seed and Draw+i").  A presence penalty is
applied from a per-sequence bitmap of the tokens the reply already holds (qwen3/chat.go:410-437).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .options import Options


class DeviceSampler:
    def __init__(self, vocab: int, max_batch: int, device, ops=None):
        if ops is None:
            from .. import ops as _ops
            ops = _ops
        self.ops = ops
        self.vocab = vocab
        self.max_batch = max_batch
        self.device = torch.device(device)
        self.words = (vocab + 31) // 32
        self.seen = torch.zeros((max_batch, self.words), dtype=torch.int32, device=self.device)
        self._opts: List[Optional[Options]] = [None] * max_batch
        self._seed = [0] * max_batch
        self._draws = [0] * max_batch

    def start(self, row: int, options: Options, seed: int) -> None:
        """Bind batch row ``row`` (a lane of the running batch) to a new sequence."""
        self._opts[row] = options
        self._seed[row] = seed & 0xFFFFFFFFFFFFFFFF
        self._draws[row] = 0
        if options.Presence != 0:
            self.seen[row].zero_()

    def select(self, logits: torch.Tensor, rows: Sequence[int]) -> List[int]:
        """One token for each live row, on the host; ``logits[i]`` belongs to batch row ``rows[i]``."""
        return self.select_device(logits, rows).tolist()

    def select_device(self, logits: torch.Tensor, rows: Sequence[int]) -> torch.Tensor:
        """The same, left on the device as int32."""
        n = len(rows)
        opts = [self._opts[r] for r in rows]
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        any_presence = any(o.Presence != 0 for o in opts)
        rows_dev = None
        if any_presence:
            rows_dev = torch.tensor(list(rows), dtype=torch.int32, device=self.device)
            pres = torch.tensor([o.Presence for o in opts], dtype=torch.float32, device=self.device)
            self.ops.presence_penalty(logits, self.seen, rows_dev, pres)
        if all(not (o.Temperature > 0) for o in opts):
            self.ops.argmax(logits, out)
        else:
            f = np.empty((2, n), dtype=np.float32)
            k = np.empty(n, dtype=np.int32)
            s = np.empty((2, n), dtype=np.uint64)
            for i, (r, o) in enumerate(zip(rows, opts)):
                f[0, i], f[1, i], k[i] = o.Temperature, o.TopP, o.TopK
                s[0, i], s[1, i] = self._seed[r], self._draws[r]
            fd = torch.from_numpy(f).to(self.device)
            kd = torch.from_numpy(k).to(self.device)
            sd = torch.from_numpy(s.view(np.int64)).to(self.device)
            self.ops.sample(logits, fd[0], kd, fd[1], sd[0], sd[1], out)
        if any_presence:
            self.ops.mark_seen(out, self.vocab, self.seen, rows_dev)
        for r in rows:
            self._draws[r] += 1
        return out
