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
    """Options, seeds and draw counters live on the device, one entry per batch row; ``start``
    changes a row's entries on the host and the next selection uploads the changed table once.
    The kernel advances the draw counters itself, so a decode step uploads nothing."""

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
        # host mirror of the per-row table: temperature, top_p, presence | top_k | seed, draws
        self._f = np.zeros((3, max_batch), dtype=np.float32)
        self._k = np.zeros(max_batch, dtype=np.int32)
        self._s = np.zeros((2, max_batch), dtype=np.uint64)
        self._f_dev = torch.zeros((3, max_batch), dtype=torch.float32, device=self.device)
        self._k_dev = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self._s_dev = torch.zeros((2, max_batch), dtype=torch.int64, device=self.device)
        self._dirty = False
        self._rows_dev = {}
        nbytes = ops.sample_scratch_bytes(max_batch, vocab)
        self._scratch = torch.zeros(nbytes, dtype=torch.uint8, device=self.device) if nbytes else None

    def start(self, row: int, options: Options, seed: int) -> None:
        """Bind batch row ``row`` (a lane of the running batch) to a new sequence."""
        if self._dirty is False and any(o is not None for o in self._opts):
            # the device holds the draw counters of the rows that are running: bring them back
            # before the table is written again
            self._s[1] = self._s_dev[1].cpu().numpy().view(np.uint64)
        self._opts[row] = options
        self._f[0, row], self._f[1, row], self._f[2, row] = options.Temperature, options.TopP, options.Presence
        self._k[row] = options.TopK
        self._s[0, row] = seed & 0xFFFFFFFFFFFFFFFF
        self._s[1, row] = 0
        self._dirty = True
        if options.Presence != 0:
            self.seen[row].zero_()

    def draws(self, row: int) -> int:
        """How many tokens batch row ``row`` has drawn (reads the device)."""
        if self._dirty:
            return int(self._s[1, row])
        return int(self._s_dev[1, row].item())

    def _sync_table(self) -> None:
        if self._dirty:
            self._f_dev.copy_(torch.from_numpy(self._f))
            self._k_dev.copy_(torch.from_numpy(self._k))
            self._s_dev.copy_(torch.from_numpy(self._s.view(np.int64)))
            self._dirty = False

    def _rows(self, rows: Sequence[int]) -> torch.Tensor:
        key = tuple(rows)
        t = self._rows_dev.get(key)
        if t is None:
            if len(self._rows_dev) > 256:
                self._rows_dev.clear()
            t = torch.tensor(list(rows), dtype=torch.int32, device=self.device)
            self._rows_dev[key] = t
        return t

    def select(self, logits: torch.Tensor, rows: Sequence[int]) -> List[int]:
        """One token for each live row, on the host; ``logits[i]`` belongs to batch row ``rows[i]``."""
        return self.select_device(logits, rows).tolist()

    def select_device(self, logits: torch.Tensor, rows: Sequence[int]) -> torch.Tensor:
        """The same, left on the device as int32."""
        n = len(rows)
        opts = [self._opts[r] for r in rows]
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        any_presence = any(o.Presence != 0 for o in opts)
        greedy = all(not (o.Temperature > 0) for o in opts)
        if greedy and not any_presence:
            self.ops.argmax(logits, out)
            return out
        self._sync_table()
        rows_dev = self._rows(rows)
        if any_presence:
            self.ops.presence_penalty(logits, self.seen, rows_dev, self._f_dev[2], indexed=True)
        if greedy:
            self.ops.argmax(logits, out)
        else:
            self.ops.sample(logits, self._f_dev[0], self._k_dev, self._f_dev[1], self._s_dev[0], self._s_dev[1], out,
                            opt_row=rows_dev, advance=True, scratch=self._scratch)
        if any_presence:
            self.ops.mark_seen(out, self.vocab, self.seen, rows_dev)
        return out
