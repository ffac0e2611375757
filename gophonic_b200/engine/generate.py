"""The generation loop above the step function.

Requests are served in batches.  A batch starts together: every prompt of the batch goes
through one step; after that each live sequence goes on by one token a step.  A sequence ends
when it draws a stop token (which is not part of its reply: qwen3/chat.go:340-341) or has
produced its MaxTokens (qwen3/chat.go:305-312, 343); it leaves the batch at once and its slot
and pages go back to the cache, while the others go on (qwen3asr/batch.go:178-249 keeps the same
alive/finished bookkeeping for its lanes).  No request joins a running batch; when the batch is
empty the next one starts, reusing the slots, until no request is left.

The loop decides; it computes nothing.  It talks to an *engine* (``new_sequence``, ``step``,
``end_sequence``, ``room``) and a *sampler* (``start``, ``select``), so its decisions are tested
without a GPU.

If the engine can take a step's tokens from where the sampler left them (``step_from``,
``fetch_tokens``) and the sampler can leave them there (``select_device``), the loop runs one step
ahead of what it has read: step k + 1 is enqueued for every sequence that step k cannot end by
length, then the tokens of step k are read and handled while step k + 1 runs.  A sequence that
drew a stop token in step k has then run one step for nothing; its result is dropped.  Replies,
callbacks and their order are the same as without the overlap.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Iterable, List, Optional, Sequence, Tuple

from ..sampling.options import Options


@dataclass
class Request:
    index: int
    prompt: List[int]
    options: Options
    budget: int                      # most tokens this reply may have
    seed: int
    reply: List[int] = field(default_factory=list)
    slot: Optional[int] = None       # given by the caller (with ``keep_slot``) or taken by the loop
    row: Optional[int] = None        # lane of the running batch (the sampler's row)
    finished: Optional[str] = None   # "stop" | "length"
    # A request that continues a sequence its caller owns (a chat session's slot): ``prompt`` holds
    # only the tokens the cache does not hold yet, and the slot is not given back at the end.
    keep_slot: bool = False
    # every token the loop fed to the engine after the prompt, in order: with ``prompt`` what the
    # slot holds more than before (a stop token that a step ran ahead of is among them)
    fed: List[int] = field(default_factory=list)


@dataclass
class GenerationStats:
    batches: int = 0
    prefill_tokens: int = 0
    decode_steps: int = 0
    decoded_tokens: int = 0


class GenerationError(ValueError):
    pass


class Generator:
    def __init__(self, engine, sampler, max_batch: int, context: int, stop_ids: Iterable[int] = (),
                 page: int = 64):
        """``context``: most tokens one sequence may hold (prompt + reply)."""
        if max_batch <= 0:
            raise GenerationError(f"max_batch {max_batch}")
        self.engine = engine
        self.sampler = sampler
        self.max_batch = max_batch
        self.context = context
        self.stop_ids = frozenset(int(s) for s in stop_ids)
        self.page = page
        self.stats = GenerationStats()
        # an engine that can lend its captured step's own output buffer is asked to: every step's
        # logits are consumed by the sampler before the next step is issued
        self._lend = {"borrow": True} if getattr(engine, "lends_logits", False) else {}

    # ---- planning ------------------------------------------------------------------------
    def _budget(self, prompt_len: int, options: Options) -> int:
        """Room for the reply: the context left, bounded by MaxTokens (qwen3/chat.go:305-312)."""
        room = self.context - prompt_len
        if options.MaxTokens > 0:
            room = min(room, options.MaxTokens)
        return room

    def _pages(self, r: Request) -> int:
        # the last drawn token is never fed back, so a sequence holds at most prompt + budget - 1
        held = len(r.prompt) + max(r.budget - 1, 0)
        return (held + self.page - 1) // self.page

    def plan_batch(self, pending: Sequence[Request], free_pages: int) -> int:
        """How many of the pending requests, in order, start together: at most ``max_batch``, and
        only as many as can grow to their full length in the pages that are free."""
        n, used = 0, 0
        for r in pending[:self.max_batch]:
            need = self._pages(r)
            if used + need > free_pages:
                break
            used += need
            n += 1
        if n == 0 and pending:
            raise GenerationError(f"request {pending[0].index} needs {self._pages(pending[0])} pages of "
                                  f"{self.page} tokens and the cache has {free_pages} free")
        return n

    # ---- the loop ------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], options=None,
                 on_token: Optional[Callable[[int, int], None]] = None) -> List[List[int]]:
        """Replies (token ids) for ``prompts``, in order.  ``options``: one ``Options`` for all, or
        one per prompt.  Request i draws with seed ``Options.Seed + i``.  ``on_token(i, token)`` is
        called for every token of request i as it is drawn."""
        if options is None:
            options = Options()
        opts = list(options) if isinstance(options, (list, tuple)) else [options] * len(prompts)
        if len(opts) != len(prompts):
            raise GenerationError(f"{len(opts)} option sets for {len(prompts)} prompts")
        pending: List[Request] = []
        for i, (p, o) in enumerate(zip(prompts, opts)):
            o.validate()
            p = [int(t) for t in p]
            if not p:
                raise GenerationError(f"request {i}: empty prompt")
            budget = self._budget(len(p), o)
            if budget <= 0:
                raise GenerationError(f"request {i}: a prompt of {len(p)} tokens fills the context of {self.context}")
            pending.append(Request(i, p, o, budget, (o.Seed + i) & 0xFFFFFFFFFFFFFFFF))
        results: List[List[int]] = [[] for _ in prompts]
        while pending:
            n = self.plan_batch(pending, self.engine.room())
            batch, pending = pending[:n], pending[n:]
            self._run_batch(batch, on_token)
            for r in batch:
                results[r.index] = r.reply
        return results

    def run(self, batch: List[Request], on_token=None) -> None:
        """Run requests the caller made itself as one batch that starts together: each request's
        ``prompt`` in one step, then one token each, until every request has finished.  A request
        with ``keep_slot`` continues the sequence in its ``slot`` and keeps it afterwards."""
        if not batch or len(batch) > self.max_batch:
            raise GenerationError(f"a batch of {len(batch)} requests (at most {self.max_batch})")
        self._run_batch(batch, on_token)

    def _run_batch(self, batch: List[Request], on_token) -> None:
        if all(hasattr(self.engine, a) for a in ("step_from", "fetch_tokens")) and hasattr(self.sampler, "select_device"):
            return self._run_batch_ahead(batch, on_token)
        self.stats.batches += 1
        live: List[Request] = []
        try:
            for row, r in enumerate(batch):
                self._begin(r, row)
                live.append(r)
            # all prompts in one step
            logits = self.engine.step([(r.slot, r.prompt) for r in live], **self._lend)
            self.stats.prefill_tokens += sum(len(r.prompt) for r in live)
            while True:
                tokens = self.sampler.select(logits, [r.row for r in live])
                still: List[Request] = []
                for r, t in zip(live, tokens):
                    self._take(r, int(t), on_token)
                    if r.finished is None:
                        still.append(r)
                    else:
                        self._release(r)
                live = still
                if not live:
                    break
                # one token each
                logits = self.engine.step([(r.slot, [r.reply[-1]]) for r in live], **self._lend)
                for r in live:
                    r.fed.append(r.reply[-1])
                self.stats.decode_steps += 1
                self.stats.decoded_tokens += len(live)
        finally:
            for r in batch:
                self._release(r)

    def _run_batch_ahead(self, batch: List[Request], on_token) -> None:
        """The same batch with the next step enqueued before the last one's tokens are read."""
        self.stats.batches += 1
        try:
            live: List[Request] = []
            for row, r in enumerate(batch):
                self._begin(r, row)
                live.append(r)
            logits = self.engine.step([(r.slot, r.prompt) for r in live], **self._lend)
            self.stats.prefill_tokens += sum(len(r.prompt) for r in live)
            drawn = self.sampler.select_device(logits, [r.row for r in live])   # tokens of `live`, on the device
            fetch = self.engine.fetch_tokens(drawn)
            while True:
                # `drawn` holds the unread tokens of `live`, in order (entries of sequences that ended a
                # step ago are there too and are skipped).  Who goes on if nobody draws a stop token:
                # everyone whose reply the unread token does not fill.
                ahead = [(i, r) for i, r in enumerate(live) if r.finished is None and len(r.reply) + 1 < r.budget]
                nxt = None
                if ahead:
                    logits = self.engine.step_from([r.slot for _, r in ahead], drawn, [i for i, _ in ahead], **self._lend)
                    nxt_drawn = self.sampler.select_device(logits, [r.row for _, r in ahead])
                    nxt = ([r for _, r in ahead], nxt_drawn, self.engine.fetch_tokens(nxt_drawn))
                # read and handle the tokens of the step before while the one just enqueued runs
                going = 0
                fed_ahead = {id(r) for _, r in ahead}
                for r, t in zip(live, fetch.wait()):
                    if r.finished is not None:
                        continue  # it drew a stop token a step ago: this entry ran for nothing
                    if id(r) in fed_ahead:
                        r.fed.append(int(t))   # the step just enqueued stores it, whatever it turns out to be
                    self._take(r, int(t), on_token)
                    if r.finished is None:
                        going += 1
                    else:
                        self._release(r)
                if nxt is None:
                    break
                live, drawn, fetch = nxt
                if going == 0:
                    fetch.wait()  # every sequence of the enqueued step has ended: its tokens are dropped
                    break
                self.stats.decode_steps += 1
                self.stats.decoded_tokens += going
        finally:
            for r in batch:
                self._release(r)

    def _begin(self, r: Request, row: int) -> None:
        if not r.keep_slot:
            r.slot = self.engine.new_sequence()
        elif r.slot is None:
            raise GenerationError(f"request {r.index} keeps its slot and has none")
        r.row = row
        self.sampler.start(row, r.options, r.seed)

    def _release(self, r: Request) -> None:
        """Give the sequence's slot and pages back, unless its caller owns them."""
        if r.slot is not None and not r.keep_slot:
            self.engine.end_sequence(r.slot)
            r.slot = None

    def _take(self, r: Request, token: int, on_token) -> None:
        if token in self.stop_ids:
            r.finished = "stop"
            return
        r.reply.append(token)
        if on_token is not None:
            on_token(r.index, token)
        if len(r.reply) >= r.budget:
            r.finished = "length"
