"""Lane "chat.Generator": conversations whose context stays evaluated between replies.

A ``ChatGenerator`` holds a loaded model; each ``Session`` is one conversation and owns one cache
slot for as long as it lives, so a new message costs only its own tokens (chat/chat.go:1-10, 69-123).
The session keeps two token lists: ``ids``, the conversation as it stands, and ``held``, the
tokens whose keys and values the slot holds.  ``Reply`` compares the two, keeps their common
prefix in the cache (``Engine.truncate``), runs what is missing in one step and then decodes one
token at a time (qwen3/chat.go:293-381: ``keep := min(kv.CommonPrefix(ids), len(ids)-1)``, then
``HiddenLastExtendInto(kv, keep, ids[keep:])``).  ``Truncate``, ``Checkpoint`` and ``Restore``
only shorten ``ids`` (qwen3/chat.go:720-757); what the cache still holds beyond is cut at the
next evaluation.

Messages are framed by a ``Template`` of token ids: a header per role, the tokens that end a
message, the tokens that open the assistant's reply, and the ids that end it
(qwen3/chat.go:102-108 builds the same from its tokenizer: ``<|im_start|>user\\n`` ... ``<|im_end|>\\n``).
With a tokenizer (``gophonic_b200.tokenizer``) the template is made from the Qwen3 strings and
messages may be text; without one (a folder that has no tokenizer.json) messages are token ids and
the template is empty unless the caller gives one.  Tool calls, ``Finished`` and speculative
drafting are not part of this lane.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Union

from .engine.generate import GenerationError, Generator, Request
from .sampling.options import Options as ChatOptions

ChatLane = "chat.Generator"

# chat/chat.go:21-31
System, User, Assistant, ToolResult = 0, 1, 2, 3
_ROLES = (System, User, Assistant, ToolResult)


class ErrClosed(RuntimeError):
    """The session or its generator was closed (chat/chat.go ErrClosed)."""


@dataclass
class Template:
    """Token ids that frame the messages of a conversation."""
    header: Dict[int, List[int]] = field(default_factory=dict)   # role -> tokens before the message
    end: List[int] = field(default_factory=list)                 # after every message (<|im_end|>, newline)
    result_end: List[int] = field(default_factory=list)          # between a tool result and ``end``
    answer: List[int] = field(default_factory=list)              # opens the assistant's reply
    stop: List[int] = field(default_factory=list)                # ids that end a reply (not part of it)

    @classmethod
    def qwen3(cls, tokenizer, thinking_block: bool = True) -> "Template":
        """The Qwen3 chat frame from its strings (qwen3/chat.go:86-108, 141-146): a non-thinking
        reply opens with an empty thinking block where the model's template has one."""
        im_end, end_text = tokenizer.added_id("<|im_end|>"), tokenizer.added_id("<|endoftext|>")
        if im_end is None or end_text is None:
            raise ValueError("the tokenizer lacks <|im_end|> or <|endoftext|>")
        enc = tokenizer.encode
        answer = "<|im_start|>assistant\n" + ("<think>\n\n</think>\n\n" if thinking_block else "")
        return cls(header={System: enc("<|im_start|>system\n"), User: enc("<|im_start|>user\n"),
                           Assistant: enc("<|im_start|>assistant\n"),
                           ToolResult: enc("<|im_start|>user\n<tool_response>\n")},
                   end=[im_end] + enc("\n"), result_end=enc("\n</tool_response>"), answer=enc(answer),
                   stop=[im_end, end_text])


def common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
    """Length of the longest common prefix (internal/qwen3lm/evaluator.go:218-226)."""
    n = min(len(a), len(b))
    for i in range(n):
        if a[i] != b[i]:
            return i
    return n


@dataclass
class ReplyStats:
    kept: int = 0             # tokens of the conversation the cache already held
    prefill_tokens: int = 0   # tokens evaluated before the first token of the reply was drawn
    decoded_tokens: int = 0


class ChatGenerator:
    """A loaded model that holds conversations.  Sessions share the engine, the sampler and the
    cache; one reply runs at a time (qwen3/chat.go:296-301 takes the generator's lock likewise)."""

    def __init__(self, engine, sampler, context: int, template: Optional[Template] = None, tokenizer=None,
                 on_close: Optional[Callable[[], None]] = None):
        self.engine = engine
        self.sampler = sampler
        self.context = context
        self.tokenizer = tokenizer
        self.template = template if template is not None else Template()
        self._loop = Generator(engine, sampler, 1, context, self.template.stop)
        self._lock = threading.Lock()
        self._sessions: List["Session"] = []
        self._on_close = on_close
        self.closed = False

    def NewSession(self, system: Union[None, str, Sequence[int]] = None) -> "Session":
        """Start a conversation, with ``system`` as its system message when not empty."""
        if self.closed:
            raise ErrClosed("the generator is closed")
        s = Session(self)
        self._sessions.append(s)
        if system is not None and len(system) > 0:
            s.Add(System, system)
        return s

    def Close(self) -> None:
        for s in list(self._sessions):
            s.Close()
        self.closed = True
        if self._on_close is not None:
            self._on_close()
            self._on_close = None


class Session:
    """One conversation.  Not safe for concurrent use; sessions of one generator may be used from
    different threads and share its model."""

    def __init__(self, generator: ChatGenerator):
        self.g = generator
        self.ids: List[int] = []        # the conversation's tokens
        self.held: List[int] = []       # the tokens whose keys and values the slot holds
        self.slot: Optional[int] = None
        self.reply_at = -1              # where the last reply's tokens start in ids, or -1
        self.reply_len = 0
        self.closed = False
        self.stats = ReplyStats()

    # ---- building the conversation ---------------------------------------------------------
    def _tokens(self, content: Union[str, Sequence[int]]) -> List[int]:
        if isinstance(content, str):
            if self.g.tokenizer is None:
                raise ValueError("this model has no tokenizer: messages are lists of token ids")
            return self.g.tokenizer.encode(content)
        toks = [int(t) for t in content]
        vocab = self.g.engine.vocab
        for t in toks:
            if not 0 <= t < vocab:
                raise ValueError(f"token id {t} is outside [0, {vocab})")
        return toks

    def Add(self, role: int, content: Union[str, Sequence[int]]) -> None:
        """Append a complete message without replying."""
        self._open()
        if role not in _ROLES:
            raise ValueError(f"unknown role {role}")
        t = self.g.template
        body = self._tokens(content)
        self.ids += t.header.get(role, []) + body
        if role == ToolResult:
            self.ids += t.result_end
        self.ids += t.end
        self.reply_at = -1

    def Checkpoint(self) -> int:
        """A mark of the conversation as it is."""
        return len(self.ids)

    def Restore(self, mark: int) -> None:
        """Back to a mark: everything added since is forgotten; what stays evaluated is reused."""
        self._open()
        if not 0 <= mark <= len(self.ids):
            raise ValueError(f"mark {mark} outside the conversation's {len(self.ids)} tokens")
        del self.ids[mark:]
        self.reply_at = -1

    def Truncate(self, n: int) -> None:
        """Shorten the last reply to its first ``n`` tokens, as when only part of it was heard (the
        reference counts bytes of text and rounds down to a token: qwen3/chat.go:720-741; with a
        tokenizer ``n`` counts bytes here too)."""
        self._open()
        if self.reply_at < 0:
            raise ValueError("no reply to truncate")
        if n < 0:
            raise ValueError(f"cannot keep {n} of a reply")
        keep = min(n, self.reply_len)
        if self.g.tokenizer is not None:
            keep, size = 0, 0
            while keep < self.reply_len:
                size += len(self.g.tokenizer.piece(self.ids[self.reply_at + keep]))
                if size > n:
                    break
                keep += 1
        del self.ids[self.reply_at + keep:]
        self.ids += self.g.template.end
        self.reply_len = keep

    # ---- evaluating ------------------------------------------------------------------------
    def _sync_cache(self, upto: int) -> int:
        """Cut the slot back to what it shares with ``ids[:upto]``; return how many tokens stay."""
        eng = self.g.engine
        if self.slot is None:
            self.slot = eng.new_sequence()
            self.held = []
        keep = min(common_prefix(self.held, self.ids[:upto]), upto)
        if keep < len(self.held):
            eng.truncate(self.slot, keep)
            del self.held[keep:]
        return keep

    def Prefill(self) -> None:
        """Evaluate the conversation as it stands, so that the next Reply starts at once."""
        self._open()
        with self.g._lock:
            keep = self._sync_cache(len(self.ids))
            if keep < len(self.ids):
                self.g.engine.step([(self.slot, self.ids[keep:])], [[]])
                self.held = list(self.ids)

    def Reply(self, options: Optional[ChatOptions] = None, on_token: Optional[Callable[[int], None]] = None,
              writer=None) -> List[int]:
        """Generate the assistant's next message; returns its token ids.  ``on_token(id)`` is called
        for each token as it is drawn; ``writer.write(text)`` receives the decoded pieces when the
        model has a tokenizer.  The message ends when the model ends it (a stop id of the template,
        not part of the reply), after ``MaxTokens`` tokens, or when the context is full; what was
        generated by then stays in the conversation as a complete message."""
        self._open()
        options = options or ChatOptions()
        options.validate()
        g, t = self.g, self.g.template
        with g._lock:
            if g.closed:
                raise ErrClosed("the generator is closed")
            mark = len(self.ids)
            self.ids += t.answer
            start = len(self.ids)
            room = g.context - start - len(t.end)
            if options.MaxTokens > 0:
                room = min(room, options.MaxTokens)
            if room <= 0 or start == 0:
                del self.ids[mark:]
                if start == 0:
                    raise GenerationError("the conversation is empty")
                raise GenerationError("the conversation fills the context")
            # the last token is always evaluated anew: its logits start the reply
            keep = self._sync_cache(start - 1)
            decoder = _PieceDecoder(g.tokenizer, writer) if (writer is not None and g.tokenizer is not None) else None

            def emit(_index: int, token: int) -> None:
                if on_token is not None:
                    on_token(token)
                if decoder is not None:
                    decoder.take(token)
            r = Request(0, self.ids[keep:], options, room, options.Seed & 0xFFFFFFFFFFFFFFFF, slot=self.slot, keep_slot=True)
            try:
                g._loop.run([r], emit)
            except BaseException:
                # what the slot holds is no longer known: start it over at the next evaluation
                g.engine.truncate(self.slot, 0)
                self.held = []
                del self.ids[mark:]
                raise
            g.engine.check_kernels()
            self.held = self.ids[:keep] + r.prompt + r.fed
            self.ids += r.reply
            self.reply_at, self.reply_len = start, len(r.reply)
            self.ids += t.end
            if decoder is not None:
                decoder.flush()
            self.stats = ReplyStats(kept=keep, prefill_tokens=len(r.prompt), decoded_tokens=len(r.reply))
            return list(r.reply)

    # ---- ending ----------------------------------------------------------------------------
    def _open(self) -> None:
        if self.closed or self.g.closed:
            raise ErrClosed("the session is closed")

    def Close(self) -> None:
        if self.closed:
            return
        self.closed = True
        if self.slot is not None:
            with self.g._lock:
                self.g.engine.end_sequence(self.slot)
            self.slot = None
        self.ids, self.held = [], []
        if self in self.g._sessions:
            self.g._sessions.remove(self)


class _PieceDecoder:
    """Writes the text of a reply in pieces that end on UTF-8 boundaries (qwen3/chat.go:700-717)."""

    def __init__(self, tokenizer, writer):
        self.tokenizer, self.writer, self.pending = tokenizer, writer, b""

    def take(self, token: int) -> None:
        self.pending += self.tokenizer.piece(token)
        n = _complete_utf8(self.pending)
        if n:
            self.writer.write(self.pending[:n].decode("utf-8", "replace"))
            self.pending = self.pending[n:]

    def flush(self) -> None:
        if self.pending:
            self.writer.write(self.pending.decode("utf-8", "replace"))
            self.pending = b""


def _complete_utf8(b: bytes) -> int:
    """Length of ``b`` without a trailing incomplete UTF-8 sequence."""
    for back in range(1, min(3, len(b)) + 1):
        c = b[len(b) - back]
        if c < 0x80:
            return len(b)
        if c >= 0xC0:   # a leading byte: how long is its sequence?
            need = 2 if c < 0xE0 else 3 if c < 0xF0 else 4
            return len(b) if back >= need else len(b) - back
    return len(b)
