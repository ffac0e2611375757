"""Byte-level BPE tokenizer read from a model folder's ``tokenizer.json``.

The pipeline is the one the Qwen family's file describes and the reference implements
(internal/qwen3lm/tokenizer.go:192-243, 506-640): added tokens are cut out of the text first, by
longest match; what lies between them is normalised to NFC, split into pieces by the file's own
regular expression, each piece's UTF-8 bytes are written in the 256-letter byte alphabet, and
neighbouring symbols are merged in the order of the file's merge list until no listed pair is
left.  No begin-of-text token is added.  Everything comes from the file: the vocabulary, the
merges, the added tokens and the split expression (compiled with the ``regex`` module, which
knows ``\\p{L}`` and look-ahead); a file that describes another pipeline (a model type other than
BPE, byte fallback, ignored merges, another normaliser, no split expression) is refused rather
than tokenised approximately.

Decoding concatenates the tokens' bytes and replaces ill-formed UTF-8 as Python's
``errors="replace"`` does (internal/qwen3lm/tokenizer.go:417-442).
"""
from __future__ import annotations

import json
import os
import unicodedata
from typing import Dict, List, Optional, Sequence, Tuple


class TokenizerError(ValueError):
    pass


def byte_alphabet() -> List[str]:
    """The letter that stands for each byte: printable Latin-1 bytes stand for themselves, the other
    68 take the code points from 256 up in byte order (internal/qwen3lm/tokenizer.go:747-760)."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    letters, extra = [""] * 256, 0
    for b in range(256):
        if b in keep:
            letters[b] = chr(b)
        else:
            letters[b] = chr(256 + extra)
            extra += 1
    return letters


class Tokenizer:
    def __init__(self, vocab: Dict[str, int], merges: Sequence[Tuple[str, str]], added: Sequence[Tuple[int, str, bool]],
                 split_regex: str, template_thinks: bool = True):
        import regex
        self.letters = byte_alphabet()
        self.byte_of = {c: b for b, c in enumerate(self.letters)}
        self.vocab = dict(vocab)
        self.ranks = {(a, b): r for r, (a, b) in enumerate(merges)}
        try:
            self.split = regex.compile(split_regex)
        except regex.error as e:
            raise TokenizerError(f"tokenizer.json: the split expression does not compile: {e}") from e
        n = max([i + 1 for i in vocab.values()] + [i + 1 for i, _, _ in added] + [0])
        if n > 1 << 24:
            raise TokenizerError("tokenizer.json: implausible vocabulary size")
        self.pieces: List[bytes] = [b""] * n
        for piece, i in vocab.items():
            if i < 0:
                raise TokenizerError(f"tokenizer.json: negative id for {piece!r}")
            try:
                self.pieces[i] = bytes(self.byte_of[c] for c in piece)
            except KeyError:
                raise TokenizerError(f"tokenizer.json: piece {piece!r} of token {i} is outside the byte alphabet") from None
        self.special = [False] * n
        self.added: Dict[str, int] = {}
        for i, content, special in added:
            self.pieces[i] = content.encode("utf-8")
            self.special[i] = bool(special)
            self.added[content] = i
        self._added_by_length = sorted(self.added, key=len, reverse=True)
        self._added_first = {c[0] for c in self.added if c}
        self.template_thinks = template_thinks
        self._cache: Dict[str, List[int]] = {}

    # ---- description -------------------------------------------------------------------------
    def tokens(self) -> int:
        return len(self.pieces)

    def added_id(self, text: str) -> Optional[int]:
        """The id of the added token whose content is exactly ``text``, or None."""
        return self.added.get(text)

    def piece(self, token: int) -> bytes:
        """The bytes of one token; nothing for an id the tokenizer does not know."""
        return self.pieces[token] if 0 <= token < len(self.pieces) else b""

    # ---- encoding ----------------------------------------------------------------------------
    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        gap_start, i, n = 0, 0, len(text)
        while i < n:
            if text[i] in self._added_first:
                hit = next((c for c in self._added_by_length if text.startswith(c, i)), None)
                if hit is not None:
                    self._encode_gap(text[gap_start:i], out)
                    out.append(self.added[hit])
                    i += len(hit)
                    gap_start = i
                    continue
            i += 1
        self._encode_gap(text[gap_start:], out)
        return out

    def _encode_gap(self, gap: str, out: List[int]) -> None:
        if not gap:
            return
        gap = unicodedata.normalize("NFC", gap)
        for m in self.split.finditer(gap):
            piece = m.group(0)
            ids = self._cache.get(piece)
            if ids is None:
                ids = self._encode_piece(piece)
                if len(self._cache) < 1 << 16:
                    self._cache[piece] = ids
            out.extend(ids)

    def _encode_piece(self, piece: str) -> List[int]:
        symbols = [self.letters[b] for b in piece.encode("utf-8")]
        while len(symbols) > 1:
            best, at = None, -1
            for k in range(len(symbols) - 1):
                r = self.ranks.get((symbols[k], symbols[k + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, k
            if best is None:
                break
            symbols[at:at + 2] = [symbols[at] + symbols[at + 1]]
        try:
            return [self.vocab[s] for s in symbols]
        except KeyError as e:
            raise TokenizerError(f"no token for the symbol {e.args[0]!r} of piece {piece!r}") from None

    # ---- decoding ----------------------------------------------------------------------------
    def decode(self, ids: Sequence[int], skip_special: bool = False) -> str:
        raw = b"".join(self.piece(int(i)) for i in ids if not (skip_special and 0 <= int(i) < len(self.special) and self.special[int(i)]))
        return raw.decode("utf-8", "replace")


def _merge_pair(m) -> Tuple[str, str]:
    """One merge of tokenizer.json: ["left", "right"] or, as older files write it, "left right"."""
    if isinstance(m, str):
        a, _, b = m.partition(" ")
        return a, b
    if isinstance(m, (list, tuple)) and len(m) == 2 and all(isinstance(x, str) for x in m):
        return m[0], m[1]
    raise TokenizerError(f"tokenizer.json: a merge is neither a pair nor a string: {m!r}")


def chat_template_text(model_dir: str) -> str:
    """The folder's chat template: ``chat_template`` of tokenizer_config.json, else
    chat_template.jinja, else nothing (qwen3/dialect.go:33-44)."""
    try:
        with open(os.path.join(model_dir, "tokenizer_config.json")) as f:
            t = json.load(f).get("chat_template")
        if isinstance(t, str) and t:
            return t
    except (OSError, ValueError):
        pass
    try:
        with open(os.path.join(model_dir, "chat_template.jinja")) as f:
            return f.read()
    except OSError:
        return ""


def load_tokenizer(model_dir: str) -> Optional[Tokenizer]:
    """The tokenizer of a model folder, or None if the folder has no tokenizer.json."""
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.exists(path):
        return None
    try:
        with open(path, encoding="utf-8") as f:
            spec = json.load(f)
    except (OSError, ValueError) as e:
        raise TokenizerError(f"cannot read {path}: {e}") from e
    model = spec.get("model") or {}
    if model.get("type") != "BPE" or model.get("ignore_merges") or model.get("byte_fallback"):
        raise TokenizerError(f"{path}: unsupported tokenizer model type={model.get('type')!r} "
                             f"ignore_merges={bool(model.get('ignore_merges'))} byte_fallback={bool(model.get('byte_fallback'))}")
    norm = (spec.get("normalizer") or {}).get("type")
    if norm != "NFC":
        raise TokenizerError(f"{path}: unsupported normalizer {norm!r}, want NFC")
    pre = spec.get("pre_tokenizer") or {}
    split_regex = None
    for node in pre.get("pretokenizers") or []:
        if node.get("type") == "Split":
            split_regex = (node.get("pattern") or {}).get("Regex")
            break
    if pre.get("type") != "Sequence" or not split_regex:
        raise TokenizerError(f"{path}: unsupported pre-tokenizer pipeline (type={pre.get('type')!r}, no split expression)")
    added = [(int(a["id"]), str(a["content"]), bool(a.get("special"))) for a in spec.get("added_tokens") or []]
    template = chat_template_text(model_dir)
    return Tokenizer(model.get("vocab") or {}, [_merge_pair(m) for m in model.get("merges") or []], added, split_regex,
                     template_thinks=(template == "" or "<think>" in template))
