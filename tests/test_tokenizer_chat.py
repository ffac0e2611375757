"""The tokenizer on a synthetic vocabulary and the chat session's bookkeeping with a scripted engine
(no GPU).  The reference's tokenizer tests compare with ids that Hugging Face's tokenizer gave for
the real Qwen3 vocabulary (internal/qwen3lm/tokenizer_test.go); that vocabulary is not available
here, so these tests check the pipeline's rules on a small vocabulary made for the purpose."""
import json
import os

import pytest

from gophonic_b200.chat import (Assistant, ChatGenerator, ErrClosed, System, Template, ToolResult, User, common_prefix)
from gophonic_b200.engine.generate import GenerationError
from gophonic_b200.sampling import Options
from gophonic_b200.tokenizer import Tokenizer, TokenizerError, byte_alphabet, load_tokenizer

SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")
MERGES = [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), ("Ġ", "w"), ("o", "r"), ("Ġw", "or"), ("Ġwor", "l"),
          ("Ġworl", "d"), ("Ã", "©"), ("Ċ", "Ċ")]
ADDED = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<|im_start|>x"]


def write_tokenizer(folder, **changes):
    letters = byte_alphabet()
    vocab = {c: i for i, c in enumerate(letters)}
    for a, b in MERGES:
        vocab[a + b] = len(vocab)
    base = len(vocab)
    spec = {"model": {"type": "BPE", "vocab": vocab, "merges": [[a, b] for a, b in MERGES[:6]] + [f"{a} {b}" for a, b in MERGES[6:]]},
            "normalizer": {"type": "NFC"},
            "pre_tokenizer": {"type": "Sequence", "pretokenizers": [{"type": "Split", "pattern": {"Regex": SPLIT}}, {"type": "ByteLevel"}]},
            "added_tokens": [{"id": base + i, "content": c, "special": i < 3} for i, c in enumerate(ADDED)]}
    for key, value in changes.items():
        node = spec
        *path, last = key.split(".")
        for k in path:
            node = node[k]
        node[last] = value
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "tokenizer.json"), "w", encoding="utf-8") as f:
        json.dump(spec, f)
    return vocab, base


def test_pieces_are_merged_in_the_order_of_the_merge_list(tmp_path):
    vocab, base = write_tokenizer(str(tmp_path))
    t = load_tokenizer(str(tmp_path))
    assert t.encode("hello world") == [vocab["hello"], vocab["Ġworld"]]
    # "hel": (h, e) outranks (l, l), which no longer applies afterwards
    assert t.encode("hel") == [vocab["he"], vocab["l"]]
    assert t.encode("llo") == [vocab["ll"], vocab["o"]]
    # digits are pieces of their own; a space joins the punctuation that follows it
    assert t.encode("12") == [vocab["1"], vocab["2"]]
    assert t.decode(t.encode("a  b!\n\nc")) == "a  b!\n\nc"
    assert vocab["ĊĊ"] in t.encode("x\n\ny")
    assert t.tokens() == base + len(ADDED)


def test_added_tokens_are_cut_out_first_by_longest_match(tmp_path):
    vocab, base = write_tokenizer(str(tmp_path))
    t = load_tokenizer(str(tmp_path))
    ids = t.encode("<|im_start|>hello<|im_end|>")
    assert ids == [base + 1, vocab["hello"], base + 2]
    assert t.encode("<|im_start|>x")[0] == base + 3                     # the longer added token wins
    assert t.added_id("<|im_end|>") == base + 2 and t.added_id("<|nope|>") is None
    assert t.decode(ids) == "<|im_start|>hello<|im_end|>" and t.decode(ids, skip_special=True) == "hello"
    assert t.encode("<|im_") == [vocab[c] for c in "<|im_"]             # an incomplete one is ordinary text


def test_text_is_normalised_and_every_byte_round_trips(tmp_path):
    vocab, _ = write_tokenizer(str(tmp_path))
    t = load_tokenizer(str(tmp_path))
    composed, decomposed = "café", "café"
    assert t.encode(composed) == t.encode(decomposed)                    # NFC before anything else
    assert vocab["Ã©"] in t.encode(composed)                             # the two bytes of é, merged
    text = "naïve 日本語 🙂 \t tab"
    assert t.decode(t.encode(text)) == text
    # half of a character decodes to the replacement character, as errors="replace" does
    ids = t.encode("🙂")
    assert len(ids) == 4 and t.decode(ids[:2]) == "�"
    assert t.piece(10 ** 9) == b""


def test_other_pipelines_are_refused(tmp_path):
    for i, (key, value, word) in enumerate([("model.type", "Unigram", "model type"), ("model.byte_fallback", True, "byte_fallback"),
                                            ("normalizer.type", "NFKC", "normalizer"), ("pre_tokenizer.type", "ByteLevel", "pre-tokenizer"),
                                            ("pre_tokenizer.pretokenizers", [{"type": "ByteLevel"}], "pre-tokenizer")]):
        d = str(tmp_path / f"bad{i}")
        write_tokenizer(d, **{key: value})
        with pytest.raises(TokenizerError, match=word):
            load_tokenizer(d)
    assert load_tokenizer(str(tmp_path / "nothing")) is None
    with pytest.raises(TokenizerError, match="outside the byte alphabet"):
        Tokenizer({"一": 0}, [], [], SPLIT)


def test_the_chat_frame_is_made_of_the_tokenizers_own_ids(tmp_path):
    vocab, base = write_tokenizer(str(tmp_path))
    t = load_tokenizer(str(tmp_path))
    assert t.template_thinks                                              # no template file: the thinking block is assumed
    frame = Template.qwen3(t)
    assert frame.header[User][0] == base + 1 and t.decode(frame.header[User]) == "<|im_start|>user\n"
    assert t.decode(frame.header[ToolResult]) == "<|im_start|>user\n<tool_response>\n"
    assert frame.end == [base + 2, vocab["Ċ"]] and frame.stop == [base + 2, base]
    assert t.decode(frame.answer) == "<|im_start|>assistant\n<think>\n\n</think>\n\n"
    with open(tmp_path / "tokenizer_config.json", "w") as f:
        json.dump({"chat_template": "{{ messages }} no thinking here"}, f)
    assert not load_tokenizer(str(tmp_path)).template_thinks
    assert t.decode(Template.qwen3(t, thinking_block=False).answer) == "<|im_start|>assistant\n"


# ---- the session's bookkeeping ---------------------------------------------------------------
class ScriptEngine:
    """One slot per sequence; records every step and truncation; 'logits' name the slot."""
    vocab = 1000

    def __init__(self):
        self.tokens = {}
        self.log = []
        self.next_slot = 0

    def new_sequence(self):
        self.next_slot += 1
        self.tokens[self.next_slot] = []
        return self.next_slot

    def end_sequence(self, slot):
        del self.tokens[slot]

    def truncate(self, slot, n):
        assert 0 <= n <= len(self.tokens[slot])
        self.log.append(("truncate", slot, n))
        del self.tokens[slot][n:]

    def step(self, entries, want=None):
        for slot, toks in entries:
            self.tokens[slot] += list(toks)
            self.log.append(("step", slot, list(toks)))
        return [slot for slot, _ in entries]

    def check_kernels(self):
        pass


class ScriptSampler:
    """Replies are scripted per call of ``start``: the k-th reply draws scripts[k], then the stop id 99."""

    def __init__(self, scripts):
        self.scripts, self.reply, self.at = scripts, -1, 0

    def start(self, row, options, seed):
        self.reply += 1
        self.at = 0

    def select(self, logits, rows):
        script = self.scripts[self.reply]
        tok = script[self.at] if self.at < len(script) else 99
        self.at += 1
        return [tok]


def make_chat(scripts, context=200, template=None):
    eng = ScriptEngine()
    template = template or Template(header={System: [1], User: [2], Assistant: [3], ToolResult: [2, 4]}, end=[99, 5],
                                    result_end=[6], answer=[3], stop=[99, 98])
    return ChatGenerator(eng, ScriptSampler(scripts), context, template), eng


def test_a_second_reply_evaluates_only_what_is_new():
    g, eng = make_chat([[10, 11], [20]])
    s = g.NewSession([7, 7])
    s.Add(User, [8])
    assert s.ids == [1, 7, 7, 99, 5, 2, 8, 99, 5]
    assert s.Reply(Options(MaxTokens=8)) == [10, 11]
    # everything in one step; then one token each; the stop token is drawn and never fed
    assert eng.log == [("step", 1, [1, 7, 7, 99, 5, 2, 8, 99, 5, 3]), ("step", 1, [10]), ("step", 1, [11])]
    assert s.ids == [1, 7, 7, 99, 5, 2, 8, 99, 5, 3, 10, 11, 99, 5] and s.held == s.ids[:12]
    assert s.stats.kept == 0 and s.stats.prefill_tokens == 10 and s.stats.decoded_tokens == 2
    eng.log.clear()
    s.Add(User, [9])
    assert s.Reply(Options(MaxTokens=8)) == [20]
    # the slot held the conversation up to the reply's last token: only the new tokens run
    assert eng.log == [("step", 1, [99, 5, 2, 9, 99, 5, 3]), ("step", 1, [20])]
    assert s.stats.kept == 12 and s.stats.prefill_tokens == 7
    assert eng.tokens[1] == s.held == s.ids[:-2]
    g.Close()
    assert eng.tokens == {}


def test_restore_and_truncate_cut_the_cache_at_the_common_prefix():
    g, eng = make_chat([[10, 11, 12], [20], [30]])
    s = g.NewSession()
    s.Add(User, [8])
    mark = s.Checkpoint()
    s.Add(User, [40, 41])                      # added speculatively
    s.Prefill()
    assert eng.log == [("step", 1, [2, 8, 99, 5, 2, 40, 41, 99, 5])]
    s.Restore(mark)
    s.Add(User, [40, 42])                      # shares "2 40" with what was dropped
    eng.log.clear()
    assert s.Reply(Options(MaxTokens=3)) == [10, 11, 12]     # ends by length: the last token is never fed
    assert eng.log[0] == ("truncate", 1, 6) and eng.log[1] == ("step", 1, [42, 99, 5, 3])
    assert s.held == [2, 8, 99, 5, 2, 40, 42, 99, 5, 3, 10, 11]
    # only the first token of the reply was heard
    s.Truncate(1)
    assert s.ids == [2, 8, 99, 5, 2, 40, 42, 99, 5, 3, 10, 99, 5]
    s.Add(User, [9])
    eng.log.clear()
    assert s.Reply() == [20]
    assert eng.log[0] == ("truncate", 1, 11) and eng.log[1] == ("step", 1, [99, 5, 2, 9, 99, 5, 3])
    with pytest.raises(ValueError, match="outside the conversation"):
        s.Restore(len(s.ids) + 1)
    s.Restore(0)
    with pytest.raises(ValueError, match="no reply"):
        s.Truncate(1)
    bare, _ = make_chat([[1]], template=Template(stop=[99]))
    with pytest.raises(GenerationError, match="empty"):
        bare.NewSession().Reply()                # no frame and no message: nothing to reply to
    s.Close()
    with pytest.raises(ErrClosed):
        s.Add(User, [1])


def test_a_reply_is_bounded_by_the_context_and_sessions_do_not_share_slots():
    g, eng = make_chat([list(range(100, 200)), [7]], context=20)
    a, b = g.NewSession(), g.NewSession()
    a.Add(User, [8] * 10)                      # 13 tokens with its frame, 14 with the reply's opening
    assert len(a.Reply()) == 20 - 14 - 2       # room for the message's end is kept
    b.Add(ToolResult, [8])
    assert b.ids == [2, 4, 8, 6, 99, 5]
    assert b.Reply() == [7]
    assert a.slot != b.slot and eng.tokens[b.slot] == [2, 4, 8, 6, 99, 5, 3, 7]
    a.Add(User, [1] * 5)
    with pytest.raises(GenerationError, match="fills the context"):
        a.Reply()
    assert a.ids[-8:] == [2, 1, 1, 1, 1, 1, 99, 5]   # the refused reply left the conversation as it was
    with pytest.raises(ValueError, match="outside"):
        a.Add(User, [1000])
    with pytest.raises(ValueError, match="no tokenizer"):
        a.Add(User, "text")
    g.Close()
    with pytest.raises(ErrClosed):
        g.NewSession()


def test_text_goes_in_and_comes_out_in_whole_characters(tmp_path):
    vocab, base = write_tokenizer(str(tmp_path))
    t = load_tokenizer(str(tmp_path))
    smile = t.encode("🙂")
    eng = ScriptEngine()
    stop = base + 2
    g = ChatGenerator(eng, ScriptSampler([t.encode("hello ") + smile + [stop]]), 200, Template.qwen3(t), t)
    s = g.NewSession("be brief")
    s.Add(User, "hello world")
    pieces = []

    class Writer:
        def write(self, text):
            pieces.append(text)
    reply = s.Reply(Options(MaxTokens=16), writer=Writer())
    assert t.decode(reply) == "hello 🙂"
    assert "".join(pieces) == "hello 🙂" and all("�" not in p for p in pieces)   # the four bytes of the face came as one piece
    assert t.decode(s.ids).startswith("<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhello world<|im_end|>\n<|im_start|>assistant\n")
    s.Truncate(5)      # five bytes of the reply were heard: "hello"
    assert t.decode(s.ids[s.reply_at:]) == "hello<|im_end|>\n"


def test_common_prefix():
    assert common_prefix([1, 2, 3], [1, 2, 4, 5]) == 2 and common_prefix([], [1]) == 0 and common_prefix([1, 2], [1, 2]) == 2
