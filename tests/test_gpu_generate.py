"""Generation through the entry point (Open / Lane / Generate and the command line) against the
plain implementation: greedy replies token for token in 32-bit, stop tokens, early ends, more
requests than a batch holds, and seeded sampling that does not depend on the batch."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests.plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lanes(model_dirs):
    import gophonic_b200 as g
    opened = {}

    def get(name, fmt, batch=4):
        key = (name, fmt, batch)
        if key not in opened:
            m = g.Open(model_dirs[name], g.Options(Format=fmt, CacheTokens=2048, Batch=batch))
            opened[key] = g.Lane(m, g.TokensGenerator)
        return opened[key]
    return get


def prompts_for(cfg, seed, lengths):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in lengths]


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_replies_equal_the_plain_ones_in_32_bit(lanes, plain_models, name):
    import gophonic_b200 as g
    cfg, w = plain_models[name]
    prompts = prompts_for(cfg, 3, [5, 11, 17, 1, 40, 7])  # six requests, batches of four: two batches
    gen = lanes(name, g.FormatF32)
    got = gen.Generate(prompts, g.ChatOptions(MaxTokens=8))
    want = [P.greedy_generate(p, 8, cfg, w) for p in prompts]
    assert got == want
    assert gen.stats.batches == 2 and gen.stats.prefill_tokens == sum(map(len, prompts))
    gen.engine.cache.check()
    assert gen.engine.cache.pages.held() == 0


def test_greedy_replies_in_bfloat16_follow_the_plain_ones(lanes, plain_models):
    """bfloat16 may flip a near-tie; up to the first difference the replies agree, and most agree fully."""
    import gophonic_b200 as g
    cfg, w = plain_models["B"]
    prompts = prompts_for(cfg, 4, [3, 9, 33, 65])
    got = lanes("B", g.FormatBF16).Generate(prompts, g.ChatOptions(MaxTokens=12))
    want = [P.greedy_generate(p, 12, cfg, w) for p in prompts]
    agree = 0
    for a, b, p in zip(got, want, prompts):
        if a == b:
            agree += 1
            continue
        k = next(i for i, (x, y) in enumerate(zip(a, b)) if x != y)
        logits = P.forward_logits(p + b[:k], cfg, w)[-1]
        top2 = np.sort(logits)[-2:]
        assert top2[1] - top2[0] < 0.05 * np.max(np.abs(logits)), "a flip that is no near-tie"
        assert a[k] == int(np.argsort(logits)[-2])
    assert agree >= 3


def test_stop_tokens_and_unequal_ends(lanes, plain_models):
    import gophonic_b200 as g
    cfg, w = plain_models["A"]
    prompts = prompts_for(cfg, 6, [4, 9, 2])
    free = [P.greedy_generate(p, 10, cfg, w) for p in prompts]
    stop = free[1][3]
    want = [P.greedy_generate(p, 10, cfg, w, stop_ids=[stop]) for p in prompts]
    assert len(want[1]) <= 3
    got = lanes("A", g.FormatF32).Generate(prompts, g.ChatOptions(MaxTokens=10), stop_ids=[stop])
    assert got == want and all(stop not in r for r in got)
    per = [g.ChatOptions(MaxTokens=2), g.ChatOptions(MaxTokens=10), g.ChatOptions(MaxTokens=5)]
    got = lanes("A", g.FormatF32).Generate(prompts, per)
    assert got == [free[0][:2], free[1], free[2][:5]]


def test_seeded_sampling_is_repeatable_and_independent_of_the_batch(lanes, plain_models):
    import gophonic_b200 as g
    cfg, w = plain_models["B"]
    prompts = prompts_for(cfg, 8, [1, 7, 23, 40])
    opts = g.ChatOptions(MaxTokens=12, Temperature=0.8, TopK=20, Seed=77)
    gen = lanes("B", g.FormatF32)
    a = gen.Generate(prompts, opts)
    b = gen.Generate(prompts, opts)
    assert a == b and all(len(r) == 12 for r in a)
    # request i of a batch draws with Seed + i: alone with that seed it replies the same
    for i in (0, 2):
        alone = gen.Generate([prompts[i]], g.ChatOptions(MaxTokens=12, Temperature=0.8, TopK=20, Seed=77 + i))
        assert alone[0] == a[i]
    c = gen.Generate(prompts, g.ChatOptions(MaxTokens=12, Temperature=0.8, TopK=20, Seed=78))
    assert c != a
    # every sampled token is among the 20 likeliest of the plain logits, and the first token follows the plain sampler
    for p, r in zip(prompts, a):
        ids = list(p)
        for t in r[:4]:
            logits = P.forward_logits(ids, cfg, w)[-1]
            assert t in np.argsort(-logits)[:20]
            ids.append(t)
    first, cand, _ = P.sample_token(P.forward_logits(prompts[1], cfg, w)[-1].astype(np.float32), 0.8, 20, 0.0, 78, 0)
    assert a[1][0] in cand and (a[1][0] == first or abs(cand.index(a[1][0]) - cand.index(first)) <= 1)


def test_presence_penalty_changes_repeats(lanes, plain_models):
    import gophonic_b200 as g
    cfg, w = plain_models["A"]
    p = prompts_for(cfg, 10, [6])
    gen = lanes("A", g.FormatF32)
    plain_reply = gen.Generate(p, g.ChatOptions(MaxTokens=24))[0]
    pen = gen.Generate(p, g.ChatOptions(MaxTokens=24, Presence=100.0))[0]
    assert len(set(pen)) == len(pen), "a huge presence penalty forbids every repeat"
    assert pen[0] == plain_reply[0]


def test_open_errors(model_dirs, tmp_path):
    import gophonic_b200 as g
    with pytest.raises(g.ErrUnsupported, match="unknown weight format"):
        g.Open(model_dirs["A"], g.Options(Format="int8"))
    with pytest.raises(ValueError, match="thread count"):
        g.Open(model_dirs["A"], g.Options(Threads=-1))
    with pytest.raises(FileNotFoundError):
        g.Open(str(tmp_path / "none"))
    (tmp_path / "x").mkdir()
    (tmp_path / "x" / "config.json").write_text(json.dumps({"architectures": ["Other"], "model_type": "other"}))
    with pytest.raises(g.ErrUnknownFormat):
        g.Open(str(tmp_path / "x"))
    m = g.Open(model_dirs["A"], g.Options(CacheTokens=256))
    assert m.Name() == "Qwen3ForCausalLM" and g.Supports(m, g.TokensGenerator) and not g.Supports(m, "speech.Transcriber")
    with pytest.raises(g.ErrUnsupported, match="does not provide"):
        g.Lane(m, "speech.Transcriber")
    m.Close()
    m.Close()


def test_command_line(model_dirs, plain_models):
    cfg, w = plain_models["A"]
    proc = subprocess.run([sys.executable, "-m", "gophonic_b200", "-model", model_dirs["A"], "-format", "f32",
                           "-max-tokens", "5", "3,9,27", "100"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    assert [l["prompt"] for l in lines] == [[3, 9, 27], [100]]
    assert [l["tokens"] for l in lines] == [P.greedy_generate(p, 5, cfg, w) for p in ([3, 9, 27], [100])]
    bad = subprocess.run([sys.executable, "-m", "gophonic_b200", "-model", "/nonexistent", "1"], cwd=ROOT,
                         capture_output=True, text=True, timeout=600)
    assert bad.returncode == 1 and "gophonic_b200:" in bad.stderr


def test_command_line_with_a_named_configuration_and_a_file_of_prompts(tmp_path):
    """-random-config NAME -weights-seed S: the model the plain implementation makes from the same
    configuration file and seed replies with the same tokens."""
    from gophonic_b200.config.presets import preset
    cfg = preset("tinyA")
    w = P.random_weights(cfg, 3)
    (tmp_path / "prompts.txt").write_text("5 6 7 8\n\n100,200\n")
    proc = subprocess.run([sys.executable, "-m", "gophonic_b200", "-random-config", "tinyA", "-weights-seed", "3", "-format", "f32",
                           "-max-tokens", "6", "-prompt-ids", str(tmp_path / "prompts.txt"), "3,9,27"],
                          cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    assert [l["prompt"] for l in lines] == [[3, 9, 27], [5, 6, 7, 8], [100, 200]]
    assert [l["tokens"] for l in lines] == [P.greedy_generate(l["prompt"], 6, cfg, w) for l in lines]


def test_running_ahead_and_reading_every_token_first_give_the_same_replies(lanes, plain_models):
    """Many requests of random lengths, budgets and stop tokens, greedy and sampled, more than a batch
    holds: the loop that runs one step ahead (the engine's own) and the loop that reads every token
    before the next step (the same engine behind a face without ``step_from``) reply alike, and the
    cache is whole afterwards."""
    import gophonic_b200 as g
    from gophonic_b200.engine.generate import Generator
    gen = lanes("A", g.FormatF32, batch=4)
    cfg, _ = plain_models["A"]
    rng = np.random.default_rng(77)
    prompts = [rng.integers(0, cfg["vocab_size"], size=int(n)).tolist() for n in rng.integers(1, 60, size=23)]
    options = [g.ChatOptions(MaxTokens=int(rng.integers(1, 30)), Temperature=float(rng.choice([0.0, 0.9])),
                             TopK=int(rng.choice([0, 5])), Presence=float(rng.choice([0.0, 0.7])), Seed=int(rng.integers(0, 1000)))
               for _ in prompts]
    stop = [int(t) for t in rng.integers(0, cfg["vocab_size"], size=60)]   # a ninth of the vocabulary stops a reply

    class ReadFirst:
        """The engine without the calls that let the loop run ahead."""

        def __init__(self, eng):
            self.new_sequence, self.end_sequence, self.step, self.room = eng.new_sequence, eng.end_sequence, eng.step, eng.room

    ahead = gen.Generate(prompts, options, stop_ids=stop)
    assert gen.engine.cache.pages.held() == 0 and gen.engine.cache.slots.held() == 0
    plain_loop = Generator(ReadFirst(gen.engine), gen.sampler, gen.batch, gen.context, stop).generate(prompts, options)
    assert ahead == plain_loop
    assert any(len(r) < o.MaxTokens for r, o in zip(ahead, options)), "some reply ended on a stop token"
    gen.engine.cache.check()
    assert gen.engine.cache.pages.held() == 0 and gen.engine.cache.slots.held() == 0


# ---- the chat lane ------------------------------------------------------------------------------
def plain_reply(ids, n_new, cfg, w, stop):
    return P.greedy_generate(ids, n_new, cfg, w, stop_ids=stop)


@pytest.mark.parametrize("name,fmt", [("A", "f32"), ("B", "f32"), ("D", "bf16")])
def test_a_conversation_keeps_its_context_between_replies(model_dirs, plain_models, name, fmt):
    """Lane "chat.Generator" over token ids: every reply equals a fresh greedy evaluation of the
    whole conversation by the plain implementation (32-bit; in bfloat16 up to a near-tie), the
    second reply evaluates only the tokens that are new, and a conversation cut back by Restore or
    Truncate goes on from what the cache still shares with it."""
    import gophonic_b200 as g
    from gophonic_b200.chat import Template, User
    cfg, w = plain_models[name]
    m = g.Open(model_dirs[name], g.Options(Format=fmt, CacheTokens=1024))
    assert g.Supports(m, g.ChatGeneratorLane)
    chat = g.Lane(m, g.ChatGeneratorLane)
    rng = np.random.default_rng(5)
    V = cfg["vocab_size"]
    stop = [int(rng.integers(0, V))]
    chat.template = Template(header={User: [1, 2]}, end=[3], answer=[4, 5], stop=stop)
    chat._loop.stop_ids = frozenset(stop)
    exact = fmt == "f32"

    def same(got, ids, n):
        want = plain_reply(ids, n, cfg, w, stop)
        if exact:
            assert got == want
        else:
            k = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), min(len(got), len(want)))
            assert k == len(want) == len(got) or k >= 1   # bfloat16 may leave the plain reply at a near-tie, not at once
    s = chat.NewSession()
    s.Add(User, rng.integers(0, V, size=70).tolist())
    first = s.Reply(g.ChatOptions(MaxTokens=9))
    same(first, s.ids[:s.reply_at], 9)
    assert s.stats.kept == 0 and s.stats.prefill_tokens == s.reply_at
    assert chat.engine.length(s.slot) == len(s.held) and s.held == s.ids[:len(s.held)]
    # a second message: only what is new is evaluated
    before = len(s.held)
    s.Add(User, rng.integers(0, V, size=11).tolist())
    second = s.Reply(g.ChatOptions(MaxTokens=6))
    same(second, s.ids[:s.reply_at], 6)
    assert s.stats.kept == min(before, s.reply_at - 1) and s.stats.prefill_tokens == s.reply_at - s.stats.kept < 25
    # a message added speculatively, evaluated, dropped, replaced
    mark = s.Checkpoint()
    s.Add(User, [7, 8, 9, 10])
    s.Prefill()
    assert chat.engine.length(s.slot) == len(s.ids)
    s.Restore(mark)
    s.Add(User, [7, 8, 11])
    third = s.Reply(g.ChatOptions(MaxTokens=5))
    same(third, s.ids[:s.reply_at], 5)
    assert s.stats.kept == mark + 4        # the frame's two tokens and 7, 8 were shared
    # the reply is cut to its first two tokens, then the conversation goes on
    if len(third) > 2:
        s.Truncate(2)
        assert s.ids[s.reply_at:] == third[:2] + [3]
    s.Add(User, [12])
    fourth = s.Reply(g.ChatOptions(MaxTokens=4))
    same(fourth, s.ids[:s.reply_at], 4)
    # a second session shares the model and the cache, not the slot
    other = chat.NewSession()
    other.Add(User, [5, 6, 7])
    same(other.Reply(g.ChatOptions(MaxTokens=4)), other.ids[:other.reply_at], 4)
    assert other.slot != s.slot
    chat.engine.cache.check()
    chat.Close()
    assert chat.engine.cache.pages.held() == 0 and chat.engine.cache.slots.held() == 0
    m.Close()


def test_a_conversation_in_text(model_dirs, plain_models, tmp_path):
    """A model folder with a tokenizer.json: messages are text, the frame is Qwen3's, the reply is
    written piece by piece, and the ids are what the plain implementation generates from the framed
    conversation."""
    import shutil
    import gophonic_b200 as g
    from gophonic_b200.chat import User
    from tests.test_tokenizer_chat import write_tokenizer
    cfg, w = plain_models["A"]
    d = str(tmp_path / "with_tokenizer")
    shutil.copytree(model_dirs["A"], d)
    vocab, base = write_tokenizer(d)
    assert base + 4 <= cfg["vocab_size"]
    m = g.Open(d, g.Options(Format="f32", CacheTokens=512))
    chat = g.Lane(m, g.ChatGeneratorLane)
    t = chat.tokenizer
    s = chat.NewSession("be brief")
    s.Add(User, "hello world")
    heard = []

    class Writer:
        def write(self, text):
            heard.append(text)
    reply = s.Reply(g.ChatOptions(MaxTokens=12), writer=Writer())
    framed = t.encode("<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhello world<|im_end|>\n"
                      "<|im_start|>assistant\n<think>\n\n</think>\n\n")
    assert s.ids[:s.reply_at] == framed
    assert reply == P.greedy_generate(framed, 12, cfg, w, stop_ids=[base + 2, base])
    assert "".join(heard) == t.decode(reply)
    chat.Close()
    m.Close()
