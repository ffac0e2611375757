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
