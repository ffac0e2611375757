"""The generation loop's decisions (no GPU), driven with a scripted engine and sampler."""
import pytest

from gophonic_b200.engine.generate import GenerationError, Generator
from gophonic_b200.sampling import Options


class ScriptEngine:
    """Hands out slots, records steps; 'logits' are just the entries so the sampler can script."""

    def __init__(self, pages=100):
        self.free = list(range(7, -1, -1))
        self.held = set()
        self.lengths = {}
        self.steps = []
        self.pages = pages
        self.max_live = 0

    def room(self):
        return self.pages - sum((n + 63) // 64 for n in self.lengths.values())

    def new_sequence(self):
        s = self.free.pop()
        assert s not in self.held
        self.held.add(s)
        self.lengths[s] = 0
        self.max_live = max(self.max_live, len(self.held))
        return s

    def end_sequence(self, slot):
        assert slot in self.held, "slot freed twice"
        self.held.remove(slot)
        del self.lengths[slot]
        self.free.append(slot)

    def step(self, entries, want=None):
        assert len({s for s, _ in entries}) == len(entries)
        for s, toks in entries:
            assert s in self.held
            self.lengths[s] += len(toks)
        self.steps.append([(s, list(t)) for s, t in entries])
        return [(s, self.lengths[s]) for s, _ in entries]


class ScriptSampler:
    """Request with seed k (its index, as Seed is 0) replies script[k]; afterwards the stop token 99."""

    def __init__(self, scripts):
        self.scripts = scripts
        self.rows = {}

    def start(self, row, options, seed):
        self.rows[row] = [seed, 0]

    def select(self, logits, rows):
        out = []
        for r in rows:
            seed, n = self.rows[r]
            script = self.scripts[seed]
            out.append(script[n] if n < len(script) else 99)
            self.rows[r][1] += 1
        return out


def run(prompts, scripts, max_batch=4, context=1000, options=None, pages=100, stop=(99,)):
    eng = ScriptEngine(pages)
    g = Generator(eng, ScriptSampler(scripts), max_batch, context, stop)
    return g.generate(prompts, options), eng, g


def test_stop_token_ends_a_reply_and_is_not_part_of_it():
    out, eng, g = run([[1, 2, 3]], {0: [5, 6, 7]})
    assert out == [[5, 6, 7]]
    # prompt in one step, then one token each; the stop token is never fed back
    assert eng.steps == [[(0, [1, 2, 3])], [(0, [5])], [(0, [6])], [(0, [7])]]
    assert not eng.held and g.stats.batches == 1 and g.stats.prefill_tokens == 3 and g.stats.decode_steps == 3


def test_shorter_requests_leave_early_and_the_rest_go_on():
    out, eng, _ = run([[1], [2, 2], [3, 3, 3]], {0: [10], 1: [20, 21, 22], 2: []})
    assert out == [[10], [20, 21, 22], []]
    assert eng.steps[0] == [(0, [1]), (1, [2, 2]), (2, [3, 3, 3])]      # start together, unequal lengths
    assert eng.steps[1] == [(0, [10]), (1, [20])]                         # request 2 stopped at once
    assert eng.steps[2] == [(1, [21])] and eng.steps[3] == [(1, [22])]    # request 0 left, 1 goes on
    assert len(eng.steps) == 4 and not eng.held


def test_max_tokens_bounds_the_reply_without_an_extra_step():
    out, eng, _ = run([[1, 1]], {0: [5, 6, 7, 8]}, options=Options(MaxTokens=2))
    assert out == [[5, 6]]
    assert eng.steps == [[(0, [1, 1])], [(0, [5])]]  # the second token is drawn and never fed


def test_context_bounds_the_reply():
    out, _, _ = run([[1] * 8], {0: list(range(10, 30))}, context=11)
    assert out == [[10, 11, 12]]
    with pytest.raises(GenerationError, match="fills the context"):
        run([[1] * 11], {0: []}, context=11)


def test_more_requests_than_the_batch_run_one_batch_after_another_reusing_slots():
    prompts = [[i + 1] for i in range(5)]
    scripts = {i: [100 + i] * (i + 1) for i in range(5)}
    out, eng, g = run(prompts, scripts, max_batch=2)
    assert out == [[100 + i] * (i + 1) for i in range(5)]
    assert g.stats.batches == 3 and eng.max_live == 2
    starts = [s for s in eng.steps if any(len(t) == 1 and t[0] < 10 for _, t in s)]
    assert [[t[0] for _, t in s] for s in starts] == [[1, 2], [3, 4], [5]]  # no request joins a running batch
    assert {s for st in eng.steps for s, _ in st} == {0, 1}                  # slots are used again


def test_batches_are_cut_to_the_free_pages():
    # each request may grow to 64 + 63 tokens = 2 pages; 5 pages hold two of them at a time
    out, eng, g = run([[1] * 64, [2] * 64, [3] * 64], {0: [7], 1: [8], 2: [9]}, max_batch=4, pages=5,
                      options=Options(MaxTokens=64))
    assert out == [[7], [8], [9]] and g.stats.batches == 2
    with pytest.raises(GenerationError, match="needs 2 pages"):
        run([[1] * 64], {0: [7]}, pages=1, options=Options(MaxTokens=64))


def test_per_request_options_and_seeds():
    seen = {}

    class S(ScriptSampler):
        def start(self, row, options, seed):
            seen[seed] = options
            super().start(row, options, seed)
    eng = ScriptEngine()
    o = [Options(Seed=10, Temperature=0.5), Options(Seed=10, TopK=3)]
    g = Generator(eng, S({10: [1], 11: [2]}), 4, 100, (99,))
    assert g.generate([[1], [2]], o) == [[1], [2]]
    assert seen[10].Temperature == 0.5 and seen[11].TopK == 3  # request i draws with Seed + i
    with pytest.raises(GenerationError, match="option sets"):
        g.generate([[1], [2]], [Options()])
    with pytest.raises(GenerationError, match="empty prompt"):
        g.generate([[]])
    with pytest.raises(ValueError, match="TopP"):
        g.generate([[1]], Options(TopP=1.5))


def test_slots_are_given_back_when_a_step_fails():
    class Boom(ScriptEngine):
        def step(self, entries, want=None):
            if len(self.steps) == 1:
                raise RuntimeError("boom")
            return super().step(entries, want)
    eng = Boom()
    g = Generator(eng, ScriptSampler({0: [1, 2], 1: [3, 4]}), 4, 100, (99,))
    with pytest.raises(RuntimeError, match="boom"):
        g.generate([[1], [2]])
    assert not eng.held


def test_on_token_streams_in_order():
    got = []
    eng = ScriptEngine()
    g = Generator(eng, ScriptSampler({0: [5, 6], 1: [7]}), 4, 100, (99,))
    g.generate([[1], [2]], on_token=lambda i, t: got.append((i, t)))
    assert got == [(0, 5), (1, 7), (0, 6)]


# ---- the loop that runs one step ahead of what it has read --------------------------------------
class AheadEngine(ScriptEngine):
    """The scripted engine with the two calls that let the loop enqueue a step before it has read
    the last one's tokens.  ``wasted`` counts entries stepped for a sequence that had already
    drawn its stop token."""

    def __init__(self, pages=100):
        super().__init__(pages)
        self.unread = 0      # fetches started and not yet waited for
        self.max_unread = 0

    def step_from(self, slots, source, positions):
        assert len(slots) == len(positions) and len(set(slots)) == len(slots)
        return self.step([(s, [source[p]]) for s, p in zip(slots, positions)])

    def fetch_tokens(self, tokens):
        eng = self
        eng.unread += 1
        eng.max_unread = max(eng.max_unread, eng.unread)

        class Fetch:
            def wait(self_inner):
                eng.unread -= 1
                return list(tokens)
        return Fetch()


class AheadSampler(ScriptSampler):
    def select_device(self, logits, rows):
        return self.select(logits, rows)


def run_ahead(prompts, scripts, max_batch=4, context=1000, options=None, pages=100, stop=(99,), on_token=None):
    eng = AheadEngine(pages)
    g = Generator(eng, AheadSampler(scripts), max_batch, context, stop)
    return g.generate(prompts, options, on_token), eng, g


CASES = [
    ([[1, 2, 3]], {0: [5, 6, 7]}, {}),
    ([[1], [2, 2], [3, 3, 3]], {0: [10], 1: [20, 21, 22], 2: []}, {}),
    ([[1, 1]], {0: [5, 6, 7, 8]}, dict(options=Options(MaxTokens=2))),
    ([[1] * 8], {0: list(range(10, 30))}, dict(context=11)),
    ([[i + 1] for i in range(5)], {i: [100 + i] * (i + 1) for i in range(5)}, dict(max_batch=2)),
    ([[1] * 64, [2] * 64, [3] * 64], {0: [7], 1: [8], 2: [9]}, dict(max_batch=4, pages=5, options=Options(MaxTokens=64))),
    ([[4], [5]], {0: [1] * 30, 1: [2] * 3}, dict(options=[Options(MaxTokens=7), Options(MaxTokens=50)])),
]


@pytest.mark.parametrize("prompts,scripts,kw", CASES)
def test_running_ahead_gives_the_same_replies_callbacks_and_counts(prompts, scripts, kw):
    plain_calls, ahead_calls = [], []
    g0 = Generator(ScriptEngine(kw.get("pages", 100)), ScriptSampler(scripts), kw.get("max_batch", 4), kw.get("context", 1000), (99,))
    want = g0.generate(prompts, kw.get("options"), lambda i, t: plain_calls.append((i, t)))
    got, eng, g = run_ahead(prompts, scripts, on_token=lambda i, t: ahead_calls.append((i, t)), **kw)
    assert got == want
    assert ahead_calls == plain_calls                       # every token, in the same order
    assert not eng.held and eng.unread == 0                 # every slot given back, every fetch read
    assert eng.max_unread <= 2                              # one step ahead, never more
    s0, s1 = g0.stats, g.stats
    assert (s1.batches, s1.prefill_tokens, s1.decode_steps, s1.decoded_tokens) == (s0.batches, s0.prefill_tokens, s0.decode_steps, s0.decoded_tokens)


def test_running_ahead_wastes_one_entry_per_stop_token_and_none_per_length_end():
    # request 0 stops by its stop token after 3 tokens: the step enqueued before that was read fed it
    # once for nothing; request 1 ends by MaxTokens, which the loop knows beforehand
    got, eng, _ = run_ahead([[1], [2]], {0: [10, 11, 12], 1: [20] * 40}, options=[Options(), Options(MaxTokens=5)])
    assert got == [[10, 11, 12], [20] * 5]
    fed0 = [t for st in eng.steps[1:] for s, t in st if s == eng.steps[0][0][0]]
    fed1 = [t for st in eng.steps[1:] for s, t in st if s == eng.steps[0][1][0]]
    assert fed0 == [[10], [11], [12], [99]]   # the stop token itself went through one step, its result dropped
    assert fed1 == [[20]] * 4                 # the fifth token is drawn and never fed
