"""The cache's bookkeeping (no GPU): no slot or page is lost, held twice or freed twice; groups
get storage of their own; refused calls change nothing."""
import random

import pytest
import torch

from gophonic_b200.cache import PAGE, Cache, CacheError, CacheFull, FreeList, pages_for
from gophonic_b200.parts.base import KVRequest, StateRequest


def make(max_tokens=64 * 10, requests=None, **kw):
    if requests is None:
        requests = [(KVRequest(2, 16), None)] * 3
    return Cache(requests, max_tokens, "cpu", torch.float32, **kw)


def test_free_list_refuses_double_free_and_unknown():
    f = FreeList(3, "slot")
    a, b = f.take(), f.take()
    assert (a, b) == (0, 1)
    f.give(a)
    with pytest.raises(CacheError, match="freed twice"):
        f.give(a)
    with pytest.raises(CacheError, match="does not exist"):
        f.give(7)
    assert f.take() == 0 and f.take() == 2
    with pytest.raises(CacheFull):
        f.take()
    f.check()


def test_pages_follow_lengths_and_come_back():
    c = make()
    s0, s1 = c.alloc_slot(), c.alloc_slot()
    c.reserve([(s0, 65), (s1, 1)])
    c.commit([(s0, 65), (s1, 1)])
    assert c.pages.held() == 3 and c.tokens_held() == 3 * PAGE
    assert c.length(s0) == 65 and c.length(s1) == 1
    assert c.block_table[s0, :2].tolist() == c._pages_of[s0]
    c.reserve([(s0, 128)])  # still two pages
    assert c.pages.held() == 3
    c.reserve([(s0, 129)])
    assert c.pages.held() == 4
    c.check()
    c.free_slot(s0)
    assert c.pages.held() == 1
    with pytest.raises(CacheError, match="freed twice"):
        c.free_slot(s0)
    with pytest.raises(CacheError, match="not live"):
        c.length(s0)
    s2 = c.alloc_slot()
    assert s2 == s0 and c.length(s2) == 0  # the slot is used again, empty
    c.check()


def test_refused_reserve_changes_nothing():
    c = make(max_tokens=64 * 4)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 64)])
    c.commit([(a, 64)])
    before = (c.pages.held(), list(c._pages_of[a]), list(c._pages_of[b]))
    with pytest.raises(CacheFull, match="needs 4 more pages"):
        c.reserve([(a, 128), (b, 64 * 3)])
    assert (c.pages.held(), list(c._pages_of[a]), list(c._pages_of[b])) == before
    with pytest.raises(CacheError, match="appears twice"):
        c.reserve([(a, 65), (a, 66)])
    with pytest.raises(CacheError, match="below its length"):
        c.reserve([(a, 10)])
    with pytest.raises(CacheError, match="not live"):
        c.reserve([(3, 10)])
    assert (c.pages.held(), list(c._pages_of[a]), list(c._pages_of[b])) == before
    c.check()


def test_truncate_returns_pages():
    c = make()
    s = c.alloc_slot()
    c.reserve([(s, 200)])
    c.commit([(s, 200)])
    c.truncate(s, 64)
    assert c.length(s) == 64 and c.pages.held() == 1
    with pytest.raises(CacheError):
        c.truncate(s, 65)
    c.check()


def test_groups_have_storage_of_their_own_and_shared_planes():
    reqs = [(KVRequest(2, 16, 0), None), (KVRequest(2, 16, 128), None), (KVRequest(2, 16, 0), None),
            (StateRequest((4, 3), torch.float32), None), (None, None), (KVRequest(2, 16, 0), 0),
            (KVRequest(1, 32, 0), None)]
    c = make(requests=reqs)
    kinds = sorted((g["kind"], tuple(g["planes"])) for g in c.groups())
    assert kinds == [("kv", (0, 2)), ("kv", (1,)), ("kv", (6,)), ("state", (3,))]
    v0, v1, v2, v5 = c.view(0), c.view(1), c.view(2), c.view(5)
    # one page and one slot beyond the pools are nobody's: rows that fill a captured step up use them
    assert v0.k.shape == (c.n_pages + 1, 2, PAGE, 16) and c.view(6).k.shape == (c.n_pages + 1, 1, PAGE, 32)
    assert v0.k.data_ptr() != v2.k.data_ptr() != v1.k.data_ptr()
    assert v1.window == 128 and v0.window == 0
    assert v5.k.data_ptr() == v0.k.data_ptr() and not v5.writable and v0.writable
    assert c.view(4) is None
    st = c.view(3)
    assert st.state.shape == (c.max_slots + 1, 4, 3) and c.block_table[c.spare_slot, 0] == c.spare_page == c.n_pages
    s = c.alloc_slot()
    st.state[s] += 5
    c.free_slot(s)
    s2 = c.alloc_slot()
    assert s2 == s and float(c.view(3).state[s2].abs().sum()) == 0  # state starts at zero again
    with pytest.raises(CacheError, match="which has none"):
        make(requests=[(None, None), (KVRequest(2, 16), 0)])


def test_max_tokens_sizes_the_pool():
    c = make(max_tokens=1000)
    assert c.n_pages == pages_for(1000) == 16
    slots = [c.alloc_slot() for _ in range(16)]
    c.reserve([(s, 1) for s in slots])  # sixteen requests of one token each hold sixteen pages
    with pytest.raises(CacheFull):
        c.reserve([(slots[0], 65)])
    with pytest.raises(CacheFull):
        c.alloc_slot()


def test_random_walk_keeps_invariants():
    rng = random.Random(3)
    c = make(max_tokens=64 * 40, max_slots=8)
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.25 and len(live) < 8:
            live[c.alloc_slot()] = 0
        elif op < 0.45 and live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            new = live[s] + rng.randint(1, 90)
            try:
                c.reserve([(s, new)])
                c.commit([(s, new)])
                live[s] = new
            except CacheFull:
                pass
        c.check()
        assert sorted(live) == c.live_slots()
        assert c.pages.held() >= sum(pages_for(n) for n in live.values())
    for s in list(live):
        c.free_slot(s)
    c.check()
    assert c.pages.held() == 0 and c.slots.held() == 0


def test_key_splits_of_single_token_attention():
    """The choice of how many pieces a sequence's keys are cut into: short contexts are not cut, a
    piece keeps at least 256 keys, few sequences are cut until every SM has work, and a batch
    that fills the machine a little more than once is cut so that its last wave is not thin."""
    from gophonic_b200.parts.attention import choose_splits
    for units in (1, 8, 64, 300, 512, 4000):
        assert choose_splits(units, 1) == 1
        assert choose_splits(units, 255) == 1
        for kv_len in (256, 1000, 4096, 32768):
            s = choose_splits(units, kv_len)
            assert 1 <= s <= max(1, min(32, kv_len // 256))
    # the cases the model was fitted to (kv heads 8, 4096 keys, 148 SMs)
    assert choose_splits(8, 4096) == 16          # one sequence
    assert choose_splits(64, 4096) == 4          # eight: 256 CTAs for 296 places
    assert choose_splits(96, 4096) == 3
    assert choose_splits(128, 4096) == 2
    assert choose_splits(256, 4096) == 1         # 32 sequences: one wave, nearly full
    assert choose_splits(384, 4096) == 3         # 48: uncut, 88 CTAs would run alone after the first 296
    assert choose_splits(512, 4096) == 1         # 64: two waves, the second well filled
    assert choose_splits(640, 4096) in (3, 4)    # 80: two full waves and 48 CTAs
    assert choose_splits(896, 4096) == 1         # 112: three waves and more are left uncut
    assert choose_splits(5000, 4096) == 1


def test_a_page_is_cleared_when_it_is_handed_out():
    """What an earlier sequence left in a page (here: NaN everywhere) is gone when the page is given
    to another one, in every plane of every group; pages nobody was given keep their contents."""
    c = make(max_tokens=64 * 6, requests=[(KVRequest(2, 16), None), (KVRequest(1, 8, 32), None), (KVRequest(2, 16), None)])
    for group in (c._k, c._v):
        for t in group.values():
            t.fill_(float("nan"))
    s = c.alloc_slot()
    c.reserve([(s, 130)])
    held = c._pages_of[s]
    assert len(held) == 3 and c.block_table[s, :3].tolist() == held
    free = [p for p in range(c.n_pages) if p not in held]
    for group in (c._k, c._v):
        for t in group.values():
            assert (t[:, held] == 0).all()
            assert torch.isnan(t[:, free]).all()
    c.commit([(s, 130)])
    c.reserve([(s, 193)])       # one more page: only that one is cleared, the sequence's own stay
    c._k[(2, 16, 0)][:, held[0]] = 5.0
    c.reserve([(s, 200)])
    assert (c._k[(2, 16, 0)][:, held[0]] == 5.0).all()
    c.check()


def test_marks_bring_a_sequence_back_with_its_state():
    c = make(max_tokens=64 * 6, requests=[(KVRequest(2, 16), None), (StateRequest((3,), torch.float32), None)])
    s = c.alloc_slot()
    c.reserve([(s, 70)])
    c.commit([(s, 70)])
    state = c.view(1).state
    state[s] = torch.tensor([1.0, 2.0, 3.0])
    mark = c.snapshot(s)
    c.reserve([(s, 200)])
    c.commit([(s, 200)])
    state[s] = torch.tensor([9.0, 9.0, 9.0])
    assert c.pages.held() == 4
    with pytest.raises(CacheError, match="cannot be truncated"):
        c.truncate(s, 70)
    c.restore(s, mark)
    assert c.length(s) == 70 and c.pages.held() == 2 and state[s].tolist() == [1.0, 2.0, 3.0]
    c.check()
    other = c.alloc_slot()
    with pytest.raises(CacheError, match="not of slot"):
        c.restore(other, mark)
    c.truncate(s, 70)      # to its own length: nothing to cut
    c.restore(s, mark)
    c.reserve([(s, 64)]) if False else None
    c.free_slot(s)
    with pytest.raises(CacheError, match="not live"):
        c.restore(s, mark)
    c.check()
