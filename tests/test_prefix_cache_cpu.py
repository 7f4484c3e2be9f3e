"""Host logic of the paged prefix cache against a restatement of the reference's entry rules.

The model below follows src/model/executor.rs of the reference: store (:1584-1636) replaces the
entry of the same key, or without key of the same tokens, and drops the oldest entry when the
deque is full; lookup without key (:1352-1375) takes the longest snapshot that is a prefix of the
prompt, later entry on ties; keyed lookup (:1425-1515) takes, among that key's entries not longer
than the prompt, the longest common prefix (zero excluded), later entry on ties; a hit moves the
entry to the back (:1388-1398).  Default 8 entries, clamped to 1..64 (:266-279).
"""
import importlib

import numpy as np
import pytest

mfk = importlib.import_module("test-burn_b200")


class Model:
    def __init__(self, max_entries):
        self.max = min(max(max_entries, 1), 64)
        self.entries = []  # (tokens tuple, key or None, pages list)

    def store(self, tokens, key, pages):
        tokens = tuple(tokens)
        if not tokens:
            return []
        freed = []
        for i, (t, k, p) in enumerate(self.entries):
            if (k == key) if key is not None else (t == tokens):
                freed += p
                del self.entries[i]
                break
        if len(self.entries) >= self.max:
            freed += self.entries.pop(0)[2]
        self.entries.append((tokens, key, list(pages)))
        return freed

    def lookup(self, prompt, key):
        prompt = tuple(prompt)
        best, best_len = None, 0
        for i, (t, k, p) in enumerate(self.entries):
            if len(t) == 0 or len(t) > len(prompt):
                continue
            if key is not None:
                if k != key:
                    continue
                m = 0
                while m < len(t) and t[m] == prompt[m]:
                    m += 1
                if m == 0:
                    continue
                if m >= best_len:
                    best, best_len = i, m
            elif t == prompt[:len(t)] and len(t) >= best_len:
                best, best_len = i, len(t)
        if best is None:
            return 0, []
        e = self.entries.pop(best)
        self.entries.append(e)
        return best_len, e[2]


def test_page_pool_counts():
    pool = mfk.PagePool(10)
    a = pool.alloc(4)
    assert sorted(a.tolist()) == [0, 1, 2, 3] and pool.free_count == 6
    pool.retain(a[:2])
    pool.release(a)
    assert pool.free_count == 8 and pool.refcount(int(a[0])) == 1 and pool.refcount(int(a[3])) == 0
    with pytest.raises(mfk.MetalError) as e:  # all or nothing
        pool.alloc(9)
    assert e.value.kind == "OutOfMemory" and pool.free_count == 8
    with pytest.raises(mfk.MetalError):
        pool.release(a[3:])  # already free
    with pytest.raises(mfk.MetalError):
        pool.retain(np.array([77], np.uint32))
    pool.release(a[:2])
    assert pool.free_count == 10
    pool.close()


def test_defaults_and_clamp():
    pool = mfk.PagePool(4096)
    assert int(mfk.lib.mf_prefix_cache_default_entries()) == 8
    for asked, kept in ((0, 1), (3, 3), (1000, 64)):
        cache = mfk.PrefixCache(pool, 16, asked)
        for i in range(70):
            pages = pool.alloc(1)
            cache.store([i + 1], pages)
            pool.release(pages)
        assert len(cache) == kept
        cache.close()
    assert pool.free_count == 4096  # destroy released what the entries held
    pool.close()


@pytest.mark.parametrize("seed", [1, 7, 42])
def test_entry_rules_follow_the_reference(seed):
    rng = np.random.default_rng(seed)
    P, n_pages = 4, 4096
    pool = mfk.PagePool(n_pages)
    cache = mfk.PrefixCache(pool, P, 5)
    model = Model(5)
    held = {}  # page id -> references held outside the library (live "sequences" + model entries)
    stems = [rng.integers(1, 6, size=12).tolist() for _ in range(3)]
    keys = [None, None, "chat-a", "chat-b"]
    for step in range(400):
        stem = stems[rng.integers(0, 3)]
        n = int(rng.integers(1, 13))
        tokens = stem[:n]
        if rng.random() < 0.3:
            tokens = tokens[:-1] + [int(rng.integers(6, 9))]
        key = keys[rng.integers(0, 4)]
        if rng.random() < 0.5:
            pages = pool.alloc((len(tokens) + P - 1) // P)
            cache.store(tokens, pages, key)
            model.store(tokens, key, pages.tolist())
            pool.release(pages)  # the sequence that produced the prefix ends; the entry keeps the pages
        else:
            prompt = tokens + rng.integers(1, 6, size=int(rng.integers(0, 4))).tolist()
            got_len, got_pages = cache.lookup(prompt, key)
            want_len, want_pages = model.lookup(prompt, key)
            assert got_len == want_len
            assert got_pages.tolist() == want_pages[:(want_len + P - 1) // P]
            if got_len:
                for pg in got_pages:
                    assert pool.refcount(int(pg)) >= 2  # the entry and the caller
                pool.release(got_pages)
        assert len(cache) == len(model.entries)
        live = sum(len(p) for _, _, p in model.entries)
        assert pool.free_count == n_pages - live  # every page is either free or held by exactly the entries
    cache.close()
    assert pool.free_count == n_pages
    pool.close()


def test_partial_keyed_match_and_ties():
    pool = mfk.PagePool(64)
    cache = mfk.PrefixCache(pool, 4)
    a, b = pool.alloc(2), pool.alloc(2)
    cache.store([1, 2, 3, 4, 5, 6], a, key="k")
    cache.store([1, 2, 3, 9, 9], b)  # no key
    m, pages = cache.lookup([1, 2, 3, 4, 7, 7, 7], key="k")  # diverges after 4 tokens
    assert m == 4 and pages.tolist() == a[:1].tolist()
    pool.release(pages)
    m, pages = cache.lookup([1, 2, 3, 4, 5], key="k")  # the snapshot is longer than the prompt: rejected
    assert m == 0 and pages.size == 0
    m, pages = cache.lookup([1, 2, 3, 9, 9, 1], key="other")
    assert m == 0
    m, pages = cache.lookup([1, 2, 3, 9, 9, 1])  # without key only whole snapshots match
    assert m == 5 and pages.tolist() == b.tolist()
    pool.release(pages)
    m, _ = cache.lookup([1, 2, 3, 9], key=None)
    assert m == 0
    m, _ = cache.lookup([1, 2], key="")  # empty key never matches
    assert m == 0
    cache.close()
    pool.release(a)
    pool.release(b)
    assert pool.free_count == 64
    pool.close()
