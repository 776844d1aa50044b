"""Prefix cache bookkeeping on the host: eviction order, reference counts and cost at scale."""
import random
import time

from oxibonsai_b200.runtime.prefix_cache import PrefixCache


class Pool:
    def __init__(self):
        self.ref = {}

    def retain(self, pages):
        for p in pages:
            self.ref[p] = self.ref.get(p, 0) + 1

    def release(self, pages):
        for p in pages:
            self.ref[p] -= 1
            if self.ref[p] == 0:
                del self.ref[p]


def _oldest_leaf(pc):
    best = None
    for leaf in pc._leaves():
        if best is None or leaf.last_used < best.last_used:
            best = leaf
    return best


def test_eviction_takes_the_least_recently_used_leaf_and_every_leaf_stays_evictable():
    rng = random.Random(5)
    pool = Pool()
    pc = PrefixCache(4, 60, pool.retain, pool.release)
    page = 0
    for _ in range(1500):
        tokens = [rng.randrange(3) for _ in range(rng.randrange(4, 40))]
        if rng.random() < 0.5:
            pages = pc.lookup(tokens)
            assert all(p in pool.ref for p in pages)
        else:
            n = len(tokens) // 4
            pc.insert(tokens, list(range(page, page + n)))
            page += n
        if rng.random() < 0.1:
            want = _oldest_leaf(pc)
            stamp = want.last_used if want else None
            assert pc._evict_one() == (want is not None)
            rest = _oldest_leaf(pc)
            assert want is None or rest is None or rest.last_used >= stamp
        live = {id(n) for used, _, n in pc._heap
                if not n.children and used == n.last_used and n.parent is not None and n.parent.children.get(n.key) is n}
        assert all(id(leaf) in live for leaf in pc._leaves())
        assert pc.size == len(pool.ref) <= 60 and len(pc._heap) <= 4 * pc.size + 1025
    pc.clear()
    assert pc.size == 0 and not pool.ref and not pc.root.children


def test_a_full_cache_takes_new_prompts_without_walking_the_trie_per_page():
    rng = random.Random(1)
    pool = Pool()
    pc = PrefixCache(16, 20000, pool.retain, pool.release)
    page = 0
    for _ in range(20000 // 64 + 1):
        pc.insert([rng.randrange(50000) for _ in range(64 * 16)], list(range(page, page + 64)))
        page += 64
    assert pc.size == 20000
    t0 = time.perf_counter()
    pc.insert([rng.randrange(50000) for _ in range(4096)], list(range(page, page + 256)))       # 256 evictions
    assert pc.evict(1000) == 1000
    assert time.perf_counter() - t0 < 0.5          # ~5 ms; a walk over 20 000 nodes per evicted page took seconds
    assert pc.size == 19000 == len(pool.ref)
