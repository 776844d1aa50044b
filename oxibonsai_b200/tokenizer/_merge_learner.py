"""Greedy pair-merge learning with incremental counts.

Both trainers (``train_bpe`` and ``toolkit.BpeTrainer``; reference: crates/oxibonsai-tokenizer/src/trainer.rs) pick the most
frequent adjacent pair, merge it everywhere and repeat.  Recounting every pair of every word for each merge costs
O(merges x corpus); here the counts are kept up to date: a merge touches only the words that contain the pair (found through
an index from pairs to words), whose old pairs are subtracted and new pairs added.  The merges learned are the same as with a
full recount, ties included.
"""
from __future__ import annotations

from collections import Counter, defaultdict
from typing import Callable, Hashable, Iterator


class MergeLearner:
    """``words``: {tuple of symbols: count}.  ``make(a, b, index)`` names the symbol that merge number ``index`` creates.
    ``tie(pair)``: among pairs of equal count the one with the largest ``tie`` wins."""

    def __init__(self, words: dict[tuple, int], make: Callable[[Hashable, Hashable, int], Hashable], tie: Callable[[tuple], object]):
        self._words = [list(w) for w in words]
        self._counts = list(words.values())
        self._make, self._tie = make, tie
        self.pairs: Counter = Counter()
        self._where: dict[tuple, set[int]] = defaultdict(set)
        for i, (w, c) in enumerate(zip(self._words, self._counts)):
            for p in zip(w, w[1:]):
                self.pairs[p] += c
                self._where[p].add(i)
        self.learned = 0

    def best(self) -> tuple[tuple, int] | None:
        if not self.pairs:
            return None
        top = max(self.pairs.values())
        return max((p for p, c in self.pairs.items() if c == top), key=self._tie), top

    def merge(self, pair: tuple) -> Hashable:
        """Applies ``pair`` to every word and returns the new symbol."""
        a, b = pair
        new = self._make(a, b, self.learned)
        self.learned += 1
        pairs, where = self.pairs, self._where
        for i in where.pop(pair, ()):
            w, c = self._words[i], self._counts[i]
            out, k, hit = [], 0, False
            while k < len(w):
                if k + 1 < len(w) and w[k] == a and w[k + 1] == b:
                    out.append(new)
                    k += 2
                    hit = True
                else:
                    out.append(w[k])
                    k += 1
            if not hit:                                   # a stale index entry: an earlier merge consumed the pair here
                continue
            for p in zip(w, w[1:]):
                left = pairs[p] - c
                if left > 0:
                    pairs[p] = left
                else:
                    del pairs[p]
            for p in zip(out, out[1:]):
                pairs[p] += c
                where[p].add(i)
            self._words[i] = out
        pairs.pop(pair, None)
        return new

    def run(self, n_merges: int, min_count: int) -> Iterator[tuple[tuple, int, Hashable]]:
        """Yields (pair, count, new symbol) until ``n_merges`` were learned or the best pair is rarer than ``min_count``."""
        while self.learned < n_merges:
            found = self.best()
            if found is None or found[1] < min_count:
                return
            pair, count = found
            yield pair, count, self.merge(pair)
