"""Byte-level BPE training (reference behaviour: ``ajllm/tokenization/bpe_trainer.py:181-214``).

The learned merges must equal the reference's for the same corpus: pre-token counts are merged
greedily by pair frequency, ties go to the lexicographically *larger* pair of byte strings, and the
vocabulary is laid out as ids 0-255 = single bytes, then one id per merge, then the special tokens.

Implementation: every distinct pre-token is a mutable list of symbols with a multiplicity; pair
frequencies and a pair -> word-index inverted index are updated incrementally around each merge site
only; the best pair comes from a max-heap with lazy invalidation.
"""

from __future__ import annotations

import heapq
import os
from collections import Counter, defaultdict
from concurrent.futures import ProcessPoolExecutor
from pathlib import Path

from ajllm_b200.tokenization.pretokenize import chunk_boundaries, corpus_lines, pretokens

Pair = tuple[bytes, bytes]


class _Candidate:
    """Heap entry ordered by (higher count, then lexicographically larger pair) first."""

    __slots__ = ("count", "pair")

    def __init__(self, count: int, pair: Pair) -> None:
        self.count, self.pair = count, pair

    def __lt__(self, other: "_Candidate") -> bool:
        if self.count != other.count:
            return self.count > other.count
        return self.pair > other.pair


def _count_range(path: str, start: int, end: int, special_tokens: list[str]) -> Counter:
    with open(path, "rb") as handle:
        handle.seek(start)
        text = handle.read(end - start).decode("utf-8", errors="ignore")
    counts: Counter = Counter()
    for token in pretokens(text, special_tokens, keep_special=False):
        counts[token.encode("utf-8")] += 1
    return counts


def count_pretokens(input_path: str | Path, special_tokens: list[str], parallel: bool = True,
                    num_processes: int | None = None, chunk_size_bytes: int = 8 << 20) -> Counter:
    """``Counter`` of pre-token byte strings, counted serially or over document-aligned byte ranges."""
    path = Path(input_path)
    if not parallel or not special_tokens:
        counts: Counter = Counter()
        for line in corpus_lines(str(path)):
            for token in pretokens(line, special_tokens, keep_special=False):
                counts[token.encode("utf-8")] += 1
        return counts
    if chunk_size_bytes < 1:
        raise ValueError("chunk_size_bytes must be positive")
    size = path.stat().st_size
    wanted = max(1, -(-size // chunk_size_bytes))
    with path.open("rb") as handle:
        cuts = chunk_boundaries(handle, wanted, max(special_tokens, key=len).encode("utf-8"))
    ranges = list(zip(cuts[:-1], cuts[1:]))
    workers = min(num_processes or (os.cpu_count() or 1), max(1, len(ranges)))
    counts = Counter()
    if workers <= 1 or len(ranges) <= 1:
        for start, end in ranges:
            counts.update(_count_range(str(path), start, end, special_tokens))
        return counts
    with ProcessPoolExecutor(max_workers=workers) as pool:
        for part in pool.map(_count_range, [str(path)] * len(ranges), [r[0] for r in ranges],
                             [r[1] for r in ranges], [special_tokens] * len(ranges)):
            counts.update(part)
    return counts


def learn_merges(word_counts: Counter, num_merges: int) -> list[Pair]:
    words: list[list[bytes]] = []
    weights: list[int] = []
    for token, count in word_counts.items():
        words.append([bytes([b]) for b in token])
        weights.append(count)
    pair_count: dict[Pair, int] = defaultdict(int)
    where: dict[Pair, set[int]] = defaultdict(set)
    for index, symbols in enumerate(words):
        for pair in zip(symbols, symbols[1:]):
            pair_count[pair] += weights[index]
            where[pair].add(index)
    heap = [_Candidate(count, pair) for pair, count in pair_count.items()]
    heapq.heapify(heap)
    merges: list[Pair] = []
    while len(merges) < num_merges and heap:
        top = heapq.heappop(heap)
        if pair_count.get(top.pair, 0) != top.count or top.count <= 0:
            continue                      # stale entry
        left, right = top.pair
        joined = left + right
        touched: set[Pair] = set()
        for index in list(where.get(top.pair, ())):
            symbols, weight = words[index], weights[index]
            # remove this word's contribution, rewrite it, add the new contribution
            for pair in zip(symbols, symbols[1:]):
                pair_count[pair] -= weight
                touched.add(pair)
            for pair in set(zip(symbols, symbols[1:])):
                where[pair].discard(index)
            merged: list[bytes] = []
            cursor = 0
            while cursor < len(symbols):
                if cursor + 1 < len(symbols) and symbols[cursor] == left and symbols[cursor + 1] == right:
                    merged.append(joined)
                    cursor += 2
                else:
                    merged.append(symbols[cursor])
                    cursor += 1
            words[index] = merged
            for pair in zip(merged, merged[1:]):
                pair_count[pair] += weight
                where[pair].add(index)
                touched.add(pair)
        merges.append(top.pair)
        for pair in touched:
            count = pair_count.get(pair, 0)
            if count > 0:
                heapq.heappush(heap, _Candidate(count, pair))
            else:
                pair_count.pop(pair, None)
                where.pop(pair, None)
    return merges


def train_bpe(input_path: str | Path, vocab_size: int, special_tokens: list[str] | None = None, parallel: bool = True,
              num_processes: int | None = None, chunk_size_bytes: int = 8 << 20) -> tuple[dict[int, bytes], list[Pair]]:
    special_tokens = list(special_tokens or [])
    floor = 256 + len(special_tokens)
    if vocab_size < floor:
        raise ValueError(f"vocab_size must be at least {floor}")
    counts = count_pretokens(input_path, special_tokens, parallel, num_processes, chunk_size_bytes)
    merges = learn_merges(counts, vocab_size - floor)
    vocab = {i: bytes([i]) for i in range(256)}
    for left, right in merges:
        vocab[len(vocab)] = left + right
    for token in special_tokens:
        vocab[len(vocab)] = token.encode("utf-8")
    return vocab, merges
