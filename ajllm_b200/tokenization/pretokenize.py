"""Pre-tokenisation shared by BPE training and encoding (reference: ``ajllm/tokenization/corpus.py``).

Text is cut at special tokens first (they never take part in merges), and each remaining segment is
split with the GPT-2 pattern. ``chunk_boundaries`` finds byte offsets at which a large corpus can be
split for worker processes without cutting a document: every interior boundary is moved forward to the
next occurrence of the document separator.
"""

from __future__ import annotations

import os
from collections.abc import Iterator
from typing import BinaryIO

import regex

GPT2_SPLIT = regex.compile(r"""'(?:[sdmt]|ll|ve|re)| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+""")


def special_splitter(special_tokens: list[str]) -> regex.Pattern[str] | None:
    """Capturing alternation of the special tokens, longest first so overlapping tokens resolve greedily."""
    if not special_tokens:
        return None
    ordered = sorted(special_tokens, key=len, reverse=True)
    return regex.compile("(" + "|".join(regex.escape(token) for token in ordered) + ")")


def pretokens(text: str, special_tokens: list[str], keep_special: bool) -> Iterator[str]:
    splitter = special_splitter(special_tokens)
    if splitter is None:
        for match in GPT2_SPLIT.finditer(text):
            yield match.group(0)
        return
    specials = frozenset(special_tokens)
    for piece in splitter.split(text):
        if not piece:
            continue
        if piece in specials:
            if keep_special:
                yield piece
            continue
        for match in GPT2_SPLIT.finditer(piece):
            yield match.group(0)


def corpus_lines(path: str) -> Iterator[str]:
    with open(path, encoding="utf-8") as handle:
        yield from handle


def chunk_boundaries(handle: BinaryIO, wanted_chunks: int, separator: bytes, probe_bytes: int = 4096) -> list[int]:
    """Sorted, de-duplicated byte offsets ``[0, ..., size]``; interior offsets sit on ``separator``."""
    if wanted_chunks < 1:
        raise ValueError("desired_num_chunks must be positive")
    handle.seek(0, os.SEEK_END)
    size = handle.tell()
    if size == 0:
        return [0]
    step = max(1, size // wanted_chunks)
    cuts = {0, size}
    for index in range(1, wanted_chunks):
        cursor = index * step
        found = size
        while cursor < size:
            handle.seek(cursor)
            window = handle.read(probe_bytes)
            if not window:
                break
            hit = window.find(separator)
            if hit >= 0:
                found = cursor + hit
                break
            cursor += probe_bytes
        cuts.add(found)
    handle.seek(0)
    return sorted(cuts)
