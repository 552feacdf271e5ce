"""Byte-level BPE encoder / decoder (reference: ``ajllm/tokenization/tokenizer.py:92-388``).

Encoding: special tokens map straight to their ids; every other pre-token is split into bytes and the
applicable merge of lowest rank is applied until none applies. Pre-tokens longer than
``max_pretoken_bytes`` follow ``long_pretoken_strategy``: ``bpe`` (merge anyway), ``byte_fallback`` (emit
raw byte ids, counted in the statistics) or ``error``. Files are encoded to native-endian ``uint32`` by
worker processes over newline-aligned, UTF-8-safe byte ranges; parts are concatenated in order and
moved into place atomically, so parallel and serial output are byte-identical. Per-pre-token results
are memoised, which the reference does not do.
"""

from __future__ import annotations

import codecs
import os
import shutil
import tempfile
from array import array
from collections.abc import Iterable, Iterator
from concurrent.futures import ProcessPoolExecutor
from pathlib import Path

from ajllm_b200.tokenization.pretokenize import pretokens
from ajllm_b200.tokenization.serialization import load_vocab_and_merges

LONG_PRETOKEN_STRATEGIES = ("bpe", "byte_fallback", "error")
_CACHE_LIMIT = 1 << 18


def new_encoding_stats() -> dict[str, int]:
    return {"fallback_pretoken_count": 0, "fallback_bytes": 0, "largest_pretoken_bytes": 0}


def _fold_stats(into: dict[str, int], part: dict[str, int]) -> None:
    into["fallback_pretoken_count"] += part["fallback_pretoken_count"]
    into["fallback_bytes"] += part["fallback_bytes"]
    into["largest_pretoken_bytes"] = max(into["largest_pretoken_bytes"], part["largest_pretoken_bytes"])


class Tokenizer:
    def __init__(self, vocab: dict[int, bytes], merges: list[tuple[bytes, bytes]],
                 special_tokens: list[str] | None = None, max_pretoken_bytes: int | None = None,
                 long_pretoken_strategy: str = "bpe") -> None:
        self.vocab = dict(vocab)
        self.merges = list(merges)
        self.special_tokens = list(special_tokens or [])
        self.id_to_token = self.vocab
        self.token_to_id = {token: token_id for token_id, token in self.vocab.items()}
        self.merge_rank = {pair: rank for rank, pair in enumerate(self.merges)}
        self.max_pretoken_bytes = max_pretoken_bytes
        self.long_pretoken_strategy = long_pretoken_strategy
        self._check_long_options(max_pretoken_bytes, long_pretoken_strategy)
        self.last_encoding_stats = new_encoding_stats()
        self._memo: dict[bytes, tuple[int, ...]] = {}
        absent = [t for t in self.special_tokens if t.encode("utf-8") not in self.token_to_id]
        if absent:
            raise ValueError(f"Special tokens are missing from the vocabulary: {absent}")

    @classmethod
    def from_files(cls, vocab_path: str | Path, merges_path: str | Path,
                   special_tokens: list[str] | None = None) -> "Tokenizer":
        vocab, merges = load_vocab_and_merges(vocab_path, merges_path)
        return cls(vocab, merges, special_tokens)

    # ---------------------------------------------------------------- core
    def _check_long_options(self, max_bytes: int | None, strategy: str) -> None:
        if strategy not in LONG_PRETOKEN_STRATEGIES:
            raise ValueError("long_pretoken_strategy must be one of: " + ", ".join(sorted(LONG_PRETOKEN_STRATEGIES)))
        if max_bytes is not None and max_bytes <= 0:
            raise ValueError("max_pretoken_bytes must be positive or None")
        if strategy == "byte_fallback" and any(bytes([b]) not in self.token_to_id for b in range(256)):
            raise ValueError("byte_fallback requires all 256 byte tokens in the vocabulary")

    def _merge_bytes(self, data: bytes) -> tuple[int, ...]:
        cached = self._memo.get(data)
        if cached is not None:
            return cached
        parts = [bytes([b]) for b in data]
        rank_of = self.merge_rank
        while len(parts) > 1:
            best_rank, best_at = None, -1
            for at in range(len(parts) - 1):
                rank = rank_of.get((parts[at], parts[at + 1]))
                if rank is not None and (best_rank is None or rank < best_rank):
                    best_rank, best_at = rank, at
            if best_rank is None:
                break
            parts[best_at:best_at + 2] = [parts[best_at] + parts[best_at + 1]]
        ids = tuple(self.token_to_id[part] for part in parts)
        if len(self._memo) < _CACHE_LIMIT:
            self._memo[data] = ids
        return ids

    def encode_iter(self, text: str, *, max_pretoken_bytes: int | None = None,
                    long_pretoken_strategy: str | None = None, stats: dict[str, int] | None = None) -> Iterator[int]:
        limit = self.max_pretoken_bytes if max_pretoken_bytes is None else max_pretoken_bytes
        strategy = self.long_pretoken_strategy if long_pretoken_strategy is None else long_pretoken_strategy
        self._check_long_options(limit, strategy)
        tally = stats if stats is not None else new_encoding_stats()
        for key, value in new_encoding_stats().items():
            tally.setdefault(key, value)
        specials = frozenset(self.special_tokens)
        for piece in pretokens(text, self.special_tokens, keep_special=True):
            if piece in specials:
                yield self.token_to_id[piece.encode("utf-8")]
                continue
            data = piece.encode("utf-8")
            if len(data) > tally["largest_pretoken_bytes"]:
                tally["largest_pretoken_bytes"] = len(data)
            if limit is not None and len(data) > limit:
                if strategy == "error":
                    raise ValueError(f"Pre-token is {len(data)} bytes, exceeding max_pretoken_bytes={limit}")
                if strategy == "byte_fallback":
                    tally["fallback_pretoken_count"] += 1
                    tally["fallback_bytes"] += len(data)
                    for b in data:
                        yield self.token_to_id[bytes([b])]
                    continue
            yield from self._merge_bytes(data)
        if stats is None:
            self.last_encoding_stats = tally

    def encode(self, text: str, *, max_pretoken_bytes: int | None = None,
               long_pretoken_strategy: str | None = None) -> list[int]:
        return list(self.encode_iter(text, max_pretoken_bytes=max_pretoken_bytes,
                                     long_pretoken_strategy=long_pretoken_strategy))

    def encode_lines(self, lines: Iterable[str]) -> Iterator[int]:
        for line in lines:
            yield from self.encode_iter(line)

    def decode(self, token_ids: Iterable[int]) -> str:
        return b"".join(self.id_to_token[int(t)] for t in token_ids).decode("utf-8", errors="replace")

    # ---------------------------------------------------------------- files
    @staticmethod
    def file_chunk_ranges(file_name: str | Path, chunk_size: int) -> list[tuple[int, int]]:
        """Byte ranges that end after a newline when one exists in the window, else on a UTF-8 boundary."""
        if chunk_size < 4:
            raise ValueError("chunk_size must be at least 4 bytes")
        ranges: list[tuple[int, int]] = []
        with Path(file_name).open("rb") as handle:
            begin = 0
            while True:
                handle.seek(begin)
                window = handle.read(chunk_size)
                if not window:
                    break
                cut = window.rfind(b"\n") + 1
                if cut == 0:
                    cut = len(window)
                    if len(window) == chunk_size:
                        # do not split a multi-byte character, nor a "\r\n" pair
                        while cut > 0 and (window[cut - 1] & 0xC0) == 0x80:
                            cut -= 1
                        if cut > 0 and window[cut - 1] >= 0xC0:
                            cut -= 1
                        if cut == 0:
                            cut = len(window)
                            while cut > 0 and (window[cut - 1] & 0xC0) == 0x80:
                                cut -= 1
                            cut -= 1
                        if cut > 0 and window[cut - 1] == 0x0D:
                            cut -= 1
                if cut <= 0:
                    raise ValueError("chunk_size is too small for a UTF-8 character")
                ranges.append((begin, begin + cut))
                begin += cut
        return ranges

    _file_chunk_ranges = file_chunk_ranges

    def encode_file_to_disk(self, input_path: str | Path, output_path: str | Path, chunk_size: int = 16 << 20,
                            parallel: bool = True, num_processes: int | None = None, buffer_tokens: int = 65_536,
                            max_pretoken_bytes: int | None = 8192,
                            long_pretoken_strategy: str = "byte_fallback") -> int:
        source, target = Path(input_path), Path(output_path)
        target.parent.mkdir(parents=True, exist_ok=True)
        if chunk_size < 4:
            raise ValueError("chunk_size must be at least 4 bytes")
        if buffer_tokens <= 0:
            raise ValueError("buffer_tokens must be positive")
        self._check_long_options(max_pretoken_bytes, long_pretoken_strategy)
        self.last_encoding_stats = new_encoding_stats()
        ranges = self.file_chunk_ranges(source, chunk_size)
        if not ranges:
            target.write_bytes(b"")
            return 0
        workers = min(num_processes or (os.cpu_count() or 1), len(ranges))
        fd, scratch = tempfile.mkstemp(prefix=f".{target.name}.", suffix=".tmp", dir=target.parent)
        os.close(fd)
        total = 0
        try:
            if not parallel or workers <= 1:
                total = self._encode_serial(source, Path(scratch), buffer_tokens, max_pretoken_bytes,
                                            long_pretoken_strategy)
            else:
                with tempfile.TemporaryDirectory(prefix="tokenizer-chunks-", dir=target.parent) as part_dir:
                    jobs = [(i, str(source), lo, hi, str(Path(part_dir) / f"{i:08d}.bin"))
                            for i, (lo, hi) in enumerate(ranges)]
                    init = (self.vocab, self.merges, self.special_tokens, max_pretoken_bytes,
                            long_pretoken_strategy, buffer_tokens)
                    with ProcessPoolExecutor(max_workers=workers, initializer=_worker_init, initargs=init) as pool, \
                            open(scratch, "wb") as sink:
                        for part_path, count, part_stats in pool.map(_worker_encode, jobs):
                            with open(part_path, "rb") as part:
                                shutil.copyfileobj(part, sink, length=1 << 20)
                            os.unlink(part_path)
                            total += count
                            _fold_stats(self.last_encoding_stats, part_stats)
            os.replace(scratch, target)
        except BaseException:
            if os.path.exists(scratch):
                os.unlink(scratch)
            raise
        return total

    def _encode_serial(self, source: Path, sink_path: Path, buffer_tokens: int, max_pretoken_bytes: int | None,
                       strategy: str) -> int:
        total = 0
        pending = array("I")
        with source.open(encoding="utf-8") as lines, sink_path.open("wb") as sink:
            for line in lines:
                for token_id in self.encode_iter(line, max_pretoken_bytes=max_pretoken_bytes,
                                                 long_pretoken_strategy=strategy, stats=self.last_encoding_stats):
                    pending.append(token_id)
                    total += 1
                    if len(pending) >= buffer_tokens:
                        pending.tofile(sink)
                        pending = array("I")
            if pending:
                pending.tofile(sink)
        return total

    def decode_file(self, input_path: str | Path, output_path: str | Path, chunk_tokens: int = 65_536) -> int:
        decoder = codecs.getincrementaldecoder("utf-8")(errors="replace")
        target = Path(output_path)
        target.parent.mkdir(parents=True, exist_ok=True)
        total = 0
        with Path(input_path).open("rb") as source, target.open("w", encoding="utf-8") as sink:
            while True:
                ids = array("I")
                try:
                    ids.fromfile(source, chunk_tokens)
                except EOFError:
                    pass
                if not ids:
                    break
                total += len(ids)
                sink.write(decoder.decode(b"".join(self.id_to_token[int(t)] for t in ids), final=False))
            sink.write(decoder.decode(b"", final=True))
        return total


_WORKER: Tokenizer | None = None
_WORKER_BUFFER = 65_536


def _worker_init(vocab, merges, special_tokens, max_pretoken_bytes, strategy, buffer_tokens) -> None:
    global _WORKER, _WORKER_BUFFER
    _WORKER = Tokenizer(vocab, merges, special_tokens, max_pretoken_bytes=max_pretoken_bytes,
                        long_pretoken_strategy=strategy)
    _WORKER_BUFFER = buffer_tokens


def _worker_encode(job: tuple[int, str, int, int, str]) -> tuple[str, int, dict[str, int]]:
    _, file_name, lo, hi, part_path = job
    assert _WORKER is not None, "encoder worker was not initialised"
    with open(file_name, "rb") as handle:
        handle.seek(lo)
        text = handle.read(hi - lo).decode("utf-8")
    text = text.replace("\r\n", "\n").replace("\r", "\n")   # same newline handling as text-mode reading
    stats = new_encoding_stats()
    count = 0
    pending = array("I")
    with open(part_path, "wb") as sink:
        for token_id in _WORKER.encode_iter(text, stats=stats):
            pending.append(token_id)
            count += 1
            if len(pending) >= _WORKER_BUFFER:
                pending.tofile(sink)
                pending = array("I")
        if pending:
            pending.tofile(sink)
    return part_path, count, stats
