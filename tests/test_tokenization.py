import numpy as np
import pytest

from ajllm_b200.tokenization import Tokenizer, load_vocab_and_merges, save_vocab_and_merges, train_bpe
from tests.helpers import CORPUS

SPECIAL = ["<|endoftext|>"]


@pytest.fixture
def corpus(tmp_path):
    path = tmp_path / "corpus.txt"
    path.write_text(CORPUS, encoding="utf-8")
    return path


def test_round_trip_vocab_layout_and_special_tokens(corpus, tmp_path):
    vocab, merges = train_bpe(corpus, 300, SPECIAL, parallel=False)
    assert len(vocab) == 256 + len(merges) + 1
    assert all(vocab[i] == bytes([i]) for i in range(256))
    assert vocab[len(vocab) - 1] == b"<|endoftext|>"
    tok = Tokenizer(vocab, merges, SPECIAL)
    text = "Voices in the café — “done”. 日本語 <|endoftext|> tail"
    ids = tok.encode(text)
    assert tok.decode(ids) == text
    assert ids.count(len(vocab) - 1) == 1
    save_vocab_and_merges(vocab, merges, tmp_path / "v.json", tmp_path / "m.txt")
    v2, m2 = load_vocab_and_merges(tmp_path / "v.json", tmp_path / "m.txt")
    assert v2 == vocab and m2 == merges


def test_parallel_training_equals_serial(corpus):
    serial = train_bpe(corpus, 290, SPECIAL, parallel=False)
    parallel = train_bpe(corpus, 290, SPECIAL, parallel=True, num_processes=2, chunk_size_bytes=200)
    assert serial == parallel


def test_parallel_file_encoding_is_byte_identical(corpus, tmp_path):
    vocab, merges = train_bpe(corpus, 290, SPECIAL, parallel=False)
    tok = Tokenizer(vocab, merges, SPECIAL)
    n1 = tok.encode_file_to_disk(corpus, tmp_path / "a.uint32", parallel=False)
    n2 = tok.encode_file_to_disk(corpus, tmp_path / "b.uint32", chunk_size=97, parallel=True, num_processes=2)
    a, b = (tmp_path / "a.uint32").read_bytes(), (tmp_path / "b.uint32").read_bytes()
    assert n1 == n2 and a == b and len(a) == 4 * n1
    ids = np.frombuffer(a, dtype=np.uint32)
    assert tok.decode(ids.tolist()) == CORPUS
    assert tok.decode_file(tmp_path / "a.uint32", tmp_path / "back.txt") == n1
    assert (tmp_path / "back.txt").read_text(encoding="utf-8") == CORPUS


def test_long_pretoken_policies(corpus):
    vocab, merges = train_bpe(corpus, 280, SPECIAL, parallel=False)
    tok = Tokenizer(vocab, merges, SPECIAL)
    text = "x" * 50 + " ok"
    stats: dict = {}
    ids = list(tok.encode_iter(text, max_pretoken_bytes=10, long_pretoken_strategy="byte_fallback", stats=stats))
    assert stats["fallback_pretoken_count"] == 1 and stats["fallback_bytes"] == 50 and stats["largest_pretoken_bytes"] == 50
    assert tok.decode(ids) == text
    with pytest.raises(ValueError):
        tok.encode(text, max_pretoken_bytes=10, long_pretoken_strategy="error")
    with pytest.raises(ValueError):
        tok.encode(text, long_pretoken_strategy="nonsense")


def test_chunk_ranges_never_split_characters(tmp_path):
    path = tmp_path / "u.txt"
    path.write_text("é" * 40 + "\r\n" + "日" * 30, encoding="utf-8")
    data = path.read_bytes()
    for size in (4, 5, 7, 16):
        ranges = Tokenizer.file_chunk_ranges(path, size)
        assert ranges[0][0] == 0 and ranges[-1][1] == len(data)
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        for lo, hi in ranges:
            data[lo:hi].decode("utf-8")


@pytest.mark.needs_reference
def test_merges_and_ids_equal_the_reference(corpus, reference_path):
    from ajllm.tokenization.bpe_trainer import train_bpe as ref_train
    from ajllm.tokenization.tokenizer import Tokenizer as RefTokenizer

    ours = train_bpe(corpus, 300, SPECIAL, parallel=False)
    theirs = ref_train(corpus, 300, SPECIAL, parallel=False)
    assert ours[0] == theirs[0] and ours[1] == theirs[1]
    assert Tokenizer(*ours, SPECIAL).encode(CORPUS) == RefTokenizer(*theirs, SPECIAL).encode(CORPUS)
