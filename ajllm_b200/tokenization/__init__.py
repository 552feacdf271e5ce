"""Byte-level BPE: training, serialisation, encoding and decoding."""

from ajllm_b200.tokenization.bpe_trainer import train_bpe
from ajllm_b200.tokenization.serialization import load_vocab_and_merges, save_vocab_and_merges
from ajllm_b200.tokenization.tokenizer import Tokenizer

__all__ = ["train_bpe", "load_vocab_and_merges", "save_vocab_and_merges", "Tokenizer"]
