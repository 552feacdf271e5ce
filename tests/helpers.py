"""Builders shared by the CPU tests: a throw-away project tree and tiny model configs."""

from __future__ import annotations

from pathlib import Path

import yaml

from ajllm_b200.config import LoadedConfig

TINY_MODEL = {"name": "tiny", "context_length": 16, "d_model": 32, "num_layers": 2, "num_heads": 4, "num_kv_heads": 2,
              "d_ff": 64, "position_encoding": {"type": "rope", "theta": 10000},
              "normalization": {"type": "rmsnorm", "placement": "pre"}, "feed_forward": {"type": "swiglu"}}

CORPUS = ("The lighthouse keeper counted seven copper coins before the bells rang.\n"
          "A small robot painted green lanterns — just once — and smiled.\n<|endoftext|>\n"
          "The night train followed the river until the tide turned, 3 times!\n"
          "Voices in the café remembered a song without words: “done”.\n<|endoftext|>\n") * 6


def make_project(root: Path) -> Path:
    (root / "pyproject.toml").write_text("[project]\nname='scratch'\n", encoding="utf-8")
    for sub in ("datasets", "tokenizers", "models", "runs"):
        (root / "configs" / sub).mkdir(parents=True, exist_ok=True)
    (root / "data").mkdir(exist_ok=True)
    (root / "data" / "train.txt").write_text(CORPUS, encoding="utf-8")
    (root / "data" / "validation.txt").write_text(CORPUS[: len(CORPUS) // 3], encoding="utf-8")
    (root / "configs" / "datasets" / "toy.yaml").write_text(yaml.safe_dump(
        {"name": "toy", "splits": {"train": "data/train.txt", "validation": "data/validation.txt"}}))
    (root / "configs" / "tokenizers" / "toy_bpe.yaml").write_text(yaml.safe_dump(
        {"name": "toy_bpe", "vocab_size": 290, "special_tokens": ["<|endoftext|>"],
         "pretokenization": {"parallel": False}}))
    (root / "configs" / "models" / "tiny.yaml").write_text(yaml.safe_dump(TINY_MODEL))
    return root


def loaded(root: Path, data: dict) -> LoadedConfig:
    return LoadedConfig(data, root / "configs" / "runs" / "inline.yaml", root, root / "configs")


def base_run(root: Path) -> dict:
    return {
        "dataset": yaml.safe_load((root / "configs/datasets/toy.yaml").read_text()),
        "tokenizer": yaml.safe_load((root / "configs/tokenizers/toy_bpe.yaml").read_text()),
        "model": dict(TINY_MODEL),
    }


def prepare_artifacts(root: Path) -> None:
    from ajllm_b200.workflows import tokenizer_encode, tokenizer_train

    tokenizer_train.run(loaded(root, {**base_run(root), "split": "train"}))
    tokenizer_encode.run(loaded(root, {**base_run(root), "encoding": {"parallel": False}}))


def train_config(root: Path, **training) -> dict:
    cfg = base_run(root)
    cfg.update({
        "experiment": "unit",
        "training": {"batch_size": 2, "max_steps": 2, **training},
        "optimizer": {"max_lr": 1e-3},
        "logging": {"log_interval": 1, "eval_interval": 1, "eval_batches": 1, "checkpoint_interval": 1},
        "runtime": {"device": "cpu", "seed": 3},
    })
    return cfg
