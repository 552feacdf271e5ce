"""``tokenizer train``: learn a byte-level BPE vocabulary and register it as an artifact
(reference: ``ajllm/workflows/tokenizer_train.py:23-65``). The manifest additionally records the
sha256 of ``vocab.json`` / ``merges.txt`` and their joint fingerprint."""

from __future__ import annotations

from typing import Any

from ajllm_b200.artifacts import ArtifactPaths, file_sha256, fingerprint_of, write_manifest
from ajllm_b200.config import LoadedConfig, check_dataset, check_tokenizer
from ajllm_b200.tokenization import save_vocab_and_merges, train_bpe
from ajllm_b200.workflows.common import dump_yaml, project_path


def run(config: LoadedConfig) -> dict[str, Any]:
    data = config.data
    dataset, tokenizer = data["dataset"], data["tokenizer"]
    check_dataset(dataset)
    check_tokenizer(tokenizer)
    split = str(data.get("split", "train"))
    if split not in dataset["splits"]:
        raise ValueError(f"Dataset has no '{split}' split")
    corpus = project_path(config.project_root, dataset["splits"][split])
    out_dir = ArtifactPaths(config.project_root).tokenizer(tokenizer["name"])
    out_dir.mkdir(parents=True, exist_ok=True)
    specials = list(tokenizer.get("special_tokens", []) or [])
    pre = tokenizer.get("pretokenization", {}) or {}
    vocab, merges = train_bpe(corpus, int(tokenizer["vocab_size"]), specials,
                              parallel=bool(pre.get("parallel", True)), num_processes=pre.get("num_processes"),
                              chunk_size_bytes=int(pre.get("chunk_size_bytes", 8 << 20)))
    save_vocab_and_merges(vocab, merges, out_dir / "vocab.json", out_dir / "merges.txt")
    dump_yaml(out_dir / "resolved_config.yaml", data)
    hashes = {name: file_sha256(out_dir / name) for name in ("vocab.json", "merges.txt")}
    manifest = {
        "name": tokenizer["name"], "dataset": dataset["name"], "source_split": split, "source_path": str(corpus),
        "source_size_bytes": corpus.stat().st_size, "vocab_size": len(vocab), "special_tokens": specials,
        "merge_count": len(merges), "files": {"vocab": "vocab.json", "merges": "merges.txt"},
        "hashes": hashes, "fingerprint": fingerprint_of(hashes),
    }
    write_manifest(out_dir / "manifest.json", "tokenizer", manifest)
    return {"output_dir": str(out_dir), **manifest}
