"""``tokenizer encode``: turn dataset splits into native-endian ``uint32`` token files
(reference: ``ajllm/workflows/tokenizer_encode.py:23-83``). Each split entry also records its sha256 and
the manifest records the fingerprint of the tokenizer that produced it, which ``lm train`` verifies."""

from __future__ import annotations

from typing import Any

from ajllm_b200.artifacts import ArtifactPaths, file_sha256, open_tokenizer_artifact, write_manifest
from ajllm_b200.config import LoadedConfig, check_dataset, check_tokenizer
from ajllm_b200.tokenization import Tokenizer
from ajllm_b200.workflows.common import dump_yaml, project_path


def run(config: LoadedConfig) -> dict[str, Any]:
    data = config.data
    dataset, tokenizer_cfg = data["dataset"], data["tokenizer"]
    check_dataset(dataset)
    check_tokenizer(tokenizer_cfg)
    tok_dir, tok_manifest = open_tokenizer_artifact(config.project_root, tokenizer_cfg["name"])
    tokenizer = Tokenizer.from_files(tok_dir / tok_manifest["files"]["vocab"], tok_dir / tok_manifest["files"]["merges"],
                                     tok_manifest.get("special_tokens", []))
    out_dir = ArtifactPaths(config.project_root).encoded(dataset["name"], tokenizer_cfg["name"])
    out_dir.mkdir(parents=True, exist_ok=True)
    enc = data.get("encoding", {}) or {}
    max_bytes = enc.get("max_pretoken_bytes", 8192)
    strategy = str(enc.get("long_pretoken_strategy", "byte_fallback"))
    splits: dict[str, Any] = {}
    for split in data.get("splits", list(dataset["splits"])):
        if split not in dataset["splits"]:
            raise ValueError(f"Dataset has no '{split}' split")
        source = project_path(config.project_root, dataset["splits"][split])
        target = out_dir / f"{split}.uint32"
        count = tokenizer.encode_file_to_disk(
            source, target, chunk_size=int(enc.get("chunk_size", 16 << 20)), parallel=bool(enc.get("parallel", True)),
            num_processes=enc.get("num_processes"), buffer_tokens=int(enc.get("buffer_tokens", 65_536)),
            max_pretoken_bytes=None if max_bytes is None else int(max_bytes), long_pretoken_strategy=strategy)
        splits[split] = {"path": target.name, "token_count": count, "size_bytes": target.stat().st_size,
                         "source_path": str(source), "encoding_stats": dict(tokenizer.last_encoding_stats),
                         "sha256": file_sha256(target)}
    dump_yaml(out_dir / "resolved_config.yaml", data)
    manifest = {
        "dataset": dataset["name"], "tokenizer": tokenizer_cfg["name"], "vocab_size": tok_manifest["vocab_size"],
        "dtype": "uint32", "byte_order": "native",
        "encoding": {"max_pretoken_bytes": max_bytes, "long_pretoken_strategy": strategy},
        "tokenizer_fingerprint": tok_manifest.get("fingerprint"), "splits": splits,
    }
    write_manifest(out_dir / "manifest.json", "encoded_dataset", manifest)
    return {"output_dir": str(out_dir), **manifest}
