"""Resolve named artifacts and verify what their manifests promise.

The reference registry only joins a path with ``read_manifest`` (``ajllm/artifacts/registry.py:12-19``)
although its README describes hash verification. Here a manifest that lists ``hashes`` is checked
against the files on disk, and an encoded dataset that records the tokenizer fingerprint it was
produced with is checked against the tokenizer artifact that a training run is about to use.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any

from ajllm_b200.artifacts.layout import ArtifactPaths
from ajllm_b200.artifacts.manifests import file_sha256, fingerprint_of, read_manifest


class LineageError(ValueError):
    """An artifact on disk does not match its manifest, or two artifacts do not belong together."""


def _verify_hashes(directory: Path, manifest: dict[str, Any]) -> None:
    recorded = manifest.get("hashes")
    if not isinstance(recorded, dict):
        return
    for name, expected in recorded.items():
        target = directory / name
        if not target.is_file():
            raise LineageError(f"{directory}: manifest lists {name}, which is missing")
        if file_sha256(target) != expected:
            raise LineageError(f"{directory}: {name} does not match the sha256 in its manifest")
    declared = manifest.get("fingerprint")
    if declared is not None and declared != fingerprint_of(recorded):
        raise LineageError(f"{directory}: manifest fingerprint does not match its hash table")


def open_tokenizer_artifact(project_root: Path, name: str, verify: bool = True) -> tuple[Path, dict[str, Any]]:
    directory = ArtifactPaths(project_root).tokenizer(name)
    manifest = read_manifest(directory / "manifest.json")
    if verify:
        _verify_hashes(directory, manifest)
    return directory, manifest


def open_encoded_artifact(project_root: Path, dataset: str, tokenizer: str,
                          verify: bool = True) -> tuple[Path, dict[str, Any]]:
    directory = ArtifactPaths(project_root).encoded(dataset, tokenizer)
    manifest = read_manifest(directory / "manifest.json")
    if verify:
        for split, entry in (manifest.get("splits") or {}).items():
            digest = entry.get("sha256") if isinstance(entry, dict) else None
            if digest is not None and file_sha256(directory / entry["path"]) != digest:
                raise LineageError(f"{directory}: split '{split}' does not match the sha256 in its manifest")
    return directory, manifest


def check_lineage(tokenizer_manifest: dict[str, Any], encoded_manifest: dict[str, Any]) -> None:
    """Refuse to train on tokens that were produced by a different tokenizer build."""
    want = encoded_manifest.get("tokenizer_fingerprint")
    have = tokenizer_manifest.get("fingerprint")
    if want is not None and have is not None and want != have:
        raise LineageError(
            "encoded dataset was produced with a different tokenizer build "
            f"(dataset records {want[:12]}…, tokenizer is {have[:12]}…)"
        )
