"""Machine-readable manifests (reference: ``ajllm/artifacts/manifests.py:11-30``).

Every manifest carries ``schema_version``, ``artifact_type`` and ``created_at`` followed by the
payload. The reference's committed manifests also carry ``hashes`` / ``fingerprint`` fields that none
of its code computes; here ``file_sha256`` and ``fingerprint_of`` produce them and the registry
verifies them.
"""

from __future__ import annotations

import hashlib
import json
import os
from datetime import datetime, timezone
from pathlib import Path
from typing import Any


def file_sha256(path: str | Path, chunk_bytes: int = 1 << 20) -> str:
    digest = hashlib.sha256()
    with Path(path).open("rb") as handle:
        while block := handle.read(chunk_bytes):
            digest.update(block)
    return digest.hexdigest()


def fingerprint_of(hashes: dict[str, str]) -> str:
    """Order-independent digest of a ``{file name: sha256}`` table."""
    digest = hashlib.sha256()
    for name in sorted(hashes):
        digest.update(name.encode("utf-8") + b"\0" + hashes[name].encode("ascii") + b"\n")
    return digest.hexdigest()


def write_manifest(path: str | Path, artifact_type: str, payload: dict[str, Any]) -> Path:
    target = Path(path)
    target.parent.mkdir(parents=True, exist_ok=True)
    document = {
        "schema_version": 1,
        "artifact_type": artifact_type,
        "created_at": datetime.now(timezone.utc).isoformat(),
    }
    document.update(payload)
    scratch = target.with_name(target.name + ".tmp")
    with scratch.open("w", encoding="utf-8") as handle:
        json.dump(document, handle, indent=2, ensure_ascii=False)
    os.replace(scratch, target)
    return target


def read_manifest(path: str | Path) -> dict[str, Any]:
    source = Path(path)
    if not source.is_file():
        raise FileNotFoundError(f"Artifact manifest does not exist: {source}")
    with source.open("r", encoding="utf-8") as handle:
        return json.load(handle)
