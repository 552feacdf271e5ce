"""Artifact locations, manifests with content hashes, and lineage checks."""

from ajllm_b200.artifacts.layout import ArtifactPaths, new_run_id
from ajllm_b200.artifacts.manifests import file_sha256, fingerprint_of, read_manifest, write_manifest
from ajllm_b200.artifacts.registry import LineageError, open_encoded_artifact, open_tokenizer_artifact

__all__ = [
    "ArtifactPaths", "new_run_id", "file_sha256", "fingerprint_of", "read_manifest", "write_manifest",
    "LineageError", "open_encoded_artifact", "open_tokenizer_artifact",
]
