import json

import pytest
import yaml

from ajllm_b200.artifacts import ArtifactPaths, file_sha256, fingerprint_of, read_manifest, write_manifest
from ajllm_b200.artifacts.registry import LineageError, check_lineage, open_tokenizer_artifact
from ajllm_b200.config import ConfigError, check_model, check_parallel, check_tokenizer, load_run_config, set_dotted_value
from tests.helpers import make_project


def test_base_inheritance_component_resolution_and_deep_merge(tmp_path):
    root = make_project(tmp_path)
    runs = root / "configs" / "runs"
    (runs / "parent.yaml").write_text(yaml.safe_dump(
        {"dataset": "toy", "tokenizer": "toy_bpe", "model": "tiny", "optimizer": {"max_lr": 1e-3, "beta1": 0.9},
         "training": {"batch_size": 4}}))
    (runs / "child.yaml").write_text(yaml.safe_dump({"base": "parent.yaml", "optimizer": {"max_lr": 5e-4}, "experiment": "x"}))
    cfg = load_run_config(runs / "child.yaml")
    assert cfg.data["optimizer"] == {"max_lr": 5e-4, "beta1": 0.9}
    assert cfg.data["model"]["d_model"] == 32 and cfg.data["model"]["name"] == "tiny"
    assert cfg.data["dataset"]["splits"]["train"] == "data/train.txt"
    assert cfg.data["_meta"]["project_root"] == str(root.resolve())
    assert cfg.project_root == root.resolve()


def test_circular_base_and_missing_files_are_rejected(tmp_path):
    root = make_project(tmp_path)
    runs = root / "configs" / "runs"
    (runs / "a.yaml").write_text("base: b.yaml\n")
    (runs / "b.yaml").write_text("base: a.yaml\n")
    with pytest.raises(ConfigError, match="Circular"):
        load_run_config(runs / "a.yaml")
    with pytest.raises(ConfigError):
        load_run_config(runs / "nope.yaml")
    (runs / "bad.yaml").write_text("model: missing_component\n")
    with pytest.raises(ConfigError):
        load_run_config(runs / "bad.yaml")


def test_dotted_override_and_validators():
    cfg = {"optimizer": {"max_lr": 1.0}}
    set_dotted_value(cfg, "optimizer.max_lr", 0.5)
    set_dotted_value(cfg, "new.deep.key", 3)
    assert cfg == {"optimizer": {"max_lr": 0.5}, "new": {"deep": {"key": 3}}}
    with pytest.raises(ConfigError):
        set_dotted_value({"a": 1}, "a.b", 2)
    with pytest.raises(ConfigError):
        check_model({"name": "m", "context_length": 8, "d_model": 30, "num_layers": 1, "num_heads": 4})
    with pytest.raises(ConfigError):
        check_model({"name": "m", "context_length": 8, "d_model": 32, "num_layers": 1, "num_heads": 4, "num_kv_heads": 3})
    with pytest.raises(ConfigError):
        check_tokenizer({"name": "t", "vocab_size": 256, "special_tokens": ["<s>"]})
    assert check_parallel({"tp": 2}, 8) == {"tp": 2, "ep": 1, "fsdp": 4, "pp": 1, "cp": 1}
    with pytest.raises(ConfigError):
        check_parallel({"tp": 3}, 8)


def test_manifest_hashes_and_lineage(tmp_path):
    root = make_project(tmp_path)
    folder = ArtifactPaths(root).tokenizer("tok")
    folder.mkdir(parents=True)
    (folder / "vocab.json").write_text("{}")
    hashes = {"vocab.json": file_sha256(folder / "vocab.json")}
    write_manifest(folder / "manifest.json", "tokenizer", {"hashes": hashes, "fingerprint": fingerprint_of(hashes)})
    manifest = read_manifest(folder / "manifest.json")
    assert manifest["schema_version"] == 1 and manifest["artifact_type"] == "tokenizer" and "created_at" in manifest
    open_tokenizer_artifact(root, "tok")
    (folder / "vocab.json").write_text('{"tampered": 1}')
    with pytest.raises(LineageError):
        open_tokenizer_artifact(root, "tok")
    with pytest.raises(LineageError):
        check_lineage({"fingerprint": "aaa"}, {"tokenizer_fingerprint": "bbb"})
    check_lineage({"fingerprint": "aaa"}, {"tokenizer_fingerprint": "aaa"})
    check_lineage({}, {})


def test_run_paths_layout(tmp_path):
    paths = ArtifactPaths(tmp_path)
    run = paths.training_run("d", "t", "m", "exp", "fixed")
    assert run == tmp_path / "runs" / "training" / "d" / "t" / "m" / "exp" / "fixed"
    auto = paths.task_run("sweeps", "s")
    assert auto.parent == tmp_path / "runs" / "sweeps" / "s" and len(auto.name.split("_")[1]) == 8
    assert json.dumps(str(auto))
