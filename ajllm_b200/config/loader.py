"""Composable YAML run configs.

Behaviour follows the reference loader (``ajllm/config/loader.py:27-113``): a config may name a
``base:`` file (relative to itself, resolved recursively, cycles rejected); mappings merge key by
key with the child winning; ``dataset`` / ``tokenizer`` / ``model`` may be either an inline mapping
or the name of ``configs/{datasets,tokenizers,models}/<name>.yaml``; ``_meta`` records where the
config came from. The project root is the nearest ancestor that holds ``configs/`` together with
``pyproject.toml`` (the reference's marker, ``loader.py:47-51``).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import yaml


class ConfigError(ValueError):
    """A config file is missing, malformed or inconsistent."""


@dataclass(frozen=True)
class LoadedConfig:
    """Resolved configuration plus the paths that were used to resolve it."""

    data: dict[str, Any]
    source: Path
    project_root: Path
    config_root: Path

    def replace_data(self, data: dict[str, Any]) -> "LoadedConfig":
        return LoadedConfig(data, self.source, self.project_root, self.config_root)


_COMPONENT_DIRS = {"dataset": "datasets", "tokenizer": "tokenizers", "model": "models"}


def _read_mapping(path: Path) -> dict[str, Any]:
    if not path.is_file():
        raise ConfigError(f"Configuration file does not exist: {path}")
    with path.open("r", encoding="utf-8") as handle:
        loaded = yaml.safe_load(handle)
    if loaded is None:
        return {}
    if not isinstance(loaded, dict):
        raise ConfigError(f"Top-level YAML value must be a mapping: {path}")
    return loaded


def merge_mappings(lower: dict[str, Any], upper: dict[str, Any]) -> dict[str, Any]:
    """Recursive merge; ``upper`` wins, nested mappings are merged rather than replaced."""
    merged = copy.deepcopy(lower)
    for key, value in upper.items():
        if isinstance(value, dict) and isinstance(merged.get(key), dict):
            merged[key] = merge_mappings(merged[key], value)
        else:
            merged[key] = copy.deepcopy(value)
    return merged


def _resolve_chain(path: Path, stack: tuple[Path, ...] = ()) -> dict[str, Any]:
    path = path.resolve()
    if path in stack:
        raise ConfigError(f"Circular base configuration reference: {path}")
    current = _read_mapping(path)
    parent = current.pop("base", None)
    if parent is None:
        return current
    parent_path = (path.parent / str(parent)).resolve()
    return merge_mappings(_resolve_chain(parent_path, stack + (path,)), current)


def find_project_root(start: Path) -> Path:
    for folder in (start.parent, *start.parents):
        if (folder / "configs").is_dir() and (folder / "pyproject.toml").is_file():
            return folder
    raise ConfigError(f"Could not find a project root above {start}")


def _inline_component(config: dict[str, Any], key: str, config_root: Path) -> None:
    value = config.get(key)
    if value is None or isinstance(value, dict):
        return
    if not isinstance(value, str):
        raise ConfigError(f"'{key}' must be a component name or mapping")
    component = _resolve_chain(config_root / _COMPONENT_DIRS[key] / f"{value}.yaml")
    component.setdefault("name", value)
    config[key] = component


def load_run_config(path: str | Path) -> LoadedConfig:
    source = Path(path).expanduser().resolve()
    if not source.is_file():
        raise ConfigError(f"Configuration file does not exist: {source}")
    project_root = find_project_root(source)
    config_root = project_root / "configs"
    data = _resolve_chain(source)
    for key in _COMPONENT_DIRS:
        _inline_component(data, key, config_root)
    data["_meta"] = {"source": str(source), "project_root": str(project_root)}
    return LoadedConfig(data, source, project_root, config_root)


def set_dotted_value(config: dict[str, Any], dotted_key: str, value: Any) -> None:
    """``set_dotted_value(cfg, "optimizer.max_lr", 1e-3)``; intermediate mappings are created."""
    *parents, leaf = dotted_key.split(".")
    node = config
    for name in parents:
        nxt = node.setdefault(name, {})
        if not isinstance(nxt, dict):
            raise ConfigError(f"Cannot override '{dotted_key}': '{name}' is not a mapping")
        node = nxt
    node[leaf] = value


def get_dotted_value(config: dict[str, Any], dotted_key: str, default: Any = None) -> Any:
    node: Any = config
    for name in dotted_key.split("."):
        if not isinstance(node, dict) or name not in node:
            return default
        node = node[name]
    return node
