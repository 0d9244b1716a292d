"""Configuration files as JSON or YAML (src/lmms_engine/utils/config_loader.py:8-68 of the reference).

A relative path that does not exist from the working directory is looked up from the enclosing project roots
(directories that hold a ``pyproject.toml`` or a ``.git``), so that ``examples/...`` paths work from any sub-folder."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any

import yaml

SUFFIXES = (".json", ".yaml", ".yml")


def resolve_config_path(config_path: str) -> Path:
    path = Path(config_path)
    if path.exists() or path.is_absolute():
        return path
    here = Path.cwd()
    for folder in (here, *here.parents):
        if (folder / "pyproject.toml").exists() or (folder / ".git").exists():
            if (folder / path).exists():
                return folder / path
    return path


def load_config(config_path: str) -> Any:
    path = resolve_config_path(config_path)
    if not path.exists():
        raise FileNotFoundError(f"configuration file not found: {config_path}")
    suffix = path.suffix.lower()
    if suffix not in SUFFIXES:
        raise ValueError(f"unsupported configuration format '{suffix}' (use .json, .yaml or .yml)")
    with open(path) as f:
        return json.load(f) if suffix == ".json" else yaml.safe_load(f)


def save_config(config: Any, config_path: str) -> None:
    path = Path(config_path)
    suffix = path.suffix.lower()
    if suffix not in SUFFIXES:
        raise ValueError(f"unsupported configuration format '{suffix}' (use .json, .yaml or .yml)")
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w") as f:
        if suffix == ".json":
            json.dump(config, f, indent=2)
        else:
            yaml.safe_dump(config, f, default_flow_style=False, sort_keys=False)
