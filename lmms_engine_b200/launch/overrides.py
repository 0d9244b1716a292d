"""A small, dependency-free implementation of the Hydra command-line grammar the engine's
launch scripts use: ``a.b.c=value`` (set), ``+a.b=value`` (add), ``++a.b=value`` (force),
``~a.b`` (delete), ``--config-path DIR --config-name NAME``, and ``hydra.*`` / ``hydra/...``
namespace overrides (accepted and ignored).  Values are parsed as YAML, so lists, dicts,
``null``, numbers and booleans work as in Hydra.  The reference uses hydra-core itself
(src/lmms_engine/launch/cli.py:141-155)."""
from __future__ import annotations

import os
import re
from typing import Any, Dict, List, Optional, Tuple

import yaml


def _parse_value(text: str) -> Any:
    try:
        val = yaml.safe_load(text)
    except yaml.YAMLError:
        return text
    if isinstance(val, str):  # YAML 1.1 does not read "1e-3" as a float; Hydra does
        try:
            return float(val) if re.fullmatch(r"[+-]?(\d+\.?\d*|\.\d+)([eE][+-]?\d+)", val) else val
        except ValueError:
            return val
    return val


def _set(cfg: Dict[str, Any], dotted: str, value: Any, must_exist: bool) -> None:
    keys = dotted.split(".")
    cur = cfg
    for k in keys[:-1]:
        if k not in cur or not isinstance(cur[k], dict):
            if must_exist and k not in cur:
                raise KeyError(f"override '{dotted}': key '{k}' does not exist (use +{dotted}=... to add)")
            cur[k] = {} if not isinstance(cur.get(k), dict) else cur[k]
        cur = cur[k]
    if must_exist and keys[-1] not in cur:
        raise KeyError(f"override '{dotted}': key does not exist (use +{dotted}=... to add)")
    cur[keys[-1]] = value


def _delete(cfg: Dict[str, Any], dotted: str) -> None:
    keys = dotted.split(".")
    cur = cfg
    for k in keys[:-1]:
        cur = cur.get(k, {})
    cur.pop(keys[-1], None)


def split_argv(argv: List[str]) -> Tuple[Optional[str], Optional[str], List[str]]:
    """Pull ``--config-path/--config-name`` (and their ``-cp/-cn`` short forms) out of argv."""
    cp = cn = None
    rest: List[str] = []
    i = 0
    while i < len(argv):
        a = argv[i]
        if a in ("--config-path", "-cp") and i + 1 < len(argv):
            cp = argv[i + 1]
            i += 2
        elif a.startswith("--config-path="):
            cp = a.split("=", 1)[1]
            i += 1
        elif a in ("--config-name", "-cn") and i + 1 < len(argv):
            cn = argv[i + 1]
            i += 2
        elif a.startswith("--config-name="):
            cn = a.split("=", 1)[1]
            i += 1
        else:
            rest.append(a)
            i += 1
    return cp, cn, rest


def apply_overrides(cfg: Dict[str, Any], overrides: List[str], strict: bool = False) -> Dict[str, Any]:
    for ov in overrides:
        if ov.startswith("hydra.") or ov.startswith("hydra/") or ov.startswith("+hydra") or ov.startswith("~hydra"):
            continue  # Hydra runtime namespace: nothing to configure here
        if ov.startswith("~"):
            _delete(cfg, ov[1:].split("=", 1)[0])
            continue
        if "=" not in ov:
            raise ValueError(f"cannot parse override '{ov}' (expected key=value)")
        key, val = ov.split("=", 1)
        force = key.startswith("++")
        add = key.startswith("+") and not force
        key = key.lstrip("+")
        _set(cfg, key, _parse_value(val), must_exist=strict and not (add or force))
    return cfg


def load_config_file(config_path: Optional[str], config_name: Optional[str], default_file: str) -> Dict[str, Any]:
    if config_name is None and config_path is None:
        path = default_file
    else:
        name = config_name or "default_config"
        if not name.endswith((".yaml", ".yml")):
            name += ".yaml"
        path = os.path.join(config_path or os.path.dirname(default_file), name)
    with open(path) as f:
        return yaml.safe_load(f) or {}
