"""Registries: architecture name -> model, and part kind -> part class.

One table maps the ``architectures[0]`` string of a config.json to the code that reads
that architecture's keys and lowers them to a ``ModelSpec``.  The reference has no such
table: its ``SUPPORTED`` list only silences a warning (crates/model/src/config.rs:9-30,
:513-518) and the block kind is read off the tensors present.  Part tables let a mixer,
feed-forward, norm, position encoding or block defined outside this package be built by
kind without touching the package.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict

from .config.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    read_config: Callable[[Dict[str, Any]], Any]      # config.json dict -> typed config
    to_spec: Callable[[Any], ModelSpec]               # typed config -> ModelSpec
    model_types: tuple = ()


_ARCHITECTURES: Dict[str, Architecture] = {}
_PARTS: Dict[str, Dict[str, type]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
}


class UnknownArchitecture(KeyError):
    pass


def register_architecture(name: str, read_config, to_spec, model_types=()) -> None:
    _ARCHITECTURES[name] = Architecture(name, read_config, to_spec, tuple(model_types))


def architectures() -> Dict[str, Architecture]:
    return dict(_ARCHITECTURES)


def resolve_architecture(raw: Dict[str, Any]) -> Architecture:
    """Pick the architecture for a config.json dict: ``architectures[0]``, else ``model_type``."""
    names = raw.get("architectures") or []
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = raw.get("model_type")
    if not names and mt is not None:
        for a in _ARCHITECTURES.values():
            if mt in a.model_types:
                return a
    raise UnknownArchitecture(
        f"no model registered for architectures={names!r} model_type={mt!r}; "
        f"known: {sorted(_ARCHITECTURES)}")


def load_config(model_dir: str):
    """Read ``model_dir/config.json`` -> (Architecture, typed config, ModelSpec)."""
    path = os.path.join(model_dir, "config.json")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    arch = resolve_architecture(raw)
    cfg = arch.read_config(raw)
    return arch, cfg, arch.to_spec(cfg)


def register_part(family: str, kind: str, cls: type) -> None:
    if family not in _PARTS:
        raise KeyError(f"unknown part family '{family}'; one of {sorted(_PARTS)}")
    _PARTS[family][kind] = cls


def part_class(family: str, kind: str) -> type:
    try:
        return _PARTS[family][kind]
    except KeyError:
        raise KeyError(f"no {family} of kind '{kind}' is registered; "
                       f"known: {sorted(_PARTS.get(family, {}))}") from None


def _register_builtin() -> None:
    from .config.qwen2 import Qwen2Config
    register_architecture("Qwen2ForCausalLM", Qwen2Config.from_dict,
                          lambda c: c.to_model_spec(), model_types=("qwen2",))


_register_builtin()
