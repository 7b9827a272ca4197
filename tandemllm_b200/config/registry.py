"""One registry from an architecture's name to its configuration reader and its model.

A model folder's family is chosen by its own config.json (`architectures` first, then `model_type`,
top level or under `text_config`), never by a file name; an unknown one is refused with the list of
registered names (engine/models/__init__.py:29-114 in the reference). An entry holds two callables:

  read_config(raw: dict, folder: str, generation: dict | None) -> config   (typed; has `.to_spec()`
                                                                            and `.to_dict()`)
  build_model(spec: ModelSpec, runtime) -> model                            (default: the generic decoder)

Adding an architecture is one `register(Architecture(...))` call from its own module; nothing here
or in the engine changes.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable

from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    architectures: tuple[str, ...]
    model_types: tuple[str, ...]
    read_config: Callable[..., Any]
    build_model: Callable[..., Any] | None = None    # None: tandemllm_b200.parts.model.DecoderModel


REGISTRY: dict[str, Architecture] = {}


def register(arch: Architecture) -> Architecture:
    REGISTRY[arch.name] = arch
    return arch


def unregister(name: str) -> None:
    REGISTRY.pop(name, None)


def architecture_of(raw: dict) -> Architecture:
    names = [str(a) for a in (raw.get("architectures") or [])]
    types = [str(raw.get("model_type", "")), str((raw.get("text_config") or {}).get("model_type", ""))]
    for arch in REGISTRY.values():
        if any(a in arch.architectures for a in names) or any(t in arch.model_types for t in types if t):
            return arch
    what = names[0] if names else (types[0] or types[1] or "<no architectures, no model_type>")
    known = ", ".join(f"{a.name} ({', '.join(a.architectures)})" for a in REGISTRY.values())
    raise ValueError(f"unknown architecture {what!r}: this engine runs {known}")


def resolve_model_folder(path: str) -> str:
    """A folder with config.json, or the parent of `snapshots/*/` that holds one
    (engine/config.py:21-30 in the reference)."""
    if os.path.isfile(os.path.join(path, "config.json")):
        return path
    snaps = os.path.join(path, "snapshots")
    if os.path.isdir(snaps):
        for name in sorted(os.listdir(snaps)):
            if os.path.isfile(os.path.join(snaps, name, "config.json")):
                return os.path.join(snaps, name)
    raise FileNotFoundError(f"{path}: no config.json here or under snapshots/*/")


def read_model_config(folder: str):
    """(architecture, typed config) of a model folder."""
    folder = resolve_model_folder(folder)
    with open(os.path.join(folder, "config.json")) as f:
        raw = json.load(f)
    generation = None
    gpath = os.path.join(folder, "generation_config.json")
    if os.path.isfile(gpath):
        with open(gpath) as f:
            generation = json.load(f)
    arch = architecture_of(raw)
    return arch, arch.read_config(raw, folder, generation)


def spec_of(config: Any) -> ModelSpec:
    return config if isinstance(config, ModelSpec) else config.to_spec()
