"""One registry from an architecture's name to how its model is described.

The reference keys its registry by ``model_type`` and maps to a model class
(kvcore/model/model_loader/default_loader.py:32-36, 64-70).  Here the value is a function
from the raw config.json dict to a ``ModelSpec``; the generic builder assembles the model
from that.  The key is ``architectures[0]`` (or the string ``architecture``) of config.json, with
``model_type`` as a fallback.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping

from .config_json import ConfigError, read_config_json
from .model_spec import ModelSpec

SpecFactory = Callable[..., ModelSpec]


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    spec_from_config: SpecFactory
    model_types: tuple[str, ...] = ()
    # an architecture some of whose sizes are only a tensor's shape: its factory then takes a second argument,
    # the shapes of the folder's tensors by name (None when there is no folder)
    reads_tensor_shapes: bool = False


_ARCHITECTURES: dict[str, ArchitectureEntry] = {}


def register_architecture(
    name: str,
    spec_from_config: SpecFactory,
    *,
    model_types: tuple[str, ...] = (),
    replace: bool = False,
    reads_tensor_shapes: bool = False,
) -> None:
    """Add an architecture: ``spec_from_config(config_json_dict) -> ModelSpec``; with
    ``reads_tensor_shapes`` the factory is called as ``spec_from_config(config_json_dict, shapes)``."""
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = ArchitectureEntry(name, spec_from_config, tuple(model_types), bool(reads_tensor_shapes))


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def resolve_architecture(raw: Mapping[str, Any]) -> ArchitectureEntry:
    names = raw.get("architectures") or raw.get("architecture") or []
    if isinstance(names, str):
        names = [names]
    for name in names:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    model_type = raw.get("model_type")
    if model_type is not None:
        for entry in _ARCHITECTURES.values():
            if model_type in entry.model_types:
                return entry
    raise ConfigError(
        f"unsupported architecture: architectures={list(names)!r}, model_type={model_type!r}; "
        f"supported: {', '.join(registered_architectures())}"
    )


def model_spec_from_config(raw: Mapping[str, Any],
                           tensor_shapes: Mapping[str, tuple[int, ...]] | None = None) -> ModelSpec:
    entry = resolve_architecture(raw)
    if entry.reads_tensor_shapes:
        return entry.spec_from_config(raw, tensor_shapes)
    return entry.spec_from_config(raw)


def folder_tensor_shapes(folder: str | Path) -> dict[str, tuple[int, ...]] | None:
    """Name -> shape of every tensor in the folder's safetensors files (their headers only); None when the
    folder holds no weights (a model that is filled with random numbers in place)."""
    from ..weights.safetensors_io import SafetensorsFile, weight_files

    try:
        files = weight_files(folder)
    except FileNotFoundError:
        return None
    shapes: dict[str, tuple[int, ...]] = {}
    for path in files:
        with SafetensorsFile(path) as handle:
            shapes.update({name: entry.shape for name, entry in handle.entries.items()})
    return shapes


def model_spec_from_folder(folder: str | Path) -> ModelSpec:
    raw = read_config_json(folder)
    if resolve_architecture(raw).reads_tensor_shapes:
        return model_spec_from_config(raw, folder_tensor_shapes(folder))
    return model_spec_from_config(raw)


def _register_stock_architectures() -> None:
    from .llama import LlamaConfig

    register_architecture(
        "LlamaForCausalLM",
        lambda raw: LlamaConfig.from_dict(raw).to_model_spec(),
        model_types=("llama",),
    )
    from .toposun import ARCHITECTURE, ToposunConfig

    register_architecture(ARCHITECTURE, lambda raw: ToposunConfig.from_dict(raw).to_model_spec())
    from .pipesun import ARCHITECTURE as PIPESUN, PipesunConfig

    register_architecture(PIPESUN, lambda raw: PipesunConfig.from_dict(raw).to_model_spec())
    from .dutivik import ARCHITECTURE as DUTIVIK, DutivikConfig

    register_architecture(DUTIVIK, lambda raw, shapes=None: DutivikConfig.from_dict(raw, shapes).to_model_spec(),
                          reads_tensor_shapes=True)
    from .rubuvik import ARCHITECTURE as RUBUVIK, RubuvikConfig

    register_architecture(RUBUVIK, lambda raw: RubuvikConfig.from_dict(raw).to_model_spec())


_register_stock_architectures()

__all__ = [
    "ArchitectureEntry",
    "folder_tensor_shapes",
    "model_spec_from_config",
    "model_spec_from_folder",
    "register_architecture",
    "registered_architectures",
    "resolve_architecture",
    "unregister_architecture",
]
