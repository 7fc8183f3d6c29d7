"""The one table from an architecture's name (``architectures[0]`` of config.json) to its
typed configuration and its model specification.

The reference picks a class with if/else on substrings and on
``num_hidden_layers / num_key_value_heads == 16`` (cpmcu/common/utils.py:33-64, 147-162).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

from .config.base import ConfigError, architecture_name, read_config_json
from .parts.base import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                                   # has from_dict(dict) and to_dict()
    model_spec: Callable[[Any], ModelSpec]              # typed config -> specification
    adapt_tensor: Optional[Callable[[Any, str, Any], List[Tuple[str, Any]]]] = None
    ignore_tensor: Optional[Callable[[str], bool]] = None
    # (typed config, {tensor name: shape}) -> typed config: fills in sizes that the configuration leaves to the
    # checkpoint's tensors; called by ``load_config`` when the folder holds a checkpoint
    fit_config: Optional[Callable[[Any, Dict[str, Tuple[int, ...]]], Any]] = None


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    _ARCHITECTURES[arch.name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


_plugins_loaded: set = set()


def load_plugins(modules=None) -> List[str]:
    """Imports the named modules (default: the comma-separated list in the environment variable
    ``CPMCU_PLUGINS``), each once.  A plug-in is any importable module that registers parts or architectures when
    it is imported; this is how a model that the package does not know is reached from the command line and
    from ``bin/trace_run`` without a change to the package."""
    import importlib
    import os

    if modules is None:
        modules = [m.strip() for m in os.environ.get("CPMCU_PLUGINS", "").split(",") if m.strip()]
    done = []
    for m in modules:
        if m not in _plugins_loaded:
            _plugins_loaded.add(m)
            importlib.import_module(m)
            done.append(m)
    return done


def architecture(name: str) -> Architecture:
    load_plugins()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture '{name}'; known: {sorted(_ARCHITECTURES)}") from None


def known_architectures() -> List[str]:
    load_plugins()
    return sorted(_ARCHITECTURES)


def load_config(model_dir: str):
    """(architecture, typed configuration) of a model folder."""
    data = read_config_json(model_dir)
    arch = architecture(architecture_name(data))
    config = arch.config_class.from_dict(data)
    if arch.fit_config is not None:
        import os
        from .weights.safetensors_io import SafetensorsError, SafetensorsFile, model_files
        shapes: Dict[str, Tuple[int, ...]] = {}
        try:
            for path in (model_files(model_dir) if os.path.isdir(model_dir) else []):
                f = SafetensorsFile(path)
                shapes.update({name: entry[1] for name, entry in f.entries.items()})
                f.close()
        except (SafetensorsError, OSError):
            shapes = {}                      # the loader reports a broken checkpoint in its own words
        if shapes:
            config = arch.fit_config(config, shapes)
    return arch, config


def _register_builtin() -> None:
    from .config.minicpm import MiniCPMConfig
    from .models import minicpm4

    register_architecture(Architecture(
        name="MiniCPMForCausalLM",
        config_class=MiniCPMConfig,
        model_spec=minicpm4.model_spec,
        adapt_tensor=minicpm4.split_fused_tensors,
        ignore_tensor=minicpm4.ignored_tensor,
    ))
    from .config.reravik import ReravikConfig
    from .models import reravik

    register_architecture(Architecture(name=ReravikConfig.architecture, config_class=ReravikConfig, model_spec=reravik.model_spec))
    from .config.mufevik import MufevikConfig
    from .models import mufevik

    register_architecture(Architecture(name=MufevikConfig.architecture, config_class=MufevikConfig, model_spec=mufevik.model_spec,
                                       fit_config=mufevik.fit_config_to_checkpoint))
    from .config.kipizen import KipizenConfig
    from .models import kipizen

    register_architecture(Architecture(name=KipizenConfig.architecture, config_class=KipizenConfig, model_spec=kipizen.model_spec))
    from .config.lukelorn import LukelornConfig
    from .models import lukelorn

    register_architecture(Architecture(name=LukelornConfig.architecture, config_class=LukelornConfig, model_spec=lukelorn.model_spec,
                                       fit_config=lukelorn.fit_config_to_checkpoint))


_register_builtin()
