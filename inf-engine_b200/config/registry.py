"""One registry from an architecture's name to its configuration and model.

The reference keeps a dictionary from a repository id to a preset
(engine/config.py:256-274) and matches folder names to presets
(main.py:113-134).  Here the key is ``architectures[0]`` of ``config.json``;
an unknown name is an error that lists the known ones, never a silent
fall-back (scripts/generate_llama.py:39-43 falls back to the 1B preset).

Adding an architecture is one ``register_architecture`` call with a function
from the ``config.json`` dictionary to a typed configuration that has a
``model_spec()`` method.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from .llama import ConfigError, LlamaConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict], object]   # config.json dict -> typed config with .model_spec()


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, parse_config: Callable[[dict], object]) -> None:
    ARCHITECTURES[name] = Architecture(name, parse_config)


def get_architecture(name: str) -> Architecture:
    try:
        return ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; known: {', '.join(sorted(ARCHITECTURES))}"
        ) from None


def parse_config_dict(d: dict):
    """Typed configuration of a ``config.json`` dictionary, chosen by its architecture."""
    archs = d.get("architectures")
    if not archs:
        raise ConfigError("config.json has no 'architectures' entry")
    return get_architecture(str(archs[0])).parse_config(d)


def detect_config(model_dir: str | Path):
    """Read ``<model_dir>/config.json`` and return the typed configuration."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in {model_dir}")
    with open(path) as f:
        return parse_config_dict(json.load(f))


_PRESET_DIR = Path(__file__).resolve().parent / "presets"


def preset_names() -> list[str]:
    return sorted(p.stem for p in _PRESET_DIR.glob("*.json"))


def get_preset(name: str):
    """A named configuration kept as a ``config.json`` file under ``presets/``
    (the sizes of engine/config.py:77-133 and two tiny test models)."""
    path = _PRESET_DIR / f"{name}.json"
    if not path.is_file():
        raise KeyError(f"unknown preset {name!r}; available: {preset_names()}")
    with open(path) as f:
        return parse_config_dict(json.load(f))


# the reference's accessor name (engine/config.py:271-274)
get_llama_config = get_preset

register_architecture("LlamaForCausalLM", LlamaConfig.from_hf_dict)
