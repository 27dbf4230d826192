"""One registry from an architecture's name to its configuration class.

``config.json`` names its architecture in ``architectures[0]``; the class
registered under that name parses the file's own keys and describes the model
as a ``ModelSpec``.  The reference matches ``general.architecture`` the same
way and refuses the rest by name (crates/nncpu/src/model/load.rs:895-942).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, Dict

from ..errors import BadFormat, UnsupportedModel

_ARCHITECTURES: Dict[str, type] = {}


def register_architecture(name: str) -> Callable[[type], type]:
    """Class decorator.  The class needs ``from_dict(dict)``, ``to_dict()``
    and ``model_spec()``; see ``Qwen3Config`` for the shape of one."""
    def deco(cls: type) -> type:
        _ARCHITECTURES[name] = cls
        cls.architecture = name
        return cls
    return deco


def architectures() -> list:
    return sorted(_ARCHITECTURES)


def config_class(name: str) -> type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise UnsupportedModel(
            f"architecture {name!r} is not supported (supported: {', '.join(architectures())})"
        ) from None


def config_from_dict(d: dict):
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise BadFormat('config.json has no "architectures": ["..."] entry')
    return config_class(archs[0]).from_dict(d)


def _generation_stop_ids(folder) -> list:
    """The ``eos_token_id`` entries of ``generation_config.json``, if the folder has one: checkpoints keep the
    whole set of tokens that end a reply there, while ``config.json`` names one
    (the reference's set: crates/nncpu/src/tokenizer/mod.rs:385-405)."""
    path = Path(folder) / "generation_config.json"
    if not path.exists():
        return []
    try:
        g = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise BadFormat(f"{path} is not JSON: {e}") from None
    eos = g.get("eos_token_id") if isinstance(g, dict) else None
    eos = eos if isinstance(eos, list) else ([] if eos is None else [eos])
    for e in eos:
        if isinstance(e, bool) or not isinstance(e, int):
            raise BadFormat(f'{path}: "eos_token_id" holds {e!r}')
    return eos


def load_config(folder):
    """The typed configuration of the model folder ``folder``: ``config.json``, with the stop tokens of
    ``generation_config.json`` added to its ``eos_token_id``."""
    path = Path(folder) / "config.json"
    try:
        d = json.loads(path.read_text())
    except FileNotFoundError:
        raise BadFormat(f"{path} does not exist") from None
    except json.JSONDecodeError as e:
        raise BadFormat(f"{path} is not JSON: {e}") from None
    if not isinstance(d, dict):
        raise BadFormat(f"{path} does not hold a JSON object")
    extra = _generation_stop_ids(folder)
    if extra:
        own = d.get("eos_token_id")
        own = own if isinstance(own, list) else ([] if own is None else [own])
        d = dict(d, eos_token_id=own + [e for e in extra if e not in own])
    return config_from_dict(d)
