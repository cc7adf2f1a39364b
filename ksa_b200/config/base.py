"""Configuration base: typed, validated, JSON/YAML round-trippable.

Every config is a pydantic model that rejects unknown fields and validates on
assignment.  A config file names its class in a ``"__class__"`` key and
:func:`load_config` dispatches on it, so the JSON files written for the
reference trainer (``muse/config/base.py:200-319``) load here unchanged.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Callable, Dict, Optional, Type

import yaml
from pydantic import BaseModel, ConfigDict

_CONFIG_CLASSES: Dict[str, Type["BaseConfig"]] = {}


def register_config(cls: Type["BaseConfig"]) -> Type["BaseConfig"]:
    """Class decorator: make ``cls`` reachable from a ``"__class__"`` key."""
    _CONFIG_CLASSES[cls.__name__] = cls
    return cls


class BaseConfig(BaseModel):
    model_config = ConfigDict(
        extra="forbid",
        validate_assignment=True,
        use_enum_values=True,
        arbitrary_types_allowed=True,
    )

    # ---- serialisation -------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        out = self.model_dump()
        out["__class__"] = type(self).__name__
        return out

    def to_json(self, indent: int = 2) -> str:
        return json.dumps(self.to_dict(), indent=indent, ensure_ascii=False)

    def to_yaml(self) -> str:
        return yaml.safe_dump(self.to_dict(), sort_keys=False)

    def save(self, path: str) -> None:
        p = Path(path)
        p.parent.mkdir(parents=True, exist_ok=True)
        text = self.to_yaml() if p.suffix in (".yml", ".yaml") else self.to_json()
        p.write_text(text, encoding="utf-8")

    def merge(self, overrides: Dict[str, Any]) -> "BaseConfig":
        """Return a new config with ``overrides`` applied on top of this one."""
        data = self.model_dump()
        data.update({k: v for k, v in overrides.items() if k != "__class__"})
        return type(self)(**data)

    # ---- construction --------------------------------------------------
    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "BaseConfig":
        return cls(**{k: v for k, v in data.items() if k != "__class__"})

    @classmethod
    def from_json(cls, text: str) -> "BaseConfig":
        return cls.from_dict(json.loads(text))

    @classmethod
    def load(cls, path: str) -> "BaseConfig":
        return cls.from_dict(_read_mapping(path))


def _read_mapping(path: str) -> Dict[str, Any]:
    p = Path(path)
    text = p.read_text(encoding="utf-8")
    if p.suffix in (".yml", ".yaml"):
        data = yaml.safe_load(text)
    else:
        data = json.loads(text)
    if not isinstance(data, dict):
        raise ValueError(f"{path}: a config file must hold a mapping, got {type(data).__name__}")
    return data


def load_config(path_or_dict, default_class: Optional[str] = None) -> BaseConfig:
    """Load a config from a JSON/YAML file (or a dict), picking the class from ``"__class__"``."""
    data = path_or_dict if isinstance(path_or_dict, dict) else _read_mapping(path_or_dict)
    name = data.get("__class__", default_class)
    if name is None:
        raise ValueError("config has no '__class__' key and no default class was given")
    if name not in _CONFIG_CLASSES:
        raise KeyError(f"unknown config class {name!r}; known: {sorted(_CONFIG_CLASSES)}")
    return _CONFIG_CLASSES[name].from_dict(data)


def config_classes() -> Dict[str, Type[BaseConfig]]:
    return dict(_CONFIG_CLASSES)
