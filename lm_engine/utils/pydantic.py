"""Strict base class of every argument section (unknown keys are errors)."""

from __future__ import annotations

from enum import Enum
from typing import Any

from pydantic import BaseModel, ConfigDict


def _plain(value: Any) -> Any:
    """Turn enums, classes, nested argument objects and containers into YAML/JSON-friendly values."""
    if isinstance(value, BaseArgs):
        return value.to_dict()
    if isinstance(value, Enum):
        return value.value
    if isinstance(value, type):
        return value.__name__
    if isinstance(value, dict):
        return {k: _plain(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [_plain(v) for v in value]
    return value


class BaseArgs(BaseModel):
    """pydantic v2 model with ``extra="forbid"`` (parity: lm_engine/utils/pydantic.py:11-34)."""

    model_config = ConfigDict(extra="forbid", protected_namespaces=(), arbitrary_types_allowed=True)

    def to_dict(self) -> dict:
        return {name: _plain(getattr(self, name)) for name in type(self).model_fields}
