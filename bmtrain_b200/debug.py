"""Tiny key/value scratch store used by the inspect tooling (reference: ``bmtrain/debug.py:1-33``)."""
from typing import Any, Dict

_store: Dict[str, Any] = {}


def clear() -> None:
    _store.clear()


def set(key: str, value: Any) -> None:  # noqa: A001 - API parity
    _store[key] = value


def get(key: str, default: Any = None) -> Any:
    return _store.get(key, default)


def append(key: str, value: Any) -> None:
    _store.setdefault(key, []).append(value)


def extend(key: str, values) -> None:
    _store.setdefault(key, []).extend(values)
