"""Registries of part classes by kind, one per role.

A configuration names parts by these keys (``PartSpec.kind``); ``build_part`` makes
the object. Registering a new class under a new key is all it takes to make it
available to any architecture.
"""
from __future__ import annotations

ROLES = ("norm", "position", "mixer", "ffn", "block", "embedding", "head")
_REGISTRY: dict = {r: {} for r in ROLES}


def register_part(role: str, kind: str, cls=None):
    """``register_part("mixer", "attention", GQAAttention)`` or as a class decorator."""
    if role not in _REGISTRY:
        raise ValueError(f"unknown part role {role!r}; roles: {ROLES}")

    def put(c):
        _REGISTRY[role][kind] = c
        return c

    return put(cls) if cls is not None else put


def unregister_part(role: str, kind: str) -> None:
    _REGISTRY[role].pop(kind, None)


def known_parts(role: str) -> list:
    return sorted(_REGISTRY[role])


def build_part(role: str, spec):
    """Instantiate the part ``spec`` (a ``PartSpec``) names; its params are constructor keywords."""
    try:
        cls = _REGISTRY[role][spec.kind]
    except KeyError:
        raise ValueError(f"no {role} part registered as {spec.kind!r}; known: {known_parts(role)}") from None
    return cls(prefix=spec.prefix, **spec.params)
