"""Registries of parts, one for each role.  A part is chosen by name, layer by
layer, from what the architecture's description says; a new part is added by
registering a class under a new name, from anywhere (a test file included),
with no change to the files of this package.
"""
from __future__ import annotations

from typing import Callable, Dict

ROLES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_REGISTRIES: Dict[str, Dict[str, type]] = {r: {} for r in ROLES}


def register(role: str, name: str, *, replace: bool = False) -> Callable[[type], type]:
    if role not in _REGISTRIES:
        raise KeyError(f"unknown role {role!r}; roles: {', '.join(ROLES)}")

    def deco(cls: type) -> type:
        if name in _REGISTRIES[role] and not replace:
            raise KeyError(f"{role} {name!r} is already registered")
        _REGISTRIES[role][name] = cls
        cls.kind = name
        return cls
    return deco


def lookup(role: str, name: str) -> type:
    try:
        return _REGISTRIES[role][name]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[role])) or "(none)"
        raise KeyError(f"no {role} named {name!r}; registered: {known}") from None


def registered(role: str) -> list:
    return sorted(_REGISTRIES[role])


def build(role: str, spec) -> "object":
    """Instantiate the part that ``spec`` (a PartSpec) names, nested parts first."""
    cls = lookup(role, spec.kind)
    nested = {}
    for slot, sub in spec.parts.items():
        sub_role = getattr(cls, "nested_roles", {}).get(slot)
        if sub_role is None:
            raise KeyError(f"{role} {spec.kind!r} has no nested part {slot!r}")
        nested[slot] = build(sub_role, sub)
    part = cls(**spec.params, **nested)
    part.prefix = spec.prefix
    return part
