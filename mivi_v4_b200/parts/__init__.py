"""Parts that layers are put together from, and their registries.  Importing
this package registers the parts that ship with it."""
from . import block, embedding, feed_forward, mixers, norm, position  # noqa: F401  (registration)
from .base import Part
from .registry import build, lookup, register, registered
from .spec import ModelSpec, ParamSpec, PartSpec, ScheduleEntry

__all__ = ["Part", "build", "lookup", "register", "registered", "ModelSpec", "ParamSpec", "PartSpec",
           "ScheduleEntry"]
