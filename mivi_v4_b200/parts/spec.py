"""Data that describes a model: which parts it is made of, with which sizes
and constants, under which tensor names, and in which order its layers run.

An architecture file turns its typed configuration into one ``ModelSpec``; the
engine builds the parts from it through the registries.  Nothing in here knows
a particular architecture.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class ParamSpec:
    """One tensor of a part as the checkpoint stores it.

    role: ``matrix`` - an operand of a matrix product or an embedding table;
    runs in the model's dtype unless the file stores it in 32-bit.
    ``vector`` - norm weights, biases, convolution taps; the kernels read
    these in 32-bit, and widening them is exact.  ``table`` - integers, kept
    as int32.
    init: which distribution the random-weights mode draws it from
    (``linear`` N(0, 0.02), ``conv`` N(0, 0.2), ``norm`` 1 + N(0, 0.1),
    ``bias`` N(0, 0.02), ``zeros``).
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "linear"


@dataclass
class PartSpec:
    kind: str                                   # name in the part's registry
    params: dict = field(default_factory=dict)  # constructor arguments (sizes, constants)
    prefix: str = ""                            # tensor-name prefix in the checkpoint
    parts: Dict[str, "PartSpec"] = field(default_factory=dict)   # nested parts (a mixer's position encoding)


@dataclass
class ScheduleEntry:
    """One step of the layer order.  ``block`` indexes ``ModelSpec.blocks`` (a
    block may appear more than once); ``cache_of`` names an EARLIER schedule
    position whose cache this entry reads instead of keeping its own."""
    block: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    blocks: List[PartSpec]                      # role "block"; its nested parts are norms, mixer, feed-forward
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    # tensors that a checkpoint may carry although the model does not use them
    ignorable: Tuple[str, ...] = ()
    stop_token_ids: Tuple[int, ...] = ()
    max_positions: Optional[int] = None
