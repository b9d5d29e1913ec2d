"""A model put together from a description: embedding, blocks, the order in
which the blocks run, final norm, head.  Nothing here is specific to an
architecture; the architecture's file supplies the ``ModelSpec``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import architectures  # noqa: F401  (registers the architectures that ship with the package)
from ..cache import CachePlan, plan_cache
from ..config import architecture_for
from ..ops import kernels as K
from ..ops.linear import end_norms_carried
from ..parts import ModelSpec, ParamSpec, build


class _AfterLastBlock:
    """What the last block sees as the block after it: the final norm, offered as a link when the
    head's product can carry it (a step of few tokens with every row's logits wanted)."""

    def __init__(self, model):
        self.model = model

    def entry_link(self, step):
        m = self.model
        if (step.carry_norms and end_norms_carried(step.n_tokens) and step.out_rows_all
                and hasattr(m.final_norm, "link") and hasattr(m.head, "carries_norm")
                and m.head.carries_norm(step, m.embedding)):
            return m.final_norm.link(step, "final")
        return None


class Model:
    def __init__(self, spec: ModelSpec, config=None):
        self.spec, self.config = spec, config
        self.hidden_size, self.vocab_size = spec.hidden_size, spec.vocab_size
        self.embedding = build("embedding", spec.embedding)
        self.blocks = [build("block", b) for b in spec.blocks]
        self.final_norm = build("norm", spec.final_norm)
        self.head = build("head", spec.head)
        self.schedule = list(spec.schedule)
        for pos, e in enumerate(self.schedule):
            if not (0 <= e.block < len(self.blocks)):
                raise ValueError(f"schedule position {pos} names block {e.block}; the model has "
                                 f"{len(self.blocks)} blocks")
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None

    # ---- parameters -------------------------------------------------------
    def parts(self) -> List:
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    @property
    def graph_safe(self) -> bool:
        """Whether a step's launches may be recorded once and replayed: every part says so."""
        def walk(p):
            return getattr(p, "graph_safe", True) and all(walk(sub) for sub in p.nested().values())
        return all(walk(p) for p in self.parts())

    def named_param_specs(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for p in self.parts():
            for name, spec in p.named_param_specs().items():
                if name in out:
                    raise ValueError(f"two parts claim the tensor {name!r}")
                out[name] = spec
        return out

    def load_params(self, named: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        for p in self.parts():
            p.load_named(named)
        self.dtype, self.device = dtype, torch.device(device)

    def weight_extents(self) -> Dict[int, int]:
        """Address -> bytes of every tensor that the parts hold (each once): the memory that lives
        as long as the model does."""
        seen: Dict[int, int] = {}

        def walk(p):
            for v in vars(p).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen[v.data_ptr()] = v.numel() * v.element_size()
            for sub in p.nested().values():
                walk(sub)
        for p in self.parts():
            walk(p)
        return seen

    def weight_bytes(self) -> int:
        """Bytes of every tensor that one step reads (each counted once)."""
        return sum(self.weight_extents().values())

    # ---- cache --------------------------------------------------------------
    def cache_plan(self) -> CachePlan:
        needs = [self.blocks[e.block].cache_need() for e in self.schedule]
        return plan_cache(needs, [e.cache_of for e in self.schedule])

    # ---- one step ---------------------------------------------------------------
    def forward(self, step, cache) -> Optional[torch.Tensor]:
        """Run the step's tokens through every scheduled block and return the
        logits at ``step.out_rows`` (float32 [n_out, vocab]), or None if no
        logits are wanted."""
        # In steps of few tokens the norms between products ride on those products; so do the two at
        # the ends: the embedding writes the first block's first norm, the head applies the final one.
        first = self.blocks[self.schedule[0].block] if self.schedule else None
        link = first.entry_link(step) if (hasattr(first, "entry_link") and getattr(self.embedding, "emits_norm", False)
                                          and end_norms_carried(step.n_tokens)) else None
        with K.profile_stage("embedding"):
            if link is not None:
                x = self.embedding.forward(step, emit=link)
                step.leave_link(link)
            else:
                x = self.embedding.forward(step)
        for pos, entry in enumerate(self.schedule):
            block = self.blocks[entry.block]
            view = cache.view(pos, step.page_tables)
            if hasattr(block, "entry_link"):
                # a block that can hand its last norm on to the next one is told which block that is
                nxt = self.blocks[self.schedule[pos + 1].block] if pos + 1 < len(self.schedule) else \
                    (_AfterLastBlock(self) if step.n_out else None)
                block.forward(x, step, view, after=nxt)
            else:
                block.forward(x, step, view)
        if step.n_out == 0:
            return None
        with K.profile_stage("logits"):
            link = step.take_link(self.final_norm)
            if link is not None:
                return self.head.forward(link.xg, step, self.embedding, scale=link)
            f = step.ws.get("final", (step.n_out, self.hidden_size), step.dtype)
            self.final_norm.forward(x, f, rows=step.out_rows)
            return self.head.forward(f, step, self.embedding)


def describe_config(config_dict: dict):
    arch = architecture_for(config_dict)
    config = arch.config_from_dict(config_dict)
    return config, arch.describe(config)


def expected_tensors(config_dict: dict) -> Dict[str, ParamSpec]:
    """The checkpoint's name table for this configuration."""
    config, spec = describe_config(config_dict)
    return Model(spec, config).named_param_specs()
