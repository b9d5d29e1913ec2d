"""What every part is: a bag of named parameters with declared shapes, built
from sizes and constants alone.  No part knows which model it is in.

Interfaces by role (``step`` is an engine.step.StepContext, ``resid`` the
32-bit residual stream [N, hidden] that a part adds its result to in place):

norm          forward(x_f32[N, dim], out_dtype, step, rows=None) -> [n, dim]
position      rotary() -> (inv_freq f32[hd/2], style) or None
mixer         cache_need() -> KVNeed | StateNeed | None | a list of those
              forward(u[N, hidden], resid, step, cache_view) -> None   (a list of views for a list of needs)
feed_forward  forward(g[N, hidden], resid, step) -> None; one that overrides cache_need() is also passed
              view=<its view or list of views>
block         cache_need(); forward(resid, step, cache_view) -> None
embedding     forward(step) -> resid f32[N, hidden]
head          forward(f[n, hidden], step, embedding) -> logits f32[n, vocab]
"""
from __future__ import annotations

from typing import Dict

from .spec import ParamSpec


class Part:
    kind = "?"
    prefix = ""
    nested_roles: Dict[str, str] = {}
    # False for a part whose forward reads device values on the host or launches work that depends
    # on the step's host-side lists: a model with such a part runs its decode steps launch by launch
    # instead of replaying a recorded CUDA graph.
    graph_safe = True

    def cache_need(self):
        """What this part keeps per sequence between steps: None, a KVNeed, a StateNeed, or a list of those."""
        return None

    def carries_norm(self, step):
        """(accepts, emits): whether, in this step, the part's first product can take rows that still
        lack their norm's scale (``forward(..., scale=link)``) and whether its last product, the one
        that adds into the residual stream, can write the next norm's rows (``forward(..., emit=link)``).
        A mixer or feed-forward that answers (False, False), the default, is never passed either."""
        return False, False

    def scratch(self, step, name: str, shape, dtype):
        """A buffer from the step's workspace under a name of this part's kind: parts of different kinds
        never share one, so a part may hold its buffers across a call into another part.  (Layers of the
        same kind do share them: a layer is done with its buffers when the next one starts.)"""
        return step.ws.get(f"{getattr(self, 'kind', type(self).__name__)}.{name}", shape, dtype)

    def param_specs(self) -> Dict[str, ParamSpec]:
        """Local tensor name (appended to ``prefix``) -> how the checkpoint stores it."""
        return {}

    def nested(self) -> Dict[str, "Part"]:
        return {}

    def named_param_specs(self) -> Dict[str, ParamSpec]:
        out = {self.prefix + k: v for k, v in self.param_specs().items()}
        for sub in self.nested().values():
            out.update(sub.named_param_specs())
        return out

    def load(self, tensors: Dict[str, "object"]) -> None:
        """Take this part's tensors (keyed by local name, already on the device
        and in their run dtype) and lay them out as its kernels want them."""
        for k, v in tensors.items():
            setattr(self, k.replace(".", "_"), v)

    def load_named(self, named: Dict[str, "object"]) -> None:
        mine = {k: named[self.prefix + k] for k in self.param_specs()}
        self.load(mine)
        for sub in self.nested().values():
            sub.load_named(named)
