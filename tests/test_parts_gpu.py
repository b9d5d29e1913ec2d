"""Each part alone against the plain function of the same name, and the
generality of the arrangement: a toy mixer with state of its own that is
registered, built and stepped from this file alone; a layer order that names a
block twice; a layer that reads another layer's cache; a window."""
import math
from dataclasses import dataclass
from typing import List

import pytest
import torch

import plain_lfm2 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_step(lens, starts, slots, dtype, ws=None, page_rows=None):
    from mivi_v4_b200.engine.step import StepContext, Workspace
    return StepContext(slots=slots, starts=starts, token_lists=[[0] * n for n in lens], out_rows=[],
                       page_rows=page_rows or {}, dtype=dtype, ws=ws or Workspace(DEV))


def rnd(*shape, scale=1.0, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed + len(shape) + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


# largest error allowed, as a fraction of the largest value of the expected result
TOL = {torch.float32: 2e-5, torch.bfloat16: 1e-2}


def near(got, want, dtype):
    got, want = got.double().cpu(), want.double().cpu()
    return (got - want).abs().max().item() <= TOL[dtype] * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_rmsnorm_part(dtype):
    from mivi_v4_b200.parts import PartSpec, build
    n = build("norm", PartSpec("rmsnorm", dict(dim=200, eps=1e-6)))
    w = rnd(200) * 0.1 + 1
    n.load({"weight": w.to(DEV)})
    x = rnd(5, 200, scale=2.0).to(DEV)
    out = torch.empty(5, 200, dtype=dtype, device=DEV)
    n.forward(x, out)
    assert near(out, P.plain_rms_norm(x.double().cpu(), w.double(), 1e-6), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("H,F", [(64, 192), (200, 144)])
def test_swiglu_part(dtype, H, F):
    from mivi_v4_b200.parts import PartSpec, build
    ff = build("feed_forward", PartSpec("swiglu", dict(hidden=H, ff=F)))
    w1, w3, w2 = (rnd(F, H, scale=0.1, seed=1, dtype=dtype), rnd(F, H, scale=0.1, seed=2, dtype=dtype),
                  rnd(H, F, scale=0.1, seed=3, dtype=dtype))
    ff.load({"w1.weight": w1.to(DEV), "w3.weight": w3.to(DEV), "w2.weight": w2.to(DEV)})
    g = rnd(7, H, dtype=dtype)
    resid = rnd(7, H, seed=9).to(DEV)
    before = resid.double().cpu()
    ff.forward(g.to(DEV), resid, make_step([7], [0], [0], dtype))
    want = before + P.plain_swiglu(g.double(), w1.double(), w3.double(), w2.double())
    assert near(resid, want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("H,k,bias", [(64, 3, False), (96, 4, True)])
def test_short_conv_part_whole_and_cut(dtype, H, k, bias):
    from mivi_v4_b200.cache import StateView
    from mivi_v4_b200.parts import PartSpec, build
    m = build("mixer", PartSpec("short_conv", dict(hidden=H, kernel=k, bias=bias)))
    t = {"in_proj.weight": rnd(3 * H, H, scale=0.1, seed=1, dtype=dtype), "conv.weight": rnd(H, 1, k, scale=0.3, seed=2),
         "out_proj.weight": rnd(H, H, scale=0.1, seed=3, dtype=dtype)}
    if bias:
        t.update({"in_proj.bias": rnd(3 * H, scale=0.1, seed=4), "conv.bias": rnd(H, scale=0.1, seed=5),
                  "out_proj.bias": rnd(H, scale=0.1, seed=6)})
    m.load({n: v.to(DEV) for n, v in t.items()})
    assert m.cache_need().shape == (k - 1, H)
    T = 9
    u = rnd(T, H, dtype=dtype)
    d = lambda n: t[n].double() if n in t else None
    want = P.plain_short_conv(u.double(), d("in_proj.weight"), d("conv.weight"), d("out_proj.weight"),
                              d("in_proj.bias"), d("conv.bias"), d("out_proj.bias"))
    for cuts in ([T], [4, 5], [1] * T):
        state = torch.zeros(3, k - 1, H, device=DEV)
        view = StateView(state, True, m.cache_need())
        outs, done = [], 0
        for n in cuts:
            resid = torch.zeros(n, H, device=DEV)
            m.forward(u[done:done + n].to(DEV).contiguous(), resid, make_step([n], [done], [2], dtype), view)
            outs.append(resid)
            done += n
        assert near(torch.cat(outs), want, dtype), cuts
        assert float(state[:2].abs().sum()) == 0           # only its own slot was touched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("style", ["interleaved", "half_split"])
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 0), (3, 1, 32, 0), (5, 5, 48, 0), (4, 2, 16, 5)])
def test_gqa_part_whole_and_cut(dtype, style, nh, nkv, hd, window):
    from mivi_v4_b200.cache import KVView
    from mivi_v4_b200.parts import PartSpec, build
    H, eps, theta, page = nh * hd, 1e-5, 1e4, 16
    spec = PartSpec("gqa", dict(hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=hd, qk_norm_eps=eps, window=window),
                    parts={"position": PartSpec("rope", dict(head_dim=hd, theta=theta, style=style))})
    m = build("mixer", spec)
    t = {"q_proj.weight": rnd(nh * hd, H, scale=0.15, seed=1, dtype=dtype),
         "k_proj.weight": rnd(nkv * hd, H, scale=0.15, seed=2, dtype=dtype),
         "v_proj.weight": rnd(nkv * hd, H, scale=0.15, seed=3, dtype=dtype),
         "out_proj.weight": rnd(H, nh * hd, scale=0.15, seed=4, dtype=dtype),
         "q_layernorm.weight": rnd(hd, scale=0.1, seed=5) + 1, "k_layernorm.weight": rnd(hd, scale=0.1, seed=6) + 1}
    m.load({n: v.to(DEV) for n, v in t.items()})
    T = 40
    u = rnd(T, H, dtype=dtype)
    want = P.plain_attention(u.double(), *(t[n].double() for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight",
                                                                   "out_proj.weight", "q_layernorm.weight",
                                                                   "k_layernorm.weight")),
                             nh=nh, nkv=nkv, hd=hd, eps=eps, theta=theta, style=style, window=window)
    table = torch.tensor([[5, 2, 7, 0]], dtype=torch.int32)
    for cuts in ([T], [17, 23], [30] + [1] * 10):
        pool = torch.zeros(8, 2, nkv, page, hd, dtype=dtype, device=DEV)
        outs, done = [], 0
        for n in cuts:
            step = make_step([n], [done], [0], dtype, page_rows={0: table.tolist()})
            view = KVView(pool, step.page_tables[0], page, True, m.cache_need())
            resid = torch.zeros(n, H, device=DEV)
            m.forward(u[done:done + n].to(DEV).contiguous(), resid, step, view)
            outs.append(resid)
            done += n
        assert near(torch.cat(outs), want, dtype), cuts


# ------------------------------------------------------------------ toy parts
def register_toy_parts():
    """A mixer with state of its own (a running sum of its inputs, passed through one matrix), and
    an architecture that uses it - all defined here, none of it in the package."""
    from mivi_v4_b200.cache import StateNeed
    from mivi_v4_b200.config import register_architecture
    from mivi_v4_b200.ops.linear import linear
    from mivi_v4_b200.parts import ModelSpec, ParamSpec, Part, PartSpec, ScheduleEntry, register

    @register("mixer", "toy_running_sum", replace=True)
    class RunningSum(Part):
        graph_safe = False                      # its forward loops over the step's slots on the host

        def __init__(self, hidden: int, decay: float):
            self.hidden, self.decay = hidden, decay

        def param_specs(self):
            return {"mix.weight": ParamSpec((self.hidden, self.hidden))}

        def load(self, t):
            self.w = t["mix.weight"]

        def cache_need(self):
            return StateNeed((self.hidden,))

        def forward(self, u, resid, step, view):
            # s_t = decay * s_{t-1} + u_t per sequence, carried in the slot's state; out = s W^T
            s_all = torch.empty(u.shape, dtype=torch.float32, device=u.device)
            row = 0
            for slot, n in zip(step.host_slots, step.host_lens):
                s = view.state[slot]
                for i in range(n):
                    s = self.decay * s + u[row + i].float()
                    s_all[row + i] = s
                view.state[slot] = s
                row += n
            linear(s_all.to(step.dtype), self.w, resid, accumulate=True)

    @register("mixer", "toy_sum_and_count", replace=True)
    class SumAndCount(Part):
        """A mixer with TWO states of different shape and dtype: the running sum above (float32 [hidden]) and
        the number of tokens seen so far, kept with its negative in bfloat16 [1, 2].  out = s_t W^T * (1 +
        count_t / 100).  It asks the cache for a list of needs and gets a list of views."""
        graph_safe = False

        def __init__(self, hidden: int, decay: float):
            self.hidden, self.decay = hidden, decay

        def param_specs(self):
            return {"mix.weight": ParamSpec((self.hidden, self.hidden))}

        def load(self, t):
            self.w = t["mix.weight"]

        def cache_need(self):
            return [StateNeed((self.hidden,)), StateNeed((1, 2), torch.bfloat16)]

        def forward(self, u, resid, step, views):
            sums, counts = views
            assert counts.state.dtype == torch.bfloat16 and tuple(counts.state.shape[1:]) == (1, 2)
            s_all = torch.empty(u.shape, dtype=torch.float32, device=u.device)
            row = 0
            for slot, n in zip(step.host_slots, step.host_lens):
                s, c = sums.state[slot], counts.state[slot].float()
                for i in range(n):
                    s = self.decay * s + u[row + i].float()
                    c = c + torch.tensor([[1.0, -1.0]], device=u.device)
                    s_all[row + i] = s * (1.0 + c[0, 0] / 100.0)
                sums.state[slot] = s
                counts.state[slot] = c.to(torch.bfloat16)
                assert float(c[0, 0]) == -float(c[0, 1])
                row += n
            linear(s_all.to(step.dtype), self.w, resid, accumulate=True)

    @register("feed_forward", "toy_top1_experts", replace=True)
    class Top1Experts(Part):
        """A feed-forward with routing: every token goes to the one expert whose router logit is
        largest and gets relu(g Wup^T) Wdown^T times that expert's softmax weight."""
        graph_safe = False                      # which rows an expert gets is decided on the host

        def __init__(self, hidden: int, ff: int, experts: int):
            self.hidden, self.ff, self.experts = hidden, ff, experts

        def param_specs(self):
            H, F = self.hidden, self.ff
            out = {"router.weight": ParamSpec((self.experts, H), "vector", "conv")}
            for e in range(self.experts):
                out[f"experts.{e}.up.weight"] = ParamSpec((F, H))
                out[f"experts.{e}.down.weight"] = ParamSpec((H, F))
            return out

        def load(self, t):
            self.router = t["router.weight"]
            self.up = [t[f"experts.{e}.up.weight"] for e in range(self.experts)]
            self.down = [t[f"experts.{e}.down.weight"] for e in range(self.experts)]

        def forward(self, g, resid, step):
            logits = g.float() @ self.router.float().T                    # router logits in 32-bit
            prob = torch.softmax(logits, dim=-1)
            top = logits.argmax(dim=-1)
            for e in range(self.experts):
                rows = (top == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                h = torch.empty(rows.numel(), self.ff, dtype=torch.float32, device=g.device)
                linear(g[rows].contiguous(), self.up[e], h)
                y = torch.empty(rows.numel(), self.hidden, dtype=torch.float32, device=g.device)
                linear(torch.relu(h).to(step.dtype), self.down[e], y)
                resid.index_add_(0, rows, y * prob[rows, e, None])

    @register("feed_forward", "toy_counted", replace=True)
    class CountedFeedForward(Part):
        """A feed-forward with state per sequence: relu(g Wup^T) Wdown^T times (1 + tokens seen so far / 50).
        It overrides ``cache_need`` and is handed its view by the block."""
        graph_safe = False

        def __init__(self, hidden: int, ff: int):
            self.hidden, self.ff = hidden, ff

        def param_specs(self):
            return {"up.weight": ParamSpec((self.ff, self.hidden)), "down.weight": ParamSpec((self.hidden, self.ff))}

        def load(self, t):
            self.up, self.down = t["up.weight"], t["down.weight"]

        def cache_need(self):
            return StateNeed((1,))

        def forward(self, g, resid, step, view=None):
            assert view is not None and tuple(view.state.shape[1:]) == (1,)
            factor = torch.empty(g.shape[0], 1, dtype=torch.float32, device=g.device)
            row = 0
            for slot, n in zip(step.host_slots, step.host_lens):
                seen = float(view.state[slot, 0])
                factor[row:row + n, 0] = 1.0 + (seen + torch.arange(1, n + 1, device=g.device)) / 50.0
                view.state[slot, 0] = seen + n
                row += n
            h = torch.empty(g.shape[0], self.ff, dtype=torch.float32, device=g.device)
            linear(g, self.up, h)
            y = torch.empty(g.shape[0], self.hidden, dtype=torch.float32, device=g.device)
            linear(torch.relu(h).to(step.dtype), self.down, y)
            resid.add_(y * factor)

    @register("position", "toy_stretched_rope", replace=True)
    class StretchedRope(Part):
        """Another position encoding: a rotation whose pair i turns by pos / factor^(i / pairs) * theta^(-2i/hd),
        so that the slow pairs are stretched more than the fast ones."""

        def __init__(self, head_dim: int, theta: float, factor: float):
            self.head_dim, self.theta, self.factor = head_dim, theta, factor
            self.table = None

        def rotary(self, device):
            if self.table is None:              # made once: a recorded step may not copy from the host
                self.table = stretched_inv_freq(self.head_dim, self.theta, self.factor).to(torch.float32).to(device)
            return self.table, False

        def score_scale(self):
            return 1.0 + 0.1 * math.log(self.factor)    # the scores are sharpened to make up for the stretch

    @dataclass
    class ToyConfig:
        hidden_size: int
        vocab_size: int
        ff: int
        decay: float
        layer_types: List[str]
        schedule: List[list]
        eps: float = 1e-5
        heads: int = 2
        kv_heads: int = 1
        window: int = 0
        experts: int = 3
        stretch: float = 4.0

        @classmethod
        def from_dict(cls, d):
            return cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d})

    def describe(c: ToyConfig) -> ModelSpec:
        H = c.hidden_size
        hd = H // c.heads
        blocks = []
        for i, kind in enumerate(c.layer_types):
            pre = f"toy.{i}."
            ffn = PartSpec("swiglu", dict(hidden=H, ff=c.ff), prefix=pre + "ff.")
            if kind.endswith("+routed"):
                kind = kind[:-len("+routed")]
                ffn = PartSpec("toy_top1_experts", dict(hidden=H, ff=c.ff, experts=c.experts), prefix=pre + "moe.")
            if kind.endswith("+counted"):
                kind = kind[:-len("+counted")]
                ffn = PartSpec("toy_counted", dict(hidden=H, ff=c.ff), prefix=pre + "cnt.")
            if kind == "sum":
                mixer = PartSpec("toy_running_sum", dict(hidden=H, decay=c.decay), prefix=pre + "sum.")
            elif kind == "sum2":
                mixer = PartSpec("toy_sum_and_count", dict(hidden=H, decay=c.decay), prefix=pre + "sum.")
            elif kind == "attn_stretched":
                mixer = PartSpec("gqa", dict(hidden=H, n_heads=c.heads, n_kv_heads=c.kv_heads, head_dim=hd,
                                             qk_norm_eps=None, window=0, shared_kv=False), prefix=pre + "attn.",
                                 parts={"position": PartSpec("toy_stretched_rope",
                                                             dict(head_dim=hd, theta=1e4, factor=c.stretch))})
            elif kind in ("attn", "attn_shared"):
                mixer = PartSpec("gqa", dict(hidden=H, n_heads=c.heads, n_kv_heads=c.kv_heads, head_dim=hd,
                                             qk_norm_eps=None, window=c.window, shared_kv=kind == "attn_shared"),
                                 prefix=pre + "attn.",
                                 parts={"position": PartSpec("rope", dict(head_dim=hd, theta=1e4))})
            else:
                mixer = PartSpec("short_conv", dict(hidden=H, kernel=2), prefix=pre + "conv.")
            blocks.append(PartSpec("prenorm", prefix=pre, parts={
                "mixer_norm": PartSpec("rmsnorm", dict(dim=H, eps=c.eps), prefix=pre + "n1."), "mixer": mixer,
                "ffn_norm": PartSpec("rmsnorm", dict(dim=H, eps=c.eps), prefix=pre + "n2."),
                "ffn": ffn}))
        return ModelSpec(hidden_size=H, vocab_size=c.vocab_size,
                         embedding=PartSpec("table", dict(vocab=c.vocab_size, hidden=H), prefix="toy.embed."),
                         blocks=blocks, schedule=[ScheduleEntry(b, src) for b, src in c.schedule],
                         final_norm=PartSpec("rmsnorm", dict(dim=H, eps=c.eps), prefix="toy.norm."),
                         head=PartSpec("linear", dict(vocab=c.vocab_size, hidden=H, tied=True), prefix="toy.head."))

    register_architecture("ToyForCausalLM", ToyConfig.from_dict, describe, replace=True)


def stretched_inv_freq(hd, theta, factor):
    i = torch.arange(hd // 2, dtype=torch.float64)
    return 1.0 / (torch.tensor(theta, dtype=torch.float64) ** (2.0 * i / hd)) / factor ** (i / (hd // 2))


def plain_stretched_attention(u, wq, wk, wv, wo, nh, nkv, hd, theta, factor):
    """Causal grouped-query attention whose rotation uses stretched_inv_freq (pairs (2i, 2i+1))."""
    T = u.shape[0]
    ang = torch.arange(T, dtype=torch.float64)[:, None] * stretched_inv_freq(hd, theta, factor)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rot(v):
        out = torch.empty_like(v)
        a, b = v[..., 0::2], v[..., 1::2]
        out[..., 0::2], out[..., 1::2] = a * c - b * s, a * s + b * c
        return out

    q, k, v = rot((u @ wq.T).view(T, nh, hd)), rot((u @ wk.T).view(T, nkv, hd)), (u @ wv.T).view(T, nkv, hd)
    out = torch.zeros(T, nh, hd, dtype=torch.float64)
    for h in range(nh):
        g = h // (nh // nkv)
        sc = (q[:, h] @ k[:, g].T) / hd ** 0.5 * (1.0 + 0.1 * math.log(factor))
        sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        out[:, h] = torch.softmax(sc, -1) @ v[:, g]
    return out.reshape(T, nh * hd) @ wo.T


def toy_plain(cfg, w, tokens, margins=None):
    """The toy architecture, whole sequence, with the plain functions.  ``margins``: a list that
    receives, per token, the smallest gap between the two largest router logits it met."""
    f = lambda n: w[n].double()
    H, hd = cfg["hidden_size"], cfg["hidden_size"] // cfg.get("heads", 2)
    x = f("toy.embed.weight")[torch.tensor(tokens)]
    kvs = {}
    gap = torch.full((len(tokens),), float("inf"), dtype=torch.float64)
    for pos, (b, src) in enumerate(cfg["schedule"]):
        kind, pre = cfg["layer_types"][b], f"toy.{b}."
        routed = kind.endswith("+routed")
        kind = kind[:-len("+routed")] if routed else kind
        counted = kind.endswith("+counted")
        kind = kind[:-len("+counted")] if counted else kind
        u = P.plain_rms_norm(x, f(pre + "n1.weight"), 1e-5)
        if kind == "attn_stretched":
            x = x + plain_stretched_attention(u, f(pre + "attn.q_proj.weight"), f(pre + "attn.k_proj.weight"),
                                              f(pre + "attn.v_proj.weight"), f(pre + "attn.out_proj.weight"),
                                              cfg.get("heads", 2), cfg.get("kv_heads", 1), hd, 1e4,
                                              cfg.get("stretch", 4.0))
        elif kind in ("sum", "sum2"):
            s, rows = torch.zeros(H, dtype=torch.float64), []
            for t in range(len(tokens)):
                s = cfg["decay"] * s + u[t]
                rows.append(s * (1.0 + (t + 1) / 100.0) if kind == "sum2" else s)
            x = x + torch.stack(rows) @ f(pre + "sum.mix.weight").T
        elif kind in ("attn", "attn_shared"):
            kw = dict(nh=cfg.get("heads", 2), nkv=cfg.get("kv_heads", 1), hd=hd, eps=1e-5, theta=1e4,
                      style="interleaved", window=cfg.get("window", 0))
            if kind == "attn":
                out, kvs[pos] = P.plain_attention(u, f(pre + "attn.q_proj.weight"), f(pre + "attn.k_proj.weight"),
                                                  f(pre + "attn.v_proj.weight"), f(pre + "attn.out_proj.weight"),
                                                  None, None, return_kv=True, **kw)
            else:
                out = P.plain_attention(u, f(pre + "attn.q_proj.weight"), None, None, f(pre + "attn.out_proj.weight"),
                                        None, None, kv=kvs[src], **kw)
            x = x + out
        else:
            x = x + P.plain_short_conv(u, f(pre + "conv.in_proj.weight"), f(pre + "conv.conv.weight"),
                                       f(pre + "conv.out_proj.weight"))
        g = P.plain_rms_norm(x, f(pre + "n2.weight"), 1e-5)
        if routed:
            logits = g @ f(pre + "moe.router.weight").T
            prob, top = torch.softmax(logits, -1), logits.argmax(-1)
            two = logits.topk(2, dim=-1).values
            gap = torch.minimum(gap, two[:, 0] - two[:, 1])
            y = torch.zeros_like(x)
            for t in range(len(tokens)):
                e = int(top[t])
                hid = torch.relu(g[t] @ f(pre + f"moe.experts.{e}.up.weight").T)
                y[t] = hid @ f(pre + f"moe.experts.{e}.down.weight").T * prob[t, e]
            x = x + y
        elif counted:
            t = torch.arange(1, len(tokens) + 1, dtype=torch.float64)[:, None]
            x = x + (torch.relu(g @ f(pre + "cnt.up.weight").T) @ f(pre + "cnt.down.weight").T) * (1.0 + t / 50.0)
        else:
            x = x + P.plain_swiglu(g, f(pre + "ff.w1.weight"), f(pre + "ff.w3.weight"), f(pre + "ff.w2.weight"))
    if margins is not None:
        margins.append(gap)
    return P.plain_rms_norm(x, f("toy.norm.weight"), 1e-5) @ f("toy.embed.weight").T


TOYS = {
    # a mixer with state of its own between two kinds the package ships
    "state": dict(layer_types=["sum", "conv", "sum"], schedule=[[0, None], [1, None], [2, None]]),
    # a mixer with two states of different shape and dtype (a list of cache needs), run twice
    "two_states": dict(layer_types=["sum2", "attn"], schedule=[[0, None], [1, None], [0, None]]),
    # a feed-forward with state of its own, beside a mixer with one state, two states, and keys and values
    "ffn_state": dict(layer_types=["sum+counted", "sum2+counted", "attn+counted"], schedule=[[0, None], [1, None], [2, None]]),
    # the layer order is data: block 0 runs twice (same weights, a cache of its own each time)
    "twice": dict(layer_types=["conv", "attn", "sum"], schedule=[[0, None], [1, None], [0, None], [2, None], [1, None]]),
    # the last attention layer has no keys and values of its own and reads the first one's cache
    "shared": dict(layer_types=["attn", "conv", "attn_shared"], schedule=[[0, None], [1, None], [2, 0]]),
    # a window: its keys form a cache group of their own and its pages are given back on the way
    "window": dict(layer_types=["attn", "sum"], schedule=[[0, None], [1, None]], window=24),
    # a feed-forward with routing (the last layer's, so that a token routed otherwise by a rounding
    # error spoils its own logits only; such tokens, with a gap under 0.05 between the two best
    # router logits, are left out of the comparison)
    "routed": dict(layer_types=["conv", "attn+routed"], schedule=[[0, None], [1, None]]),
    # another position encoding inside the attention the package ships
    "position": dict(layer_types=["attn_stretched", "conv"], schedule=[[0, None], [1, None]]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("toy", list(TOYS))
def test_toy_architecture_registered_from_the_test(toy, dtype, tmp_path):
    from safetensors.torch import load_file
    from mivi_v4_b200 import Engine, load_model, write_random_model
    register_toy_parts()
    cfg = dict(architectures=["ToyForCausalLM"], hidden_size=48, vocab_size=97, ff=80, decay=0.9, heads=3, kv_heads=1,
               **TOYS[toy])
    folder = write_random_model(str(tmp_path / toy), cfg, seed=3)
    w = load_file(str(tmp_path / toy / "model.safetensors"))
    g = torch.Generator().manual_seed(1)
    seqs = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (70, 9, 33)]
    margins = []
    want = [toy_plain(cfg, w, s, margins) for s in seqs]
    sure = [m > 0.05 for m in margins]                 # tokens whose expert does not hang on rounding
    assert all(x.float().mean() > 0.8 for x in sure)
    eng = Engine(load_model(folder, dtype, DEV), max_tokens=1024, page_size=16)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    tol = 3e-5 if dtype == "float32" else 4e-2

    def close(a, b, what, keep=None):
        a, b = a.double().cpu(), b.double()
        if keep is not None:
            a, b = a[keep], b[keep]
        assert (a - b).abs().max() <= tol * max(1.0, b.abs().max().item()), (toy, what, (a - b).abs().max())

    # whole, then the same sequences in one unequal batch with the tail token by token
    for s, wv, ok in zip(seqs, want, sure):
        slot = eng.open()
        close(eng.step([(slot, s)], "all"), wv, "whole", ok)
        eng.close(slot)
    slots = [eng.open() for _ in seqs]
    cut = [len(s) - 5 for s in seqs]
    lg = eng.step([(sl, s[:c]) for sl, s, c in zip(slots, seqs, cut)], "last")
    for i in range(len(seqs)):
        if sure[i][cut[i] - 1]:
            close(lg[i], want[i][cut[i] - 1], "batch prompt")
    for j in range(5):
        lg = eng.step([(sl, [s[c + j]]) for sl, s, c in zip(slots, seqs, cut)], "last")
        for i in range(len(seqs)):
            if sure[i][cut[i] + j]:
                close(lg[i], want[i][cut[i] + j], f"decode {j}")
    if toy == "two_states":
        kinds = sorted((str(eng.cache.storage[g].dtype), tuple(eng.cache.storage[g].shape)) for g in eng.cache.state_groups)
        assert kinds == [("torch.bfloat16", (2, eng.cache.n_slots, 1, 2)), ("torch.float32", (2, eng.cache.n_slots, 48))]
    if toy == "window":
        kvg = eng.cache.kv_groups[0]
        assert eng.cache._get(slots[0]).pages[kvg][0] is None     # pages before the window went back
        assert eng.cache.plan.groups[kvg].need.window == 24
    for sl in slots:
        eng.close(sl)
    eng.cache.check()
    assert all(p.held_count == 0 for p in eng.cache.pages.values())
    del tdt
