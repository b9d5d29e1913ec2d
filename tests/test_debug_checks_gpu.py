"""The build with index checks (MIVI_DEBUG_CHECKS=1): kernels that turn a page-table entry or a slot number
into an address compare it with the bound declared for the launch, never use an index outside it, and set the
device's error flag instead, which the host reports as a ``KernelError``.

Nothing here can fault even if a check were wrong: the tensor handed to a kernel is the first half of a larger
tensor that the test owns, the bad index points into the second half, and the declared bound is the first
half's size.  The test then also asks that the second half is untouched.  It runs in a process of its own,
because the checked build is chosen when the library is loaded."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r'''
import sys, tempfile
import torch
sys.path.insert(0, %(root)r); sys.path.insert(0, %(tests)r)
from mivi_v4_b200.ops import kernels as K
from mivi_v4_b200.ops.build import DEBUG_CHECKS
from mivi_v4_b200.engine.step import Workspace
assert DEBUG_CHECKS and K.DEBUG_CHECKS
dev = "cuda:0"
ints = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)

def flagged(what):
    try:
        K.check_device_errors()
    except K.KernelError as e:
        assert "outside its bounds" in str(e), str(e)
        return
    raise AssertionError(what + ": an index outside the declared bound went unreported")

def clean(what):
    K.check_device_errors()          # raises if the flag is set

nh, nkv, hd, page = 4, 2, 32, 16
for dtype in (torch.float32, torch.bfloat16):
    big = torch.zeros(8, 2, nkv, page, hd, dtype=dtype, device=dev)
    pool = big[:4]                                     # what the kernels are told the cache is: 4 pages
    # a token at position 17 of a sequence whose second block is said to lie in page 6
    table = ints([[1, 6, 0, 0]])
    qkv = torch.randn(1, (nh + 2 * nkv) * hd, device=dev)
    q = torch.empty(1, nh * hd, dtype=dtype, device=dev)
    K.qk_prepare(qkv, None, None, 1e-5, None, False, ints([17]), ints([0]), table, pool, q, nh, nkv, hd)
    flagged("qk_prepare")
    assert torch.isfinite(q.float()).all() and float(q.float().abs().max()) > 0      # the queries were still written
    assert float(big.float().abs().max()) == 0.0, "qk_prepare wrote although its page was out of bounds"
    # the same token with a page inside the bound: written, nothing reported
    K.qk_prepare(qkv, None, None, 1e-5, None, False, ints([17]), ints([0]), ints([[1, 3, 0, 0]]), pool, q, nh, nkv, hd)
    clean("qk_prepare in bounds")
    assert float(big[3].float().abs().max()) > 0 and float(big[4:].float().abs().max()) == 0.0
    # reads: a query at position 20 whose second block is said to lie in page 6
    big.normal_()
    keep = big[4:].clone()
    out = torch.empty_like(q)
    K.attention_decode(q, pool, table, ints([20]), ints([0]), out, nh, nkv, hd, 0.2, 0, Workspace(dev))
    flagged("attention_decode")
    K.attention_generic(q, pool, table, ints([20]), ints([0]), out, nh, nkv, hd, 0.2, 0)
    flagged("attention_generic")
    if dtype == torch.bfloat16:
        qs = torch.randn(21, nh * hd, device=dev).to(dtype)
        outs = torch.empty_like(qs)
        K.attention_prefill(qs, pool, table, ints([0, 21]), ints([0]), outs, 1, nh, nkv, hd, 0.2, 0)
        flagged("attention_prefill")
    assert torch.equal(big[4:], keep)
    K.attention_decode(q, pool, ints([[1, 3, 0, 0]]), ints([20]), ints([0]), out, nh, nkv, hd, 0.2, 0, Workspace(dev))
    clean("attention_decode in bounds")

# slots: the state of 4 sequences inside a tensor of 8; the step names slot 6
H, k = 64, 3
state_big = torch.zeros(8, k - 1, H, device=dev)
state = state_big[:4]
taps = torch.randn(H, k, device=dev)
p = torch.randn(1, 3 * H, device=dev)
z = torch.empty(1, H, device=dev)
K.shortconv(p, taps, None, state, ints([5]), ints([0]), ints([0, 1]), ints([6]), ints([5]), ints([1]), z, 1, decode=True)
flagged("shortconv, one token")
p3 = torch.randn(3, 3 * H, device=dev)
z3 = torch.empty(3, H, device=dev)
K.shortconv(p3, taps, None, state, ints([5, 6, 7]), ints([0, 0, 0]), ints([0, 3]), ints([6]), ints([5]), ints([3]), z3, 1)
flagged("shortconv, three tokens")
assert float(state_big.abs().max()) == 0.0, "shortconv wrote state although its slot was out of bounds"
K.shortconv(p, taps, None, state, ints([5]), ints([0]), ints([0, 1]), ints([2]), ints([5]), ints([1]), z, 1, decode=True)
clean("shortconv in bounds")
assert float(state_big[2].abs().max()) > 0 and float(state_big[4:].abs().max()) == 0.0

# the whole engine in this build: right logits, nothing reported, no recorded steps
from helpers import assert_close, plain_logits, plain_noise, write_model
from tiny_configs import TINY_F, prompts
from mivi_v4_b200 import Engine, load_model
with tempfile.TemporaryDirectory() as tmp:
    folder = write_model(tmp, TINY_F, 5, init="loud")
    toks = prompts(TINY_F["vocab_size"], [150], seed=2)[0]
    for dtype in (torch.float32, torch.bfloat16):
        eng = Engine(load_model(folder, dtype, dev), max_tokens=512)
        assert not eng.cuda_graphs
        s = eng.open()
        rows = [eng.step([(s, toks[:130])], "all")] + [eng.step([(s, [t])], "last") for t in toks[130:]]
        assert_close(torch.cat(rows), plain_logits(folder, toks), dtype, "checked build", noise=plain_noise(folder, toks, dtype))
        eng.close(s)
        torch.cuda.synchronize()
        eng.check_errors()
        clean("engine")
print("checked build ok")
'''


def test_out_of_bounds_indices_are_skipped_and_reported():
    env = dict(os.environ, MIVI_DEBUG_CHECKS="1")
    script = SCRIPT % dict(root=ROOT, tests=os.path.join(ROOT, "tests"))
    proc = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env, timeout=900)
    assert proc.returncode == 0 and "checked build ok" in proc.stdout, proc.stdout[-1500:] + proc.stderr[-3000:]
