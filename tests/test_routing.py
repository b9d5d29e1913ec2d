"""Which kernel a product goes to is decided on the host from its shape alone (``ops/linear.py``): these are
the decisions for the five products of the LFM2.5-1.2B layer sizes, as measured when the rule was made."""
import torch

from mivi_v4_b200.ops import linear as L


def w(n, k):
    return torch.empty(n, k, dtype=torch.bfloat16, device="meta")


IN_PROJ, OUT_PROJ, GATE_UP, DOWN, QKV = w(6144, 2048), w(2048, 2048), w(16384, 2048), w(2048, 8192), w(3072, 2048)


def test_products_whose_k_must_be_cut_go_to_the_swapped_kernel():
    for rows in (65, 128, 256, 512, 1024):
        assert L.swap_takes(rows, DOWN), rows                  # K = 8,192: one block walking it alone takes 50 us
    assert not L.swap_takes(2048, DOWN)
    for rows in (65, 128, 256, 512):
        assert L.swap_takes(rows, OUT_PROJ), rows
    assert not L.swap_takes(1024, OUT_PROJ)
    assert L.swap_takes(128, IN_PROJ) and L.swap_takes(256, IN_PROJ) and not L.swap_takes(512, IN_PROJ)
    assert L.swap_takes(256, QKV) and L.swap_takes(512, QKV) and not L.swap_takes(1024, QKV)
    # the widest product fills the device with its row tiles alone from about a hundred rows on
    assert L.swap_takes(65, GATE_UP) and not L.swap_takes(128, GATE_UP) and not L.swap_takes(2048, GATE_UP)


def test_which_products_may_carry_a_norm():
    # every tensor-core kernel applies a scale; only the weight-streaming ones emit by default
    for rows in (1, 64, 65, 700, 2048, 30000):
        assert L.norm_link_ok(rows, IN_PROJ) and L.norm_link_ok(rows, GATE_UP)
    for rows in (1, 64, 65, 512):
        assert L.norm_link_ok(rows, OUT_PROJ, emits=True) and L.norm_link_ok(rows, DOWN, emits=True)
    assert not L.norm_link_ok(2048, OUT_PROJ, emits=True) and not L.norm_link_ok(2048, DOWN, emits=True)
    # float32 weights, or rows of a length that is no multiple of 8, never
    assert not L.norm_link_ok(8, torch.empty(64, 64, device="meta"))
    assert not L.norm_link_ok(8, w(64, 60))
