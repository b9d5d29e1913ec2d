"""The step workspace: named buffers that grow on demand, and the views of them that it hands out."""
import torch

from mivi_v4_b200.engine.step import Workspace


def test_views_are_kept_and_follow_their_buffer():
    ws = Workspace("cpu")
    a = ws.get("x", (4, 8), torch.float32)
    assert ws.get("x", (4, 8), torch.float32) is a                   # the same view for the same request
    b = ws.get("x", (2, 8), torch.float32)
    assert b.data_ptr() == a.data_ptr() and tuple(b.shape) == (2, 8)  # a smaller view of the same buffer
    gen = ws.generation
    big = ws.get("x", (16, 8), torch.float32)                        # the buffer has to grow: a new one
    assert ws.generation == gen + 1 and big.data_ptr() != a.data_ptr()
    again = ws.get("x", (4, 8), torch.float32)
    assert again is not a and again.data_ptr() == big.data_ptr()     # old views are not handed out again
    assert ws.get("x", (4, 8), torch.bfloat16).dtype == torch.bfloat16   # another dtype is another buffer
    assert ws.get("x", (4, 8), torch.float32) is again


def test_zeroed_buffers_replace_their_views_too():
    ws = Workspace("cpu")
    z = ws.get_zeroed("t", (8,), torch.int32)
    assert not z.any()
    v = ws.get("t", (8,), torch.int32)
    assert v.data_ptr() == z.data_ptr()
    z2 = ws.get_zeroed("t", (64,), torch.int32)                      # grows: the view kept for "t" is dropped
    assert not z2.any() and ws.get("t", (8,), torch.int32).data_ptr() == z2.data_ptr()
