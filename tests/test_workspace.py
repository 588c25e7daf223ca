"""The step's scratch memory: named buffers that live as long as the engine, and the views of them."""
import torch

from nanoinfer_b200.parts.base import Workspace


def test_views_are_remembered_and_follow_a_buffer_that_grows():
    ws = Workspace(torch.device("cpu"))
    a = ws.get("x", (4, 8), torch.float32)
    assert ws.get("x", (4, 8), torch.float32) is a                 # the same view again
    b = ws.get("x", (2, 8), torch.float32)                         # another shape: the same memory
    assert b.data_ptr() == a.data_ptr() and b.shape == (2, 8)
    big = ws.get("x", (16, 8), torch.float32)                      # the buffer grows: old views are dropped
    again = ws.get("x", (4, 8), torch.float32)
    assert again is not a and again.data_ptr() == big.data_ptr()
    assert ws.get("x", (4, 8), torch.bfloat16).dtype == torch.bfloat16
    assert ws.nbytes() == 4 * 8 * 2                                # (another dtype under the same name replaces the buffer)


def test_zeroed_buffers_start_at_zero_and_keep_what_is_written():
    ws = Workspace(torch.device("cpu"))
    c = ws.get_zeroed("counters", (5,), torch.int32)
    assert c.tolist() == [0] * 5
    c[2] = 7
    assert ws.get_zeroed("counters", (5,), torch.int32)[2] == 7    # not zeroed again
    assert ws.get_zeroed("counters", (9,), torch.int32).tolist() == [0] * 9   # grown: zero again
