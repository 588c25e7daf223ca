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


def test_a_replaced_buffer_is_kept_until_released_and_the_generation_tells():
    """A captured graph holds raw addresses: a buffer that must grow is retired, not freed, and the
    generation goes up so that the holder of graphs can drop them before the memory is let go."""
    ws = Workspace(torch.device("cpu"))
    ws.reserve("partials", 100, torch.float32)
    a = ws.get("partials", (10, 10), torch.float32)
    assert ws.generation == 0 and not ws.retired
    assert ws.get("partials", (5, 4), torch.float32).data_ptr() == a.data_ptr()    # smaller: nothing moves
    assert ws.generation == 0
    b = ws.get("partials", (11, 10), torch.float32)                                # larger: replaced
    assert ws.generation == 1 and len(ws.retired) == 1 and ws.retired[0].data_ptr() == a.data_ptr()
    assert b.data_ptr() != a.data_ptr()
    z = ws.get_zeroed("arrivals", (4,), torch.int32)
    assert ws.generation == 1                                                      # a first request is no replacement
    ws.get_zeroed("arrivals", (8,), torch.int32)
    assert ws.generation == 2 and ws.retired[1].data_ptr() == z.data_ptr()
    ws.release_retired()
    assert not ws.retired and ws.generation == 2
    ws.reserve("arrivals", 4, torch.int32, zeroed=True)                            # already large enough
    assert ws.generation == 2
