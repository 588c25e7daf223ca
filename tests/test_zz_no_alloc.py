"""The decode attention entry point that allocates nothing (nib_attention_decode_static).

Some hosts may not ask the driver for device memory once they are running: they gave the whole GPU
to a pool of their own at start-up, or they call from inside a stream callback or a real-time loop,
or their sandbox forbids it.  For them the library carries its scratch memory inside itself.  This
test calls that entry point through its exported C symbol, twice in a row on the same inputs and once
on others, and checks each result against the ordinary entry point, which takes its scratch from the
caller, and against the plain attention formula of the tests (so that the two entry points cannot
be wrong together).  It also checks that a call too large for the built-in scratch is refused, not run.

The file is named to be collected last, so that a run that stops at the first failure has already
run every other test; it passes alone in a fresh process as well."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _case(seed, n_rows, n_head, hd, lengths, dtype):
    g = torch.Generator().manual_seed(seed)
    ps = 16
    n_pages = sum(-(-n // ps) for n in lengths) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_blocks = max(-(-n // ps) for n in lengths)
    table = torch.full((n_rows, max_blocks), -1, dtype=torch.int32)
    cache = (torch.randn(n_pages, 2, n_head, ps, hd, generator=g)).to(dtype)
    for e, n in enumerate(lengths):
        for b in range(-(-n // ps)):
            table[e, b] = perm.pop()
    q = torch.randn(n_rows, n_head * hd, generator=g).to(dtype)
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32)
    return (q.to(DEV), cache.to(DEV), table.to(DEV), torch.arange(n_rows, dtype=torch.int32, device=DEV),
            positions.to(DEV))


def _plain(q, cache, table, lengths, n_head, hd, scale):
    """The plain attention of each row over its request's keys, gathered from the pages by hand."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import plain_gpt2 as P
    ps = cache.shape[3]
    rows = []
    for e, n in enumerate(lengths):
        pages = table[e, :-(-n // ps)].long().cpu()
        kv = cache.cpu().double()[pages]                                  # [blocks, 2, heads, page, hd]
        k = kv[:, 0].permute(0, 2, 1, 3).reshape(-1, n_head * hd)[:n]     # [positions, heads * hd]
        v = kv[:, 1].permute(0, 2, 1, 3).reshape(-1, n_head * hd)[:n]
        rows.append(P.causal_attention(q[e:e + 1].cpu().double(), k, v, n_head, n_head, scale=scale, window=0,
                                       q_pos0=n - 1))
    return torch.cat(rows)


def _static_call(lib, q, cache, table, row_entry, positions, out, n_head, scale, chunk, n_splits, status):
    fn = lib.nib_attention_decode_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    n_pages, _, n_kv_head, page_size, head_dim = cache.shape
    dt = 0 if q.dtype == torch.float32 else 1
    return fn(dt, q.data_ptr(), q.stride(0), cache.data_ptr(), out.data_ptr(), out.stride(0), table.data_ptr(),
              table.shape[1], None, row_entry.data_ptr(), positions.data_ptr(), q.shape[0], n_head, n_kv_head,
              head_dim, page_size, n_pages, ctypes.c_float(scale), 0, chunk, n_splits, status.data_ptr(),
              torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_static_scratch_entry_matches_the_ordinary_one(dtype, tol):
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.base import Workspace
    lib = ops.library().raw
    status = ops.status_word()
    n_head, hd = 6, 64
    scale = 1.0 / math.sqrt(hd)
    ws = Workspace(torch.device(DEV))
    for seed, lengths in ((1, [700, 333, 64, 1]), (1, [700, 333, 64, 1]), (2, [90, 513, 1000, 17])):
        n_rows = len(lengths)
        q, cache, table, row_entry, positions = _case(seed, n_rows, n_head, hd, lengths, dtype)
        want = torch.zeros_like(q)
        ops.attention_decode(q, cache, want, table, row_entry, positions, n_rows, n_head, scale, 0, status,
                             max(lengths), ws)
        chunk, n_splits = ops.decode_split(n_rows, n_head, max(lengths))
        assert n_splits > 1                                   # the scratch is really used
        got = torch.full_like(q, 7.0)
        rc = _static_call(lib, q, cache, table, row_entry, positions, got, n_head, scale, chunk, n_splits, status)
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert (got.float() - want.float()).abs().max().item() <= tol
        plain = _plain(q, cache, table, lengths, n_head, hd, scale)
        assert (got.cpu().double() - plain).abs().max().item() <= tol


def test_static_scratch_refuses_what_does_not_fit():
    from nanoinfer_b200.kernels import ops
    lib = ops.library().raw
    lims = (ctypes.c_longlong(), ctypes.c_longlong())
    lib.nib_attention_decode_static_limits.restype = None
    lib.nib_attention_decode_static_limits(ctypes.byref(lims[0]), ctypes.byref(lims[1]))
    max_floats = lims[0].value
    assert max_floats == 1 << 20 and lims[1].value == 1 << 14
    n_head, hd = 6, 64
    q, cache, table, row_entry, positions = _case(3, 4, n_head, hd, [40, 40, 40, 40], torch.float32)
    out = torch.full_like(q, 3.0)
    n_splits = max_floats // (4 * n_head * (hd + 2)) + 1       # one split too many for the array
    rc = _static_call(lib, q, cache, table, row_entry, positions, out, n_head, 0.125, 16, n_splits, ops.status_word())
    assert rc == -4                                            # NIB_ERR_STATIC_SCRATCH_TOO_SMALL
    torch.cuda.synchronize()
    assert (out == 3.0).all()                                  # nothing was launched
