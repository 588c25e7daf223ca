"""Each kernel alone against its plain formula, at sizes other than the engine's models:
widths and vocabularies that are no power of two, head sizes in steps of 8, grouped key/value
heads, windows, pages scattered over the pool."""
import math

import pytest
import torch

import plain_gpt2 as P

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from nanoinfer_b200.kernels import ops as o
    return o


def gen(seed=0):
    return torch.Generator().manual_seed(seed)


def attention_plan(ctx):
    from nanoinfer_b200.parts.attention import AttentionPlan
    return AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0, device=torch.device(DEV))


class Ctx:
    """The few fields of a StepContext that the attention kernels read."""

    def __init__(self, row_entry, positions, starts=None):
        self.row_entry = torch.tensor(row_entry, dtype=torch.int32, device=DEV)
        self.positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
        self.n_rows = len(positions)
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.n_entries = max(row_entry) + 1
        starts = starts or [row_entry.index(e) for e in range(self.n_entries)] + [len(row_entry)]
        self.host_entry_start = starts
        self.host_entry_pos0 = [positions[s] for s in starts[:-1]]
        self.entry_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        self.entry_pos0 = torch.tensor(self.host_entry_pos0, dtype=torch.int32, device=DEV)
        self.max_q_len = max(b - a for a, b in zip(starts, starts[1:]))
        self.max_kv_len = max(positions) + 1
        self.max_rows = self.n_rows
        from nanoinfer_b200.parts.base import Workspace
        self.workspace = Workspace(torch.device(DEV))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C", [100, 768, 1600])
def test_embed_adds_positions(dtype, C):
    V, Pn, T = 777, 300, 37
    g = gen(1)
    wte, wpe = torch.randn(V, C, generator=g).to(dtype), torch.randn(Pn, C, generator=g).to(dtype)
    tok = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    pos = torch.randint(0, Pn, (T,), generator=g, dtype=torch.int32)
    out = torch.full((T, C), 7.0, device=DEV)
    ops().embed(tok.to(DEV), wte.to(DEV), out, wpe.to(DEV), pos.to(DEV))
    want = wte.float()[tok.long()] + wpe.float()[pos.long()]
    assert torch.equal(out.cpu(), want)
    ops().embed(tok.to(DEV), wte.to(DEV), out)
    assert torch.equal(out.cpu(), wte.float()[tok.long()])


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C, eps", [(120, 1e-6), (768, 1e-5), (1600, 1e-5), (5000, 1e-3)])
def test_layernorm_two_pass_and_gather(out_dtype, C, eps):
    g = gen(2)
    x = (torch.randn(40, C, generator=g) * 3 + 50.0)             # a large mean punishes one-pass variance
    gamma, beta = torch.randn(C, generator=g), torch.randn(C, generator=g)
    rows = torch.tensor([39, 0, 7, 7, 21], dtype=torch.int32)
    out = torch.zeros(40, C, dtype=out_dtype, device=DEV)
    ops().layernorm(x.to(DEV), gamma.to(DEV), beta.to(DEV), eps, out, 40)
    want = P.layernorm(x.double(), gamma.double(), beta.double(), eps)
    tol = 2e-5 if out_dtype == torch.float32 else 3e-2
    assert (out.cpu().double() - want).abs().max() < tol * max(1.0, float(want.abs().max()))
    out2 = torch.zeros(5, C, dtype=out_dtype, device=DEV)
    ops().layernorm(x.to(DEV), gamma.to(DEV), beta.to(DEV), eps, out2, 5, rows.to(DEV))
    assert torch.equal(out2.cpu(), out.cpu()[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M, N, K", [(1, 96, 768), (37, 70, 3072), (130, 257, 100), (64, 1000, 120)])
@pytest.mark.parametrize("act", ["none", "tanh", "erf"])
def test_linear_simt(dtype, M, N, K, act):
    g = gen(3)
    a = (torch.randn(M, K, generator=g) * 0.5).to(dtype)
    w = (torch.randn(N, K, generator=g) * 0.05).to(dtype)
    b = torch.randn(N, generator=g)
    out = torch.zeros(M, N, dtype=dtype, device=DEV)
    o = ops()
    o.linear_simt(a.to(DEV), w.to(DEV), b.to(DEV), out, M, act=o.ACT_CODES[act])
    y = a.double() @ w.double().T + b.double()
    want = {"none": lambda u: u, "tanh": P.gelu_tanh, "erf": P.gelu_erf}[act](y)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (out.cpu().double() - want).abs().max() < tol
    # the residual epilogue adds into a 32-bit stream, rows beyond M untouched
    x = torch.randn(M + 3, N, generator=g)
    xd = x.to(DEV)
    o.linear_simt(a.to(DEV), w.to(DEV), b.to(DEV), xd, M, residual=True)
    assert (xd.cpu().double()[:M] - (x.double()[:M] + y)).abs().max() < tol
    assert torch.equal(xd.cpu()[M:], x[M:])


def test_linear_rows_do_not_depend_on_the_batch():
    g = gen(4)
    a, w = torch.randn(70, 200, generator=g), torch.randn(130, 200, generator=g)
    o = ops()
    full = torch.zeros(70, 130, device=DEV)
    o.linear_simt(a.to(DEV), w.to(DEV), None, full, 70)
    one = torch.zeros(1, 130, device=DEV)
    o.linear_simt(a[41:42].to(DEV), w.to(DEV), None, one, 1)
    assert torch.equal(one[0], full[41])
    # steps of at most 16 rows run on a kernel of their own (a thread per feature, K in chunks of 64 asked
    # for ahead): every output is still one accumulator in index order, so the bits are those of the tiled
    # kernel; with bias, both activations and the residual sum, and sizes that no tile divides
    bias = torch.randn(130, generator=g)
    for act in (o.ACT_NONE, o.ACT_GELU_TANH, o.ACT_GELU_ERF):
        for residual in (False, True):
            base = torch.randn(70, 130, generator=g).to(DEV)
            full = base.clone()
            o.linear_simt(a.to(DEV), w.to(DEV), bias.to(DEV), full, 70, act, residual)
            for m0, n in ((0, 1), (3, 5), (20, 8), (33, 13), (50, 16)):
                few = base[m0:m0 + n].clone()
                o.linear_simt(a[m0:m0 + n].to(DEV), w.to(DEV), bias.to(DEV), few, n, act, residual)
                assert torch.equal(few, full[m0:m0 + n]), (act, residual, m0, n)


def paged_case(dtype, n_head, n_kv_head, hd, page_size, lengths, q_lens, seed):
    """Requests of the given lengths whose last q_lens tokens are this step's rows; pages are dealt
    out in a shuffled order so that a request's blocks lie scattered."""
    g = gen(seed)
    n_pages = sum(-(-n // page_size) for n in lengths) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_blocks = max(-(-n // page_size) for n in lengths) + 1
    table = torch.full((len(lengths), max_blocks), -1, dtype=torch.int32)
    cache = torch.zeros(n_pages, 2, n_kv_head, page_size, hd)
    ks, vs, qs, row_entry, positions = [], [], [], [], []
    for e, (n, nq) in enumerate(zip(lengths, q_lens)):
        k, v = torch.randn(n, n_kv_head * hd, generator=g), torch.randn(n, n_kv_head * hd, generator=g)
        q = torch.randn(nq, n_head * hd, generator=g)
        k, v, q = k.to(dtype).float(), v.to(dtype).float(), q.to(dtype).float()
        ks.append(k); vs.append(v); qs.append(q)
        for b in range(-(-n // page_size)):
            table[e, b] = perm.pop()
        for j in range(n):
            page = int(table[e, j // page_size])
            cache[page, 0, :, j % page_size] = k[j].view(n_kv_head, hd)
            cache[page, 1, :, j % page_size] = v[j].view(n_kv_head, hd)
        row_entry += [e] * nq
        positions += list(range(n - nq, n))
    return dict(cache=cache.to(dtype), table=table, ks=ks, vs=vs, qs=qs, row_entry=row_entry, positions=positions)


ATT_CASES = [
    # n_head, n_kv_head, head_dim, page, lengths, q_lens, window
    (4, 4, 16, 16, [1, 17, 50], [1, 17, 3], 0),
    (5, 5, 24, 16, [40, 33, 2], [40, 1, 2], 0),
    (6, 2, 64, 16, [130, 64, 65], [1, 64, 2], 0),
    (3, 1, 128, 8, [70, 9], [5, 9], 0),
    (4, 2, 32, 16, [100, 45, 16], [100, 1, 16], 24),
    (2, 2, 80, 16, [300], [1], 0),
    # single tokens over long ranges: many splits per (row, head); with and without a window
    (12, 12, 64, 16, [1024, 1000, 513], [1, 1, 1], 0),
    (4, 2, 64, 16, [700, 300, 5], [1, 1, 1], 100),
    (1, 1, 256, 16, [90], [1], 0),
    # prompt portions of several 64-row tiles that continue an earlier part of the request
    (2, 2, 64, 16, [200], [130], 0),
    (4, 1, 32, 32, [260, 90], [200, 90], 50),
    (2, 2, 128, 16, [150, 64, 65], [150, 64, 2], 0),
    (3, 3, 48, 16, [100, 31], [37, 1], 0),
    # head size 64 in bfloat16 goes to the tcgen05 kernel: tiles of 128 rows, a window, pages of 32,
    # grouped heads, portions that begin in the middle of a page and of a tile
    (12, 12, 64, 16, [1024, 300], [1024, 200], 0),
    (4, 2, 64, 32, [400, 150], [333, 150], 90),
    (2, 1, 64, 16, [515, 2], [257, 2], 0),
    (3, 3, 64, 48, [200, 129, 128], [100, 129, 128], 130),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ATT_CASES)
def test_attention_over_scattered_pages(dtype, case):
    n_head, n_kv_head, hd, ps, lengths, q_lens, window = case
    c = paged_case(dtype, n_head, n_kv_head, hd, ps, lengths, q_lens, seed=hd + len(lengths))
    scale = 0.7 / math.sqrt(hd)
    want = torch.cat([
        P.causal_attention(q.double(), k.double(), v.double(), n_head, n_kv_head, scale=scale, window=window,
                           q_pos0=len(k) - len(q))
        for q, k, v in zip(c["qs"], c["ks"], c["vs"])])
    q = torch.cat(c["qs"]).to(dtype).to(DEV)
    out = torch.zeros_like(q)
    ctx = Ctx(c["row_entry"], c["positions"])
    ops().attention(q, c["cache"].to(DEV), out, c["table"].to(DEV), ctx, n_head, scale, window, attention_plan(ctx))
    assert int(ctx.status.item()) == 0
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (out.cpu().double() - want).abs().max() < tol


@pytest.mark.parametrize("case", [c for c in ATT_CASES if c[2] == 64 and max(c[5]) > 1])
def test_both_prefill_attention_kernels_at_head_size_64(case):
    """Head size 64 is taken by the tcgen05 kernel; the warp-level MMA kernel (which serves the other
    head sizes) and the tcgen05 kernel are each called directly here and must both agree with the
    plain attention on the rows of the prompt portions."""
    o = ops()
    n_head, n_kv_head, hd, ps, lengths, q_lens, window = case
    c = paged_case(torch.bfloat16, n_head, n_kv_head, hd, ps, lengths, q_lens, seed=hd + len(lengths))
    scale = 0.7 / math.sqrt(hd)
    want = torch.cat([
        P.causal_attention(q.double(), k.double(), v.double(), n_head, n_kv_head, scale=scale, window=window,
                           q_pos0=len(k) - len(q))
        for q, k, v in zip(c["qs"], c["ks"], c["vs"])])
    q = torch.cat(c["qs"]).to(torch.bfloat16).to(DEV)
    ctx = Ctx(c["row_entry"], c["positions"])
    plan = attention_plan(ctx)
    rows = [t for e in range(len(lengths)) if q_lens[e] > 1
            for t in range(ctx.host_entry_start[e], ctx.host_entry_start[e + 1])]
    cache, table = c["cache"].to(DEV), c["table"].to(DEV)
    assert o.library().nib_attention_prefill_tc_supported(hd, ps) and o.library().nib_attention_prefill_supported(hd)
    for kernel in ("tcgen05", "mma"):
        out = torch.zeros_like(q)
        if kernel == "tcgen05":
            o.attention_prefill_tc(q, cache, out, table, plan.wide_tiles, plan.n_wide_tiles, ctx.entry_start,
                                   ctx.entry_pos0, ctx.n_rows, n_head, scale, window, ctx.status)
        else:
            o.attention_prefill(q, cache, out, table, plan.tiles, plan.n_tiles, ctx.entry_start, ctx.entry_pos0,
                                n_head, scale, window, ctx.status)
        assert int(ctx.status.item()) == 0, kernel
        assert (out.cpu().double()[rows] - want[rows]).abs().max() < 2e-2, kernel


DECODE_CASES = [
    # n_head, n_kv_head, head_dim, page, lengths (one single-token row each), window
    (12, 12, 64, 16, [1024, 1000, 513, 1], 0),
    (6, 2, 64, 16, [130, 64, 65, 17], 0),
    (5, 5, 24, 16, [40, 33, 2], 0),
    (3, 1, 128, 32, [70, 9, 300], 0),
    (4, 2, 32, 16, [100, 45, 16], 24),
    (2, 2, 96, 48, [300, 31], 0),
    (4, 2, 64, 16, [700, 300, 5], 100),
    (2, 2, 80, 16, [250, 16], 0),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", DECODE_CASES)
def test_both_decode_attention_kernels_at_every_split(dtype, case):
    """Single decoded tokens over scattered pages, each kernel called directly with 1 to 16 splits of the
    keys: the streaming kernel (both dtypes, every head size) and, in bfloat16 at head sizes 32, 64,
    96 and 128, the kernel that takes 16 keys at a time with warp-level MMAs; against the plain
    attention.  Positions past a row's own in its last page hold NaN, as a page that was used before
    may: a key that is not the row's must not reach the result, not even times zero."""
    o = ops()
    n_head, n_kv_head, hd, ps, lengths, window = case
    c = paged_case(dtype, n_head, n_kv_head, hd, ps, lengths, [1] * len(lengths), seed=3 * hd + len(lengths))
    for e, n in enumerate(lengths):                     # poison what lies behind each request's last position
        if n % ps:
            c["cache"][int(c["table"][e, (n - 1) // ps]), :, :, n % ps:] = float("nan")
    scale = 0.7 / math.sqrt(hd)
    want = torch.cat([
        P.causal_attention(q.double(), k.double(), v.double(), n_head, n_kv_head, scale=scale, window=window,
                           q_pos0=len(k) - 1)
        for q, k, v in zip(c["qs"], c["ks"], c["vs"])])
    q = torch.cat(c["qs"]).to(dtype).to(DEV)
    ctx = Ctx(c["row_entry"], c["positions"])
    cache, table = c["cache"].to(DEV), c["table"].to(DEV)
    n_rows, max_keys = len(lengths), (min(max(lengths), window) if window else max(lengths))
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    lib = o.library()
    dt = 0 if dtype == torch.float32 else 1
    stream = torch.cuda.current_stream().cuda_stream
    kernels = ["streaming"]
    if dtype == torch.bfloat16 and lib.nib_attention_decode_mma_supported(hd, ps):
        kernels.append("mma")
    assert ("mma" in kernels) == (dtype == torch.bfloat16 and hd in (32, 64, 96, 128))
    scratch = torch.zeros(o.DECODE_RESIDENT_BLOCKS * (hd + 2), device=DEV)
    counters = torch.zeros(o.DECODE_RESIDENT_BLOCKS, dtype=torch.int32, device=DEV)
    if "mma" in kernels:
        kernels += ["mma, splits in a cluster", "mma, ring 2", "mma, ring 3", "mma, ring 4", "mma, ring 2, splits in a cluster",
                    "mma, ring 3, splits in a cluster"]
    for kernel in kernels:
        for ns in (1, 2, 5, 16) if "cluster" not in kernel else (2, 3, 4, 5, 6, 7, 8, 11, 16):
            chunk = max(16, -(-(-(-max_keys // ns)) // 16) * 16)
            n_splits = -(-max_keys // chunk)
            if n_rows * n_head * n_splits > o.DECODE_RESIDENT_BLOCKS:
                continue
            out = torch.full_like(q, 7.0)
            if "cluster" in kernel and not 2 <= n_splits <= (8 if "ring" in kernel else 16):
                continue                     # (beyond the portable cluster size of 8 there is no ring)
            args = (q.data_ptr(), q.stride(0), cache.data_ptr(), scratch.data_ptr(), out.data_ptr(), out.stride(0),
                    table.data_ptr(), table.shape[1], None, ctx.row_entry.data_ptr(), ctx.positions.data_ptr(), n_rows,
                    n_head, n_kv_head, hd, ps, cache.shape[0], scale, window, chunk, n_splits, counters.data_ptr(),
                    ctx.status.data_ptr())
            code = lib.nib_attention_decode(dt, *args, stream) if kernel == "streaming" else \
                lib.nib_attention_decode_mma(*args, int("cluster" in kernel),
                                             int(kernel.split("ring ")[1][0]) if "ring" in kernel else 0, stream)
            assert code == 0 and int(ctx.status.item()) == 0, (kernel, n_splits)
            diff = (out.cpu().double() - want).abs().max()
            assert diff < tol, f"{kernel}, {n_splits} splits: {float(diff):.3e}"     # (NaN fails here too)
            assert int(counters.abs().sum().item()) == 0     # found zero, left zero


def test_attention_finds_one_far_key_among_hundreds():
    """One key far back is made to match the query: the output must be that key's value, whichever
    page it lies on."""
    n_head, hd, ps, n = 2, 64, 16, 600
    for far in (0, 15, 16, 17, 255, 256, 431, 598):
        c = paged_case(torch.float32, n_head, n_head, hd, ps, [n], [1], seed=far)
        k, v, q = c["ks"][0], c["vs"][0], c["qs"][0]
        page = int(c["table"][0, far // ps])
        for h in range(n_head):
            c["cache"][page, 0, h, far % ps] = 40.0 * q[0, h * hd:(h + 1) * hd] / q[0, h * hd:(h + 1) * hd].norm()
        out = torch.zeros(1, n_head * hd, device=DEV)
        ctx = Ctx(c["row_entry"], c["positions"])
        ops().attention(q.to(DEV), c["cache"].to(DEV), out, c["table"].to(DEV), ctx, n_head, 1.0, 0, attention_plan(ctx))
        assert (out.cpu() - v[far]).abs().max() < 1e-3, f"key {far} was not found"


def test_kv_append_writes_the_right_slots():
    o = ops()
    for dtype in (torch.float32, torch.bfloat16):
        n_kv_head, hd, ps = 3, 24, 16
        kv = n_kv_head * hd
        T = 21
        g = gen(9)
        src = torch.randn(T, 40 + 2 * kv, generator=g).to(dtype)
        table = torch.tensor([[5, 2, -1], [0, 7, 3]], dtype=torch.int32)
        row_entry = [0] * 4 + [1] * 17
        positions = [14, 15, 16, 17] + list(range(20, 37))
        cache = torch.zeros(8, 2, n_kv_head, ps, hd, dtype=dtype, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        o.kv_append(src.to(DEV), 40, 40 + kv, cache, table.to(DEV),
                    torch.tensor(row_entry, dtype=torch.int32, device=DEV),
                    torch.tensor(positions, dtype=torch.int32, device=DEV), T, status)
        want = torch.zeros(8, 2, n_kv_head, ps, hd, dtype=dtype)
        for t in range(T):
            page = int(table[row_entry[t], positions[t] // ps])
            want[page, 0, :, positions[t] % ps] = src[t, 40:40 + kv].view(n_kv_head, hd)
            want[page, 1, :, positions[t] % ps] = src[t, 40 + kv:].view(n_kv_head, hd)
        assert torch.equal(cache.cpu(), want) and int(status.item()) == 0
        # a page index outside the pool is reported, not followed
        bad = table.clone(); bad[1, 1] = 99
        o.kv_append(src.to(DEV), 40, 40 + kv, cache, bad.to(DEV),
                    torch.tensor(row_entry, dtype=torch.int32, device=DEV),
                    torch.tensor(positions, dtype=torch.int32, device=DEV), T, status)
        assert int(status.item()) == o.STATUS_BAD_PAGE


def test_argmax_ties_and_odd_vocabulary():
    V = 50257
    lg = torch.randn(5, V, generator=gen(5))
    lg[1, 40000] = lg[1, 123] = 9.0
    lg[2, V - 1] = 11.0
    lg[3, :] = 0.25
    out = torch.zeros(5, dtype=torch.int32, device=DEV)
    padded = torch.zeros(5, V + 15, device=DEV)
    padded[:, :V] = lg.to(DEV)
    ops().argmax(padded[:, :V], out, 5)
    assert out.tolist() == [P.argmax(lg[i]) for i in range(5)] and out.tolist()[1:4] == [123, V - 1, 0]


@pytest.mark.parametrize("teams, R", [(False, 8), (True, 8), (True, 24), (True, 48)])
@pytest.mark.parametrize("V", [1000, 50257])
def test_sampling_follows_the_reference_walk(V, teams, R):
    """``teams``: a sampled row is the work of one block, or of the blocks of a cluster: eight of them
    for a few rows, four or two where that many teams still fit the device at once (24 and 48 rows)."""
    o = ops()
    lg = torch.randn(R, V, generator=gen(6)) * 2.5
    for r in range(4, R, 8):
        lg[r, :] = lg[r, 0]                                         # all equal: every walk is a tie
    # rows 6 and 7 (of every eight): a low temperature spreads the scaled logits far beyond the span in which
    # tokens have mass; row 6 keeps so many that the k-th largest lies among the massless ones
    temps = [[0.8, 1.0, 0.0, 1.3, 1.0, 0.6, 0.3, 0.05][r % 8] for r in range(R)]
    topk = [[40, 0, 5, 7, 3, V + 5, 2 * V // 5, 0][r % 8] for r in range(R)]
    seeds = [[42, 7, 1, 99, 5, 2 ** 40 + 3, 11, 12][r % 8] + 1000 * (r // 8) for r in range(R)]
    slots = torch.tensor([(5 * r + 3) % R for r in range(R)], dtype=torch.int32, device=DEV)   # (5 and R coprime)
    t_dev = torch.zeros(R, device=DEV); k_dev = torch.zeros(R, dtype=torch.int32, device=DEV)
    rng = torch.zeros(R, dtype=torch.int64, device=DEV)
    for r, sl in enumerate(slots.tolist()):
        t_dev[sl], k_dev[sl], rng[sl] = temps[r], topk[r], seeds[r]
    plain = [P.XorShiftSampler(temps[r], topk[r], seeds[r]) for r in range(R)]
    out = torch.zeros(R, dtype=torch.int32, device=DEV)
    scratch = torch.zeros(2 * R, dtype=torch.int64, device=DEV)
    dev = lg.to(DEV)
    agree = total = 0
    for _ in range(12 if R == 8 else (4 if V == 1000 else 1)):      # (the plain walk over 50257 tokens is slow)
        o.sample(dev, R, slots, t_dev, k_dev, rng, out, scratch, teams=teams)
        got = out.tolist()
        want = [plain[r].sample(lg[r]) for r in range(R)]
        for r in range(R):
            if r % 8 == 2:
                assert got[r] == want[r]                            # greedy row
            elif r % 8 == 4:
                assert 0 <= got[r] < 3                              # ties: the three lowest indices are kept
            else:
                total += 1
                agree += int(got[r] == want[r])
    # the walks agree except where r falls within rounding of a boundary between two tokens
    assert agree >= total - max(1, R // 8)
    for r, sl in enumerate(slots.tolist()):                         # the generator words advanced alike
        if temps[r] > 0:
            assert (int(rng[sl].item()) & (2 ** 64 - 1)) == plain[r].rng
    assert len(set(slots.tolist())) == R


TC_SHAPES = [
    # M, N, K: few rows take the swapped orientation (weights on the MMA's M side), many rows the plain one
    (1, 96, 768), (8, 2304, 768), (37, 70, 3072), (64, 1000, 120), (128, 257, 64), (16, 50257, 64),
    (129, 768, 768), (300, 200, 200), (2048, 2304, 768), (515, 1000, 3072), (130, 50, 72),
]


@pytest.mark.parametrize("M, N, K", TC_SHAPES)
def test_linear_tensor_cores(M, N, K):
    """tcgen05 GEMM against a float64 product of the same bfloat16 inputs: every epilogue, both
    output types, sizes that are no multiple of any tile."""
    o = ops()
    g = gen(M * 7 + N)
    a = (torch.randn(M + 2, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    ad, wd, bd = a.to(DEV), w.to(DEV), b.to(DEV)
    assert o.linear_tc_supported(ad, wd)
    y = a[:M].double() @ w.double().T + b.double()
    scale = float(y.abs().max())
    for act, fn in (("none", lambda u: u), ("tanh", P.gelu_tanh), ("erf", P.gelu_erf)):
        out = torch.full((M + 2, N), 3.0, dtype=torch.bfloat16, device=DEV)
        o.linear_tc(ad, wd, bd, out, M, act=o.ACT_CODES[act])
        want = fn(y)
        assert (out.cpu().double()[:M] - want).abs().max() < 1e-2 * max(1.0, scale), act
        assert (out.cpu()[M:] == 3.0).all()                          # rows beyond M are untouched
    # 32-bit output into a pitched buffer (the logits), without bias
    pitch = (N + 15) // 16 * 16 + 16
    buf = torch.full((M, pitch), -7.0, device=DEV)
    o.linear_tc(ad, wd, None, buf[:, :N], M)
    assert (buf.cpu().double()[:, :N] - (y - b.double())).abs().max() < 2e-3 * max(1.0, scale)
    assert (buf.cpu()[:, N:] == -7.0).all()
    # residual: added into the 32-bit stream
    x = torch.randn(M + 2, N, generator=g)
    xd = x.to(DEV)
    o.linear_tc(ad, wd, bd, xd, M, residual=True)
    assert (xd.cpu().double()[:M] - (x.double()[:M] + y)).abs().max() < 2e-3 * max(1.0, scale)
    assert torch.equal(xd.cpu()[M:], x[M:])
    assert int(o.status_word().item()) == 0


def test_linear_falls_back_when_rows_are_not_16_byte_multiples():
    o = ops()
    g = gen(11)
    a, w = torch.randn(5, 36, generator=g).to(torch.bfloat16), torch.randn(20, 36, generator=g).to(torch.bfloat16)
    ad, wd = a.to(DEV), w.to(DEV)
    assert not o.linear_tc_supported(ad, wd)                         # K = 36: 72-byte rows
    out = torch.zeros(5, 20, dtype=torch.bfloat16, device=DEV)
    o.linear(ad, wd, None, out, 5)
    assert (out.cpu().double() - a.double() @ w.double().T).abs().max() < 0.1


@pytest.mark.parametrize("M, n_head, n_kv_head, hd", [(1, 4, 4, 16), (8, 12, 12, 64), (20, 3, 1, 48), (37, 6, 2, 32), (64, 12, 12, 64), (128, 5, 5, 24)])
def test_fused_qkv_projection_writes_queries_and_cache(M, n_head, n_kv_head, hd):
    """The small-step q/k/v projection: queries to the output, keys and values into scattered pages."""
    o = ops()
    g = gen(M + hd)
    C, ps = 64 + 8 * n_head, 16
    q_dim, kv_dim = n_head * hd, n_kv_head * hd
    N = q_dim + 2 * kv_dim
    a = (torch.randn(M, C, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, C, generator=g) * 0.1).to(torch.bfloat16)
    b = torch.randn(N, generator=g) * 0.1
    # each row is the next token of a request of its own, at a position of its own
    positions = torch.randint(0, 200, (M,), generator=g).tolist()
    n_pages = M * 13 + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((M, 13), -1, dtype=torch.int32)
    for e in range(M):
        table[e, positions[e] // ps] = perm.pop()
    cache = torch.zeros(n_pages, 2, n_kv_head, ps, hd, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    status = o.status_word()
    done = o.linear_qkv(a.to(DEV), w.to(DEV), b.to(DEV), out, M, q_dim, cache, table.to(DEV),
                        torch.arange(M, dtype=torch.int32, device=DEV),
                        torch.tensor(positions, dtype=torch.int32, device=DEV), status)
    assert done and int(status.item()) == 0
    y = (a.double() @ w.double().T + b.double())
    assert (out.cpu().double()[:, :q_dim] - y[:, :q_dim]).abs().max() < 2e-2
    want = torch.zeros(n_pages, 2, n_kv_head, ps, hd, dtype=torch.float64)
    for e in range(M):
        page = int(table[e, positions[e] // ps])
        want[page, 0, :, positions[e] % ps] = y[e, q_dim:q_dim + kv_dim].view(n_kv_head, hd)
        want[page, 1, :, positions[e] % ps] = y[e, q_dim + kv_dim:].view(n_kv_head, hd)
    assert (cache.cpu().double() - want).abs().max() < 2e-2
    assert (out.cpu()[:, q_dim:] == 0).all()            # key and value columns of the buffer are not written


SMALL_SHAPES = [(1, 96, 768), (8, 2304, 768), (8, 3072, 768), (37, 70, 3072), (64, 1000, 120), (128, 257, 64),
                (16, 768, 3072), (5, 50257, 64), (8, 4800, 1600), (13, 200, 2048), (3, 96, 1104),
                # 17 to 64 rows: row blocks of 16, the norm folded into each
                (24, 2304, 768), (32, 3072, 768), (64, 2304, 768), (50, 3072, 1024), (20, 4800, 1600), (40, 96, 768),
                (17, 1000, 1104),
                # 65 to 128 rows: up to eight row blocks
                (100, 2304, 768), (128, 768, 768), (96, 3072, 1024), (65, 70, 768)]


@pytest.mark.parametrize("M, N, K", SMALL_SHAPES)
@pytest.mark.parametrize("folded", [False, True])
@pytest.mark.parametrize("kernel", ["dispatch", "tensor_core"])
def test_small_step_product_with_folded_layernorm_and_split_k(M, N, K, folded, kernel):
    """Steps of at most 128 rows, through the dispatcher (warp-level MMA kernel up to 64 rows) and through
    the tcgen05 kernel with all its options: K split over blocks (partial tiles summed by the last
    block, or reduce-added for the residual) and the LayerNorm before the product folded in."""
    o = ops()

    def product(a, wd, bd, out, M, act=0, residual=False, norm=None):
        if kernel == "dispatch":
            o.linear(a, wd, bd, out, M, act=act, residual=residual, norm=norm)
        else:
            assert o.linear_small_tc(a, norm, wd, bd, out, M, act, residual, split=True)

    from nanoinfer_b200.parts.base import Workspace
    g = gen(M * 3 + N + K)
    x = torch.randn(M + 5, K, generator=g) * 2.0 + 0.5
    gamma, beta = 1 + 0.1 * torch.randn(K, generator=g), 0.1 * torch.randn(K, generator=g)
    rows = torch.randperm(M + 5, generator=g)[:M].to(torch.int32)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    xn = P.layernorm(x.double(), gamma.double(), beta.double(), 1e-5)[rows.long()]
    xn16 = xn.to(torch.bfloat16)
    y = xn16.double() @ w.double().T + b.double()
    scale = max(1.0, float(y.abs().max()))
    ws = Workspace(torch.device(DEV))
    wd, bd = w.to(DEV), b.to(DEV)

    def activations():
        if folded:
            return None, o.NormInput(x.to(DEV), gamma.to(DEV), beta.to(DEV), 1e-5, ws, torch.bfloat16,
                                     rows=rows.to(DEV))
        return xn16.to(DEV), None

    for act, fn in (("none", lambda u: u), ("tanh", P.gelu_tanh)):
        a, norm = activations()
        out = torch.full((M + 2, N), 3.0, dtype=torch.bfloat16, device=DEV)
        product(a, wd, bd, out, M, act=o.ACT_CODES[act], norm=norm)
        assert (out.cpu().double()[:M] - fn(y)).abs().max() < 1.5e-2 * scale, act
        assert (out.cpu()[M:] == 3.0).all()
    a, norm = activations()
    res = torch.randn(M + 2, N, generator=g)
    rd = res.to(DEV)
    product(a, wd, bd, rd, M, residual=True, norm=norm)
    assert (rd.cpu().double()[:M] - (res.double()[:M] + y)).abs().max() < 4e-3 * scale
    assert torch.equal(rd.cpu()[M:], res[M:])
    a, norm = activations()
    pitch = (N + 15) // 16 * 16
    buf = torch.full((M, pitch), -7.0, device=DEV)
    product(a, wd, None, buf[:, :N], M, norm=norm)
    assert (buf.cpu().double()[:, :N] - (y - b.double())).abs().max() < 4e-3 * scale
    assert (buf.cpu()[:, N:] == -7.0).all()
    assert int(o.status_word().item()) == 0
    # the same call twice gives the same bits: the splits are summed in a fixed order
    a, norm = activations()
    out1 = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    product(a, wd, bd, out1, M, norm=norm)
    a, norm = activations()
    out2 = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    product(a, wd, bd, out2, M, norm=norm)
    assert torch.equal(out1, out2)


@pytest.mark.parametrize("M, N, K", [(17, 96, 768), (32, 2304, 768), (33, 70, 1024), (64, 3072, 768), (64, 130, 264),
                                     (28, 400, 1600), (100, 2304, 768), (128, 96, 1024), (65, 768, 768)])
def test_few_row_product_in_row_blocks_gives_each_row_its_own_bits(M, N, K):
    """Beyond 16 rows the step is cut into row blocks of 16, each normalising its own rows: a row's
    results are the bits it gets in a step of its own, whichever block it falls into."""
    o = ops()
    from nanoinfer_b200.parts.base import Workspace
    g = gen(7 * M + N + K)
    x = torch.randn(M + 3, K, generator=g) * 1.5 - 0.3
    gamma, beta = 1 + 0.1 * torch.randn(K, generator=g), 0.1 * torch.randn(K, generator=g)
    rows = torch.randperm(M + 3, generator=g)[:M].to(torch.int32)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    ws = Workspace(torch.device(DEV))
    xd, gd, bed, wd, bd, rd = x.to(DEV), gamma.to(DEV), beta.to(DEV), w.to(DEV), b.to(DEV), rows.to(DEV)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    norm = o.NormInput(xd, gd, bed, 1e-5, ws, torch.bfloat16, rows=rd)
    assert o.linear_skinny(None, norm, wd, bd, out, M), "the kernel refused the shape"
    xn = P.layernorm(x.double(), gamma.double(), beta.double(), 1e-5)[rows.long()].to(torch.bfloat16)
    y = xn.double() @ w.double().T + b.double()
    assert (out.cpu().double() - y).abs().max() < 1.5e-2 * max(1.0, float(y.abs().max()))
    for m in sorted(m for m in {0, 1, 15, 16, 31, 32, M // 2, M - 2, M - 1} if m < M):
        alone = torch.zeros(1, N, dtype=torch.bfloat16, device=DEV)
        one = o.NormInput(xd, gd, bed, 1e-5, ws, torch.bfloat16, rows=rd[m:m + 1].contiguous())
        assert o.linear_skinny(None, one, wd, bd, alone, 1)
        assert torch.equal(alone[0], out[m]), f"row {m}"
    assert int(o.status_word().item()) == 0


SPLIT_SHAPES = [(1, 96, 768), (8, 768, 3072), (16, 768, 768), (20, 100, 1000), (33, 70, 3072), (64, 1000, 264),
                (64, 768, 3072), (48, 2304, 768), (80, 768, 3072), (128, 100, 1000)]


@pytest.mark.parametrize("M, N, K", SPLIT_SHAPES)
@pytest.mark.parametrize("split", [0, 1, 2, 4, 8])
def test_few_row_product_with_k_split_over_a_cluster(M, N, K, split):
    """The warp-level MMA kernel for steps of at most 64 rows, with K split over the blocks of a
    cluster (their sums exchanged through distributed shared memory): every epilogue, rows and
    columns beside the result untouched, the same bits twice, and a split that would leave a block
    without work refused."""
    o = ops()
    g = gen(M * 7 + N + K + split)
    a = (torch.randn(M, K, generator=g) * 0.7).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    y = a.double() @ w.double().T + b.double()
    scale = max(1.0, float(y.abs().max()))
    ad, wd, bd = a.to(DEV), w.to(DEV), b.to(DEV)
    k_per = (-(-K // max(split, 1)) + 31) // 32 * 32
    if split > 1 and (split - 1) * k_per >= K:
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        with pytest.raises(o.KernelError):
            o.linear_skinny(ad, None, wd, bd, out, M, split=split)
        return
    # the step's rows of a block's slice of K must fit in shared memory: else the kernel declines
    row_tiles = 1 if M <= 8 else 2                        # (more than 16 rows: row blocks of 16)
    pitch = k_per + ((32 - k_per % 64) + 64) % 64
    if split and row_tiles * 8 * pitch * 2 + 10 * row_tiles * 128 * 4 > 200 * 1024:
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        assert not o.linear_skinny(ad, None, wd, bd, out, M, split=split)
        assert (out == 0).all()
        return
    for act, fn in (("none", lambda u: u), ("tanh", P.gelu_tanh), ("erf", P.gelu_erf)):
        out = torch.full((M + 2, N), 3.0, dtype=torch.bfloat16, device=DEV)
        assert o.linear_skinny(ad, None, wd, bd, out, M, act=o.ACT_CODES[act], split=split)
        assert (out.cpu().double()[:M] - fn(y)).abs().max() < 1.5e-2 * scale, act
        assert (out.cpu()[M:] == 3.0).all()
    res = torch.randn(M + 2, N, generator=g)
    rd = res.to(DEV)
    assert o.linear_skinny(ad, None, wd, bd, rd, M, residual=True, split=split)
    assert (rd.cpu().double()[:M] - (res.double()[:M] + y)).abs().max() < 4e-3 * scale
    assert torch.equal(rd.cpu()[M:], res[M:])
    pitch = (N + 15) // 16 * 16
    buf = torch.full((M, pitch), -7.0, device=DEV)
    assert o.linear_skinny(ad, None, wd, None, buf[:, :N], M, split=split)
    assert (buf.cpu().double()[:, :N] - (y - b.double())).abs().max() < 4e-3 * scale
    assert (buf.cpu()[:, N:] == -7.0).all()
    out1 = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    out2 = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    assert o.linear_skinny(ad, None, wd, bd, out1, M, split=split)
    assert o.linear_skinny(ad, None, wd, bd, out2, M, split=split)
    assert torch.equal(out1, out2)
    # a row's result does not depend on the rows beside it
    if M > 1:
        alone = torch.zeros(1, N, dtype=torch.bfloat16, device=DEV)
        assert o.linear_skinny(ad[M - 1:], None, wd, bd, alone, 1, split=split or 1)
        assert (alone.cpu().double() - out1.cpu().double()[M - 1:]).abs().max() < 1.5e-2 * scale
    assert int(o.status_word().item()) == 0


PAIR_SHAPES = [(256, 256, 64), (2048, 2304, 768), (2000, 3072, 768), (513, 1000, 264), (1024, 768, 3072), (300, 200, 72)]


@pytest.mark.parametrize("M, N, K", PAIR_SHAPES)
@pytest.mark.parametrize("bq", [0, 128, 192, 256])
def test_product_by_pairs_of_blocks(M, N, K, bq):
    """The tcgen05 product for many rows by pairs of blocks that share one 256-row MMA: every epilogue,
    ragged edges in rows and columns, K split over blocks for the residual sum, rows and columns beside
    the result untouched."""
    o = ops()
    g = gen(M + N + K + bq)
    a = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    y = a.double() @ w.double().T + b.double()
    scale = max(1.0, float(y.abs().max()))
    ad, wd, bd = a.to(DEV), w.to(DEV), b.to(DEV)
    if bq > N and bq > 128:
        bq = 128
    for act, fn in (("none", lambda u: u), ("tanh", P.gelu_tanh), ("erf", P.gelu_erf)):
        out = torch.full((M + 2, N), 3.0, dtype=torch.bfloat16, device=DEV)
        assert o.linear_tc_pair(ad, wd, bd, out, M, act=o.ACT_CODES[act], bq=bq)
        assert (out.cpu().double()[:M] - fn(y)).abs().max() < 1.5e-2 * scale, act
        assert (out.cpu()[M:] == 3.0).all()
    for splits in (0, 1, 2):
        res = torch.randn(M + 2, N, generator=g)
        rd = res.to(DEV)
        assert o.linear_tc_pair(ad, wd, bd, rd, M, residual=True, bq=bq, splits=splits)
        assert (rd.cpu().double()[:M] - (res.double()[:M] + y)).abs().max() < 4e-3 * scale, splits
        assert torch.equal(rd.cpu()[M:], res[M:])
    pitch = (N + 15) // 16 * 16 + 16
    buf = torch.full((M, pitch), -7.0, device=DEV)
    if (N * 4) % 16 == 0:
        assert o.linear_tc_pair(ad, wd, None, buf[:, :N], M, bq=bq)
        assert (buf.cpu().double()[:, :N] - (y - b.double())).abs().max() < 4e-3 * scale
        assert (buf.cpu()[:, N:] == -7.0).all()
    assert int(o.status_word().item()) == 0


def test_product_by_pairs_declines_what_it_cannot_take():
    o = ops()
    a = torch.zeros(100, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(100, 128, dtype=torch.bfloat16, device=DEV)
    assert not o.linear_tc_pair(a, w, None, out, 100)                    # fewer than 256 rows
    a = torch.zeros(256, 36, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128, 36, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(256, 128, dtype=torch.bfloat16, device=DEV)
    assert not o.linear_tc_pair(a, w, None, out, 256)                    # 72-byte rows


@pytest.mark.parametrize("n_head, n_kv_head, hd, lens", [(12, 12, 64, [1024, 700, 324]), (6, 2, 32, [1600]),
                                                         (4, 4, 16, [513, 500, 600]), (12, 12, 64, [130, 1, 126]),
                                                         (25, 25, 64, [300, 41]), (8, 2, 48, [257])])
def test_fused_qkv_projection_for_many_rows(n_head, n_kv_head, hd, lens):
    """The q/k/v projection of prompt portions by the pair kernel: queries to the output, keys and values
    from the epilogue into the rows' slots of scattered pages (portions that start in mid-page)."""
    o = ops()
    g = gen(sum(lens) + hd)
    M, ps = sum(lens), 16
    C = 64 + 8 * n_head
    q_dim, kv_dim = n_head * hd, n_kv_head * hd
    N = q_dim + 2 * kv_dim
    a = (torch.randn(M, C, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, C, generator=g) * 0.1).to(torch.bfloat16)
    b = torch.randn(N, generator=g) * 0.1
    pos0 = [5 + 11 * e for e in range(len(lens))]                      # each portion continues a request
    max_blocks = max(-(-(p0 + n) // ps) for p0, n in zip(pos0, lens)) + 1
    n_pages = sum(-(-(p0 + n) // ps) for p0, n in zip(pos0, lens)) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((len(lens), max_blocks), -1, dtype=torch.int32)
    row_entry, positions = [], []
    for e, (p0, n) in enumerate(zip(pos0, lens)):
        for blk in range(-(-(p0 + n) // ps)):
            table[e, blk] = perm.pop()
        row_entry += [e] * n
        positions += list(range(p0, p0 + n))
    cache = torch.zeros(n_pages, 2, n_kv_head, ps, hd, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    status = o.status_word()
    done = o.linear_qkv(a.to(DEV), w.to(DEV), b.to(DEV), out, M, q_dim, cache, table.to(DEV),
                        torch.tensor(row_entry, dtype=torch.int32, device=DEV),
                        torch.tensor(positions, dtype=torch.int32, device=DEV), status)
    if q_dim % 64:
        assert not done and (out == 0).all() and (cache == 0).all()    # declined: nothing was written
        return
    assert done and int(status.item()) == 0
    y = (a.double() @ w.double().T + b.double())
    assert (out.cpu().double()[:, :q_dim] - y[:, :q_dim]).abs().max() < 3e-2
    want = torch.zeros(n_pages, 2, n_kv_head, ps, hd, dtype=torch.float64)
    for t in range(M):
        page = int(table[row_entry[t], positions[t] // ps])
        want[page, 0, :, positions[t] % ps] = y[t, q_dim:q_dim + kv_dim].view(n_kv_head, hd)
        want[page, 1, :, positions[t] % ps] = y[t, q_dim + kv_dim:].view(n_kv_head, hd)
    assert (cache.cpu().double() - want).abs().max() < 3e-2
    assert (out.cpu()[:, q_dim:] == 0).all()            # key and value columns of the buffer are not written
