"""Trace replay on the GPU: the same requests replayed whole, with the last 32 tokens one by one,
in portions of changing size, and mixed with other requests so that pages are used again, in
32-bit and in bfloat16; every logits row is compared with the plain implementation."""
import pytest
import torch

from conftest import TINY, random_tokens
from trace_util import TraceSession, max_diff, max_kl

pytestmark = pytest.mark.gpu

# Tolerances on logits of magnitude ~1 (attention sharpened, see conftest.sharpen_attention).
# 32-bit: the bound the engine is built to.  bfloat16: weights, activations and cache are rounded
# to 8 bits of mantissa; measured differences on these models stay below 0.04.
TOL = {"float32": 1e-4, "bfloat16": 6e-2}
# KL(plain || engine) of the next-token distribution, per position: the second measure the reference
# applies to a reduced-precision path (crates/core/tests/reference.rs:29-45; its bound for 8-bit
# weights is 1e-2).  Measured on these models (whole prompts of the tiny, the 768-wide and the whole
# GPT-2 small model): at most 1.2e-5 in bfloat16 and 1e-12 in 32-bit.
KL_BOUND = {"float32": 1e-10, "bfloat16": 1e-4}
TORCH_DTYPE = {"float32": torch.float32, "bfloat16": torch.bfloat16}

LENGTHS = {"A": [97, 128, 70, 45, 33, 18], "B": [64, 50, 37, 22, 60, 9]}


def round64(n):
    return -(-n // 64) * 64


def requests_of(name):
    vocab = TINY[name]["vocab_size"]
    return {f"r{i}": random_tokens(vocab, n, 100 + i) for i, n in enumerate(LENGTHS[name])}


def check(session, reqs, model_dir, plain_logits, tol, ids=None):
    worst = 0.0
    for rid in (ids or reqs):
        toks = reqs[rid]
        got = session.stacked(rid, len(toks))
        ref = plain_logits(model_dir, toks)
        d = max_diff(got, ref)
        worst = max(worst, d)
        assert d <= tol, f"request {rid} ({len(toks)} tokens): max |logit difference| {d:.3e} > {tol}"
        kl = max_kl(ref, got)
        bound = KL_BOUND["float32" if tol == TOL["float32"] else "bfloat16"]
        assert kl <= bound, f"request {rid}: KL(plain || engine) {kl:.3e} > {bound}"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_alone_whole_tail_and_portions(name, dtype, model_dirs, plain_logits, tmp_path):
    model_dir = model_dirs(name, TORCH_DTYPE[dtype])
    vocab = TINY[name]["vocab_size"]
    reqs = requests_of(name)
    longest = max(len(t) for t in reqs.values())

    # (1) each request alone and whole, logits at every position
    s = TraceSession(model_dir, dtype, tmp_path / "whole", round64(longest), vocab)
    for rid, toks in reqs.items():
        s.step([(rid, toks, range(len(toks)))], end=[rid])
    s.close()
    check(s, reqs, model_dir, plain_logits, TOL[dtype])

    # (2) most of it in one step, the last 32 tokens one by one
    s = TraceSession(model_dir, dtype, tmp_path / "tail", round64(longest), vocab)
    for rid, toks in reqs.items():
        head = max(len(toks) - 32, 1)
        s.step([(rid, toks[:head], range(head))])
        for p in range(head, len(toks)):
            s.step([(rid, toks[p:p + 1], [0])], end=[rid] if p == len(toks) - 1 else [])
        if head == len(toks):
            s.step([], end=[rid])
    s.close()
    check(s, reqs, model_dir, plain_logits, TOL[dtype])

    # (3) portions of changing size, down to two tokens and one
    sizes = [5, 2, 16, 3, 1, 17, 2, 31, 4, 1, 2, 9]
    s = TraceSession(model_dir, dtype, tmp_path / "portions", round64(longest), vocab)
    for rid, toks in reqs.items():
        p, k = 0, 0
        while p < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - p)
            s.step([(rid, toks[p:p + n], range(n))], end=[rid] if p + n == len(toks) else [])
            p, k = p + n, k + 1
    s.close()
    check(s, reqs, model_dir, plain_logits, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_requests_with_few_pages(name, dtype, model_dirs, plain_logits, tmp_path):
    """Up to four live requests, portions of some beside single tokens of others, some left out of
    a step; the pool holds just what the live ones need, so ended requests' pages are used again."""
    model_dir = model_dirs(name, TORCH_DTYPE[dtype])
    vocab = TINY[name]["vocab_size"]
    reqs = requests_of(name)
    order = list(reqs)
    # plan: each request has a cut list; a "wave" runs four at a time, the next starts when one ends
    cuts = {"r0": [30, 1, 1, 7], "r1": [2, 40, 1, 1, 1], "r2": [1, 1, 20, 3], "r3": [17, 2, 1], "r4": [8, 1, 1, 5],
            "r5": [3, 1, 2]}
    live, waiting, done_pos = [], list(order), {}
    peak = 0
    steps = []
    progress = {r: 0 for r in order}
    cut_idx = {r: 0 for r in order}
    tick = 0
    while live or waiting:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        entries, ended = [], []
        for j, rid in enumerate(list(live)):
            if (tick + j) % 5 == 4 and len(live) > 1:
                continue                                  # left out of this step, goes on later
            toks = reqs[rid]
            c = cuts[rid]
            n = min(c[cut_idx[rid] % len(c)], len(toks) - progress[rid])
            entries.append((rid, toks[progress[rid]:progress[rid] + n], range(n)))
            progress[rid] += n
            cut_idx[rid] += 1
            if progress[rid] == len(toks):
                ended.append(rid)
                live.remove(rid)
        peak = max(peak, sum(round64(progress[r]) for r in set(live) | set(ended)))
        steps.append((entries, ended))
        tick += 1
    s = TraceSession(model_dir, dtype, tmp_path / "mixed", peak, vocab, extra=["--log-pages"])
    for entries, ended in steps:
        s.step(entries, end=ended)
    s.close()
    # the pool is so small that pages come back into use: some page id was held by two requests
    # (one after the other), and never by two at the same time
    owners = {}
    for held in s.pages():
        now = [(p, rid) for rid, groups in held.items() for p in groups[0]]
        assert len(set(p for p, _ in now)) == len(now), "a page is held by two requests at once"
        for p, rid in now:
            owners.setdefault(p, set()).add(rid)
    assert any(len(r) >= 2 for r in owners.values()), "no page was used again: the pool is too large for this test"
    assert any(len(e) >= 3 and min(len(t) for _, t, _ in e) == 1 and max(len(t) for _, t, _ in e) > 1
               for e, _ in steps), "the plan must mix portions with single tokens"
    check(s, reqs, model_dir, plain_logits, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_small_layer_sizes_long_prompts_in_one_step(dtype, model_dirs, plain_logits, tmp_path):
    """GPT-2 small's layer sizes: two long prompts in ONE step of 1700 rows (in bfloat16 that is the
    step that runs the paired tensor-memory products, whose q/k/v epilogue writes the cache, and the
    tensor-memory attention over several requests), a third request's prompt in portions beside
    their decoded tokens, then single tokens up to the last position of the context.  Attention is
    sharpened less than in the tiny models: 64-wide heads of a 768-wide model give larger scores."""
    model_dir = model_dirs("WIDE", TORCH_DTYPE[dtype], sharpen=2.5)
    vocab = TINY["WIDE"]["vocab_size"]
    reqs = {"r0": random_tokens(vocab, 1024, 300), "r1": random_tokens(vocab, 733, 301),
            "r2": random_tokens(vocab, 200, 302)}
    s = TraceSession(model_dir, dtype, tmp_path / "wide", 1024 + 768 + 256, vocab)
    want0 = [0, 1, 127, 128, 129, 500, 998, 999]
    want1 = [0, 15, 16, 255, 256, 698, 699]
    s.step([("r0", reqs["r0"][:1000], want0), ("r1", reqs["r1"][:700], want1)])
    # a third prompt in portions (130, then 70) beside single tokens of the two
    s.step([("r0", reqs["r0"][1000:1001], [0]), ("r2", reqs["r2"][:130], [0, 127, 129]),
            ("r1", reqs["r1"][700:701], [0])])
    s.step([("r2", reqs["r2"][130:], [0, 69]), ("r1", reqs["r1"][701:702], [0]), ("r0", reqs["r0"][1001:1002], [0])],
           end=["r2"])
    # a portion of 20 beside single tokens, then single tokens to the end (r0 ends at position 1023)
    s.step([("r1", reqs["r1"][702:722], range(20)), ("r0", reqs["r0"][1002:1003], [0])])
    for p in range(1003, 1024):
        entries = [("r0", reqs["r0"][p:p + 1], [0])]
        q = 722 + (p - 1003)
        if q < 733:
            entries.append(("r1", reqs["r1"][q:q + 1], [0]))
        s.step(entries, end=(["r0"] if p == 1023 else []) + (["r1"] if q == 732 else []))
    s.close()
    worst = 0.0
    for rid, toks in reqs.items():
        ref = plain_logits(model_dir, toks)
        for pos, row in s.logits[rid].items():
            d = max_diff(row, ref[pos])
            worst = max(worst, d)
            assert d <= TOL[dtype], f"request {rid} position {pos}: max |logit difference| {d:.3e} > {TOL[dtype]}"
    assert set(s.logits["r0"]) == set(want0) | set(range(1000, 1024))
    assert set(s.logits["r1"]) == set(want1) | set(range(700, 733))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_xl_layer_sizes(dtype, model_dirs, plain_logits, tmp_path):
    """GPT-2 XL's layer sizes, one layer: four prompts of about 400 tokens in one step of 1600 rows,
    then the four decode side by side."""
    model_dir = model_dirs("XLW", TORCH_DTYPE[dtype], sharpen=2.0)
    vocab = TINY["XLW"]["vocab_size"]
    lens = [420, 407, 399, 412]
    reqs = {f"r{i}": random_tokens(vocab, n, 400 + i) for i, n in enumerate(lens)}
    first = [393, 400, 381, 396]                      # rows of the first step: 1570 in all
    s = TraceSession(model_dir, dtype, tmp_path / "xl", 4 * 448, vocab)
    s.step([(r, reqs[r][:n], [0, 1, 63, 64, n - 1]) for r, n in zip(reqs, first)])
    at = dict(zip(reqs, first))
    while at:
        entries = [(r, reqs[r][p:p + 1], [0]) for r, p in at.items()]
        ended = [r for r, p in at.items() if p + 1 == len(reqs[r])]
        s.step(entries, end=ended)
        at = {r: p + 1 for r, p in at.items() if r not in ended}
    s.close()
    for rid, toks in reqs.items():
        ref = plain_logits(model_dir, toks)
        for pos, row in s.logits[rid].items():
            d = max_diff(row, ref[pos])
            assert d <= TOL[dtype], f"request {rid} position {pos}: max |logit difference| {d:.3e} > {TOL[dtype]}"
        assert len(s.logits[rid]) == 5 + len(toks) - first[int(rid[1:])]


def compare_rows(s, reqs, model_dir, plain_logits, dtype, device="cpu"):
    """Every logits row that was asked for against the plain implementation; returns (rows, worst)."""
    rows, worst = 0, 0.0
    for rid, toks in reqs.items():
        if rid not in s.logits:
            continue
        ref = plain_logits(model_dir, toks, device=device)
        for pos, row in s.logits[rid].items():
            d = max_diff(row, ref[pos])
            assert d <= TOL[dtype], f"request {rid} position {pos}: max |logit difference| {d:.3e} > {TOL[dtype]}"
            kl = max_kl(ref[pos], row)
            assert kl <= KL_BOUND[dtype], f"request {rid} position {pos}: KL(plain || engine) {kl:.3e}"
            rows, worst = rows + 1, max(worst, d)
    return rows, worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, sharpen", [("WIDE", 2.5), ("XLW", 2.0)])
def test_dozens_of_requests_decode_side_by_side_at_real_widths(name, sharpen, dtype, model_dirs, plain_logits, tmp_path):
    """Sixty-four, then forty, then twenty-four live requests decode side by side at GPT-2 small's
    and GPT-2 XL's layer widths, after prompts of different lengths that came in mixed steps: the
    steps of 17 to 64 rows are those of a loaded server (a norm kernel of its own, the few-row
    product with K split over blocks or the tensor-memory product with the weights on the M side,
    batches padded to a graph's shape)."""
    model_dir = model_dirs(name, TORCH_DTYPE[dtype], sharpen=sharpen)
    vocab = TINY[name]["vocab_size"]
    base = [random_tokens(vocab, 150, 700 + i) for i in range(8)]          # a request is a prefix of one of these
    n_req = 64
    prompt_len = [20 + (29 * i) % 101 for i in range(n_req)]                # 20..120
    ids = [f"q{i}" for i in range(n_req)]
    total = {rid: prompt_len[i] + (6 if i < 24 else 4 if i < 40 else 2) for i, rid in enumerate(ids)}
    reqs = {rid: base[i % 8][:total[rid]] for i, rid in enumerate(ids)}
    s = TraceSession(model_dir, dtype, tmp_path / "many", n_req * 192, vocab, extra=["--max-requests", "64"])
    # prompts, sixteen requests a step, each wanting its last row; the second group beside decoded tokens of the first
    at = {}
    for g in range(0, n_req, 16):
        entries = [(ids[i], reqs[ids[i]][:prompt_len[i]], [prompt_len[i] - 1]) for i in range(g, g + 16)]
        if g == 16:
            entries += [(ids[i], reqs[ids[i]][at[ids[i]]:at[ids[i]] + 1], [0]) for i in range(0, 16)]
            for i in range(0, 16):
                at[ids[i]] += 1
        s.step(entries)
        for i in range(g, g + 16):
            at[ids[i]] = prompt_len[i]
    live = list(ids)
    sizes = []
    while live:
        ended = [rid for rid in live if at[rid] + 1 == total[rid]]
        s.step([(rid, reqs[rid][at[rid]:at[rid] + 1], [0]) for rid in live], end=ended)
        sizes.append(len(live))
        for rid in live:
            at[rid] += 1
        live = [rid for rid in live if rid not in ended]
    s.close()
    assert 64 in sizes and 40 in sizes and 24 in sizes
    # (a request is a prefix of its base sequence, and a position's logits depend on nothing after it:
    # the plain implementation runs once for each of the eight)
    rows, _ = compare_rows(s, {rid: base[i % 8] for i, rid in enumerate(ids)}, model_dir, plain_logits, dtype)
    assert rows == n_req + sum(total[rid] - prompt_len[i] for i, rid in enumerate(ids))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_medium_layer_sizes(dtype, model_dirs, plain_logits, tmp_path):
    """GPT-2 medium's layer sizes (width 1024, sixteen heads, inner 4096), two layers: a long prompt in
    one step, a mixed step (a portion beside single tokens), then single tokens side by side."""
    model_dir = model_dirs("MEDW", TORCH_DTYPE[dtype], sharpen=2.5)
    vocab = TINY["MEDW"]["vocab_size"]
    reqs = {"r0": random_tokens(vocab, 930, 800), "r1": random_tokens(vocab, 310, 801), "r2": random_tokens(vocab, 40, 802)}
    s = TraceSession(model_dir, dtype, tmp_path / "med", 960 + 320 + 64, vocab)
    s.step([("r0", reqs["r0"][:900], [0, 127, 128, 511, 899])])
    s.step([("r1", reqs["r1"][:300], [0, 63, 64, 299]), ("r0", reqs["r0"][900:901], [0]), ("r2", reqs["r2"][:2], [0, 1])])
    s.step([("r2", reqs["r2"][2:33], range(31)), ("r0", reqs["r0"][901:902], [0]), ("r1", reqs["r1"][300:301], [0])])
    at = {"r0": 902, "r1": 301, "r2": 33}
    while at:
        ended = [r for r, p in at.items() if p + 1 == len(reqs[r])]
        s.step([(r, reqs[r][p:p + 1], [0]) for r, p in at.items()], end=ended)
        at = {r: p + 1 for r, p in at.items() if r not in ended}
    s.close()
    rows, _ = compare_rows(s, reqs, model_dir, plain_logits, dtype)
    assert rows == 5 + 4 + 2 + 31 + (930 - 900) + (310 - 300) + (40 - 33)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_real_vocabulary_inside_a_step(dtype, model_dirs, plain_logits, tmp_path):
    """One layer of GPT-2 small's sizes with the vocabulary of 50257: logits wanted at three rows of a
    prompt (the head's few-row product over 50257 features, whose pitch is no multiple of a tile),
    then for eight requests that decode side by side, then at forty rows of a portion (the head
    through the tensor-memory product with the vocabulary on its M side)."""
    model_dir = model_dirs("V50K", TORCH_DTYPE[dtype], sharpen=2.5)
    vocab = TINY["V50K"]["vocab_size"]
    reqs = {f"r{i}": random_tokens(vocab, 30 + 7 * i, 820 + i) for i in range(8)}
    reqs["p"] = random_tokens(vocab, 70, 830)
    s = TraceSession(model_dir, dtype, tmp_path / "v50k", 9 * 128, vocab, extra=["--max-requests", "9"])
    s.step([("r0", reqs["r0"][:27], [0, 13, 26])])
    s.step([(f"r{i}", reqs[f"r{i}"][:27 + 7 * i], []) for i in range(1, 8)])
    for t in range(3):
        s.step([(f"r{i}", reqs[f"r{i}"][27 + 7 * i + t:28 + 7 * i + t], [0]) for i in range(8)],
               end=[f"r{i}" for i in range(8)] if t == 2 else [])
    s.step([("p", reqs["p"][:30], [])])
    s.step([("p", reqs["p"][30:], range(40))], end=["p"])
    s.close()
    rows, _ = compare_rows(s, reqs, model_dir, plain_logits, dtype)
    assert rows == 3 + 24 + 40


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gpt2_small_whole_against_the_plain_implementation(dtype, model_dirs, plain_logits, tmp_path):
    """The model the benchmark runs, whole: twelve layers, width 768, the vocabulary of 50257, random
    weights with sharpened attention.  A prompt of 700 tokens in one step, a second request's prompt
    in portions beside the first one's decoded tokens, then both side by side.  The plain
    implementation's float64 formulas run on the GPU here (on the CPU this model takes minutes)."""
    model_dir = model_dirs("SMALL", TORCH_DTYPE[dtype], sharpen=2.0)
    vocab = TINY["SMALL"]["vocab_size"]
    reqs = {"a": random_tokens(vocab, 716, 850), "b": random_tokens(vocab, 150, 851)}
    s = TraceSession(model_dir, dtype, tmp_path / "small", 768 + 192, vocab)
    s.step([("a", reqs["a"][:700], [0, 1, 255, 256, 699])])
    s.step([("a", reqs["a"][700:701], [0]), ("b", reqs["b"][:97], [0, 96])])
    s.step([("b", reqs["b"][97:140], [0, 42]), ("a", reqs["a"][701:702], [0])])
    for t in range(10):
        s.step([("a", reqs["a"][702 + t:703 + t], [0]), ("b", reqs["b"][140 + t:141 + t], [0])],
               end=["b"] if t == 9 else [])
    for p in range(712, 716):
        s.step([("a", reqs["a"][p:p + 1], [0])], end=["a"] if p == 715 else [])
    s.close()
    rows, worst = compare_rows(s, reqs, model_dir, plain_logits, dtype, device="cuda")
    assert rows == 5 + 1 + 2 + 2 + 1 + 20 + 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_thousands_of_keys_behind_a_decoded_token(dtype, model_dirs, plain_logits, tmp_path):
    """A request of 4600 tokens (portions of 2000, 2000 and 568, then 32 single tokens) beside a short one
    that decodes in the same steps: the long row's keys are cut into more splits than one cluster
    merges (they meet through scratch), and the short row has keys for the first split only.  The
    attention is sharpened so that single far keys carry the result."""
    model_dir = model_dirs("FAR", TORCH_DTYPE[dtype], sharpen=3.0)
    vocab = TINY["FAR"]["vocab_size"]
    if dtype == "bfloat16":
        from nanoinfer_b200.kernels import ops
        chunk, n_splits = 256, 18    # what the rule below must give for 4608 keys and 2 rows of 2 heads
        assert ops.DECODE_DEEP_KEYS == 512 and ops.decode_split(2, 2, 4608, at_most=18) == (chunk, n_splits)
    reqs = {"far": random_tokens(vocab, 4600, 410), "near": random_tokens(vocab, 60, 411)}
    s = TraceSession(model_dir, dtype, tmp_path / "far", 4608 + 64, vocab)
    s.step([("far", reqs["far"][:2000], [0, 1999])])
    s.step([("far", reqs["far"][2000:4000], [0, 1999]), ("near", reqs["near"][:28], [27])])
    s.step([("far", reqs["far"][4000:4568], [0, 567])])
    for i in range(32):
        s.step([("near", reqs["near"][28 + i:29 + i], [0]), ("far", reqs["far"][4568 + i:4569 + i], [0])],
               end=["far", "near"] if i == 31 else [])
    s.close()
    rows, worst = compare_rows(s, reqs, model_dir, plain_logits, dtype)
    assert rows == 6 + 1 + 64
