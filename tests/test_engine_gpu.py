"""The engine as a user calls it: greedy generation through the entry point against the plain
implementation, long decoding, the first tokens of a sequence, sampling with seeds, and the
scheduler driving the real step function with few pages."""
import pytest
import torch

from conftest import TINY, random_tokens

pytestmark = pytest.mark.gpu


def engine(model_dir, dtype, **kw):
    import nanoinfer_b200 as nb
    return nb.Engine(model_dir, dtype=dtype, check_status=True, **kw)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_the_plain_implementation(name, model_dirs):
    """The tiny workloads: A: prompts of 1, 7 and 33 tokens, 16 new tokens each;
    B: prompts of 2, 5, 17 and 40, 20 new tokens, prompts cut into portions of 8 beside decodes."""
    import nanoinfer_b200 as nb
    from plain_gpt2 import PlainGPT2
    d = model_dirs(name, torch.float32)
    vocab = TINY[name]["vocab_size"]
    lens, n_new, budget = ([1, 7, 33], 16, None) if name == "A" else ([2, 5, 17, 40], 20, 8)
    prompts = [random_tokens(vocab, n, 40 + i) for i, n in enumerate(lens)]
    plain = PlainGPT2(d)
    want = [plain.greedy(p, n_new) for p in prompts]
    eng = engine(d, "float32", max_batch=4, max_rows=64, prefill_budget=budget)
    got = eng.generate(prompts, nb.SamplingParams(max_new_tokens=n_new, temperature=0.0))
    assert got == want
    assert eng.cache.pages_used() == [0] and eng.cache.slots.n_free == 4
    # bfloat16: the same tokens except where two logits are within rounding of each other
    eng16 = engine(model_dirs(name, torch.bfloat16), "bfloat16", max_batch=4, max_rows=64, prefill_budget=budget)
    plain16 = PlainGPT2(model_dirs(name, torch.bfloat16))
    got16 = eng16.generate(prompts, nb.SamplingParams(max_new_tokens=n_new, temperature=0.0))
    for p, g in zip(prompts, got16):
        w = plain16.greedy(p, n_new)
        first_diff = next((i for i, (a, b) in enumerate(zip(g, w)) if a != b), n_new)
        if first_diff < n_new:  # a flip must be a near-tie in the plain logits
            lg = plain16.logits(p + w[:first_diff])[-1]
            assert float(lg[w[first_diff]] - lg[g[first_diff]]) < 0.05
        assert first_diff >= 1


def test_greedy_generation_of_a_dozen_requests_with_padded_batches(model_dirs):
    """Twelve requests of different output lengths through the entry point (one step ahead of its
    reads): batches of 12, 11, 10 and 9 single tokens are padded to 16 rows and share graphs; the
    tokens are the plain implementation's."""
    import nanoinfer_b200 as nb
    from plain_gpt2 import PlainGPT2
    d = model_dirs("A", torch.float32)
    prompts = [random_tokens(512, 2 + (5 * i) % 9, 140 + i) for i in range(12)]
    n_new = [6 + i for i in range(12)]
    plain = PlainGPT2(d)
    eng = engine(d, "float32", max_batch=16, max_rows=64)
    reqs = [eng.add_request(p, nb.SamplingParams(max_new_tokens=n, temperature=0.0)) for p, n in zip(prompts, n_new)]
    while eng.has_work():
        eng.step()
    assert eng.runner.padded_steps >= 5
    for r, p, n in zip(reqs, prompts, n_new):
        assert r.output == plain.greedy(p, n)
    assert eng.cache.pages_used() == [0] and eng.cache.slots.n_free == 16
    eng.cache.check()


def test_long_decoding_and_the_first_tokens(model_dirs, plain_logits):
    """One token at a time from position 0 to the end of a 640-position context: the first tokens
    (one key, one page) and the last (hundreds of keys, forty pages)."""
    from nanoinfer_b200 import load_model
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.engine import ModelRunner, StepItem
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 6e-2)):
        d = model_dirs("LONG", dtype)
        toks = random_tokens(TINY["LONG"]["vocab_size"], 640, 77)
        want = plain_logits(d, toks)
        m = load_model(d, dtype, "cuda")
        cache = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=640, max_requests=2, page_size=16,
                             dtype=dtype, device=torch.device("cuda"), max_positions=m.max_positions)
        runner = ModelRunner(m, cache, max_rows=64, max_entries=2)
        r = cache.open_request()
        worst = 0.0
        for p, t in enumerate(toks):
            lg = runner.step([StepItem(r, [t], [0])])
            diff = float((lg[0].cpu() - want[p]).abs().max())
            assert diff <= tol, f"{dtype}: position {p}: {diff:.3e}"
            worst = max(worst, diff)
        with pytest.raises(Exception, match="context full"):
            runner.step([StepItem(r, [1], [0])])
        cache.close_request(r)
        cache.check()


def test_step_refuses_bad_input_and_changes_nothing(model_dirs):
    from nanoinfer_b200 import load_model
    from nanoinfer_b200.cache import CacheManager, PoolExhausted
    from nanoinfer_b200.engine import BadToken, ContextFull, ModelRunner, StepError, StepItem, TooManyRows
    d = model_dirs("A", torch.float32)
    m = load_model(d, torch.float32, "cuda")
    cache = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=64, max_requests=3, page_size=16,
                         dtype=torch.float32, device=torch.device("cuda"), max_positions=m.max_positions)
    runner = ModelRunner(m, cache, max_rows=80, max_entries=3)
    a, b = cache.open_request(), cache.open_request()
    runner.step([StepItem(a, [1, 2, 3], [2])])
    state = (a.n_tokens, list(a.blocks[0]), cache.pages_free())
    for items, err in [
        ([StepItem(a, [512], [0])], BadToken), ([StepItem(a, [], [])], StepError),
        ([StepItem(a, [1], [1])], StepError), ([StepItem(a, [1], []), StepItem(a, [2], [])], StepError),
        ([StepItem(a, [1] * 81, [])], TooManyRows), ([StepItem(a, [1] * 30, []), StepItem(b, [1] * 40, [])], PoolExhausted),
    ]:
        with pytest.raises(err):
            runner.step(items)
        assert (a.n_tokens, list(a.blocks[0]), cache.pages_free()) == state and b.n_tokens == 0
    cache.close_request(b)
    with pytest.raises(StepError):
        runner.step([StepItem(b, [1], [])])
    big = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=512, max_requests=1, page_size=16,
                       dtype=torch.float32, device=torch.device("cuda"), max_positions=m.max_positions)
    r2 = ModelRunner(m, big, max_rows=256, max_entries=1)
    c = big.open_request()
    with pytest.raises(ContextFull):
        r2.step([StepItem(c, [1] * 129, [])])


def test_graph_table_keeps_the_most_recently_used_shapes(model_dirs):
    """A table of two graphs under steps of three shapes by turns: old graphs make room, every step
    gives the logits that the step function gives without graphs."""
    from nanoinfer_b200 import load_model
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.engine import ModelRunner, StepItem
    m = load_model(model_dirs("A", torch.float32), torch.float32, "cuda")

    def run(use_graphs):
        cache = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=3 * 64, max_requests=3, page_size=16,
                             dtype=torch.float32, device=torch.device("cuda"), max_positions=m.max_positions)
        runner = ModelRunner(m, cache, max_rows=64, max_entries=3, use_graphs=use_graphs, max_graphs=2)
        reqs = [cache.open_request() for _ in range(3)]
        for i, r in enumerate(reqs):
            runner.step([StepItem(r, random_tokens(512, 5 + 3 * i, 60 + i), [])])
        out = []
        for turn in range(18):
            live = reqs[:turn % 3 + 1]               # one, two, three rows, and again
            out.append(runner.step([StepItem(r, [(7 * turn + 3 * i) % 512], [0]) for i, r in enumerate(live)]).cpu().clone())
        return out, runner

    plain, _ = run(False)
    got, runner = run(True)
    assert len(runner._graphs) == 2 and runner.graph_replays >= 6
    for a, b in zip(plain, got):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_graphs_survive_larger_steps_between_their_replays(dtype, model_dirs, plain_logits):
    """A captured graph holds the raw addresses of the step's scratch.  Eight requests with hundreds
    of keys decode side by side (the keys are split over blocks, so the partial results and arrival
    counters go through scratch) until their step is captured; then forty rows, then sixty-four rows
    with a sampler, then the eight again, replayed.  No scratch buffer may have moved in between:
    every logits row is the plain implementation's, and the step function reports no replacement.
    Then a step that does make a buffer grow (logits at 200 places of a prompt): the graphs are
    dropped, captured anew, and the eight rows are still right."""
    from plain_gpt2 import XorShiftSampler
    from nanoinfer_b200 import load_model
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.engine import ModelRunner, StepItem
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.sampling import Sampler, SamplingParams
    tol = 1e-4 if dtype == torch.float32 else 6e-2
    d = model_dirs("LONG", dtype)
    vocab, n_head = TINY["LONG"]["vocab_size"], TINY["LONG"]["n_head"]
    m = load_model(d, dtype, "cuda")
    base = [random_tokens(vocab, 340, 500 + i) for i in range(8)]
    want = [plain_logits(d, b) for b in base]
    lens = [260 + (37 * i) % 41 for i in range(64)]               # 260..300 tokens are in the cache at first
    cache = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=64 * 352, max_requests=64, page_size=16,
                         dtype=dtype, device=torch.device("cuda"), max_positions=m.max_positions, padding=True)
    runner = ModelRunner(m, cache, max_rows=1280, max_entries=64)
    sampler = Sampler(cache.slots)
    generation = runner.workspace.generation
    reqs = [cache.open_request() for _ in range(64)]
    for i in range(0, 64, 4):
        runner.step([StepItem(reqs[j], base[j % 8][:lens[j]], []) for j in range(i, i + 4)])
    at = list(lens)
    assert ops.decode_split(8, n_head, 512)[1] > 1 and ops.decode_split(64, n_head, 512)[1] > 1

    def decode(ids, sampler=None):
        out = runner.step([StepItem(reqs[j], [base[j % 8][at[j]]], [0]) for j in ids], sampler=sampler)
        for j in ids:
            at[j] += 1
        return out

    def check(ids, logits):
        for row, j in enumerate(ids):
            diff = float((logits[row].float().cpu() - want[j % 8][at[j] - 1]).abs().max())
            assert diff <= tol, f"request {j} at position {at[j] - 1}: {diff:.3e}"

    eight, forty, all64 = list(range(8)), list(range(40)), list(range(64))
    for _ in range(3):                                            # uncaptured, captured, replayed
        check(eight, decode(eight))
    replays = runner.graph_replays
    assert replays >= 2
    for _ in range(2):
        check(forty, decode(forty))
    # sixty-four rows through the sampler: even slots greedy, odd ones with a temperature
    plain_samplers = {}
    for j in all64:
        sp = SamplingParams(temperature=0.0 if j % 2 == 0 else 0.8, top_k=0 if j % 4 == 1 else 12, seed=900 + j)
        sampler.set_request(reqs[j].slot, sp)
        plain_samplers[j] = XorShiftSampler(sp.temperature, sp.top_k, sp.seed)
    differ = 0
    for _ in range(2):
        toks = decode(all64, sampler).tolist()
        for j in all64:
            ref = want[j % 8][at[j] - 1]
            tok = plain_samplers[j].sample(ref)
            if dtype == torch.float32:
                differ += int(toks[j] != tok)     # may differ where a draw falls within rounding of a boundary
            elif j % 2 == 0 and toks[j] != tok:   # bfloat16: the greedy rows, unless two logits are nearly tied
                assert float(ref[tok] - ref[toks[j]]) < 2 * tol, f"request {j}: greedy token {toks[j]}, plain {tok}"
    assert differ <= 1, f"{differ} of 128 tokens differ from the plain sampler"
    for _ in range(3):                                            # the eight again: their graph is replayed
        check(eight, decode(eight))
    assert runner.graph_replays >= replays + 3
    assert runner.workspace.generation == generation and runner.graph_drops == 0, "a scratch buffer was replaced"
    # now make a buffer grow: logits at 200 places of one prompt are more rows than the scratch was sized for
    cache.close_request(reqs[63])
    r = cache.open_request()
    lg = runner.step([StepItem(r, base[3][:200], range(200))])
    assert float((lg.float().cpu() - want[3][:200]).abs().max()) <= tol
    assert runner.workspace.generation > generation
    for _ in range(3):                                            # dropped, run plainly, captured again
        check(eight, decode(eight))
    assert runner.graph_drops == 1 and not runner.workspace.retired
    cache.check()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batches_padded_to_a_graph_shape_give_the_same_logits(dtype, model_dirs, plain_logits):
    """Eleven, then ten, then nine requests decode side by side: the step function fills the batch
    up to sixteen rows with rows of no request (so that the three sizes share one graph); the real
    rows' logits are those of the plain implementation, and of a step function that does not pad."""
    from nanoinfer_b200 import load_model
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.engine import ModelRunner, StepItem
    d = model_dirs("B", dtype)
    m = load_model(d, dtype, "cuda")
    prompts = [random_tokens(1000, 3 + 2 * i, 80 + i) for i in range(11)]
    more = [random_tokens(1000, 12, 95 + i) for i in range(11)]

    def run(padding):
        cache = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=11 * 48, max_requests=11, page_size=16,
                             dtype=dtype, device=torch.device("cuda"), max_positions=m.max_positions, padding=padding)
        runner = ModelRunner(m, cache, max_rows=64, max_entries=16)
        reqs = [cache.open_request() for _ in range(11)]
        for r, p in zip(reqs, prompts):
            runner.step([StepItem(r, p, [])])
        rows = {i: [] for i in range(11)}
        for t in range(12):
            live = range(11 - t // 4)                         # 11, 10, then 9 rows
            out = runner.step([StepItem(reqs[i], [more[i][t]], [0]) for i in live])
            assert out.shape[0] == len(live)
            for k, i in enumerate(live):
                rows[i].append(out[k].float().cpu().clone())
        cache.check()
        return rows, runner

    padded, runner = run(True)
    exact, runner_exact = run(False)
    assert runner.padded_steps == 12 and runner_exact.padded_steps == 0
    assert runner.graph_replays >= 10 and sum(1 for k in runner._graphs if k[0] == k[1]) == 1   # (T == E: single tokens)
    tol = 1e-4 if dtype == torch.float32 else 6e-2
    for i in range(11):
        ref = plain_logits(d, prompts[i] + more[i])
        for t, (a, b) in enumerate(zip(padded[i], exact[i])):
            assert (a - ref[len(prompts[i]) + t]).abs().max() <= tol
            assert (a - b).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompts_of_nearly_one_length_share_a_graph(dtype, model_dirs, plain_logits):
    """Prompts of 67, 70, 75, 80 and 66 tokens, each a step of its own: the step function fills every one up
    to 80 rows with rows of no request, so that the second is captured and the others replay its graph.
    Logits at the prompts' ends and at places inside them, and the tokens decoded afterwards (the cache
    holds exactly each request's keys), are those of the plain implementation; a step that is not
    filled up gives the same."""
    from nanoinfer_b200 import load_model
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.engine import ModelRunner, StepItem
    tol = 1e-4 if dtype == torch.float32 else 6e-2
    d = model_dirs("A", dtype)
    m = load_model(d, dtype, "cuda")
    lens = [67, 70, 75, 80, 66]
    toks = [random_tokens(512, n + 6, 700 + i) for i, n in enumerate(lens)]
    want = [plain_logits(d, t) for t in toks]
    cache = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=5 * 96, max_requests=5, page_size=16,
                         dtype=dtype, device=torch.device("cuda"), max_positions=m.max_positions, padding=True)
    runner = ModelRunner(m, cache, max_rows=128, max_entries=8)
    reqs = [cache.open_request() for _ in lens]
    for i, n in enumerate(lens):
        places = [0, 15, 16, n - 1]
        out = runner.step([StepItem(reqs[i], toks[i][:n], places)])
        for k, p in enumerate(places):
            diff = float((out[k].float().cpu() - want[i][p]).abs().max())
            assert diff <= tol, f"prompt of {n} tokens, position {p}: {diff:.3e}"
    assert runner.row_padded_steps == 4 and runner.graph_replays >= 3          # (80 rows need no filling)
    assert sum(1 for k in runner._graphs if k[0] == 80) == 1
    for t in range(6):                                                         # then all five decode side by side
        out = runner.step([StepItem(reqs[i], [toks[i][lens[i] + t]], [0]) for i in range(5)])
        for i in range(5):
            diff = float((out[i].float().cpu() - want[i][lens[i] + t]).abs().max())
            assert diff <= tol, f"request {i}, decoded token {t}: {diff:.3e}"
    cache.check()
    # the same first prompt through a step function without graphs (nothing is filled up): the same logits
    cache2 = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=96, max_requests=1, page_size=16,
                          dtype=dtype, device=torch.device("cuda"), max_positions=m.max_positions)
    plain_runner = ModelRunner(m, cache2, max_rows=128, max_entries=1, use_graphs=False)
    out = plain_runner.step([StepItem(cache2.open_request(), toks[0][:67], [66])])
    assert plain_runner.row_padded_steps == 0
    assert float((out[0].float().cpu() - want[0][66]).abs().max()) <= tol


def test_sampling_with_seeds_is_reproducible_and_independent_of_the_batch(model_dirs):
    import nanoinfer_b200 as nb
    d = model_dirs("A", torch.float32, sharpen=0.0)
    prompts = [random_tokens(512, n, 60 + i) for i, n in enumerate([5, 9, 3])]
    params = [nb.SamplingParams(max_new_tokens=12, temperature=0.9, top_k=20, seed=100 + i) for i in range(3)]
    eng = engine(d, "float32", max_batch=4, max_rows=64)
    together = eng.generate(prompts, params)
    alone = [engine(d, "float32", max_batch=1, max_rows=64).generate([p], [sp])[0] for p, sp in zip(prompts, params)]
    assert together == alone
    other = eng.generate(prompts[:1], [nb.SamplingParams(max_new_tokens=12, temperature=0.9, top_k=20, seed=5)])
    assert other[0] != together[0]
    # the walk is the reference sampler's: replay request 0 with the plain sampler on the plain logits
    from plain_gpt2 import PlainGPT2, XorShiftSampler
    plain, s = PlainGPT2(d), XorShiftSampler(0.9, 20, 100)
    toks = list(prompts[0])
    differ = 0
    for k in range(12):
        lg = plain.logits(toks)[-1].float()
        t = s.sample(lg)
        differ += int(t != together[0][k])
        toks.append(together[0][k])      # go on from the engine's token: the generators stay in step
    # the walks agree except where a draw falls within rounding of the boundary between two tokens
    # (the rule of the kernel's own test): at most one of the twelve
    assert differ <= 1, f"{differ} of 12 sampled tokens differ from the reference walk"


def test_sampling_over_the_real_vocabulary_together_and_alone(model_dirs):
    """Temperature 0.8 over a vocabulary of 50257 through the entry point (a sampled row is shared by
    a cluster of blocks there): eight requests together give the tokens that each gives alone, and a
    request's first token is the plain sampler's on the plain logits."""
    import nanoinfer_b200 as nb
    from plain_gpt2 import PlainGPT2, XorShiftSampler
    d = model_dirs("V50K", torch.float32, sharpen=2.5)
    prompts = [random_tokens(50257, 4 + 3 * i, 860 + i) for i in range(8)]
    params = [nb.SamplingParams(max_new_tokens=6, temperature=0.8, top_k=0 if i % 2 else 40, seed=300 + i)
              for i in range(8)]
    together = engine(d, "float32", max_batch=8, max_rows=64).generate(prompts, params)
    alone_engine = engine(d, "float32", max_batch=1, max_rows=64)
    alone = [alone_engine.generate([p], [sp])[0] for p, sp in zip(prompts, params)]
    assert together == alone
    plain = PlainGPT2(d)
    first = [XorShiftSampler(0.8, sp.top_k, sp.seed).sample(plain.logits(p)[-1].float()) for p, sp in
             zip(prompts[:3], params[:3])]
    assert sum(int(a != b[0]) for a, b in zip(first, together)) <= 1     # (a draw within rounding of a boundary)


def test_few_pages_preemption_gives_the_same_tokens(model_dirs):
    """With a pool too small for all requests the scheduler preempts and recomputes; greedy tokens
    must be what an ample pool gives."""
    import nanoinfer_b200 as nb
    d = model_dirs("A", torch.float32)
    prompts = [random_tokens(512, n, 80 + i) for i, n in enumerate([14, 14, 14, 30, 3])]
    sp = nb.SamplingParams(max_new_tokens=40, temperature=0.0)
    ample = engine(d, "float32", max_batch=4, max_rows=64).generate(prompts, sp)
    tight = engine(d, "float32", max_batch=4, max_rows=64, max_tokens=144, prefill_budget=16)
    got = tight.generate(prompts, sp)
    assert got == ample
    assert tight.scheduler.stats.preemptions >= 1
    assert tight.cache.pages_used() == [0]


def test_running_a_step_ahead_of_the_reads_gives_the_same_tokens(model_dirs):
    """With ``run_ahead`` a step is launched before the host has read the tokens of the step before
    (they go from sampler to embedding on the device).  Tokens, end reasons and what comes back to
    the pool must be those of the engine that reads every step: greedy and sampled, with end tokens
    that cut requests short, and with so few pages that requests are preempted meanwhile."""
    import nanoinfer_b200 as nb
    d = model_dirs("A", torch.float32, sharpen=0.0)
    prompts = [random_tokens(512, n, 90 + i) for i, n in enumerate([14, 14, 14, 30, 3, 22])]
    base = engine(d, "float32", max_batch=4, max_rows=64, run_ahead=False)
    greedy = base.generate(prompts, nb.SamplingParams(max_new_tokens=40, temperature=0.0))
    # end tokens taken from what is generated: one early, one late, one never
    eos = [greedy[0][3], greedy[1][30], None, None, greedy[4][11], None]
    params = [nb.SamplingParams(max_new_tokens=40, temperature=0.0 if i % 2 == 0 else 0.8, top_k=30, seed=7 + i,
                                eos_token_id=e) for i, e in enumerate(eos)]
    for kw in (dict(), dict(max_tokens=128, prefill_budget=16)):
        outs = {}
        for ahead in (False, True):
            eng = engine(d, "float32", max_batch=4, max_rows=64, run_ahead=ahead, **kw)
            reqs = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]
            ended = []
            while eng.has_work():
                ended += eng.step()
            assert sorted(r.id for r in ended) == sorted(r.id for r in reqs)
            assert all(t >= 0 for r in reqs for t in r.output)
            assert eng.cache.pages_used() == [0] and eng.cache.slots.n_free == 4
            outs[ahead] = [(r.output, r.finish_reason) for r in reqs]
            if kw:
                assert eng.scheduler.stats.preemptions >= 1
        assert outs[True] == outs[False]
        assert outs[True][0][1] == "eos" and len(outs[True][0][0]) <= 4


def test_serving_benchmark_runs_both_policies_to_the_end(model_dirs):
    """The serving workload through the continuous scheduler and through static batching: every request
    generates exactly its output length under both, and continuous batching needs fewer iterations."""
    from nanoinfer_b200 import serve_bench as sb
    d = model_dirs("A", torch.bfloat16)
    reqs = sb.workload(24, 2, 40, 2, 30, 0.0, 3, 512)
    eng = engine(d, "bfloat16", max_batch=4, max_rows=64, prefill_budget=32, max_tokens=4 * 80 + 128)
    stat = sb.run_static(eng, reqs)
    cont = sb.run_continuous(eng, reqs)
    for o in (stat, cont):
        assert [l.generated for l in o.logs] == [r.out_len for r in reqs]
        assert all(0.0 <= l.admitted <= l.first_token <= l.finished <= o.makespan for l in o.logs)
    assert len(cont.iters) < len(stat.iters)
    s = sb.summarise("continuous", reqs, cont, 16)
    assert s["generated_tokens"] == sum(r.out_len for r in reqs) and s["throughput_tok_s"] > 0
    if s["preemptions"] == 0:   # every token but a request's last goes through the model once
        assert s["rows_computed"] == sum(len(r.prompt) + r.out_len - 1 for r in reqs)
    assert eng.cache.pages_used() == [0] and eng.cache.slots.n_free == 4


def test_command_line_generate_prints_the_tokens_of_the_entry_point(model_dirs, capsys):
    """``generate`` streams token ids as the host reads them; they are those of ``Engine.generate``,
    greedy and sampled with the reference's option names."""
    import nanoinfer_b200 as nb
    from nanoinfer_b200 import cli
    d = model_dirs("A", torch.float32)
    prompt = random_tokens(512, 9, 123)
    ids = ",".join(str(t) for t in prompt)
    for extra, params in ((["--temperature", "0.0"], nb.SamplingParams(max_new_tokens=14, temperature=0.0)),
                          (["--temperature", "0.9", "--top-k", "25", "--seed", "5"],
                           nb.SamplingParams(max_new_tokens=14, temperature=0.9, top_k=25, seed=5))):
        assert cli.main(["--weights", d, "generate", "--dtype", "float32", "--prompt-ids", ids, "--tokens", "14"]
                        + extra) == 0
        printed = [int(t) for t in capsys.readouterr().out.split()]
        want = engine(d, "float32", max_batch=1, max_rows=64).generate([prompt], params)[0]
        assert printed == want and len(printed) == 14 and all(t >= 0 for t in printed)


def test_command_line_random_weights_writes_a_loadable_folder(tmp_path):
    import nanoinfer_b200 as nb
    from nanoinfer_b200 import cli
    out = str(tmp_path / "m")
    assert cli.main(["random-weights", "--config", "gpt2-tiny-b", "--seed", "3", "--out", out, "--dtype", "float32"]) == 0
    eng = engine(out, "float32", max_batch=2, max_rows=32)
    got = eng.generate([[1, 2, 3]], nb.SamplingParams(max_new_tokens=4, temperature=0.0))
    assert len(got[0]) == 4


def test_command_line_generates_from_text_and_writes_a_trace(tmp_path, capsys):
    """The command line as the reference's: a model folder from ``random-weights`` (with the byte
    tokenizer, so that text can be given), ``generate --prompt TEXT`` with a profile and a trace file,
    the same tokens from ``--prompt-ids``, and a clear answer when the tokenizer's files are absent."""
    import json
    from nanoinfer_b200.cli import main
    d = str(tmp_path / "m")
    assert main(["random-weights", "--config", "gpt2-tiny-a", "--seed", "4", "--out", d, "--dtype", "float32",
                 "--tokenizer"]) == 0
    capsys.readouterr()
    trace = str(tmp_path / "trace.jsonl")
    assert main(["--weights", d, "generate", "--dtype", "float32", "--prompt", "Hi é", "--tokens", "6", "--profile",
                 "--trace-out", trace]) == 0
    out, err = capsys.readouterr()
    assert out.startswith("Hi é") and "of roof" in err and "decode" in err
    lines = [json.loads(l) for l in open(trace)]
    assert lines[0]["t"] == "run_start" and lines[0]["prompt_tokens"] == list("Hi é".encode())
    assert lines[-1]["t"] == "run_end" and lines[-1]["n_gen"] == 6 and lines[-1]["n_prompt"] == 5
    ops_seen = {l["op"] for l in lines if l["t"] == "op"}
    assert {"qkv", "attn", "attn_proj", "fc", "fc_proj", "lm_head", "embed", "sample"} <= ops_seen
    assert all(l["flops"] >= 0 and l["bytes"] > 0 and l["dur_us"] > 0 for l in lines if l["t"] == "op")
    tokens = [l["id"] for l in lines if l["t"] == "token"]
    assert len(tokens) == 6
    ids = ",".join(str(b) for b in "Hi é".encode())
    assert main(["--weights", d, "generate", "--dtype", "float32", "--prompt-ids", ids, "--tokens", "6"]) == 0
    out, _ = capsys.readouterr()
    assert [int(t) for t in out.split()] == tokens
    import os
    os.remove(os.path.join(d, "merges.txt"))
    assert main(["--weights", d, "generate", "--prompt", "Hi"]) == 2
    assert "merges.txt" in capsys.readouterr().err
