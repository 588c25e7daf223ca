"""The scheduler's decisions (no GPU): admission, portions under the token budget, decoding,
finishing and freeing, and what happens when pages run out."""
import random

from nanoinfer_b200.cache import CacheManager
from nanoinfer_b200.engine.scheduler import FINISHED, RUNNING, WAITING, Scheduler
from nanoinfer_b200.parts.base import KVCacheSpec
from nanoinfer_b200.sampling import SamplingParams

SPEC = KVCacheSpec(2, 16)


def setup(max_tokens, max_batch=4, max_rows=64, budget=32, max_positions=128, **kw):
    cache = CacheManager([(0, SPEC), (1, SPEC)], [], max_tokens=max_tokens, max_requests=max_batch, page_size=16,
                         device=None, max_positions=max_positions)
    return cache, Scheduler(cache, max_batch=max_batch, max_rows=max_rows, prefill_budget=budget,
                            max_positions=max_positions, **kw)


def run_step(cache, s, token=7):
    """What the engine does around a step, without a model."""
    items = s.schedule()
    if items:
        cache.append([(i.request.cache, i.n_tokens) for i in items])    # must never fail
        for i in items:
            cache.commit(i.request.cache, i.n_tokens)
    ended = s.on_step_done(items, [token] * sum(1 for i in items if i.samples))
    cache.check()
    return items, ended + s.ended_without_step


def test_prompt_is_cut_under_the_budget_then_decoded():
    cache, s = setup(max_tokens=256, budget=32)
    r = s.add(list(range(70)), SamplingParams(max_new_tokens=3))
    sizes = []
    while s.has_work():
        items, _ = run_step(cache, s)
        sizes.append([(i.n_tokens, i.samples) for i in items])
    # 70 tokens as 32 + 32 + 6; only the last portion yields a token; then two single-token steps
    assert sizes == [[(32, False)], [(32, False)], [(6, True)], [(1, True)], [(1, True)]]
    assert r.output == [7, 7, 7] and r.finish_reason == "length" and r.state == FINISHED
    assert cache.pages_used() == [0] and cache.slots.n_free == 4


def test_decode_rows_first_and_prompts_share_the_rest():
    cache, s = setup(max_tokens=512, budget=40, max_rows=42)
    a = s.add([1] * 5, SamplingParams(max_new_tokens=10))
    run_step(cache, s)                                             # a is prefilled
    b = s.add([2] * 30, SamplingParams(max_new_tokens=2))
    c = s.add([3] * 30, SamplingParams(max_new_tokens=2))
    items, _ = run_step(cache, s)
    got = [(i.request.id, i.n_tokens) for i in items]
    assert got == [(a.id, 1), (b.id, 30), (c.id, 10)]              # one decode row, then 40 prompt tokens
    items, _ = run_step(cache, s)
    assert [(i.request.id, i.n_tokens, i.samples) for i in items] == [(a.id, 1, True), (b.id, 1, True), (c.id, 20, True)]


def test_a_lone_short_portion_takes_turns_with_the_decoded_tokens():
    """With ``portions_alone`` a single short prompt portion beside decoded tokens runs as a step of its
    own, then the decoded tokens as one of theirs: never two portion steps in a row while tokens wait,
    and nothing of this for two portions at once, for a long one, or without the switch."""
    cache, s = setup(max_tokens=2048, max_batch=4, max_rows=512, budget=512, max_positions=600)
    s.portions_alone = True
    a = s.add([1] * 5, SamplingParams(max_new_tokens=40))
    run_step(cache, s)                                             # a is prefilled (alone anyway)
    b = s.add([2] * 30, SamplingParams(max_new_tokens=20))
    kinds = []
    for _ in range(3):
        items, _ = run_step(cache, s)
        kinds.append([(i.request.id, i.n_tokens) for i in items])
    # the portion alone (it is the whole prompt: b has its first token), then both decode together
    assert kinds == [[(b.id, 30)], [(a.id, 1), (b.id, 1)], [(a.id, 1), (b.id, 1)]]
    # two arrivals one after the other: portion, tokens, portion, tokens
    c = s.add([3] * 40, SamplingParams(max_new_tokens=5))
    items, _ = run_step(cache, s)
    assert [(i.request.id, i.n_tokens) for i in items] == [(c.id, 40)]
    d = s.add([4] * 20, SamplingParams(max_new_tokens=5))
    items, _ = run_step(cache, s)                                  # the tokens' turn: d waits a step
    assert sorted((i.request.id, i.n_tokens) for i in items) == sorted([(a.id, 1), (b.id, 1), (c.id, 1)])
    items, _ = run_step(cache, s)
    assert [(i.request.id, i.n_tokens) for i in items] == [(d.id, 20)]
    while s.has_work():
        run_step(cache, s)
    # a long portion, and two portions at once, share their step with the decoded tokens as before
    cache, s = setup(max_tokens=4096, max_batch=4, max_rows=1024, budget=1024, max_positions=600)
    s.portions_alone = True
    a = s.add([1] * 5, SamplingParams(max_new_tokens=40))
    run_step(cache, s)
    b = s.add([2] * 300, SamplingParams(max_new_tokens=2))
    items, _ = run_step(cache, s)
    assert [(i.request.id, i.n_tokens) for i in items] == [(a.id, 1), (b.id, 300)]
    c = s.add([3] * 30, SamplingParams(max_new_tokens=2))
    d = s.add([4] * 30, SamplingParams(max_new_tokens=2))
    items, _ = run_step(cache, s)
    assert [(i.request.id, i.n_tokens) for i in items] == [(a.id, 1), (b.id, 1), (c.id, 30), (d.id, 30)]
    while s.has_work():
        run_step(cache, s)
    assert cache.pages_used() == [0]


def test_row_limit_bounds_the_budget():
    cache, s = setup(max_tokens=1024, max_batch=4, max_rows=10, budget=100)
    a = s.add([1] * 3, SamplingParams(max_new_tokens=50))
    b = s.add([1] * 3, SamplingParams(max_new_tokens=50))
    run_step(cache, s)
    s.add([2] * 40, SamplingParams(max_new_tokens=1))
    items, _ = run_step(cache, s)
    assert sum(i.n_tokens for i in items) == 10 and [i.n_tokens for i in items] == [1, 1, 8]


def test_admission_is_first_come_first_served_with_headroom():
    cache, s = setup(max_tokens=96, max_batch=4)                   # 6 pages
    a = s.add([1] * 40, SamplingParams(max_new_tokens=4))          # pages(41) = 3
    b = s.add([1] * 40, SamplingParams(max_new_tokens=4))          # needs 3 + 1 headroom: 3 free after a -> waits
    c = s.add([1] * 2, SamplingParams(max_new_tokens=4))           # would fit, but may not overtake b
    run_step(cache, s)
    assert a.state == RUNNING and b.state == WAITING and c.state == WAITING
    while a.state != FINISHED:
        run_step(cache, s)
    run_step(cache, s)
    assert b.state == RUNNING and c.state == RUNNING and b.admitted_order < c.admitted_order


def test_eos_and_context_full_end_a_request():
    cache, s = setup(max_tokens=512, max_positions=20)
    a = s.add([1] * 4, SamplingParams(max_new_tokens=50, eos_token_id=9))
    b = s.add([1] * 15, SamplingParams(max_new_tokens=50))
    run_step(cache, s, token=5)
    items, ended = run_step(cache, s, token=9)
    assert a in ended and a.finish_reason == "eos" and a.output == [5, 9]
    while b.state != FINISHED:
        run_step(cache, s, token=5)
    assert b.finish_reason == "context_full" and len(b.prompt) + len(b.output) == 21
    assert cache.pages_used() == [0]


def test_when_pages_run_out_the_newest_request_is_preempted_and_recomputed():
    cache, s = setup(max_tokens=64, max_batch=3, headroom_pages=0)          # 4 pages
    a = s.add([1] * 14, SamplingParams(max_new_tokens=40))
    b = s.add([2] * 14, SamplingParams(max_new_tokens=40))
    c = s.add([3] * 14, SamplingParams(max_new_tokens=40))
    run_step(cache, s)                                                      # a, b, c hold a page each; one spare
    assert [r.state for r in (a, b, c)] == [RUNNING] * 3
    preempted_seen = False
    for _ in range(400):
        if not s.has_work():
            break
        items, _ = run_step(cache, s)
        assert items, "a step must always make progress"
        if c.n_preemptions and not preempted_seen:
            preempted_seen = True
            assert c.state == WAITING and c.cache is None and c.n_computed == 0 and s.waiting[0] is c
            kept = len(c.output)
    assert preempted_seen and s.stats.preemptions >= 1
    assert a.n_preemptions == 0                                             # the oldest never loses its pages
    for r in (a, b, c):
        assert r.finish_reason == "length" and len(r.output) == 40         # nothing is lost by recomputing
    assert kept >= 1 and cache.pages_used() == [0] and cache.slots.n_free == 3


def test_a_request_that_can_never_fit_ends_with_too_long():
    cache, s = setup(max_tokens=32, max_batch=2)                            # 2 pages
    a = s.add([1] * 40, SamplingParams(max_new_tokens=4))                   # pages(41) = 3 > 2
    b = s.add([1] * 20, SamplingParams(max_new_tokens=30))                  # fits, then outgrows the pool alone
    items, ended = run_step(cache, s)
    assert a in ended and a.finish_reason == "too_long" and a.output == []
    while s.has_work():
        run_step(cache, s)
    assert b.finish_reason == "too_long" and len(b.prompt) + len(b.output) - 1 <= 32
    assert cache.pages_used() == [0]


def test_portions_shrink_to_the_pages_that_are_left():
    cache, s = setup(max_tokens=64, max_batch=2, budget=64, headroom_pages=0)   # 4 pages
    a = s.add([1] * 30, SamplingParams(max_new_tokens=20))
    run_step(cache, s)                                                          # a holds 2 pages
    b = s.add([2] * 30, SamplingParams(max_new_tokens=1))                       # admitted: pages(31) = 2 free
    items, _ = run_step(cache, s)
    # a's decode row crosses no page edge (token 31 of page 2); b gets the two free pages
    assert [(i.request.id, i.n_tokens) for i in items] == [(a.id, 1), (b.id, 30)]


def test_random_traffic_always_finishes_everything():
    for seed in range(5):
        rng = random.Random(seed)
        cache, s = setup(max_tokens=rng.choice([112, 160, 256]), max_batch=rng.choice([2, 4]),
                         budget=rng.choice([8, 32, 64]), max_rows=64)
        reqs = [s.add([1] * rng.randint(1, 60), SamplingParams(max_new_tokens=rng.randint(1, 40))) for _ in range(15)]
        for _ in range(3000):
            if not s.has_work():
                break
            run_step(cache, s)
        assert not s.has_work()
        for r in reqs:
            assert r.state == FINISHED and r.finish_reason == "length" and len(r.output) == r.params.max_new_tokens
        assert cache.pages_used() == [0]


def test_tokens_recorded_as_stand_ins_get_their_values_one_step_later():
    """The engine runs one step ahead of its reads: a step's tokens are recorded as negative
    stand-ins (they count for lengths at once) and their values follow.  An end token that turns up
    then ends the request there and drops what was computed ahead; the pages all come back."""
    cache, s = setup(max_tokens=512, max_positions=64)
    a = s.add([1] * 4, SamplingParams(max_new_tokens=50, eos_token_id=9))
    b = s.add([1] * 6, SamplingParams(max_new_tokens=3, eos_token_id=9))
    values = {0: [5, 5], 1: [9, 9], 2: [5, 5]}    # step -> token of every sampling item; a and b end at step 1
    in_flight, step, reported = None, 0, []
    while s.has_work() or in_flight:
        items = s.schedule()
        if items:
            cache.append([(i.request.cache, i.n_tokens) for i in items])
            for i in items:
                cache.commit(i.request.cache, i.n_tokens)
                toks = i.request.next_tokens(i.n_tokens)
                # a stand-in is only ever the lone token of a decoding request, in its own slot
                assert all(t >= 0 for t in toks) or (i.n_tokens == 1 and toks[0] == -(i.request.cache.slot + 1))
            stand_ins = [-(i.request.cache.slot + 1) for i in items if i.samples]
            ended_now = s.on_step_done(items, stand_ins)
        else:
            ended_now = []
        if in_flight:
            reported += in_flight[2] + s.on_tokens_read(in_flight[0], in_flight[1])
        in_flight = (items, values.get(step, [5] * 8)[:sum(1 for i in items if i.samples)], ended_now) if items else None
        step += 1
        cache.check()
    assert a.output == [5, 9] and a.finish_reason == "eos"
    assert b.output == [5, 9] and b.finish_reason == "eos"      # not "length": the end token came first
    assert set(id(r) for r in reported) == {id(a), id(b)}
    assert all(t >= 0 for r in (a, b) for t in r.output)
    assert cache.pages_used() == [0]
    # the third token of b would have ended it by length with the same token: the reason is the end token's
    cache, s = setup(max_tokens=512, max_positions=64)
    c = s.add([1] * 3, SamplingParams(max_new_tokens=1, eos_token_id=9))
    items = s.schedule()
    cache.append([(i.request.cache, i.n_tokens) for i in items])
    cache.commit(items[0].request.cache, 3)
    assert s.on_step_done(items, [-1]) == [c] and c.finish_reason == "length" and c.output == [-1]
    assert s.on_tokens_read(items, [9]) == [] and c.finish_reason == "eos" and c.output == [9]


def _token_of(req, index):
    """The token a model would give: a function of the request and of the token's place only."""
    return 9 if (req.id * 7 + index * 3) % 11 == 0 else 5


def _run_reading_every_step(cache, s):
    while s.has_work():
        items = s.schedule()
        if items:
            cache.append([(i.request.cache, i.n_tokens) for i in items])
            for i in items:
                cache.commit(i.request.cache, i.n_tokens)
        s.on_step_done(items, [_token_of(i.request, len(i.request.output)) for i in items if i.samples])
        cache.check()


def _run_one_step_ahead(cache, s):
    """The engine's loop when it launches a step before it has read the tokens of the one before."""
    in_flight, ended = None, []

    def read():
        nonlocal in_flight, ended
        if in_flight is not None:
            items, values, done = in_flight
            in_flight = None
            ended += done + s.on_tokens_read(items, values)

    while s.has_work() or in_flight is not None:
        while True:
            items = s.schedule()
            ended += s.ended_without_step
            if in_flight is not None and any(i.n_tokens > 1 and any(t < 0 for t in i.request.next_tokens(i.n_tokens))
                                             for i in items):
                read()      # a portion must not hold a stand-in
                continue
            break
        if not items:
            read()
            continue
        cache.append([(i.request.cache, i.n_tokens) for i in items])
        for i in items:
            cache.commit(i.request.cache, i.n_tokens)
        values = [_token_of(i.request, len(i.request.output)) for i in items if i.samples]
        done = s.on_step_done(items, [-(i.request.cache.slot + 1) for i in items if i.samples])
        flight = (items, values, done)
        read()
        in_flight = flight
        cache.check()
    return ended


def test_an_end_token_read_after_its_request_was_preempted_ends_it_in_the_queue_too():
    """A request can be preempted while its newest token is still a stand-in.  When the value turns
    out to be its end token, the request must leave the waiting queue: it is neither admitted again
    nor reported twice, and its output ends at the end token."""
    for seed in range(40):
        rng = random.Random(seed)
        lens = [(rng.randint(1, 40), rng.randint(2, 30)) for _ in range(6)]
        outs = []
        for run in (_run_reading_every_step, _run_one_step_ahead):
            cache, s = setup(max_tokens=96, max_batch=4, max_rows=48, budget=24, max_positions=80)
            reqs = [s.add([1] * p, SamplingParams(max_new_tokens=n, eos_token_id=9)) for p, n in lens]
            ended = run(cache, s)
            assert not s.waiting and not s.running and cache.pages_used() == [0]
            for r in reqs:
                assert r.state == FINISHED and all(t >= 0 for t in r.output)
                assert 9 not in r.output[:-1]
            if ended is not None:
                assert sorted(r.id for r in ended) == sorted(r.id for r in reqs)    # each reported once
            outs.append([(r.output, r.finish_reason) for r in reqs])
        assert outs[0] == outs[1]
    # the order named in the scheduler's own words: stand-in recorded, preempted, then the end token is read
    cache, s = setup(max_tokens=512, max_positions=64)
    a = s.add([1] * 4, SamplingParams(max_new_tokens=50, eos_token_id=9))
    b = s.add([1] * 4, SamplingParams(max_new_tokens=50, eos_token_id=9))
    items = s.schedule()
    cache.append([(i.request.cache, i.n_tokens) for i in items])
    for i in items:
        cache.commit(i.request.cache, i.n_tokens)
    s.on_step_done(items, [-(i.request.cache.slot + 1) for i in items])
    s._preempt(b)
    assert b in s.waiting and b.state == WAITING
    assert s.on_tokens_read(items, [5, 9]) == [b]
    assert b not in s.waiting and b not in s.running and b.state == FINISHED and b.output == [9]
    assert [i.request for i in s.schedule()] == [a]


def test_next_tokens_is_a_slice_of_prompt_and_output():
    _, s = setup(max_tokens=512)
    r = s.add([1, 2, 3, 4], SamplingParams())
    r.output = [5, 6, 7]
    for done in range(7):
        r.n_computed = done
        for n in range(1, 8 - done):
            assert r.next_tokens(n) == r.tokens[done:done + n]


def test_serving_workload_is_seeded_and_within_its_bounds():
    from nanoinfer_b200.serve_bench import XorShift, workload
    a = workload(50, 3, 40, 2, 9, 25.0, 7, 1000)
    b = workload(50, 3, 40, 2, 9, 25.0, 7, 1000)
    c = workload(50, 3, 40, 2, 9, 25.0, 8, 1000)
    assert [(r.arrival, r.prompt, r.out_len) for r in a] == [(r.arrival, r.prompt, r.out_len) for r in b]
    assert [r.prompt for r in a] != [r.prompt for r in c]
    assert all(3 <= len(r.prompt) <= 40 and 2 <= r.out_len <= 9 and all(0 <= t < 1000 for t in r.prompt) for r in a)
    assert all(x.arrival < y.arrival for x, y in zip(a, a[1:]))
    assert 50 / a[-1].arrival == __import__("pytest").approx(25.0, rel=0.5)      # about `rate` arrivals a second
    assert all(r.arrival == 0.0 for r in workload(5, 3, 4, 2, 3, 0.0, 1, 10))
    # the generator is the reference's xorshift64 (13, 7, 17) on seed * 0x9e3779b97f4a7c15 | 1
    g = XorShift(7)
    s = ((7 * 0x9E3779B97F4A7C15) & (2 ** 64 - 1)) | 1
    s ^= (s << 13) & (2 ** 64 - 1); s ^= s >> 7; s ^= (s << 17) & (2 ** 64 - 1)
    assert g.next() == s
