"""The scheduler's decisions, with the cache manager but without a GPU.

A stand-in for the step function takes pages exactly as the real one does (admit, extend, release
behind the window) and "samples" a token that is a fixed function of all tokens of the request so
far, so that a recomputed request must reproduce its earlier output."""
import random

import pytest

from lucciola_b200.cache import CacheGroup, CacheManager
from lucciola_b200.engine.request import Request, Status
from lucciola_b200.engine.scheduler import Scheduler
from lucciola_b200.sampling import SamplingParams

VOCAB = 97


def next_token(tokens):
    h = 17
    for t in tokens:
        h = (h * 31 + t + 1) % 1000003
    return h % VOCAB


def make(pages=64, page=4, budget=16, seqs=8, max_len=256, chunk=0, eos=(), window=0, **kw):
    groups = [CacheGroup(2, 16, 0, (0,))] + ([CacheGroup(2, 16, window, (1,))] if window else [])
    m = CacheManager(groups, page, pages, seqs)
    return m, Scheduler(m, budget, seqs, max_len, chunk, eos, **kw)


def run_step(m, s, log=None):
    plan = s.schedule()
    sampled = []
    for e in plan:
        r = e.request
        if not m.has_request(r.rid):
            m.admit(r.rid)
        assert m.length(r.rid) == e.start == r.num_computed
        assert m.extend(r.rid, e.start + e.num_tokens), "the scheduler planned more than the pool has"
        if e.sample:
            sampled.append(next_token(r.tokens[:e.start + e.num_tokens]))
    for e in plan:
        m.release_behind_window(e.request.rid)
    if log is not None:
        log.append([(e.request.rid, e.start, e.num_tokens, e.sample) for e in plan])
    events = s.update(plan, sampled)
    m.check_invariants()
    return plan, events


def req(rid, n, new=8, **kw):
    rng = random.Random(rid)
    return Request(rid, [rng.randrange(VOCAB) for _ in range(n)], SamplingParams(max_new_tokens=new, **kw))


def expected_output(r):
    toks, out = list(r.prompt), []
    for _ in range(r.params.max_new_tokens):
        t = next_token(toks); out.append(t); toks.append(t)
    return out


def test_prompt_is_cut_under_the_budget_then_decoded():
    m, s = make(budget=16)
    r = req(1, 40, new=3)
    s.add_request(r)
    log = []
    while s.has_unfinished():
        run_step(m, s, log)
    assert log[:3] == [[(1, 0, 16, False)], [(1, 16, 16, False)], [(1, 32, 8, True)]]
    assert log[3:] == [[(1, 40, 1, True)], [(1, 41, 1, True)]]
    assert r.output == expected_output(r) and r.finish_reason == "length" and r.status is Status.FINISHED
    assert m.pools[0].num_free == 64 and m.num_requests() == 0


def test_decodes_go_first_and_the_rest_of_the_budget_goes_to_prompts():
    m, s = make(budget=10)
    a, b, c = req(1, 6, new=20), req(2, 7, new=20), req(3, 30, new=2)
    s.add_request(a); s.add_request(b)
    log = []
    run_step(m, s, log)                       # a whole (6) and the first 4 of b
    assert log[-1] == [(1, 0, 6, True), (2, 0, 4, False)]
    s.add_request(c)
    run_step(m, s, log)                       # a decodes; b's rest (3); c gets what is left (6)
    assert log[-1] == [(1, 6, 1, True), (2, 4, 3, True), (3, 0, 6, False)]
    run_step(m, s, log)                       # a and b decode first, then c continues with 8
    assert log[-1] == [(1, 7, 1, True), (2, 7, 1, True), (3, 6, 8, False)]


def test_portions_shortened_to_fill_whole_token_tiles():
    """token_tile 8, budget 21, portions of up to 16: beside 3 decoding requests a portion of 16 makes a step of 19 (21 with
    two tokens of the next prompt); it is shortened to 13 so that the step has 16 and ends there.  A prompt's last portion is left alone, and the output is
    what it is without the option."""
    outs = {}
    for tile in (0, 8):
        m, s = make(pages=200, budget=21, chunk=16, token_tile=tile)
        rs = [req(i, 5, new=40) for i in range(3)] + [req(9, 70, new=3), req(10, 30, new=3)]
        for r in rs[:3]:
            s.add_request(r)
        while any(not r.output for r in rs[:3]):
            run_step(m, s)
        s.add_request(rs[3])
        s.add_request(rs[4])                       # a second prompt waits: it must not fill what the shortening left
        log = []
        while s.has_unfinished():
            run_step(m, s, log)
        outs[tile] = [r.output for r in rs]
        portions = [[e for e in step if e[0] == 9 and e[2] > 1] for step in log]
        sizes = [(sum(e[2] for e in step), p[0][2]) for step, p in zip(log, portions) if p]
        if tile:
            assert sizes[:-1] and all(total % 8 == 0 for total, _ in sizes[:-1]), sizes       # every step but the prompt's last
            assert sizes[0] == (16, 13)
            assert sum(n for _, n in sizes) == 70
        else:
            assert sizes[0] == (21, 16)                   # the second prompt takes what is left of the budget
        assert all(r.output == expected_output(r) for r in rs)
    assert outs[0] == outs[8]


def test_the_release_callback_sees_every_request_that_gives_up_its_pages():
    """Whoever keeps more per request than the cache manager (the runner's converted block tables) passes `release`:
    it is called when a request finishes, is preempted or is aborted."""
    seen = []
    groups = [CacheGroup(2, 16, 0, (0,))]
    m = CacheManager(groups, 4, 10, 8)
    def release(rid):
        seen.append(rid)
        if m.has_request(rid):
            m.release(rid)
    s = Scheduler(m, 16, 8, 256, 0, (), release=release)
    rs = [req(i, 9, new=16) for i in range(3)]
    for r in rs:
        s.add_request(r)
    for _ in range(6):
        run_step(m, s)
    assert s.abort(rs[0].rid)
    while s.has_unfinished():
        run_step(m, s)
    assert s.num_preemptions > 0 and rs[0].rid in seen and {r.rid for r in rs} <= set(seen)
    assert len(seen) >= 3 + s.num_preemptions
    assert m.num_requests() == 0 and m.pools[0].num_free == 10


def test_prefill_chunk_option_and_several_prompts_in_one_step():
    m, s = make(budget=32, chunk=5)
    s.add_request(req(1, 12)); s.add_request(req(2, 3)); s.add_request(req(3, 9))
    log = []
    run_step(m, s, log)
    assert log[-1] == [(1, 0, 5, False), (2, 0, 3, True), (3, 0, 5, False)]


def test_stops_on_eos_max_new_tokens_and_model_length():
    m, s = make(eos=(next_token([5, 6, 7]),))
    r = Request(1, [5, 6, 7], SamplingParams(max_new_tokens=9))
    s.add_request(r)
    while s.has_unfinished():
        run_step(m, s)
    assert len(r.output) == 1 and r.finish_reason == "stop"
    r2 = Request(2, [5, 6, 7], SamplingParams(max_new_tokens=4, ignore_eos=True))
    s.add_request(r2)
    while s.has_unfinished():
        run_step(m, s)
    assert len(r2.output) == 4 and r2.finish_reason == "length"
    m, s = make(max_len=12)
    r3 = req(3, 9, new=50)
    s.add_request(r3)
    while s.has_unfinished():
        run_step(m, s)
    assert r3.length == 12 and r3.finish_reason == "length"


def test_refuses_what_can_never_run():
    m, s = make(pages=4, page=4, max_len=64)
    with pytest.raises(ValueError, match="at least one prompt token"):
        s.add_request(Request(1, [], SamplingParams()))
    with pytest.raises(ValueError, match="pages"):
        s.add_request(req(2, 10, new=10))               # 20 tokens = 5 pages > 4
    with pytest.raises(ValueError, match="nothing could be generated"):
        s.add_request(req(3, 64, new=1))
    with pytest.raises(ValueError, match="max_new_tokens"):
        s.add_request(Request(4, [1], SamplingParams(max_new_tokens=0)))
    s.add_request(req(5, 10, new=6))                    # 16 tokens = 4 pages: fits alone


def test_admission_waits_for_the_pages_of_the_whole_prompt():
    m, s = make(pages=5, page=4, budget=64)
    a = req(1, 12, new=4)
    s.add_request(a)
    run_step(m, s)                                      # a holds 3 pages
    b = req(2, 12, new=2)
    s.add_request(b)
    log = []
    run_step(m, s, log)                                 # a decodes into a 4th page; b needs 3, one is free
    assert log[-1] == [(1, 12, 1, True)] and list(s.waiting) == [b]
    while a.status is not Status.FINISHED:
        run_step(m, s, log)
    run_step(m, s, log)
    assert log[-1] == [(2, 0, 12, True)]


def test_later_portion_shrinks_to_the_free_pages():
    m, s = make(pages=6, page=4, budget=9)
    a, b = req(1, 4, new=12), req(2, 16, new=2)
    s.add_request(a); s.add_request(b)
    log = []
    run_step(m, s, log)                                 # a whole (1 page), b's first 5 (2 pages); b was admitted with 4 free
    assert log[-1] == [(1, 0, 4, True), (2, 0, 5, False)]
    run_step(m, s, log)                                 # a takes a page; b's next 8 fit the 2 pages left only up to 16
    assert log[-1] == [(1, 4, 1, True), (2, 5, 8, False)]
    run_step(m, s, log)                                 # no page left for position 16.. wait: 13..15 are in b's 4th page
    assert log[-1] == [(1, 5, 1, True), (2, 13, 3, True)]


def test_out_of_pages_preempts_the_latest_and_recomputes_it():
    m, s = make(pages=6, page=4, budget=64)
    a, b = req(1, 8, new=12), req(2, 8, new=12)          # each grows to 20 tokens = 5 pages; the pool has 6
    s.add_request(a); s.add_request(b)
    log = []
    while s.has_unfinished():
        run_step(m, s, log)
        assert len(log) < 200
    assert s.num_preemptions >= 1 and b.preemptions >= 1 and a.preemptions == 0    # the one admitted last gives way
    assert a.output == expected_output(a) and b.output == expected_output(b)
    # The recomputation runs prompt + output so far as one prompt and samples only at its end.
    recompute = [e for step in log for e in step if e[0] == 2 and e[1] == 0 and e[2] > 8]
    assert len(recompute) == 1 and recompute[0][3] is True and b.preemptions == 1
    assert m.pools[0].num_free == 6


def test_preempted_request_returns_to_the_front_of_the_queue():
    m, s = make(pages=6, page=4, budget=64)
    a, b, c = req(1, 8, new=12), req(2, 8, new=12), req(3, 4, new=2)
    s.add_request(a); s.add_request(b)
    for _ in range(3):
        run_step(m, s)
    s.add_request(c)
    while b.preemptions == 0:
        run_step(m, s)
    assert list(s.waiting)[0] is b and b.num_computed == 0 and b.status is Status.WAITING


def test_all_prompts_stuck_frees_the_latest():
    m, s = make(pages=6, page=4, budget=8, chunk=4)       # both are admitted early and are mid-prompt when the pool is empty
    a, b = req(1, 16, new=2), req(2, 16, new=2)
    s.add_request(a); s.add_request(b)
    n = 0
    while s.has_unfinished():
        run_step(m, s); n += 1
        assert n < 100
    assert a.output == expected_output(a) and b.output == expected_output(b) and s.num_preemptions >= 1


def test_abort():
    m, s = make()
    a, b = req(1, 8), req(2, 8)
    s.add_request(a); run_step(m, s); s.add_request(b)
    assert s.abort(1) and s.abort(2) and not s.abort(3)
    assert a.finish_reason == b.finish_reason == "abort" and not s.has_unfinished() and m.pools[0].num_free == 64


@pytest.mark.parametrize("seed", range(8))
def test_random_arrivals_under_pressure_finish_with_the_unpressured_output(seed):
    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    window = rng.choice([0, 0, 6])
    m, s = make(pages=rng.randint(12, 24), page=page, budget=rng.choice([8, 16, 48]), seqs=rng.choice([2, 3, 6]),
                max_len=200, chunk=rng.choice([0, 5]), window=window)
    cap = m.pools[0].num_pages * page
    reqs, pending = [], []
    for i in range(12):
        n = rng.randint(1, cap // 2)
        pending.append(req(i + 1, n, new=rng.randint(1, min(16, cap - n))))
    steps = 0
    while pending or s.has_unfinished():
        while pending and rng.random() < 0.4:
            r = pending.pop(0); s.add_request(r); reqs.append(r)
        if s.has_unfinished():
            plan, _ = run_step(m, s)
            assert plan, "work is waiting but nothing was scheduled"
            assert sum(e.num_tokens for e in plan if e.num_tokens > 1) <= s.max_tokens_per_step
            assert len(s.running) <= s.max_num_seqs
        steps += 1
        assert steps < 5000
    for r in reqs:
        assert r.status is Status.FINISHED and r.output == expected_output(r), (r.rid, r.preemptions)
    assert all(p.num_free == p.num_pages for p in m.pools) and m.num_requests() == 0


def test_a_decoding_batch_with_pages_to_spare_is_planned_as_it_stands():
    """Nobody waits, everybody decodes, every group has a free page for each: the plan is one token for each running
    request in the order of admission, and it equals what the weighing path decides when pages are short of that."""
    m, s = make(pages=64, page=4, budget=4, seqs=8)
    for rid, n in ((1, 5), (2, 9), (3, 2)):
        s.add_request(req(rid, n, new=20))
    log = []
    while any(r.remaining > 1 for r in s.running) or s.waiting:
        run_step(m, s, log)
    assert all(p.num_free >= len(s.running) for p in m.pools)
    plan, _ = run_step(m, s, log)
    assert [(e.request.rid, e.num_tokens, e.sample) for e in plan] == [(1, 1, True), (2, 1, True), (3, 1, True)]   # budget 4 does not bind
    # the same requests in a pool so small that the short cut does not apply: same plan while the pages last
    m2, s2 = make(pages=8, page=4, budget=4, seqs=8)
    for rid, n in ((1, 5), (2, 9), (3, 2)):
        s2.add_request(req(rid, n, new=20))
    while any(r.remaining > 1 for r in s2.running) or s2.waiting:
        run_step(m2, s2)
    assert not all(p.num_free >= len(s2.running) for p in m2.pools)
    plan2, _ = run_step(m2, s2)
    assert [(e.request.rid, e.start, e.num_tokens, e.sample) for e in plan2] == \
        [(e.request.rid, e.request.num_computed - 1, 1, True) for e in plan2]
    assert [e.request.rid for e in plan2] == [1, 2, 3]


def test_attention_split_counts_are_valid_and_hit_the_measured_points():
    """How many key ranges a decode attention launch is cut into is a plan made on the host: every answer must be
    launchable (a range has at least 256 keys, at most 64 ranges, powers of two where a cluster combines them), and the
    points that were measured keep their answers."""
    from lucciola_b200.ops import attention_splits
    for tiles in (1, 2, 3, 8, 12, 24, 37, 40, 48, 64, 96, 128, 500):
        for heads in (1, 2, 8):
            for span in (1, 100, 256, 1000, 4096, 8192, 32768, 131072):
                for rows in (1, 4, 16, 17, 64):
                    for wide in (0, 14):
                        s = attention_splits(tiles, heads, span, rows, wide_clusters=wide)
                        assert 1 <= s <= 64, (tiles, heads, span, rows, s)
                        assert s == 1 or span // s >= 256, (tiles, heads, span, rows, s)
                        if rows <= 16 and tiles * heads <= 296 and s < 16:
                            assert s & (s - 1) == 0, (tiles, heads, span, rows, s)
                        if rows > 16 and tiles * heads >= 148:
                            assert s == 1
    assert attention_splits(8, 8, 8192, 4) == 4            # batch 8: one wave of 256 CTAs
    assert attention_splits(64, 8, 8192, 4) == 1           # two waves that are full enough: no cutting
    assert attention_splits(40, 8, 8192, 4) == 4           # 320 tiles: a last wave of 24 CTAs would cost more than the cuts
    assert attention_splits(1, 8, 8192, 4, wide_clusters=14) == 16      # one request: 16 ranges in clusters of 16
    assert attention_splits(1, 8, 32768, 4, wide_clusters=14) > 16      # very long: more ranges through the workspace
    assert attention_splits(2, 8, 8192, 4, wide_clusters=14) == 18      # 16 clusters of 16 would not fit at once


def test_key_ranges_of_prompt_attention_are_valid_and_hit_the_measured_points():
    """Into how many key ranges the work items of the tensor-memory prompt kernel are cut is a plan made on the host too: at
    most 8, a range of 256 keys at least, none where the launch fills the SMs by itself; the measured points keep their answers."""
    from lucciola_b200.ops import attention_tcgen05_splits
    assert attention_tcgen05_splits(32, 8, 2048) == 1           # a whole prompt: the launch fills the SMs
    assert attention_tcgen05_splits(128, 8, 8192) == 1
    assert attention_tcgen05_splits(8, 8, 8192) == 2            # 64 CTAs behind a long context: two ranges make 128
    assert attention_tcgen05_splits(8, 8, 1024) == 1            # too few keys to pay for the partial results
    assert attention_tcgen05_splits(16, 8, 8192) == 1           # 128 CTAs: any cut adds a round
    assert attention_tcgen05_splits(1, 8, 65536) == 8           # one item of a few tokens behind a very long context
    assert attention_tcgen05_splits(1, 8, 512) == 1
    for tiles in range(1, 40):
        for heads in (1, 2, 8, 16):
            for span in (1, 256, 1024, 4096, 32768, 262144):
                s = attention_tcgen05_splits(tiles, heads, span)
                assert 1 <= s <= min(8, max(1, span // 256)), (tiles, heads, span, s)
