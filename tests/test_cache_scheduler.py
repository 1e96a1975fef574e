"""The cache manager's bookkeeping and the scheduler's decisions (no GPU)."""
import random

import pytest
import torch

from delta_b200.cache import CacheManager, OutOfPages, PagePool
from delta_b200.engine.scheduler import FAILED, FINISHED, RUNNING, WAITING, Scheduler
from delta_b200.parts.base import PAGE, CacheSpec, StateSpec
from delta_b200.sampling import SamplingParams


def manager(num_pages=16, page_size=4, max_slots=4, max_seq_len=64, window=None, states=None):
    specs = {0: CacheSpec((2, 2, PAGE, 8)), 1: CacheSpec((2, 2, PAGE, 8))}
    if window:
        specs[2] = CacheSpec((2, 2, PAGE, 8), window)
    return CacheManager(specs, states or {}, max_slots=max_slots, max_seq_len=max_seq_len, page_size=page_size,
                        num_pages=num_pages, dtype=torch.float32, device="cpu")


def test_pool_is_lifo_and_strict():
    p = PagePool(4)
    a = p.alloc(3)
    assert a == [0, 1, 2] and p.free_pages == 1
    p.free([1])
    assert p.alloc(1) == [1]          # the page given back last is used again first
    with pytest.raises(OutOfPages):
        p.alloc(2)
    assert p.free_pages == 1          # nothing was taken by the failed call
    p.free([0])
    with pytest.raises(ValueError, match="twice"):
        p.free([0])
    with pytest.raises(ValueError):
        p.free([7])
    p.check()
    assert sorted(PagePool(8, shuffle_seed=0).alloc(8)) == list(range(8))


def test_pool_hands_out_runs():
    """Requests that grow by one page in turns still hold aligned runs; many pages at once come in order;
    runs given back are used again first, in their order; when no run is wholly free, pages of begun runs
    are taken, and every free page can be had."""
    R = 4
    p = PagePool(128, run_pages=R)
    held = {r: [] for r in range(5)}
    for _ in range(9):                                   # five requests, a page each in turn, nine times
        for r in held:
            held[r] += p.alloc(1, after=held[r][-1] if held[r] else None)
    for r, pages in held.items():
        for j in range(0, 8, R):                         # the first two runs of every request
            assert pages[j] % R == 0 and pages[j:j + R] == list(range(pages[j], pages[j] + R)), (r, pages)
    p.check()
    big = p.alloc(10, after=None)
    assert big == list(range(big[0], big[0] + 10)) and big[0] % R == 0
    # request 1 ends: its runs come back and are the next ones handed out, in their order
    p.free(held[1])
    again = p.alloc(8)
    assert again == held[1][:8]
    p.check()
    # use the pool up: pages of begun runs are handed out too, down to the last page
    rest = p.alloc(p.free_pages)
    assert p.free_pages == 0 and len(set(rest)) == len(rest)
    with pytest.raises(OutOfPages):
        p.alloc(1)
    p.check()
    # a pool whose size is no multiple of the run
    q = PagePool(10, run_pages=4)
    assert q.alloc(10) == list(range(10))
    q.free([9, 8])
    assert q.alloc(2, after=7) == [8, 9]
    q.check()


def test_pool_under_random_orders_with_runs():
    rng = random.Random(5)
    for R, n in ((1, 13), (4, 30), (8, 64), (8, 21)):
        p = PagePool(n, run_pages=R)
        held = {}
        for step in range(600):
            if held and (rng.random() < 0.45 or p.free_pages == 0):
                r = rng.choice(list(held))
                k = rng.randint(1, len(held[r]))
                if rng.random() < 0.5:
                    gone, held[r] = held[r][:k], held[r][k:]       # a window passes the oldest pages
                else:
                    gone, held[r] = held[r], []
                p.free(gone)
                if not held[r]:
                    del held[r]
            else:
                r = rng.randint(0, 5)
                k = rng.randint(1, min(6, p.free_pages))
                got = p.alloc(k, after=held[r][-1] if held.get(r) else None)
                assert len(got) == k
                held.setdefault(r, []).extend(got)
            everything = [x for v in held.values() for x in v]
            assert len(set(everything)) == len(everything) == p.held_pages
            p.check()


def test_grow_release_reuse():
    m = manager(num_pages=6)
    s = m.acquire_slot()
    m.grow(s, 9)                      # 3 pages of 4 tokens
    assert m.pages_in_use() == {"2x2xPx8": 3}
    m.grow(s, 12)
    assert m.pages_in_use() == {"2x2xPx8": 3}     # no page in advance at a page's edge
    m.grow(s, 13)
    assert m.pages_in_use() == {"2x2xPx8": 4}
    t = m.acquire_slot()
    with pytest.raises(OutOfPages):
        m.grow(t, 12)
    assert m.pages_in_use() == {"2x2xPx8": 4}     # all or nothing
    held = m.groups["2x2xPx8"].held(s)
    m.release_slot(s)
    m.grow(t, 16)
    assert set(m.groups["2x2xPx8"].held(t)) == set(held)   # pages are used again
    with pytest.raises(ValueError, match="twice"):
        m.release_slot(s)
    m.check()


def test_requests_that_grow_in_turns_hold_runs_of_pages():
    """Six requests decode in turns, a token each; with a mixer that asks for runs of 8 tokens' pages (two
    pages of 4) every request's block table is made of aligned pairs of pages that follow one another."""
    specs = {0: CacheSpec((2, 2, PAGE, 8), run_tokens=8)}
    m = CacheManager(specs, {}, max_slots=6, max_seq_len=64, page_size=4, num_pages=96, dtype=torch.float32, device="cpu")
    slots = [m.acquire_slot() for _ in range(6)]
    for n in range(1, 41):
        for s in slots:
            m.grow(s, n)
            m.advance(s, n)
    g = m.groups["2x2xPx8"]
    for s in slots:
        pages = g.held(s)
        assert len(pages) == 10
        for j in range(0, 10, 2):
            assert pages[j] % 2 == 0 and pages[j + 1] == pages[j] + 1, pages
    m.check()


def test_layers_share_a_group_and_windows_have_their_own():
    m = manager(window=6)
    assert set(m.groups) == {"2x2xPx8", "2x2xPx8w6"}
    assert m.groups["2x2xPx8"].cache_ids == [0, 1] and m.groups["2x2xPx8w6"].cache_ids == [2]
    assert m.layer_pages(1).shape == (16 + 1, 2, 2, 4, 8)      # the pool's 16 pages and the padding slot's spare page
    s = m.acquire_slot()
    for n in range(1, 41):
        m.grow(s, n)
        m.advance(s, n)
        m.check()
        g = m.groups["2x2xPx8w6"]
        # the next query (position n) reads keys n-5 .. n; earlier pages are given back
        first_needed = max(0, n - 6 + 1) // 4
        assert int(g.first_page[s]) == first_needed
        assert len(g.held(s)) == (n + 3) // 4 - first_needed
        assert len(m.groups["2x2xPx8"].held(s)) == (n + 3) // 4
    assert m.groups["2x2xPx8w6"].pool.held_pages <= 3
    m.release_slot(s)
    assert m.pages_in_use() == {"2x2xPx8": 0, "2x2xPx8w6": 0}


def test_the_padding_slot_holds_the_spare_page_and_no_pool_page():
    m = manager(num_pages=16, page_size=4, max_slots=4)
    slots = [m.acquire_slot() for _ in range(4)]
    assert m.padding_slot not in slots and m.free_slots == 0
    for g in m.groups.values():
        assert g.table[m.padding_slot, 0] == g.spare_page == 16 and (g.table[m.padding_slot, 1:] == -1).all()
        assert g.pool.free_pages == 16          # the spare page is not one of the pool's
    assert all(int(g.table[[slots[0], m.padding_slot]][1, 0]) == 16 for g in m.groups.values())
    m.check()


def test_state_slots_are_reset_at_admission():
    m = manager(states={"toy": StateSpec((3,), torch.float32, 0.5), "count": StateSpec((), torch.int32, -1)})
    s = m.acquire_slot()
    # a row for each of the four slots and one for the padding slot, which is never handed out
    assert m.states["toy"].shape == (4 + 1, 3) and m.states["count"].shape == (4 + 1,)
    assert m.padding_slot == 4 and m.free_slots == 3
    m.states["toy"][s] = 9.0
    m.states["count"][s] = 4
    m.release_slot(s)
    s2 = m.acquire_slot()
    assert s2 == s and m.states["toy"][s].tolist() == [0.5] * 3 and int(m.states["count"][s]) == -1


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    m = manager(num_pages=24, page_size=4, max_slots=4, max_seq_len=40, window=10)
    live = {}
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and m.free_slots:
            live[m.acquire_slot()] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = min(40, live[s] + rng.randrange(1, 9))
            try:
                m.grow(s, n)
                m.advance(s, n)
                live[s] = n
            except OutOfPages:
                pass
        elif live:
            s = rng.choice(list(live))
            m.release_slot(s)
            del live[s]
        m.check()
        for g in m.groups.values():
            assert g.pool.held_pages == sum(len(g.held(s)) for s in live)
    for s in list(live):
        m.release_slot(s)
    assert all(v == 0 for v in m.pages_in_use().values())


# ---- scheduler ----------------------------------------------------------------------

def drive(sch, next_token=lambda r: 7, max_steps=10_000):
    """Runs the scheduler without a model: every sampled token comes from ``next_token``."""
    log = []
    for _ in range(max_steps):
        if not sch.has_work():
            break
        plan = sch.schedule()
        if not plan:
            break
        assert sum(x.count for x in plan) <= sch.budget
        assert len({id(x.request) for x in plan}) == len(plan)
        log.append([(x.request.id, x.start, x.count, x.samples, x.decode) for x in plan])
        sch.complete(plan, [next_token(x.request) for x in plan if x.samples])
        sch.cache.check()
    return log


def test_budget_cuts_prompts_and_decode_goes_first():
    m = manager(num_pages=64, page_size=4, max_slots=4, max_seq_len=64)
    sch = Scheduler(m, max_batch=4, max_tokens_per_step=10)
    a = sch.add_request(list(range(23)), 30)
    b = sch.add_request(list(range(5)), 12)
    log = drive(sch)
    assert log[0] == [(0, 0, 10, False, False)]
    assert log[1] == [(0, 10, 10, False, False)]
    assert log[2] == [(0, 20, 3, True, False), (1, 0, 5, True, False)]      # rest of a, then b is admitted
    assert log[3] == [(0, 23, 1, True, True), (1, 5, 1, True, True)]
    assert a.status == FINISHED and len(a.output) == 7 and a.finish_reason == "length"
    assert b.status == FINISHED and len(b.output) == 7
    assert sch.stats["prompt_tokens"] == 28 and sch.stats["generated_tokens"] == 14
    assert all(v == 0 for v in m.pages_in_use().values()) and m.free_slots == 4


def test_stop_token_and_max_new_tokens():
    m = manager(num_pages=64)
    sch = Scheduler(m, max_batch=2, max_tokens_per_step=64)
    a = sch.add_request([1, 2, 3], 40, stop_ids=[9], max_new_tokens=None)
    b = sch.add_request([1, 2, 3], 40, max_new_tokens=3)
    drive(sch, next_token=lambda r: 9 if (r is a and len(r.output) == 4) else 5)
    assert a.output == [5, 5, 5, 5, 9] and a.finish_reason == "stop token"
    assert b.output == [5, 5, 5] and b.finish_reason == "max_new_tokens"


def test_admission_waits_for_pages_then_reuses_them():
    m = manager(num_pages=8, page_size=4, max_slots=4, max_seq_len=32)
    sch = Scheduler(m, max_batch=4, max_tokens_per_step=64)
    reqs = [sch.add_request(list(range(10)), 16) for _ in range(3)]   # 3 pages for the prompt + 1 token, 4 at the end
    log = drive(sch)
    first = [r for r, *_ in log[0]]
    assert first == [0, 1]            # the third request needs 3 free pages and only 2 are left
    assert all(r.status == FINISHED and len(r.output) == 6 for r in reqs)
    assert reqs[2].start_time >= reqs[0].start_time
    assert sch.stats["preemptions"] == 0


def test_out_of_pages_preempts_the_youngest_and_recomputes():
    m = manager(num_pages=7, page_size=4, max_slots=4, max_seq_len=28)
    sch = Scheduler(m, max_batch=4, max_tokens_per_step=64)
    a = sch.add_request(list(range(11)), 24)    # 3 pages now, 6 at the end
    b = sch.add_request(list(range(11)), 24)
    log = drive(sch)
    assert a.status == FINISHED and b.status == FINISHED
    assert len(a.output) == 13 and len(b.output) == 13
    assert b.preemptions >= 1 and a.preemptions == 0          # the older request is never the victim
    # after the preemption b's prompt and what it had generated run again as one portion
    again = [row for step in log for row in step if row[0] == 1 and row[1] == 0]
    assert len(again) == 2 and again[1][2] > 11
    assert all(v == 0 for v in m.pages_in_use().values())


def test_recomputing_after_a_preemption_keeps_decode_positions_single():
    """When some part treats decode rows in a way of its own, a preempted request runs its prompt
    in portions again and every token it had generated as a decode row of its own, unsampled,
    until it is where it was."""
    m = manager(num_pages=7, page_size=4, max_slots=4, max_seq_len=28)
    sch = Scheduler(m, max_batch=4, max_tokens_per_step=64, decode_singly=True)
    a = sch.add_request(list(range(11)), 24)
    b = sch.add_request(list(range(11)), 24)
    log = drive(sch, next_token=lambda r: 100 + len(r.output))
    assert a.status == FINISHED and b.status == FINISHED and b.preemptions >= 1
    assert a.output == [100 + i for i in range(13)] and b.output == [100 + i for i in range(13)]
    rows_b = [row for step in log for row in step if row[0] == 1]
    # no portion of b ever reaches past its prompt, and positions from the prompt's end on are single decode rows
    for (_, start, count, samples, decode) in rows_b:
        assert start + count <= 11 or (count == 1 and decode)
    again = [row for row in rows_b if row[4] and not row[3]]
    assert again and all(11 <= start < 11 + 13 for (_, start, *_rest) in again)
    # a position that is computed again is not sampled again
    sampled = [start for (_, start, count, samples, _d) in rows_b if samples]
    assert len(sampled) == len(set(sampled)) == 13
    assert all(v == 0 for v in m.pages_in_use().values())


def test_prompts_first_does_not_hold_decoding_for_a_request_that_cannot_be_admitted():
    """More requests than slots with prompts first: the waiting ones cannot be admitted until a
    running one ends, so the running ones must go on decoding."""
    m = manager(num_pages=64, page_size=4, max_slots=2, max_seq_len=32)
    sch = Scheduler(m, max_batch=2, max_tokens_per_step=16)
    sch.decode_while_prefill = False
    reqs = [sch.add_request(list(range(5)), 9) for _ in range(5)]
    drive(sch, max_steps=200)
    assert all(r.status == FINISHED and len(r.output) == 4 for r in reqs)
    # the same when the pool, not the slots, keeps the third request waiting
    m = manager(num_pages=6, page_size=4, max_slots=4, max_seq_len=32)
    sch = Scheduler(m, max_batch=4, max_tokens_per_step=16)
    sch.decode_while_prefill = False
    reqs = [sch.add_request(list(range(7)), 12) for _ in range(3)]
    drive(sch, max_steps=200)
    assert all(r.status == FINISHED for r in reqs)


def test_a_cache_group_takes_any_page_layout():
    """The manager allocates what the mixer declares: keys and values per head, one vector per
    token, or keys and values of different widths packed side by side."""
    specs = {0: CacheSpec((2, 2, PAGE, 8)), 1: CacheSpec((PAGE, 24)), 2: CacheSpec((3, PAGE, 16 + 40)), 3: CacheSpec((PAGE, 24))}
    m = CacheManager(specs, {}, max_slots=2, max_seq_len=32, page_size=4, num_pages=9, dtype=torch.float32, device="cpu")
    assert set(m.groups) == {"2x2xPx8", "Px24", "3xPx56"}
    assert m.layer_pages(0).shape == (10, 2, 2, 4, 8) and m.layer_pages(1).shape == (10, 4, 24)
    assert m.layer_pages(2).shape == (10, 3, 4, 56) and m.groups["Px24"].cache_ids == [1, 3]
    s = m.acquire_slot()
    m.grow(s, 9)
    assert m.pages_in_use() == {"2x2xPx8": 3, "Px24": 3, "3xPx56": 3}
    m.release_slot(s)
    m.check()
    with pytest.raises(ValueError):
        CacheSpec((2, 4, 8))            # no token axis
    with pytest.raises(ValueError):
        CacheSpec((PAGE, 4, PAGE))      # two of them


def test_a_request_that_can_never_fit_fails_at_once():
    m = manager(num_pages=4, page_size=4, max_slots=2, max_seq_len=64)
    sch = Scheduler(m, max_batch=2, max_tokens_per_step=64)
    big = sch.add_request(list(range(30)), 40)
    too_long = sch.add_request(list(range(70)), 80)
    ok = sch.add_request(list(range(6)), 12)
    assert big.status == FAILED and "pages" in big.finish_reason
    assert too_long.status == FAILED and "limit" in too_long.finish_reason
    drive(sch)
    assert ok.status == FINISHED and len(ok.output) == 6
    res = sch.results()
    assert [r["status"] for r in res] == [FAILED, FAILED, FINISHED]
    assert set(res[2]) >= {"request_id", "status", "input_length", "output_length", "tokens_generated", "total_time", "tokens_per_second"}


def test_prompts_first_option_holds_decoding():
    m = manager(num_pages=64, page_size=4, max_slots=4, max_seq_len=64)
    sch = Scheduler(m, max_batch=4, max_tokens_per_step=8)
    sch.decode_while_prefill = False
    sch.add_request(list(range(6)), 12)
    sch.add_request(list(range(20)), 26)
    log = drive(sch)
    decode_steps = [i for i, step in enumerate(log) if any(row[4] for row in step)]
    prefill_steps = [i for i, step in enumerate(log) if any(not row[4] for row in step)]
    assert min(decode_steps) > max(prefill_steps)


@pytest.mark.parametrize("seed", range(4))
def test_random_load_finishes_everything(seed):
    rng = random.Random(seed)
    m = manager(num_pages=20, page_size=4, max_slots=3, max_seq_len=48, window=9)
    sch = Scheduler(m, max_batch=3, max_tokens_per_step=rng.choice([5, 16, 64]))
    reqs = [sch.add_request([1] * rng.randrange(1, 30), rng.randrange(8, 48)) for _ in range(12)]
    drive(sch, next_token=lambda r: rng.randrange(10))
    for r in reqs:
        assert r.status in (FINISHED, FAILED)
        if r.status == FINISHED:
            assert r.total_len >= min(r.max_length, 48) or r.finish_reason != "length"
    assert all(v == 0 for v in m.pages_in_use().values()) and m.free_slots == 3


def test_decode_graph_sizes_round_up_by_at_most_a_half():
    """Batch sizes of captured decode steps: exact up to 8, then 12, 16, 24, 32, 48, 64, ..., capped
    by the engine's largest batch."""
    from types import SimpleNamespace
    from delta_b200.engine.step import ModelRunner
    size = lambda b, most: ModelRunner.graph_batch(SimpleNamespace(cfg=SimpleNamespace(max_batch=most)), b)
    assert [size(b, 256) for b in range(1, 9)] == list(range(1, 9))
    assert [size(b, 256) for b in (9, 12, 13, 16, 17, 25, 33, 49, 64, 65, 97, 129, 200)] == \
        [12, 12, 16, 16, 24, 32, 48, 64, 64, 96, 128, 192, 256]
    for b in range(1, 257):
        assert b <= size(b, 256) <= max(8, b * 3 // 2) and size(size(b, 256), 256) == size(b, 256)
    assert size(13, 13) == 13 and size(9, 10) == 10 and size(60, 70) == 64 and size(66, 70) == 70
