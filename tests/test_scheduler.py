"""The scheduler's decisions, without a GPU: a stand-in executor reserves and commits
what each plan holds and answers with made-up tokens (reference behaviour:
tests/cpp/test_engine.cpp:50-162)."""

import pytest

from from_scratch_inference_engine_b200.cache import CacheManager, CacheNeed
from from_scratch_inference_engine_b200.engine.scheduler import Scheduler, SeqStatus
from from_scratch_inference_engine_b200.sampling import SamplingParams

NEED = CacheNeed(kv_heads=1, head_dim=16)
GREEDY = SamplingParams(temperature=0.0)


def make(num_pages, page_size=4, max_batch=8, max_step_tokens=16, prefix=False, needs=None):
    cache = CacheManager(needs or [NEED], page_size, num_pages, max_batch, prefix)
    return Scheduler(cache, max_batch, max_step_tokens), cache


def next_token(seq):
    """Stand-in model: the next token depends on the whole context only."""
    context = seq.context()
    return (sum(context) * 31 + len(context)) % 97


def run_step(s, cache, log=None):
    items = s.plan()
    tokens = []
    for item in items:
        cache.reserve(item.seq.handle, len(item.tokens))
        # the portion must continue exactly where the cache stands
        context = item.seq.context()
        at = item.seq.handle.length
        assert context[at:at + len(item.tokens)] == item.tokens
        cache.commit(item.seq.handle, len(item.tokens))
        tokens.append(next_token(item.seq) if item.samples else None)
    if log is not None:
        log.append([(i.seq.id, len(i.tokens), i.was_prefill) for i in items])
    s.finish_step(items, tokens)
    cache.check()
    return items


def run_all(s, cache, log=None, limit=10_000):
    for _ in range(limit):
        if not s.has_work():
            return
        assert run_step(s, cache, log), "no progress"
    raise AssertionError("did not finish")


def alone(prompt, max_tokens, eos_id=-1):
    s, cache = make(num_pages=64)
    rid = s.add(prompt, GREEDY, max_tokens, eos_id, seed=0)
    run_all(s, cache)
    return s.sequences[rid].output


def test_single_request_prefills_in_portions_then_decodes():
    s, cache = make(num_pages=64, max_step_tokens=16)
    rid = s.add(list(range(40)), GREEDY, 5, -1, 0)
    log = []
    run_all(s, cache, log)
    assert [step[0][1] for step in log] == [16, 16, 8, 1, 1, 1, 1]
    assert [step[0][2] for step in log] == [True, True, True, False, False, False, False]
    assert len(s.sequences[rid].output) == 5 and s.sequences[rid].status is SeqStatus.Finished
    assert cache.free_pages() == [64] and cache.slots.num_free == 8


def test_decodes_go_first_and_portions_fill_the_rest_of_the_budget():
    s, cache = make(num_pages=64, max_step_tokens=16)
    a = s.add(list(range(6)), GREEDY, 20, -1, 0)
    run_step(s, cache)                                    # a is prefilled
    b = s.add(list(range(50)), GREEDY, 3, -1, 0)
    log = []
    run_step(s, cache, log)
    assert log[0] == [(a, 1, False), (b, 15, True)]       # one decode token + 15 of the budget
    run_step(s, cache, log)
    assert log[1] == [(a, 1, False), (b, 15, True)]
    run_all(s, cache, log)
    assert s.sequences[b].output == alone(list(range(50)), 3)
    assert s.sequences[a].output == alone(list(range(6)), 20)


def test_two_concurrent_equal_each_alone():
    s, cache = make(num_pages=64)
    a = s.add([3, 1, 4, 1, 5], GREEDY, 9, -1, 0)
    b = s.add([2, 7, 1, 8, 2, 8, 1], GREEDY, 6, -1, 0)
    run_all(s, cache)
    assert s.sequences[a].output == alone([3, 1, 4, 1, 5], 9)
    assert s.sequences[b].output == alone([2, 7, 1, 8, 2, 8, 1], 6)


def test_admission_is_fcfs_and_capped_by_max_batch():
    s, cache = make(num_pages=64, max_batch=2)
    ids = [s.add([1, 2, 3], GREEDY, 4, -1, 0) for _ in range(4)]
    run_step(s, cache)
    assert s.running == ids[:2] and list(s.waiting) == ids[2:]
    run_all(s, cache)
    assert all(s.sequences[i].status is SeqStatus.Finished for i in ids)


def test_head_of_the_queue_blocks_those_behind_it():
    s, cache = make(num_pages=6, page_size=4, max_step_tokens=64)
    a = s.add(list(range(12)), GREEDY, 4, -1, 0)          # 3 pages now, 4 at the end
    run_step(s, cache)
    big = s.add(list(range(16)), GREEDY, 2, -1, 0)        # needs 4 pages at once: 3 are free
    small = s.add([1], GREEDY, 2, -1, 0)                  # would fit, but is behind `big`
    run_step(s, cache)
    assert s.running == [a] and list(s.waiting) == [big, small]
    run_all(s, cache)
    assert s.sequences[small].status is SeqStatus.Finished


def test_tight_pool_serialises():
    # one request's worth of pages: the second waits until the first is done
    s, cache = make(num_pages=2, page_size=4)
    a = s.add([1, 2, 3, 4, 5], GREEDY, 3, -1, 0)
    b = s.add([9, 8, 7, 6, 5], GREEDY, 3, -1, 0)
    log = []
    run_all(s, cache, log)
    assert all(len(step) == 1 for step in log)
    first_b = next(i for i, step in enumerate(log) if step[0][0] == b)
    assert all(step[0][0] == a for step in log[:first_b])
    assert s.sequences[a].output == alone([1, 2, 3, 4, 5], 3)
    assert s.sequences[b].output == alone([9, 8, 7, 6, 5], 3)


def test_pages_run_out_preempts_the_youngest_which_recomputes():
    # both fit at first; growing, they exhaust the pool; the younger one is preempted
    s, cache = make(num_pages=4, page_size=4, max_step_tokens=32)
    a = s.add([5, 6, 7], GREEDY, 12, -1, 0)               # ends at 14 tokens: 4 pages
    b = s.add([8, 9, 10], GREEDY, 12, -1, 0)
    log = []
    run_all(s, cache, log)
    assert s.preemptions > 0 and s.sequences[b].preempted > 0 and s.sequences[a].preempted == 0
    assert s.sequences[a].output == alone([5, 6, 7], 12)
    assert s.sequences[b].output == alone([8, 9, 10], 12)
    # after the preemption b's recompute covers prompt + output so far, as a prefill
    recomputes = [n for step in log for (rid, n, prefill) in step if rid == b and prefill]
    assert len(recomputes) >= 2 and max(recomputes[1:]) > 3
    assert cache.free_pages() == [4]


def test_preempted_request_returns_to_the_front_of_the_queue():
    s, cache = make(num_pages=4, page_size=4, max_step_tokens=32)
    a = s.add([5, 6, 7], GREEDY, 12, -1, 0)
    b = s.add([8, 9, 10], GREEDY, 12, -1, 0)
    c = s.add([1], GREEDY, 2, -1, 0)
    while s.preemptions == 0:
        run_step(s, cache)
    assert s.waiting[0] == b and s.sequences[b].status is SeqStatus.Waiting
    assert s.sequences[b].handle is None
    run_all(s, cache)
    assert s.sequences[c].output == alone([1], 2)


def test_eos_stops_and_is_kept():
    prompt = [4, 4, 4]
    free_run = alone(prompt, 10)
    eos = free_run[3]
    out = alone(prompt, 10, eos_id=eos)
    stop = free_run.index(eos)
    assert out == free_run[:stop + 1] and out[-1] == eos


def test_requests_that_can_never_fit_are_refused():
    s, _ = make(num_pages=4, page_size=4)
    with pytest.raises(ValueError, match="page pool holds 16"):
        s.add(list(range(10)), GREEDY, 8, -1, 0)          # 17 cached tokens at the end
    s.add(list(range(10)), GREEDY, 7, -1, 0)              # 16: fits exactly
    with pytest.raises(ValueError, match="empty prompt"):
        s.add([], GREEDY, 4, -1, 0)
    with pytest.raises(ValueError, match="max_tokens"):
        s.add([1], GREEDY, 0, -1, 0)


def test_prefix_cache_on_equals_off_with_hits():
    prompt = list(range(30, 43))                          # 13 tokens: three full pages
    outs = {}
    for prefix in (False, True):
        s, cache = make(num_pages=32, prefix=prefix)
        first = s.add(prompt, GREEDY, 4, -1, 0)
        run_all(s, cache)
        log = []
        second = s.add(prompt + [7, 7], GREEDY, 4, -1, 0)
        run_all(s, cache, log)
        outs[prefix] = (s.sequences[first].output, s.sequences[second].output)
        if prefix:
            assert cache.prefix_hits == 1
            assert log[0] == [(second, 3, True)]          # 12 of 15 tokens came from the cache
        else:
            assert log[0] == [(second, 15, True)]
    assert outs[False] == outs[True]


def test_prefix_hit_under_page_pressure_never_plans_more_than_is_free():
    """A cached prefix page that only the cache holds counts as free until a new request
    takes it: the plan of that step must not give the same page to a decode as well."""
    s, cache = make(num_pages=8, page_size=4, prefix=True, max_step_tokens=64)
    a = s.add(list(range(100, 109)), GREEDY, 2, -1, 0)     # 9 tokens: registers 2 full pages
    run_all(s, cache)
    assert s.sequences[a].status is SeqStatus.Finished and cache.free_pages() == [8]
    b = s.add(list(range(200, 207)), GREEDY, 12, -1, 0)    # decodes across page edges
    run_step(s, cache)
    c = s.add(list(range(100, 108)) + list(range(300, 313)), GREEDY, 2, -1, 0)   # a's prefix + 13
    run_all(s, cache)                                     # run_step reserves every planned item
    assert cache.prefix_hits == 1
    assert s.sequences[b].status is SeqStatus.Finished and s.sequences[c].status is SeqStatus.Finished
    cache.clear_prefix_cache()
    assert cache.free_pages() == [8]


@pytest.mark.parametrize("seed", range(6))
def test_prefix_cache_under_pressure_random_orders(seed):
    import random
    rng = random.Random(seed)
    s, cache = make(num_pages=12, page_size=4, prefix=True, max_step_tokens=24, max_batch=4)
    stems = [[rng.randrange(90) for _ in range(12)] for _ in range(2)]
    ids, outs = [], {}
    for k in range(14):
        prompt = stems[rng.randrange(2)][:rng.choice([4, 8, 12])] + \
            [rng.randrange(90) for _ in range(rng.randrange(1, 9))]
        ids.append((s.add(prompt, GREEDY, rng.randrange(1, 9), -1, 0), prompt))
        for _ in range(rng.randrange(3)):
            if s.has_work():
                run_step(s, cache)
    run_all(s, cache)
    for rid, prompt in ids:
        assert s.sequences[rid].output == alone(prompt, s.sequences[rid].max_tokens)
    cache.clear_prefix_cache()
    assert cache.free_pages() == [12]


def test_small_window_pool_admits_with_the_default_token_budget():
    """A windowed group's pool smaller than the first portion must not keep the request
    waiting for ever: it starts with the pages there are and its portions are cut to them."""
    needs = [NEED, CacheNeed(1, 16, window=21)]
    s, cache = make(num_pages=[64, 6], page_size=8, needs=needs, max_step_tokens=2048)
    rid = s.add(list(range(70)), GREEDY, 6, -1, 0)
    log = []
    run_all(s, cache, log)
    assert len(s.sequences[rid].output) == 6
    assert log[0][0][1] == 48                             # six pages of eight tokens
    assert cache.free_pages() == [64, 6]


def test_window_pool_that_can_never_hold_a_window_is_refused():
    needs = [NEED, CacheNeed(1, 16, window=21)]
    s, cache = make(num_pages=[64, 3], page_size=8, needs=needs)
    with pytest.raises(ValueError, match="window of 21"):
        s.add(list(range(10)), GREEDY, 4, -1, 0)


def test_shared_pages_are_looked_for_when_a_request_starts_not_when_it_is_admitted():
    """A short request has left the first two pages of a long common prefix in the cache.
    Three requests behind that prefix are admitted together; the second and third start only
    after the first has registered all of it, and must then share all six pages - not the
    two that were there when they were admitted."""
    # 19 tokens per step: exactly what the first of the three still has to run
    s, cache = make(num_pages=64, page_size=4, prefix=True, max_step_tokens=19, max_batch=8)
    stem = list(range(500, 524))                              # six pages
    early = s.add(stem[:9], GREEDY, 2, -1, 0)
    run_all(s, cache)
    ids = [s.add(stem + [900 + k, 7, 7], GREEDY, 3, -1, 0) for k in range(3)]
    shared = {}
    while s.has_work():
        run_step(s, cache)
        for rid in ids:
            handle = s.sequences[rid].handle
            if handle is not None and handle.length:
                shared.setdefault(rid, handle.shared_tokens)
    assert shared == {ids[0]: 8, ids[1]: 24, ids[2]: 24}
    assert all(s.sequences[r].output == alone(stem + [900 + k, 7, 7], 3) for k, r in enumerate(ids))


def test_release_prefix_undoes_an_acquisition():
    s, cache = make(num_pages=8, page_size=4, prefix=True)
    first = s.add(list(range(40, 49)), GREEDY, 2, -1, 0)
    run_all(s, cache)
    assert cache.free_pages() == [8]                          # two cached pages count as free
    handle = cache.open("x")
    assert cache.acquire_prefix(handle, list(range(40, 48))) == 8
    assert cache.free_pages() == [6] and cache.prefix_hits == 1
    cache.release_prefix(handle)
    assert cache.free_pages() == [8] and cache.prefix_hits == 0
    assert handle.length == 0 and handle.tables == [[]]
    cache.check()
    cache.reserve(handle, 5)
    cache.commit(handle, 5)
    with pytest.raises(RuntimeError, match="tokens of its own"):
        cache.release_prefix(handle)
    cache.close(handle)


def test_windowed_group_bounds_what_a_request_holds():
    needs = [NEED, CacheNeed(1, 16, window=8)]
    s, cache = make(num_pages=[40, 6], page_size=4, needs=needs, max_step_tokens=8)
    rid = s.add(list(range(60)), GREEDY, 30, -1, 0)
    peak = 0
    while s.has_work():
        run_step(s, cache)
        if s.sequences[rid].handle is not None:
            peak = max(peak, sum(p >= 0 for p in s.sequences[rid].handle.tables[1]))
    assert len(s.sequences[rid].output) == 30 and peak <= 5


# ------------------------------------------------------------------ overlapped steps
def run_overlapped(s, cache, limit=10_000):
    """Drives the scheduler as the engine does with overlapped steps: the next step is planned
    and 'launched' (pages reserved and committed) before the tokens of the step before it are
    known; only then are those tokens computed and recorded.  The stand-in model needs the whole
    context, so a token is computed when it is resolved - which also proves that no plan ever
    needed a token that was still pending."""
    from from_scratch_inference_engine_b200.engine.scheduler import PENDING_TOKEN
    in_flight = None
    wasted = 0

    def settle():
        nonlocal in_flight, wasted
        items = in_flight
        in_flight = None
        tokens = []
        for item in items:
            seq = item.seq
            if item.samples and seq.status is SeqStatus.Running and seq.handle is not None and seq.pending:
                context = seq.context()
                tokens.append((sum(context) * 31 + len(context)) % 97)
            else:
                wasted += bool(item.samples)
                tokens.append(None if not item.samples else 0)      # a dropped token: any value
        s.resolve_step(items, tokens)
        cache.check()

    for _ in range(limit):
        if not s.has_work() and in_flight is None:
            return wasted
        items = s.plan(can_preempt=in_flight is None)
        if not items and in_flight is not None:
            settle()
            items = s.plan()
        if not items:
            assert not s.has_work(), "no progress"
            continue
        for item in items:
            assert item.seq.status is SeqStatus.Running
            if item.source_row >= 0:
                assert item.tokens == [PENDING_TOKEN] and item.seq.pending == 1
            else:
                context = item.seq.context()
                at = item.seq.handle.length
                assert context[at:at + len(item.tokens)] == item.tokens
            cache.reserve(item.seq.handle, len(item.tokens))
            cache.commit(item.seq.handle, len(item.tokens))
        if in_flight is not None:
            settle()
        s.begin_step(items)
        in_flight = items
    raise AssertionError("did not finish")


@pytest.mark.parametrize("num_pages", [64, 9])
def test_overlapped_steps_record_the_same_tokens(num_pages):
    """With a roomy pool and with one that forces preemption: every request ends with the tokens it
    gets alone; a request that stops at an end-of-sequence token costs one dropped token."""
    prompts = [[5, 6, 7], list(range(1, 20)), [9] * 11, [3, 1, 4, 1, 5, 9, 2, 6], [8]]
    lengths = [6, 9, 4, 12, 7]
    eos_of = {3: alone(prompts[3], 12)[4]}
    want = [alone(p, n, eos_of.get(i, -1)) for i, (p, n) in enumerate(zip(prompts, lengths))]
    s, cache = make(num_pages=num_pages, max_batch=3, max_step_tokens=8)
    ids = [s.add(p, GREEDY, n, eos_of.get(i, -1), seed=0) for i, (p, n) in enumerate(zip(prompts, lengths))]
    wasted = run_overlapped(s, cache)
    assert [s.sequences[i].output for i in ids] == want
    assert len(want[3]) < 12 and wasted >= 1
    assert all(seq.pending == 0 and seq.status is SeqStatus.Finished for seq in s.sequences.values())
    assert cache.free_pages() == [num_pages]
    if num_pages == 9:
        assert s.preemptions > 0


def test_a_plan_that_would_preempt_is_given_up_while_tokens_are_pending():
    s, cache = make(num_pages=4, max_batch=2, max_step_tokens=8)          # 16 tokens of cache
    a = s.add([1] * 7, GREEDY, 8, -1, seed=0)
    b = s.add([2] * 7, GREEDY, 8, -1, seed=0)
    items = s.plan()
    for item in items:
        cache.reserve(item.seq.handle, len(item.tokens))
        cache.commit(item.seq.handle, len(item.tokens))
    s.begin_step(items)
    pending = [i for i in items if i.samples]
    assert pending and all(i.seq.pending == 1 for i in pending)
    # fill the pool: both requests now hold all four pages between them
    while True:
        items2 = s.plan(can_preempt=False)
        if not items2:
            break
        for item in items2:
            cache.reserve(item.seq.handle, len(item.tokens))
            cache.commit(item.seq.handle, len(item.tokens))
        s.resolve_step(items, [1 if i.samples else None for i in items])
        s.begin_step(items2)
        items = items2
    assert s.preemptions == 0                  # it came back empty instead of preempting
    s.resolve_step(items, [1 if i.samples else None for i in items])
    assert s.plan() and s.preemptions >= 1    # with nothing pending the youngest is preempted
    assert {s.sequences[a].status, s.sequences[b].status} == {SeqStatus.Running, SeqStatus.Waiting}


def test_key_splits_of_the_attention_launch():
    """How many key ranges a tile is cut into (host arithmetic of parts/attention.py): decoded
    tokens fill the block slots without falling under 128 keys per range and never split past 64;
    prompt tiles split only into slots that would stay empty."""
    from from_scratch_inference_engine_b200.parts.attention import attention_splits
    sms = 148
    # decoded tokens, mma.sync kernel (three blocks per SM): 32 pairs at 4,096 keys fill 444 slots
    n = attention_splits(32, 4096, sms, True)
    assert 9 <= n <= 13 and 32 * n <= 3 * sms
    assert attention_splits(4, 4096, sms, True) >= 24           # batch 1
    # a range is a whole number of 64-key tiles: 4,091 keys in ranges of two tiles are 32 ranges,
    # none of them empty (29 or 31 ranges would be three tiles each, and some ranges empty)
    assert attention_splits(4, 4091, sms, True) == 32
    for pairs, longest in ((4, 4091), (16, 4091), (32, 4091), (8, 9000), (4, 700)):
        n = attention_splits(pairs, longest, sms, True)
        tiles = -(-(-(-longest // n)) // 64)
        assert n == 1 or (n - 1) * tiles * 64 < longest <= n * tiles * 64
    assert attention_splits(4, 200, sms, True) == 1              # too short to split
    assert 32 < attention_splits(4, 100000, sms, True) <= 64     # batch 1, a very long context
    assert attention_splits(2048, 4096, sms, True) <= 2          # many pairs: waves, not splits
    # decoded tokens, tcgen05 kernel (two blocks per SM, dearer blocks): one wave unsplit
    assert attention_splits(256, 4096, sms, True, decode_slots=2, decode_fixed=530) == 1
    assert attention_splits(148, 4096, sms, True, decode_slots=2, decode_fixed=530) == 2
    # 200 requests x 2 kv heads, contexts of up to 2,560 keys (a serving step): two waves of whole
    # key ranges beat three waves of halves once the merge launch is counted
    assert attention_splits(400, 2560, sms, True, decode_slots=2, decode_fixed=530, merge_cost=1300) == 1
    assert attention_splits(400, 2560, sms, True, decode_slots=2, decode_fixed=530, merge_cost=0) == 2
    # prompt tiles: as many splits as fill the slots, none when there are tiles enough
    assert attention_splits(2 * sms, 8192, sms, False) == 1
    assert attention_splits(sms // 2, 8192, sms, False) == 4
    assert attention_splits(32, 2048, sms, False, 1) == 4        # one block per SM: 148 // 32
    assert attention_splits(32, 300, sms, False, 1) == 2         # at least 128 keys per range
