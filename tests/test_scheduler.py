"""The scheduler's decisions, on the host, with made-up tokens in place of a model
(the reference tests its scheduler the same way, tests/zedinfer/test_scheduler_sampling.cpp:64-170)."""
import pytest

from zedinfer_b200.cache import CacheManager, PagedKVNeed
from zedinfer_b200.config import GenerationConfig, SchedulerConfig
from zedinfer_b200.engine.request import InferenceRequest, RequestPhase
from zedinfer_b200.engine.scheduler import Scheduler


def make(pages=64, page_size=4, max_seq_len=256, stop=(), **kw):
    cache = CacheManager([(0, PagedKVNeed(1, 16, None)), (1, PagedKVNeed(1, 16, None))], page_size,
                         max_requests=kw.get("max_batch_requests", 64))
    cache.set_num_pages(pages)
    cfg = SchedulerConfig(kv_block_size=page_size, **kw)
    return Scheduler(cfg, cache, max_seq_len, stop), cache


def req(n, max_new=4, **kw):
    return InferenceRequest(list(range(1, n + 1)), GenerationConfig(max_new_tokens=max_new, **kw))


def run_step(s, cache, token=7):
    """Pretend to be the step function: commit the lengths, hand back one token per wanted row."""
    batch = s.schedule()
    for r in batch.decode_requests:
        cache.commit(r.cache, r.cache.length + 1)
    for r, size in zip(batch.prefill_requests, batch.prefill_chunk_sizes):
        cache.commit(r.cache, r.cache.length + size)
    tokens = [token(r) if callable(token) else token for r, _ in batch.rows_wanted()]
    done = s.process_results(batch, tokens)
    cache.check()
    return batch, done


def test_prompt_is_cut_into_portions_and_blocks_the_queue():
    s, cache = make(max_prefill_tokens=8, max_batch_tokens=64)
    a, b = req(20), req(5)
    s.submit(a), s.submit(b)
    batch, _ = run_step(s, cache)
    assert batch.prefill_requests == [a] and batch.prefill_chunk_starts == [0] and batch.prefill_chunk_sizes == [8]
    assert batch.rows_wanted() == [] and a.phase == RequestPhase.PREFILL
    batch, _ = run_step(s, cache)
    assert batch.prefill_chunk_starts == [8] and batch.prefill_chunk_sizes == [8]
    batch, _ = run_step(s, cache)                       # a's last 4 tokens, and b beside them under the budget
    assert batch.prefill_requests == [a, b] and batch.prefill_chunk_sizes == [4, 4]
    assert [r for r, _ in batch.rows_wanted()] == [a] and a.output_ids == [7] and a.phase == RequestPhase.DECODE
    batch, _ = run_step(s, cache)                       # decode first, then the rest of b
    assert batch.decode_requests == [a] and batch.prefill_requests == [b] and batch.prefill_chunk_sizes == [1]
    assert [r for r, _ in batch.rows_wanted()] == [a, b]
    assert a.output_ids == [7, 7] and b.output_ids == [7]


def test_admission_fills_every_free_place_and_never_more():
    """max_batch_requests counts live requests once: a step admits as many short prompts as there are free places
    (the reference counts those whose prompt ends in the step twice and admits half of them), a request in
    mid-prompt takes the last place, and nobody is admitted beyond the limit."""
    s, cache = make(pages=256, max_batch_requests=6, max_batch_tokens=64, max_prefill_tokens=64)
    rs = [req(3, max_new=50) for _ in range(5)] + [req(40, max_new=50)] + [req(3, max_new=50) for _ in range(3)]
    for r in rs:
        s.submit(r)
    batch, _ = run_step(s, cache)
    assert batch.prefill_requests == rs[:6] and batch.prefill_chunk_sizes == [3] * 5 + [40]
    assert len(s.active) == 6
    batch, _ = run_step(s, cache)
    assert batch.decode_requests == rs[:6] and batch.prefill_requests == [] and len(s.waiting) == 3
    s.cancel(rs[0])
    batch, _ = run_step(s, cache)                       # one place is free again: one more comes in
    assert batch.prefill_requests == [rs[6]] and len(s.active) == 6 and len(s.waiting) == 2
    # a long prompt takes the last place while it is still in portions
    s2, cache2 = make(pages=256, max_batch_requests=2, max_batch_tokens=16, max_prefill_tokens=16)
    a, b, c = req(3, max_new=50), req(30, max_new=50), req(3, max_new=50)
    for r in (a, b, c):
        s2.submit(r)
    batch, _ = run_step(s2, cache2)
    assert batch.prefill_requests == [a, b] and batch.prefill_chunk_sizes == [3, 13]
    batch, _ = run_step(s2, cache2)
    assert batch.decode_requests == [a] and batch.prefill_requests == [b] and batch.prefill_chunk_sizes == [15]
    batch, _ = run_step(s2, cache2)
    assert batch.prefill_requests == [b] and batch.prefill_chunk_sizes == [2] and len(s2.active) == 2
    batch, _ = run_step(s2, cache2)
    assert batch.decode_requests == [a, b] and batch.prefill_requests == [] and list(s2.waiting) == [c]


def test_token_budget_covers_decode_and_prefill():
    s, cache = make(max_batch_tokens=6, max_prefill_tokens=512)
    rs = [req(3, max_new=50) for _ in range(4)]
    for r in rs:
        s.submit(r)
    batch, _ = run_step(s, cache)
    assert batch.num_tokens() == 6 and batch.prefill_chunk_sizes == [3, 3]
    batch, _ = run_step(s, cache)
    assert len(batch.decode_requests) == 2 and batch.prefill_chunk_sizes == [3, 1] and batch.num_tokens() == 6


def test_finishing_by_stop_token_length_and_cancel():
    s, cache = make(stop=(99,))
    a, b, c, d = req(3, max_new=3), req(3, max_new=10), req(3, max_new=10, ignore_eos=True), req(3, max_new=10)
    for r in (a, b, c, d):
        s.submit(r)
    run_step(s, cache, token=lambda r: 99 if r in (b, c) else 5)
    assert b.phase == RequestPhase.COMPLETE and b.finish_reason == "stop" and b.output_ids == [99] and b.cache is None
    assert c.phase == RequestPhase.DECODE
    s.cancel(d)
    run_step(s, cache, token=5)
    assert d.finish_reason == "cancelled"
    run_step(s, cache, token=5)
    assert a.finish_reason == "length" and a.output_ids == [5, 5, 5]
    assert cache.num_live == 1                      # only c is left


def test_max_new_tokens_of_one():
    s, cache = make()
    a = req(5, max_new=1)
    s.submit(a)
    _, done = run_step(s, cache)
    assert done == [a] and a.finish_reason == "length" and a.output_ids == [7] and not s.has_work()
    assert cache.free_pages() == [64]


def test_request_that_can_never_fit_fails_instead_of_waiting():
    s, cache = make(pages=4, page_size=4)
    big = req(40)
    s.submit(big)
    batch = s.schedule()
    assert batch.empty() and big.phase == RequestPhase.COMPLETE and big.finish_reason == "error"
    assert "Cannot admit" in big.error and not s.has_work()


def test_admission_waits_while_others_can_free_pages():
    s, cache = make(pages=6, page_size=4)
    a, b = req(16, max_new=2), req(16, max_new=2)
    s.submit(a), s.submit(b)
    batch, _ = run_step(s, cache)
    assert batch.prefill_requests == [a]            # b does not fit beside a (4 + 4 pages > 6)
    assert b.phase == RequestPhase.WAITING and b.error is None
    run_step(s, cache)                              # a decodes and finishes by length
    assert a.finish_reason == "length"
    batch, _ = run_step(s, cache)
    assert batch.prefill_requests == [b]


def test_pages_run_out_during_decode_fail_policy():
    s, cache = make(pages=4, page_size=4, on_exhaust="fail")
    a, b = req(7, max_new=50), req(8, max_new=50)
    s.submit(a), s.submit(b)
    run_step(s, cache)                              # both prompts in: 2 + 2 pages, a has one free slot, b none
    batch, _ = run_step(s, cache)
    assert batch.decode_requests == [a]
    assert b.finish_reason == "error" and "KV cache exhausted during decode" in b.error
    assert a.phase == RequestPhase.DECODE and cache.num_live == 1


def test_pages_run_out_during_decode_preempts_the_youngest():
    s, cache = make(pages=4, page_size=4, on_exhaust="preempt")
    a, b = req(7, max_new=6), req(8, max_new=6)
    s.submit(a), s.submit(b)
    run_step(s, cache)
    batch, _ = run_step(s, cache)                   # b (the youngest) is taken off, a goes on
    assert batch.decode_requests == [a] and b.phase == RequestPhase.WAITING and b.cache is None
    assert b.stats.preemptions == 1 and s.waiting[0] is b and b.output_ids == [7]
    assert cache.free_pages() == [2]
    while a.phase != RequestPhase.COMPLETE:
        run_step(s, cache)
    # b comes back with prompt + generated as its sequence and finishes with all its tokens
    while s.has_work():
        batch, _ = run_step(s, cache)
    assert b.finish_reason == "length" and len(b.output_ids) == 6 and a.finish_reason == "length"
    assert cache.free_pages() == [4] and cache.num_live == 0


def test_the_only_request_preempts_itself_and_then_fails_for_good():
    s, cache = make(pages=2, page_size=4, on_exhaust="preempt")
    a = req(8, max_new=5)
    s.submit(a)
    run_step(s, cache)
    batch = s.schedule()                            # needs a third page: preempted, then can never fit again
    assert batch.empty() and a.finish_reason == "error" and a.stats.preemptions == 1
    assert cache.free_pages() == [2]


def test_queue_full_and_request_limit():
    s, cache = make(max_queue_size=2, max_batch_requests=1)
    s.submit(req(3)), s.submit(req(3))
    with pytest.raises(RuntimeError, match="Queue full"):
        s.submit(req(3))
    batch, _ = run_step(s, cache)
    assert len(batch.prefill_requests) == 1
    batch, _ = run_step(s, cache)
    assert len(batch.decode_requests) == 1 and batch.prefill_requests == []     # one live request at a time
    with pytest.raises(ValueError, match="at least one prompt token"):
        s.submit(InferenceRequest([]))
    with pytest.raises(ValueError, match="no room"):
        s.submit(req(256))


def test_generation_reserve_is_taken_at_admission():
    s, cache = make(pages=8, page_size=4, generation_reserve=256)
    a = req(6, max_new=9)
    s.submit(a)
    s.schedule()
    assert cache.free_pages() == [8 - 4]            # ceil((6 + 9) / 4)


def test_failed_step_fails_its_requests_and_serving_goes_on():
    s, cache = make()
    a, b = req(3), req(3)
    s.submit(a)
    batch = s.schedule()
    s.fail_batch(batch, "step failed: boom")
    assert a.finish_reason == "error" and "boom" in a.error and cache.num_live == 0
    s.submit(b)
    _, _ = run_step(s, cache)
    assert b.output_ids == [7]


def test_a_raising_stream_callback_ends_its_own_request_only():
    s, cache = make()
    seen = []

    def bad(tok):
        seen.append(tok)
        if len(seen) == 2:
            raise RuntimeError("consumer went away")
    a = InferenceRequest(list(range(1, 6)), GenerationConfig(max_new_tokens=5), stream_callback=bad)
    b = req(5, max_new=5)
    s.submit(a), s.submit(b)
    for _ in range(12):
        if not s.has_work():
            break
        run_step(s, cache)
    assert a.finish_reason == "error" and "stream callback raised" in a.error and len(a.output_ids) == 2
    assert b.finish_reason == "length" and len(b.output_ids) == 5
    cache.check()
    assert cache.num_live == 0


def test_a_preempted_request_waits_behind_the_one_in_mid_prompt():
    """Pages run out while another request is in the middle of its prompt: that request holds its pages and is the
    only one the admission looks at, so the preempted one queues behind it; both finish.  (At the very head it would
    find too few free pages with nothing running, and fail as one that can never fit.)"""
    s, cache = make(pages=8, page_size=4, max_prefill_tokens=4, max_batch_tokens=64)
    a, b = req(8, max_new=20), req(20, max_new=3)
    s.submit(a), s.submit(b)
    for _ in range(200):
        if not s.has_work():
            break
        run_step(s, cache)
    assert s.num_preemptions >= 1 and a.stats.preemptions >= 1
    assert a.finish_reason == "length" and a.error is None and len(a.output_ids) == 20
    assert b.finish_reason == "length" and len(b.output_ids) == 3
    cache.check()
    assert cache.num_live == 0


def test_random_workloads_always_finish_when_every_request_fits_alone():
    """Random prompts, limits, portion sizes and pool sizes (never smaller than the largest request needs alone):
    with preemption every request finishes with all its tokens, no page is lost, and the number of steps stays
    within what recomputation can cost."""
    import random
    rng = random.Random(4)
    for trial in range(150):
        page = rng.choice([2, 4, 8])
        n = rng.randrange(1, 10)
        prompts = [rng.randrange(1, 40) for _ in range(n)]
        news = [rng.randrange(1, 25) for _ in range(n)]
        biggest = max(-(-(p + m) // page) for p, m in zip(prompts, news))
        total = sum(-(-(p + m) // page) for p, m in zip(prompts, news))
        pages = max(biggest, int(total * rng.choice([0.3, 0.6, 1.0]))) + rng.randrange(0, 2)
        s, cache = make(pages=pages, page_size=page, max_seq_len=128, max_prefill_tokens=rng.choice([3, 8, 64]),
                        max_batch_tokens=rng.choice([16, 64]), max_batch_requests=rng.choice([2, 4, 64]))
        reqs = [req(p, max_new=m) for p, m in zip(prompts, news)]
        for r in reqs:
            s.submit(r)
        steps = 0
        while s.has_work():
            run_step(s, cache)
            steps += 1
            assert steps < 20000, (trial, "no progress")
        for r, m in zip(reqs, news):
            assert r.finish_reason == "length" and r.error is None and len(r.output_ids) == m, (trial, r.error)
        cache.check()
        assert cache.num_live == 0


def test_random_workloads_with_failures_and_cancellations_lose_no_page():
    """The reference's policy (fail the request whose decode finds no page) and requests cancelled at random moments:
    every request ends one way or another, nothing stays live, and the pool is whole."""
    import random
    rng = random.Random(11)
    for trial in range(120):
        page = rng.choice([2, 4, 8])
        n = rng.randrange(1, 10)
        prompts = [rng.randrange(1, 40) for _ in range(n)]
        news = [rng.randrange(1, 25) for _ in range(n)]
        total = sum(-(-(p + m) // page) for p, m in zip(prompts, news))
        pages = max(2, int(total * rng.choice([0.2, 0.5, 1.0])))
        s, cache = make(pages=pages, page_size=page, max_seq_len=128, max_prefill_tokens=rng.choice([3, 8, 64]),
                        max_batch_tokens=rng.choice([16, 64]), max_batch_requests=rng.choice([2, 4, 64]),
                        on_exhaust=rng.choice(["fail", "preempt"]))
        reqs = [req(p, max_new=m) for p, m in zip(prompts, news)]
        for r in reqs:
            s.submit(r)
        steps = 0
        while s.has_work():
            if rng.random() < 0.1:
                s.cancel(rng.choice(reqs))
            run_step(s, cache)
            steps += 1
            assert steps < 20000, (trial, "no progress")
        for r, m in zip(reqs, news):
            assert r.finish_reason in ("length", "error", "cancelled"), (trial, r.finish_reason)
            if r.finish_reason == "length":
                assert len(r.output_ids) == m
        cache.check()
        assert cache.num_live == 0


def test_a_prompt_longer_than_the_windowed_pool_is_admitted_and_runs_through():
    """Layers with a window have a pool of their own size (what max_batch_requests requests can hold under the step's
    token budget).  A prompt with more pages than that pool is admitted all the same: the reservation takes the
    window's group only as far as the next step reaches, and each step takes its own pages as the step function does."""
    page, window, budget = 4, 12, 8
    cache = CacheManager([(0, PagedKVNeed(1, 16, None)), (1, PagedKVNeed(1, 16, window))], page, max_requests=2,
                         max_step_tokens=budget)
    cache.set_num_pages(80)
    assert cache.groups[1].num_pages == 2 * ((window + budget + 2) // page + 1) == 12
    s = Scheduler(SchedulerConfig(kv_block_size=page, max_batch_tokens=budget, max_prefill_tokens=budget,
                                  max_batch_requests=2), cache, 256, ())
    a, b = req(100, max_new=6), req(30, max_new=3)          # 25 and 8 pages where all keys are kept
    s.submit(a), s.submit(b)
    held_most = 0
    for _ in range(200):
        batch = s.schedule()
        if batch.empty():
            break
        for r in batch.decode_requests:                     # what EngineCore.prepare and step do
            cache.ensure(r.cache, r.cache.length + 1)
            cache.commit(r.cache, r.cache.length + 1)
        for r, size in zip(batch.prefill_requests, batch.prefill_chunk_sizes):
            assert size <= budget
            cache.ensure(r.cache, r.cache.length + size)
            cache.commit(r.cache, r.cache.length + size)
        s.process_results(batch, [7] * len(batch.rows_wanted()))
        cache.check()
        held_most = max(held_most, cache.groups[1].pool.num_used)
    assert a.phase == b.phase == RequestPhase.COMPLETE and a.finish_reason == b.finish_reason == "length"
    assert len(a.output_ids) == 6 and len(b.output_ids) == 3 and s.num_preemptions == 0
    assert 0 < held_most <= 12 and cache.free_pages() == [80, 12]


# ---- the sampler's record of the table of generated tokens (host side only; the kernels are stood in for) -------
def test_the_samplers_record_of_the_generated_tokens_table(monkeypatch):
    """Which slot a request's table is in, when the host sends tokens up (a request that comes back after its slot was
    given away) and when it cannot answer (no table kept; the table behind while tokens are still on their way)."""
    import torch
    from zedinfer_b200 import ops
    from zedinfer_b200.sampling.sampler import Sampler

    class FakeRc:
        def __init__(self, slot, serial):
            self.slot, self.serial = slot, serial

    class FakeCache:
        def __init__(self):
            self.rcs = {}

        def get(self, rid):
            return self.rcs.get(rid)

    class FakeCore:
        def __init__(self, vocab):
            self.generated_counts = torch.zeros(4, vocab, dtype=torch.int32)
            self.cache = FakeCache()

    added = []

    def count_token_list(row, tokens):
        added.append(tokens.tolist())
        for t in tokens.tolist():
            row[t] += 1
    monkeypatch.setattr(ops, "count_token_list", count_token_list)
    core = FakeCore(50)
    sampler = Sampler(torch.device("cpu"), core)
    r = req(3, use_argmax=False, temperature=0.8, repetition_penalty=1.3, seed=5)
    greedy = req(3)
    plain = req(3, use_argmax=False, temperature=0.8, seed=5)
    core.cache.rcs[r.request_id] = FakeRc(slot=2, serial=11)
    assert sampler._count_slot(greedy, 0) == -1 and sampler._count_slot(plain, 0) == -1
    assert sampler._count_slot(r, 0) == 2 and (r.count_serial, r.counted) == (11, 0) and added == []
    sampler.counted([r, greedy, plain])                  # the step chose a token for each; only r keeps a table
    assert r.counted == 1 and greedy.counted == 0 and plain.counted == 0
    assert sampler._count_slot(r, 1) == 2                # a step launched ahead: one token chosen, none read yet
    r.output_ids.append(7)
    assert sampler._count_slot(r, 0) == 2 and added == []
    par, ints = sampler.params([greedy, r, plain])
    assert ints.tolist() == [[0, 0, 0], [-1, 2, -1]] and par[3].tolist() == [1.0, pytest.approx(1.3), 1.0]
    assert par[0].tolist() == [0.0, pytest.approx(0.8), pytest.approx(0.8)]
    # the table is behind while a token is still on its way: no answer, the caller takes the ordinary path
    assert sampler._count_slot(r, 2) is None and sampler.params([r], ahead=2) is None
    # taken off the GPU and back in another slot, zeroed: the host sends what was generated so far
    sampler.counted([r])
    r.output_ids.extend([9, 7])
    core.cache.rcs[r.request_id] = FakeRc(slot=0, serial=12)
    assert sampler._count_slot(r, 0) == 0 and added == [[7, 9, 7]] and (r.count_serial, r.counted) == (12, 3)
    assert core.generated_counts[0, 7] == 2 and core.generated_counts[0, 9] == 1 and int(core.generated_counts.sum()) == 3
    # no table kept: a penalised request cannot be answered, the others can
    bare = Sampler(torch.device("cpu"))
    assert bare._count_slot(r, 0) is None and bare._count_slot(plain, 0) == -1 and bare.params([r]) is None
    assert bare.params([plain, greedy])[1].tolist() == [[0, 0], [-1, -1]]
