"""The scheduler's decisions (no GPU): a fake step function stands in for the model."""
import random

import pytest

from sglang_rs_b200.cache import CacheManager
from sglang_rs_b200.engine.scheduler import Request, Scheduler, SchedulerConfig
from sglang_rs_b200.parts import PagedKV
from sglang_rs_b200.sampling import SamplingParams

FULL = ("kv", None)


def next_token(tokens):
    """A deterministic stand-in for the model: the next token depends on all tokens so far."""
    return (sum((i + 1) * t for i, t in enumerate(tokens)) * 31 + len(tokens)) % 97


def make(max_tokens=64, page_size=4, budget=16, max_running=4, stops=(), max_positions=1000, needs=None):
    cache = CacheManager(needs or [PagedKV(2, 16)], page_size=page_size, max_tokens=max_tokens,
                         max_requests=max_running, device=None)
    return Scheduler(cache, SchedulerConfig(max_running, budget, max_positions, stops)), cache


def run_step(scheduler, cache, log=None):
    """What the engine does around the scheduler, with the model faked."""
    entries = scheduler.schedule()
    sampled = []
    for entry in entries:
        handle = entry.request.handle
        assert entry.tokens == entry.request.tokens[handle.length:handle.length + len(entry.tokens)]
        cache.reserve(handle, len(entry.tokens))            # already reserved: must take nothing more
        cache.commit(handle, len(entry.tokens))
        if entry.samples:
            sampled.append(next_token(entry.request.tokens))
    if log is not None:
        log.append([(e.request.request_id, len(e.tokens), e.samples) for e in entries])
    outputs = scheduler.process_outputs(entries, sampled)
    cache.check_invariants()
    return entries, outputs


def drain(scheduler, cache, limit=10_000, log=None):
    steps = 0
    while scheduler.has_work:
        run_step(scheduler, cache, log)
        steps += 1
        assert steps < limit, "the scheduler does not make progress"
    return steps


def expected_output(prompt, n, stops=()):
    tokens, out = list(prompt), []
    for _ in range(n):
        t = next_token(tokens)
        tokens.append(t)
        out.append(t)
        if t in stops:
            break
    return out


def request(rid, prompt, **sampling):
    sampling.setdefault("max_new_tokens", 5)
    return Request(rid, list(prompt), SamplingParams(**sampling))


def test_fifo_admission_budget_cut_and_decode_rows_first():
    scheduler, cache = make(max_tokens=256, budget=16)
    a, b, c = request("a", range(10)), request("b", range(20, 40)), request("c", range(3))
    for r in (a, b, c):
        scheduler.add_request(r)
    log = []
    run_step(scheduler, cache, log)
    assert log[-1] == [("a", 10, True), ("b", 6, False)]          # budget 16: b is cut, c waits
    run_step(scheduler, cache, log)
    assert log[-1] == [("a", 1, True), ("b", 14, True), ("c", 1, False)]   # a decoded token beside portions
    run_step(scheduler, cache, log)
    assert log[-1] == [("a", 1, True), ("b", 1, True), ("c", 2, True)]
    drain(scheduler, cache)
    for r in (a, b, c):
        assert r.finished and r.finish_reason == "length" and r.output_ids == expected_output(r.prompt, 5)
    assert cache.free_pages()[FULL] == 64 and not cache.live


def test_running_limit_keeps_requests_waiting():
    scheduler, cache = make(max_tokens=256, max_running=2, budget=100)
    for i in range(4):
        scheduler.add_request(request(i, range(5), max_new_tokens=3))
    entries, _ = run_step(scheduler, cache)
    assert [e.request.request_id for e in entries] == [0, 1] and len(scheduler.waiting) == 2
    drain(scheduler, cache)
    assert cache.state_pool.free_count == 2


def test_finish_reasons():
    prompt = [1, 2, 3]
    stop = expected_output(prompt, 3)[2]
    scheduler, cache = make(stops=(stop,))
    r1, r2 = request("stop", prompt, max_new_tokens=9), request("ignore", prompt, max_new_tokens=4, ignore_eos=True)
    r3 = request("own-stop", [5, 6], max_new_tokens=9, stop_token_ids=(expected_output([5, 6], 1)[0],))
    for r in (r1, r2, r3):
        scheduler.add_request(r)
    drain(scheduler, cache)
    assert r1.finish_reason == "stop" and r1.output_ids == expected_output(prompt, 3)     # the stop token stays
    assert r2.finish_reason == "length" and len(r2.output_ids) == 4
    assert r3.finish_reason == "stop" and len(r3.output_ids) == 1
    scheduler, cache = make(max_positions=8)
    r4 = request("ctx", range(5), max_new_tokens=50)
    scheduler.add_request(r4)
    drain(scheduler, cache)
    assert r4.finish_reason == "context" and len(r4.tokens) == 8


def test_preemption_when_decoding_runs_out_of_pages():
    # 8 pages of 4 tokens: two requests of 12 + growth cannot both finish
    scheduler, cache = make(max_tokens=32, budget=64)
    old, young = request("old", range(12), max_new_tokens=12), request("young", range(50, 62), max_new_tokens=12)
    scheduler.add_request(old)
    scheduler.add_request(young)
    log = []
    drain(scheduler, cache, log=log)
    assert scheduler.stats["preemptions"] >= 1 and young.preemptions >= 1 and old.preemptions == 0
    # tokens kept, recomputed, and the outputs are what they would have been anyway
    assert old.output_ids == expected_output(old.prompt, 12)
    assert young.output_ids == expected_output(young.prompt, 12)
    assert old.finish_reason == young.finish_reason == "length"
    # after the preemption the young request's tokens (prompt and output so far) were computed again
    computed = sum(e[1] for step in log for e in step if e[0] == "young")
    assert computed > len(young.tokens), log
    assert cache.free_pages()[FULL] == 8


def test_a_portion_is_cut_to_the_free_pages_and_a_starved_request_waits():
    scheduler, cache = make(max_tokens=32, budget=20, max_running=4)    # 8 pages
    a, b = request("a", range(26), max_new_tokens=2), request("b", range(30, 56), max_new_tokens=2)
    scheduler.add_request(a)
    scheduler.add_request(b)
    log = []
    run_step(scheduler, cache, log)
    run_step(scheduler, cache, log)
    assert log == [[("a", 20, False)], [("a", 6, True), ("b", 4, False)]]      # b gets the one page left
    run_step(scheduler, cache, log)
    assert log[-1] == [("a", 1, True)]                                    # no page for b: it waits
    drain(scheduler, cache)
    assert a.output_ids == expected_output(a.prompt, 2) and b.output_ids == expected_output(b.prompt, 2)
    assert b.preemptions == 0


def test_running_requests_that_all_starve_are_resolved_by_preemption():
    scheduler, cache = make(max_tokens=32, budget=20, max_running=4)
    a, b = request("a", range(20), max_new_tokens=2), request("b", range(30, 50), max_new_tokens=2)
    scheduler.add_request(a)
    scheduler.add_request(b)
    # force the state by hand: both in the middle of their prompts, all pages taken
    a.handle, b.handle = cache.open("a"), cache.open("b")
    for r, stamp in ((a, -3), (b, -2)):
        cache.reserve(r.handle, 16); cache.commit(r.handle, 16)
        scheduler._force_running(r, r.handle, stamp)
    assert cache.free_pages()[FULL] == 0
    drain(scheduler, cache)
    assert b.preemptions >= 1 and a.preemptions == 0
    assert a.output_ids == expected_output(a.prompt, 2) and b.output_ids == expected_output(b.prompt, 2)


def test_request_that_can_never_fit_fails_alone():
    scheduler, cache = make(max_tokens=16, budget=64)
    big, small = request("big", range(40)), request("small", range(4), max_new_tokens=3)
    scheduler.add_request(big)
    scheduler.add_request(small)
    _, outputs = run_step(scheduler, cache)
    failed = [o for o in outputs if o.request_id == "big"]
    assert failed and failed[0].finished and failed[0].finish_reason == "cache_full"
    drain(scheduler, cache)
    assert small.output_ids == expected_output(small.prompt, 3)
    # one that fits at first but outgrows the whole pool while decoding
    scheduler, cache = make(max_tokens=16, budget=64)
    grow = request("grow", range(10), max_new_tokens=50)
    scheduler.add_request(grow)
    drain(scheduler, cache)
    assert grow.finish_reason == "cache_full" and len(grow.tokens) == 16 + 1
    assert cache.free_pages()[FULL] == 4


def test_abort_and_failed_step_give_pages_back():
    scheduler, cache = make(max_tokens=64, budget=8)
    a, b = request("a", range(20)), request("b", range(6))
    scheduler.add_request(a)
    scheduler.add_request(b)
    run_step(scheduler, cache)
    assert cache.free_pages()[FULL] < 16
    assert scheduler.abort("a") and not scheduler.abort("nobody")
    assert scheduler.abort("b")                                        # still waiting
    assert cache.free_pages()[FULL] == 16 and not scheduler.has_work
    _, outputs = run_step(scheduler, cache)
    assert sorted(o.request_id for o in outputs) == ["a", "b"] and all(o.finish_reason == "abort" for o in outputs)
    c = request("c", range(9))
    scheduler.add_request(c)
    entries = scheduler.schedule()
    scheduler.step_failed(entries)                                     # the model raised
    assert cache.free_pages()[FULL] == 16 and c.finished and not scheduler.has_work
    cache.check_invariants()


def test_duplicate_and_empty_requests_are_refused():
    scheduler, _ = make()
    scheduler.add_request(request("a", [1]))
    with pytest.raises(ValueError, match="queued already"):
        scheduler.add_request(request("a", [2]))
    with pytest.raises(ValueError, match="empty prompt"):
        scheduler.add_request(request("b", []))


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_with_the_right_tokens(seed):
    rng = random.Random(seed)
    needs = [PagedKV(2, 16), PagedKV(2, 16, window=9)] if seed % 2 else None
    scheduler, cache = make(max_tokens=rng.choice([48, 80, 160]), page_size=rng.choice([2, 4, 8]),
                            budget=rng.choice([5, 16, 33]), max_running=rng.choice([2, 3, 6]), needs=needs)
    requests = []
    arrivals = sorted(rng.randrange(60) for _ in range(14))
    step = 0
    while arrivals or scheduler.has_work:
        while arrivals and arrivals[0] <= step:
            arrivals.pop(0)
            r = request(len(requests), [rng.randrange(97) for _ in range(rng.randrange(1, 30))],
                        max_new_tokens=rng.randrange(1, 12))
            requests.append(r)
            scheduler.add_request(r)
        run_step(scheduler, cache)
        step += 1
        assert step < 5000
    for r in requests:
        assert r.finished and r.finish_reason == "length"
        assert r.output_ids == expected_output(r.prompt, r.sampling.max_new_tokens)
    assert all(a.free_count == a.num_pages for a in cache.allocators.values())


# ------------------------------------------------------------------------------ steps that run ahead
class FakeOverlappedEngine:
    """The engine's overlapped loop with the model faked: a step is 'launched' (pages reserved and
    committed, tokens computed but withheld), and its tokens reach the scheduler one call later."""

    def __init__(self, scheduler, cache):
        self.scheduler, self.cache = scheduler, cache
        self.in_flight = None
        self.ran_ahead = 0
        self.rows_in_vain = 0

    def launch(self, ahead):
        entries = self.scheduler.schedule(ahead=ahead)
        if not entries:
            return None
        before = {id(e.request): t for e, t in self.in_flight} if ahead else {}
        tokens = []
        for entry in entries:
            handle = entry.request.handle
            if entry.from_device:
                assert ahead and entry.tokens == [-1] and entry.request.pending == 1
                known = entry.request.tokens + [before[id(entry.request)]]      # what the device holds
            else:
                assert -1 not in entry.tokens
                known = entry.request.tokens[:handle.length + len(entry.tokens)]
            self.cache.reserve(handle, len(entry.tokens))
            self.cache.commit(handle, len(entry.tokens))
            tokens.append(next_token(known) if entry.samples else None)
        for entry in entries:
            if entry.samples:
                self.scheduler.mark_pending(entry.request)
        return list(zip(entries, tokens))

    def step(self):
        launched = None
        if self.in_flight is not None:
            running = len(self.scheduler.running)
            if all(free >= running for free in self.cache.free_pages().values()):
                launched = self.launch(ahead=True)
                self.ran_ahead += launched is not None
        outputs = []
        if self.in_flight is not None:
            entries = [e for e, _ in self.in_flight]
            outputs = self.scheduler.process_outputs(entries, [t for _, t in self.in_flight if t is not None])
            self.in_flight = None
        if launched is None:
            launched = self.launch(ahead=False)
        else:
            self.rows_in_vain += sum(e.request.finished for e, _ in launched)
        self.in_flight = launched
        self.cache.check_invariants()
        return outputs


@pytest.mark.parametrize("seed", range(6))
def test_steps_that_run_ahead_give_the_same_tokens(seed):
    """Requests of random lengths arrive over time; some stop on a stop token, so the step that ran
    ahead computed a row in vain; pools are small, so some steps cannot run ahead and some requests
    are preempted.  Every request ends with the tokens of the plain loop, and no page is lost."""
    rng = random.Random(100 + seed)
    stops = (5, 17, 60)
    scheduler, cache = make(max_tokens=rng.choice([64, 96, 200]), page_size=rng.choice([2, 4, 8]),
                            budget=rng.choice([7, 16, 33]), max_running=rng.choice([2, 4, 6]), stops=stops)
    engine = FakeOverlappedEngine(scheduler, cache)
    requests, got = [], {}
    arrivals = sorted(rng.randrange(50) for _ in range(16))
    step = 0
    while arrivals or scheduler.has_work or engine.in_flight is not None:
        while arrivals and arrivals[0] <= step:
            arrivals.pop(0)
            r = request(len(requests), [rng.randrange(97) for _ in range(rng.randrange(1, 28))],
                        max_new_tokens=rng.randrange(1, 14), ignore_eos=rng.random() < 0.3)
            requests.append(r)
            scheduler.add_request(r)
        for output in engine.step():
            got.setdefault(output.request_id, []).extend(output.token_ids)
        step += 1
        assert step < 5000
    for r in requests:
        want = expected_output(r.prompt, r.sampling.max_new_tokens, () if r.sampling.ignore_eos else stops)
        assert r.finished and r.output_ids == want and got.get(r.request_id, []) == want and r.pending == 0
        assert r.finish_reason == ("stop" if want[-1] in stops and not r.sampling.ignore_eos else "length")
    assert engine.ran_ahead > 0
    assert all(a.free_count == a.num_pages for a in cache.allocators.values())


def test_a_request_whose_pending_token_is_its_last_is_not_scheduled_ahead():
    scheduler, cache = make(max_tokens=128)
    engine = FakeOverlappedEngine(scheduler, cache)
    a, b = request("a", range(6), max_new_tokens=2), request("b", range(9), max_new_tokens=4)
    scheduler.add_request(a)
    scheduler.add_request(b)
    engine.step()                                            # both prompts; first tokens pending
    assert a.pending == b.pending == 1 and not a.output_ids
    engine.step()                                            # runs ahead: second token of each, the first arrives
    assert [e.request.request_id for e, _ in engine.in_flight] == ["a", "b"]
    assert len(a.output_ids) == 1 and a.pending == 1
    engine.step()                                            # a's pending token is its last whatever it is: only b
    assert [e.request.request_id for e, _ in engine.in_flight] == ["b"]
    while scheduler.has_work or engine.in_flight is not None:
        engine.step()
    assert a.output_ids == expected_output(a.prompt, 2) and b.output_ids == expected_output(b.prompt, 4)
    assert engine.rows_in_vain == 0


def test_a_failed_drain_after_a_run_ahead_launch_fails_both_steps():
    """The engine's own overlapped loop (``Engine._step_overlapped``) with launch and drain faked: the
    step before fails on the device after the next step was launched from its tokens.  The requests of
    both steps end as failed, nothing stays running or pending, no page is lost, and the loop of
    ``generate`` would stop."""
    from types import SimpleNamespace
    from sglang_rs_b200.engine.engine import Engine
    scheduler, cache = make(max_tokens=128)
    fake = FakeOverlappedEngine(scheduler, cache)
    engine = Engine.__new__(Engine)
    engine.scheduler, engine.cache, engine._in_flight = scheduler, cache, None
    engine._may_run_ahead = lambda: True

    def launch(before):
        fake.in_flight = None if before is None else before.pairs
        pairs = fake.launch(ahead=before is not None)
        return None if pairs is None else SimpleNamespace(entries=[e for e, _ in pairs], pairs=pairs)

    def drain():
        flight, engine._in_flight = engine._in_flight, None
        if flight is None:
            return []
        if fail["now"]:
            scheduler.step_failed(flight.entries)
            raise RuntimeError("device-side check failed")
        return scheduler.process_outputs(flight.entries, [t for _, t in flight.pairs if t is not None])
    engine._launch, engine.drain = launch, drain
    fail = {"now": False}
    a, b = request("a", range(6), max_new_tokens=8), request("b", range(9), max_new_tokens=8)
    scheduler.add_request(a)
    scheduler.add_request(b)
    engine._step_overlapped()                                # prompts launched
    engine._step_overlapped()                                # a step runs ahead, the prompts' tokens arrive
    assert a.pending == 1 and len(a.output_ids) == 1
    c = request("c", range(5), max_new_tokens=8)             # arrives now: only the step that runs ahead holds it
    scheduler.add_request(c)
    fail["now"] = True
    with pytest.raises(RuntimeError, match="device-side"):
        engine._step_overlapped()                            # launches ahead, then the step before fails
    assert engine._in_flight is None and not scheduler.has_work
    assert a.finished and b.finished and c.finished
    assert a.finish_reason == b.finish_reason == c.finish_reason == "abort"
    assert all(alloc.free_count == alloc.num_pages for alloc in cache.allocators.values())
    cache.check_invariants()


def test_decode_split_counts_follow_the_shape_only():
    """How many blocks share the keys of a (row, kv head) in the decode attention: a function of
    rows, kv heads and the longest row; within the bound that sizes the scratch memory."""
    from sglang_rs_b200 import ops
    assert ops.decode_splits(64, 8, 2100, sms=148) == 3           # 512 blocks would be 1.15 waves of 444
    assert ops.decode_splits(8, 8, 2100, sms=148) == 6            # 384 blocks: one wave
    assert ops.decode_splits(1, 8, 2100, sms=148) == 7            # five units each, merged inside a cluster
    assert ops.decode_splits(1, 8, 40, sms=148) == 1
    for rows in (1, 3, 8, 64, 200):
        for n_kv in (1, 2, 8, 32):
            for keys in (1, 64, 65, 1000, 5000, 40000):
                splits = ops.decode_splits(rows, n_kv, keys, sms=148)
                assert 1 <= splits <= ops.decode_splits_bound(keys) <= ops.DECODE_MAX_SPLITS
                assert splits == ops.decode_splits(rows, n_kv, keys, sms=148)
