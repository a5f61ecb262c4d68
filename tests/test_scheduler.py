"""The scheduler's decisions, with exact integer arithmetic instead of a model
(in the manner of the reference's fake models,
pulsarlm-core/tests/runtime/test_scheduler.cpp:306ff): the "next token" of a
request is a function of every token it has been fed, so a wrong portion, a lost
token or a wrong order changes the output."""

import torch

from pulsarlm_b200.cache.manager import CacheManager
from pulsarlm_b200.engine.scheduler import Request, Scheduler
from pulsarlm_b200.parts.spec import KVCacheNeed
from pulsarlm_b200.sampling.params import SamplingParams

VOCAB = 97


def next_token(history):
    return (sum((i + 1) * t for i, t in enumerate(history)) + 7) % VOCAB


def expected_output(prompt, n, stop=()):
    seq, out = list(prompt), []
    for _ in range(n):
        t = next_token(seq)
        out.append(t)
        seq.append(t)
        if t in stop:
            break
    return out


class FakeStepper:
    """Stands in for the GPU: checks that each entry continues its request where the
    cache says it is, and 'samples' the next token from the fed history."""

    def __init__(self, cache):
        self.cache = cache
        self.fed = {}
        self.steps = []

    def run(self, entries):
        sampled = {}
        self.steps.append([(e.request.id, len(e.tokens), e.samples) for e in entries])
        for e in entries:
            rid = e.request.id
            start = self.cache.length(rid)
            history = self.fed.setdefault(rid, [])
            if start == 0:
                history.clear()  # admitted anew (first time, or after preemption)
            assert len(history) == start, "tokens fed do not match the cached length"
            history.extend(e.tokens)
            self.cache.commit(rid, start + len(e.tokens))
            if e.samples:
                sampled[rid] = next_token(history)
        return sampled


def make(pages=64, page=4, slots=8, budget=16, stop=()):
    cache = CacheManager([KVCacheNeed(1, 4)], page, pages, slots, torch.float32, None, allocate=False)
    return cache, Scheduler(cache, stop, prefill_tokens_per_step=budget), FakeStepper(cache)


def drive(sched, stepper, limit=10000):
    ended = []
    for _ in range(limit):
        if not sched.has_work():
            return ended
        entries, gone = sched.plan()
        ended += gone
        if entries:
            ended += sched.finish_step(entries, stepper.run(entries))
    raise AssertionError("the scheduler did not finish")


def test_prompt_is_cut_under_the_budget_then_decodes():
    cache, sched, stepper = make(budget=16)
    r = Request("a", list(range(1, 41)), SamplingParams(), max_tokens=3)
    sched.add(r)
    drive(sched, stepper)
    assert stepper.steps == [[("a", 16, False)], [("a", 16, False)], [("a", 8, True)], [("a", 1, True)],
                             [("a", 1, True)]]
    assert r.output == expected_output(r.prompt, 3) and r.finish_reason == "length"
    assert not cache.open_requests() and cache.free_pages() == 64


def test_decodes_run_beside_prompt_portions_and_do_not_use_the_budget():
    cache, sched, stepper = make(budget=8)
    a = Request("a", [5, 6, 7], max_tokens=6)
    b = Request("b", list(range(1, 21)), max_tokens=2)
    sched.add(a)
    drive_one = lambda: sched.finish_step(*(lambda e: (e, stepper.run(e)))(sched.plan()[0]))  # noqa: E731
    drive_one()
    sched.add(b)
    drive(sched, stepper)
    assert stepper.steps[1] == [("a", 1, True), ("b", 8, False)]
    assert stepper.steps[2] == [("a", 1, True), ("b", 8, False)]
    assert stepper.steps[3] == [("a", 1, True), ("b", 4, True)]
    assert a.output == expected_output(a.prompt, 6) and b.output == expected_output(b.prompt, 2)


def test_budget_is_shared_in_admission_order():
    cache, sched, stepper = make(budget=10)
    for name, n in (("a", 6), ("b", 6), ("c", 6)):
        sched.add(Request(name, list(range(1, n + 1)), max_tokens=1))
    drive(sched, stepper)
    assert stepper.steps[0] == [("a", 6, True), ("b", 4, False)]
    assert stepper.steps[1] == [("b", 2, True), ("c", 6, True)]


def test_stop_token_ends_a_request_and_is_emitted():
    prompt = [3, 1, 4, 1, 5]
    full = expected_output(prompt, 10)
    cache, sched, stepper = make(stop=(full[3],))
    r = Request("a", prompt, max_tokens=10)
    sched.add(r)
    drive(sched, stepper)
    first = full.index(full[3])
    assert r.output == full[: first + 1] and r.finish_reason == "stop"
    cache2, sched2, stepper2 = make(stop=(full[3],))
    r2 = Request("a", prompt, max_tokens=10, ignore_eos=True)
    sched2.add(r2)
    drive(sched2, stepper2)
    assert r2.output == full and r2.finish_reason == "length"


def test_max_tokens_zero_runs_the_prompt_and_ends():
    cache, sched, stepper = make()
    r = Request("a", [1, 2, 3], max_tokens=0)
    sched.add(r)
    drive(sched, stepper)
    assert r.output == [] and r.finish_reason == "length" and stepper.steps == [[("a", 3, True)]]


def test_cancel_frees_at_the_next_plan():
    cache, sched, stepper = make()
    a, b = Request("a", [1, 2, 3], max_tokens=50), Request("b", [4, 5], max_tokens=50)
    sched.add(a)
    sched.add(b)
    entries, _ = sched.plan()
    sched.finish_step(entries, stepper.run(entries))
    a.cancel()
    entries, ended = sched.plan()
    assert ended == [a] and a.finish_reason == "cancelled" and [e.request.id for e in entries] == ["b"]
    assert cache.open_requests() == ["b"]


def test_waits_for_a_slot():
    cache, sched, stepper = make(slots=2)
    reqs = [Request(n, [i + 1, i + 2], max_tokens=2) for i, n in enumerate("abc")]
    for r in reqs:
        sched.add(r)
    drive(sched, stepper)
    assert [rid for rid, _, _ in stepper.steps[0]] == ["a", "b"]
    assert all(r.output == expected_output(r.prompt, 2) for r in reqs)


def test_out_of_pages_preempts_the_newest_and_recomputes_it():
    # 6 pages of 4 tokens. a and b each grow to 16 tokens = 4 pages: they cannot both.
    cache, sched, stepper = make(pages=6, page=4, budget=16)
    a = Request("a", [1, 2, 3, 4, 5, 6], max_tokens=10)
    b = Request("b", [9, 8, 7, 6, 5, 4], max_tokens=10)
    sched.add(a)
    sched.add(b)
    drive(sched, stepper)
    assert a.output == expected_output(a.prompt, 10) and b.output == expected_output(b.prompt, 10)
    assert sched.preemptions >= 1 and b.preemptions >= 1 and a.preemptions == 0
    # after preemption b's whole history (prompt + generated) was fed again as a prompt
    refeeds = [s for s in stepper.steps if any(rid == "b" and n > 6 for rid, n, _ in s)]
    assert refeeds
    assert not cache.open_requests() and cache.free_pages() == 6


def test_a_request_too_large_for_the_pool_ends_with_oom_and_others_go_on():
    cache, sched, stepper = make(pages=4, page=4, budget=64)
    big = Request("big", list(range(1, 30)), max_tokens=2)  # 29 tokens > 16
    small = Request("small", [1, 2, 3], max_tokens=2)
    sched.add(big)
    sched.add(small)
    ended = drive(sched, stepper)
    assert big.finish_reason == "oom" and big.output == []
    assert small.output == expected_output(small.prompt, 2)
    assert big in ended and cache.free_pages() == 4


def test_growing_alone_past_the_pool_ends_with_oom():
    cache, sched, stepper = make(pages=2, page=4)
    r = Request("a", [1, 2, 3], max_tokens=50)
    sched.add(r)
    drive(sched, stepper)
    assert r.finish_reason == "oom" and r.output == expected_output(r.prompt, 6)[: len(r.output)]
    assert len(r.prompt) + len(r.output) - 1 <= 8 and cache.free_pages() == 2


def test_many_requests_under_page_pressure_all_finish_right():
    import random

    rng = random.Random(3)
    cache, sched, stepper = make(pages=12, page=4, slots=4, budget=8)
    reqs = [Request(i, [rng.randrange(VOCAB) for _ in range(rng.randrange(1, 20))], max_tokens=rng.randrange(1, 12))
            for i in range(12)]
    for r in reqs:
        sched.add(r)
    drive(sched, stepper)
    for r in reqs:
        assert r.output == expected_output(r.prompt, r.max_tokens), r.id
    assert cache.free_pages() == 12


def test_more_requests_than_any_fixed_buffer_can_end_in_one_plan():
    """A queue far longer than the slots, cancelled all at once: one plan ends every
    request (its buffers grow with the number of known requests), and the few that
    ran give back what they held."""
    cache, sched, stepper = make(pages=64, slots=2)
    requests = [Request(i, [1 + i % 5, 2, 3], max_tokens=4) for i in range(700)]
    for r in requests:
        sched.add(r)
    entries, gone = sched.plan()
    assert len(entries) == 2 and not gone
    sched.finish_step(entries, stepper.run(entries))
    for r in requests:
        r.cancel()
    entries, gone = sched.plan()
    assert not entries and len(gone) == 700 and all(r.finish_reason == "cancelled" for r in requests)
    assert not sched.has_work() and cache.free_pages() == 64 and cache.stats()["slots_used"] == 0


# ---------------------------------------------------------------- steps planned while the one before runs

def drive_pipelined(sched, stepper, limit=10000, cancel_at=None):
    """As the engine with lookahead: plan and launch the next step, then settle the one before."""
    from pulsarlm_b200.engine.scheduler import FROM_DEVICE

    ended, flight, device = [], None, {}
    for step in range(limit):
        if not sched.has_work() and flight is None:
            return ended
        if cancel_at and step in cancel_at:
            cancel_at[step].cancel()
        entries, gone = sched.plan()
        ended += gone
        launched = None
        if entries:
            for e in entries:
                if e.tokens == [FROM_DEVICE]:
                    e.tokens = [device[e.request.id]]  # what the device holds: the id the earlier step drew
            epochs = {e.request.id: e.request.preemptions for e in entries}
            sampled = stepper.run(entries)
            device.update(sampled)
            sched.advance(entries)
            launched = (entries, sampled, epochs)
        if flight is not None:
            ended += sched.settle(*flight)
        flight = launched
    raise AssertionError("the scheduler did not finish")


def test_the_next_step_is_planned_while_one_runs():
    from pulsarlm_b200.engine.scheduler import FROM_DEVICE

    cache, sched, stepper = make(budget=8)
    a = Request("a", list(range(1, 20)), max_tokens=2)   # 19 tokens: portions of 8, 8, 3
    b = Request("b", [5, 6], max_tokens=1)
    sched.add(a)
    first, _ = sched.plan()
    assert [(e.request.id, len(e.tokens), e.samples) for e in first] == [("a", 8, False)]
    stepper.run(first)
    sched.advance(first)
    sched.add(b)
    second, _ = sched.plan()  # the first step is not settled: the prompt goes on where it will stand
    assert [(e.request.id, e.tokens, e.samples) for e in second] == [("a", list(range(9, 17)), False)]
    assert sched.settle(first, {}) == []
    stepper.run(second)
    sched.advance(second)
    third, _ = sched.plan()
    assert [(e.request.id, len(e.tokens), e.samples) for e in third] == [("a", 3, True), ("b", 2, True)]
    sampled = stepper.run(third)
    sched.advance(third)
    # a goes on with the token being drawn; b is drawing its only token and is not planned again
    fourth, _ = sched.plan()
    assert [(e.request.id, e.tokens, e.samples) for e in fourth] == [("a", [FROM_DEVICE], True)] and a.draw_count == 1
    fourth[0].tokens = [sampled["a"]]
    later = stepper.run(fourth)
    sched.advance(fourth)
    assert sched.plan() == ([], [])  # a's second token is its last
    assert [r.id for r in sched.settle(third, sampled)] == ["b"] and a.output == [sampled["a"]]
    assert [r.id for r in sched.settle(fourth, later)] == ["a"]
    assert a.output == expected_output(a.prompt, 2) and b.output == expected_output(b.prompt, 1)
    assert not sched.has_work() and cache.free_pages() == 64


def test_a_stop_token_drops_what_the_step_after_computed():
    prompt = [3, 4, 5]
    want = expected_output(prompt, 6)
    cache, sched, stepper = make(stop=[want[2]])
    r = Request("r", prompt, max_tokens=6)
    sched.add(r)
    drive_pipelined(sched, stepper)
    assert r.output == want[:3] and r.finish_reason == "stop"
    assert len(stepper.fed["r"]) == len(prompt) + 3  # one token more than needed was run, and dropped
    assert cache.free_pages() == 64 and cache.stats()["slots_used"] == 0


def test_pipelined_steps_under_page_pressure_give_the_same_tokens():
    import random

    preemptions = 0
    for seed in range(8):
        rng = random.Random(seed)
        stop = [rng.randrange(VOCAB) for _ in range(3)]
        cache, sched, stepper = make(pages=rng.choice([8, 10, 12, 20]), page=4, slots=rng.choice([2, 4]), budget=8,
                                     stop=stop)
        reqs = [Request(i, [rng.randrange(VOCAB) for _ in range(rng.randrange(1, 20))],
                        max_tokens=rng.randrange(0, 12), ignore_eos=rng.random() < 0.3) for i in range(14)]
        for r in reqs:
            sched.add(r)
        cancelled = reqs[rng.randrange(len(reqs))]
        drive_pipelined(sched, stepper, cancel_at={rng.randrange(3, 30): cancelled})
        for r in reqs:
            want = expected_output(r.prompt, r.max_tokens, () if r.ignore_eos else stop)
            if r is cancelled and r.finish_reason == "cancelled":
                assert r.output == want[: len(r.output)]
            else:
                assert r.output == want and r.finish_reason in ("stop", "length"), (seed, r.id)
        assert cache.free_pages() == cache.n_pages and cache.stats()["slots_used"] == 0
        preemptions += sched.preemptions
    assert preemptions > 0
