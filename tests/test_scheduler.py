"""The scheduler's decisions, on the host alone: a fake engine gives it tokens.

Policy under test (after src/scheduler/prefill.rs:163-293 and
src/scheduler/scheduler.rs:225-274, :570-578 of the reference): arrival order,
a budget of prompt tokens per step, continuation first, one token per decoding
request per step, finishing on an end id / max_tokens / max_seq_len, and, when
pages run out, waiting at the head of the queue while nothing that runs is
disturbed.
"""
import pytest

from llm_infer_rust_b200.kernels.build import load_host_runtime

rt = load_host_runtime()


def make(pages=64, page_size=4, max_running=8, max_seq=64, budget=16, eos=(), window=0, slots=None):
    groups = [rt.GroupSpec(page_size, pages, 0)]
    if window:
        groups.append(rt.GroupSpec(page_size, pages, window))
    cache = rt.CacheManager(groups, slots or max_running)
    sched = rt.Scheduler(cache, rt.SchedulerOptions(max_running, max_seq, budget), list(eos))
    return cache, sched


def params(max_tokens=4, ignore_eos=False, temperature=0.0):
    return rt.SamplingParams(temperature, -1, 1.0, ignore_eos, max_tokens, 0)


def run_step(cache, sched, token_of=lambda uid, idx: 100 + idx):
    """Plan, 'run' the step as the engine does (grow, advance), sample and commit."""
    out = list(sched.drain_outbox())
    plan = sched.plan_step()
    out += sched.drain_outbox()
    sampled = []
    for e in plan.entries:
        assert len(sched.tokens_of(e)) == e.count
        assert cache.length(e.uid) == e.start
        assert cache.grow(e.uid, e.start + e.count), "a running request ran out of pages"
        cache.advance(e.uid, e.start + e.count)
        if e.sample:
            sampled.append(token_of(e.uid, e.output_index))
    out += sched.commit_step(plan, sampled)
    assert cache.check() == ""
    return plan, out


def shape(plan):
    return [(e.uid, e.start, e.count, e.sample) for e in plan.entries]


def test_budget_cuts_the_prompt_and_the_rest_goes_first():
    cache, s = make(budget=6)
    a = s.add_request([1, 2], params())
    b = s.add_request(list(range(9)), params())
    c = s.add_request([7, 8], params())
    plan, out = run_step(cache, s)
    assert shape(plan) == [(a, 0, 2, True), (b, 0, 4, False)] and plan.prefill_tokens == 6
    assert [(o.uid, o.token) for o in out] == [(a, 100)] and s.num_pending() == 1
    plan, out = run_step(cache, s)
    # a decodes, b's continuation comes before anything new, c gets what is left of the budget
    assert shape(plan) == [(a, 2, 1, True), (b, 4, 5, True), (c, 0, 1, False)]
    plan, out = run_step(cache, s)
    assert shape(plan) == [(a, 3, 1, True), (b, 9, 1, True), (c, 1, 1, True)]
    assert plan.decode_rows == 2 and plan.prefill_tokens == 1


def test_no_budget_means_whole_prompts():
    cache, s = make(budget=0, max_seq=64)
    a = s.add_request(list(range(40)), params())
    b = s.add_request(list(range(30)), params())
    plan, _ = run_step(cache, s)
    assert shape(plan) == [(a, 0, 40, True), (b, 0, 30, True)]


def test_finish_reasons_and_the_finishing_token_is_emitted():
    cache, s = make(eos=[9], max_seq=8)
    a = s.add_request([1, 2, 3], params(max_tokens=2))
    b = s.add_request([1, 2, 3], params(max_tokens=50))
    c = s.add_request([1, 2, 3], params(max_tokens=50, ignore_eos=True))
    d = s.add_request([1, 2, 3], params(max_tokens=1))
    tokens = {a: [5, 6], b: [5, 9], c: [9, 9, 9, 9, 9, 9, 9], d: [4]}
    seen = {}
    while not s.is_idle():
        _, out = run_step(cache, s, lambda uid, idx: tokens[uid][idx])
        for o in out:
            seen.setdefault(o.uid, []).append((o.token, o.finished, o.reason))
    L, S, N = rt.FinishReason.Length, rt.FinishReason.Stop, rt.FinishReason.NotFinished
    assert seen[a] == [(5, False, N), (6, True, L)]
    assert seen[b] == [(5, False, N), (9, True, S)]
    # c ignores the end id and stops when the sequence reaches max_seq_len = 8: 3 + 5 tokens
    assert [t for t, _, _ in seen[c]] == [9] * 5 and seen[c][-1][1:] == (True, L)
    assert seen[d] == [(4, True, L)]
    assert cache.live_requests() == 0 and cache.free_pages(0) == 64


def test_empty_and_overlong_prompts_are_aborted_at_submission():
    cache, s = make(max_seq=8)
    a = s.add_request([], params())
    b = s.add_request(list(range(9)), params())
    ok = s.add_request(list(range(8)), params(max_tokens=1))
    out = s.drain_outbox()
    assert [(o.uid, o.token, o.finished, o.reason) for o in out] == \
        [(a, -1, True, rt.FinishReason.Abort), (b, -1, True, rt.FinishReason.Abort)]
    _, out = run_step(cache, s)
    assert [(o.uid, o.finished, o.reason) for o in out] == [(ok, True, rt.FinishReason.Length)]


def test_when_pages_run_out_the_head_waits_and_the_running_go_on():
    # 6 pages of 4: each request below needs ceil((6 + 7 - 1) / 4) = 3 pages for its whole life
    cache, s = make(pages=6, budget=32)
    ids = [s.add_request(list(range(6)), params(max_tokens=7, ignore_eos=True)) for _ in range(4)]
    plan, _ = run_step(cache, s)
    assert [e.uid for e in plan.entries] == ids[:2]           # the third is promised nothing
    assert s.num_pending() == 2 and cache.unpromised_pages(0) == 0
    finished_at = {}
    step = 1
    while not s.is_idle():
        plan, out = run_step(cache, s)
        step += 1
        for o in out:
            if o.finished:
                finished_at[o.uid] = step
        running = [e.uid for e in plan.entries]
        assert len(running) <= 2                              # never more than the pages allow
    assert finished_at[ids[0]] == finished_at[ids[1]] == 7    # undisturbed: 7 tokens in 7 steps
    assert finished_at[ids[2]] == finished_at[ids[3]] == 14   # admitted the step after, on the freed pages
    assert cache.free_pages(0) == 6 and cache.live_requests() == 0


def test_a_request_larger_than_the_pool_is_aborted_and_the_queue_moves_on():
    cache, s = make(pages=4, page_size=4, max_seq=64)
    big = s.add_request(list(range(10)), params(max_tokens=20))   # 29 tokens: 8 pages, the pool has 4
    small = s.add_request([1, 2], params(max_tokens=2))
    plan, out = run_step(cache, s)
    assert [(o.uid, o.reason) for o in out if o.token < 0] == [(big, rt.FinishReason.Abort)]
    assert [e.uid for e in plan.entries] == [small]


def test_max_running_req_limits_admission_and_slots_too():
    cache, s = make(max_running=2)
    ids = [s.add_request([1, 2, 3], params(max_tokens=2)) for _ in range(3)]
    plan, _ = run_step(cache, s)
    assert [e.uid for e in plan.entries] == ids[:2] and s.num_pending() == 1
    plan, _ = run_step(cache, s)                                # both finish here
    plan, _ = run_step(cache, s)
    assert [e.uid for e in plan.entries] == [ids[2]]


def test_abort_waiting_and_running():
    cache, s = make()
    a = s.add_request([1, 2, 3], params(max_tokens=9))
    b = s.add_request([1, 2, 3], params(max_tokens=9))
    assert s.abort_request(b) and not s.abort_request(b)
    _, out = run_step(cache, s)
    assert [(o.uid, o.reason) for o in out if o.token < 0] == [(b, rt.FinishReason.Abort)]
    assert s.status_of(a) == rt.Status.Decoding and cache.has(a)
    assert s.abort_request(a) and not cache.has(a)
    assert [(o.uid, o.reason) for o in s.drain_outbox()] == [(a, rt.FinishReason.Abort)]
    assert s.is_idle() and cache.free_pages(0) == 64 and not s.abort_request(12345)


def test_a_failed_step_ends_its_requests_with_error_and_frees_them():
    cache, s = make()
    a = s.add_request([1, 2, 3], params())
    b = s.add_request([4, 5], params())
    plan = s.plan_step()
    out = s.fail_step(plan)
    assert sorted((o.uid, o.token, o.reason) for o in out) == \
        [(a, -1, rt.FinishReason.Error), (b, -1, rt.FinishReason.Error)]
    assert s.is_idle() and cache.live_requests() == 0 and cache.check() == ""


def test_commit_refuses_a_wrong_number_of_tokens():
    cache, s = make()
    s.add_request([1, 2, 3], params())
    plan = s.plan_step()
    with pytest.raises(Exception):
        s.commit_step(plan, [])
    with pytest.raises(Exception):
        s.commit_step(plan, [1, 2])


def test_sampling_params_are_normalised():
    p = rt.SamplingParams(0.7, 5, 7.5, False, 0, 3).normalized()
    assert p.top_p == 1.0 and p.max_tokens == 1 and p.top_k == 5 and abs(p.temperature - 0.7) < 1e-6
    assert rt.SamplingParams(0.7, 5, float("nan"), False, 3, 0).normalized().top_p == 1.0


def test_a_windowed_group_is_promised_less_and_never_runs_dry():
    # window 8, budget 4: a long request needs only ceil((8 + 4 - 1) / 4) + 1 = 4 window pages
    cache, s = make(pages=16, page_size=4, budget=4, window=8, max_seq=64)
    a = s.add_request(list(range(30)), params(max_tokens=20, ignore_eos=True))
    steps = 0
    while not s.is_idle():
        run_step(cache, s)
        steps += 1
        if cache.has(a):
            assert cache.pages_held(a, 1) <= 4
    assert steps == 8 + 19 and cache.free_pages(1) == 16 and cache.free_pages(0) == 16


# ---------------------------------------------------------------- a step planned before the one before it has reported
def test_successor_is_one_decoded_token_for_every_request_in_the_plans_order():
    cache, s = make(budget=32)
    a = s.add_request([1, 2, 3], params(max_tokens=5))
    b = s.add_request([4, 5], params(max_tokens=5))
    plan = s.plan_step()                                     # both prompts whole, both sample
    nxt = s.successor(plan)
    assert [(e.uid, e.start, e.count, e.sample, e.output_index) for e in nxt.entries] == \
        [(a, 3, 1, True, 1), (b, 2, 1, True, 1)] and nxt.decode_rows == 2
    # what the scheduler plans after the commit is that very step
    for e in plan.entries:
        cache.grow(e.uid, e.start + e.count)
        cache.advance(e.uid, e.start + e.count)
    s.commit_step(plan, [50, 51])
    assert shape(s.plan_step()) == [(a, 3, 1, True), (b, 2, 1, True)]


def test_no_successor_when_a_decision_is_needed():
    # somebody waits
    cache, s = make(budget=4)
    s.add_request([1, 2, 3, 4], params())
    s.add_request([5, 6], params())
    plan = s.plan_step()
    assert s.num_pending() == 1 and not s.successor(plan).entries
    # a prompt is not through yet
    cache, s = make(budget=3)
    s.add_request([1, 2, 3, 4, 5], params())
    plan = s.plan_step()
    assert shape(plan) == [(1, 0, 3, False)] and not s.successor(plan).entries
    # a request ends by length with this step: max_tokens, then max_seq_len
    cache, s = make()
    s.add_request([1, 2], params(max_tokens=1))
    assert not s.successor(s.plan_step()).entries
    cache, s = make(max_seq=4)
    s.add_request([1, 2, 3], params(max_tokens=9))
    assert not s.successor(s.plan_step()).entries           # 3 prompt tokens + 1 output = max_seq_len
    cache, s = make(max_seq=5)
    s.add_request([1, 2, 3], params(max_tokens=9))
    assert len(s.successor(s.plan_step()).entries) == 1


def test_a_request_that_ends_while_its_successor_step_runs_is_a_dead_row():
    cache, s = make(eos=[99])
    a = s.add_request([1, 2], params(max_tokens=8))
    b = s.add_request([3], params(max_tokens=8))
    c = s.add_request([4, 5, 6], params(max_tokens=8))

    def run(plan):
        for e in plan.entries:
            cache.grow(e.uid, e.start + e.count)
            cache.advance(e.uid, e.start + e.count)

    plan = s.plan_step()
    run(plan)
    nxt = s.successor(plan)
    assert [e.uid for e in nxt.entries] == [a, b, c]
    run(nxt)                                                 # the engine launches it before it knows plan's tokens
    out = s.commit_step(plan, [10, 99, 12])                  # b draws the stop id
    assert [(o.uid, o.token, o.finished) for o in out] == [(a, 10, False), (b, 99, True), (c, 12, False)]
    assert s.abort_request(c)                                # and c is aborted meanwhile
    out = s.commit_step(nxt, [20, 21, 22])                   # the tokens of b and c are dropped
    assert [(o.uid, o.token) for o in out] == [(a, 20)]
    assert shape(s.plan_step()) == [(a, 3, 1, True)]
    with pytest.raises(ValueError):
        s.commit_step(nxt, [20, 21])                         # still one token for every sampling row
    assert cache.check() == ""


# ---------------------------------------------------------------- random traffic
@pytest.mark.parametrize("seed", range(16))
def test_random_traffic_keeps_every_promise(seed):
    """Requests arrive, are aborted and draw stop ids at random; steps are planned ahead wherever the scheduler
    allows it.  Whatever the order: a plan never exceeds the budget of prompt tokens or the number of rows, every
    decoding request is in every plan, a running request always gets its pages, requests start in arrival order,
    each ends once with a reason that fits, and in the end no page, promise or slot is left behind."""
    import random
    rng = random.Random(seed)
    page_size = rng.choice([1, 2, 4, 16])
    max_seq = rng.randrange(8, 48)
    pages = rng.randrange(-(-max_seq // page_size), 4 * -(-max_seq // page_size) + 2)
    max_running = rng.randrange(1, 6)
    budget = rng.choice([0, 3, 5, 16])
    window = rng.choice([0, 0, 6])
    stop = 7
    cache, s = make(pages=pages, page_size=page_size, max_running=max_running, max_seq=max_seq, budget=budget,
                    eos=[stop], window=window)
    wanted = {}                                  # uid -> (prompt length, max_tokens, ignore_eos)
    tokens, reasons, first_seen = {}, {}, []
    to_come = rng.randrange(5, 30)

    def note(out):
        for o in out:
            assert o.uid in wanted and o.uid not in reasons, "a request reported after it had ended"
            if o.token >= 0:
                tokens.setdefault(o.uid, []).append(o.token)
            else:
                assert o.finished and o.reason in (rt.FinishReason.Abort, rt.FinishReason.Error)
            if o.finished:
                reasons[o.uid] = o.reason

    def check_plan(plan, ahead):
        uids = [e.uid for e in plan.entries]
        assert len(set(uids)) == len(uids) and len(uids) <= max_running
        prompt_tokens = sum(e.count for e in plan.entries if e.start < wanted[e.uid][0])
        if not ahead:
            assert prompt_tokens == plan.prefill_tokens
            assert budget == 0 or prompt_tokens <= budget
            for uid in wanted:
                if s.status_of(uid) == rt.Status.Decoding:
                    assert uid in uids, "a decoding request was left out of a step"
        for e in plan.entries:
            if e.uid not in first_seen:
                first_seen.append(e.uid)
            assert cache.length(e.uid) == e.start
            assert cache.grow(e.uid, e.start + e.count), "a running request ran out of pages"
            cache.advance(e.uid, e.start + e.count)
            assert e.start + e.count <= max_seq

    def draw(plan):
        return [stop if rng.random() < 0.08 else rng.randrange(8, 100) for e in plan.entries if e.sample]

    flight = None                                # a step that was planned ahead and is "on the GPU"
    steps = 0
    while to_come or not s.is_idle() or flight is not None:
        steps += 1
        assert steps < 5000, "the scheduler makes no progress"
        for _ in range(min(rng.choice([0, 0, 1, 2]), to_come)):
            to_come -= 1
            n, m, ig = rng.randrange(0, max_seq + 3), rng.randrange(1, 12), rng.random() < 0.5
            uid = s.add_request([rng.randrange(8, 100) for _ in range(n)], params(max_tokens=m, ignore_eos=ig))
            wanted[uid] = (n, m, ig)
        if wanted and rng.random() < 0.1:
            victim = rng.choice(sorted(wanted))
            alive = s.status_of(victim) != rt.Status.Finished
            assert s.abort_request(victim) == alive
        note(s.drain_outbox())
        if flight is None:
            plan = s.plan_step()
            note(s.drain_outbox())
            if not plan.entries:
                assert cache.check() == ""
                continue
            check_plan(plan, ahead=False)
        else:
            plan, flight = flight, None
        following = s.successor(plan)
        if following.entries and rng.random() < 0.8:
            assert [e.uid for e in following.entries] == [e.uid for e in plan.entries]
            check_plan(following, ahead=True)
            flight = following
        if rng.random() < 0.03:
            note(s.fail_step(plan))
            if flight is not None:               # the engine drops the step that it launched ahead with it
                flight = None
        else:
            note(s.commit_step(plan, draw(plan)))
        assert cache.check() == ""

    assert cache.live_requests() == 0 and cache.free_state_slots() == max_running
    for g in range(cache.num_groups()):
        assert cache.free_pages(g) == pages and cache.unpromised_pages(g) == pages
    assert set(reasons) == set(wanted), "every request ends, once"
    assert first_seen == sorted(first_seen), "requests start in the order of their arrival"
    for uid, (n, m, ignore) in wanted.items():
        got, why = tokens.get(uid, []), reasons[uid]
        assert len(got) <= m and n + max(len(got) - 1, 0) <= max(max_seq, n)   # the last token is never cached
        if n == 0 or n > max_seq:
            assert why == rt.FinishReason.Abort and not got
        if why == rt.FinishReason.Stop:
            assert got[-1] == stop and not ignore and stop not in got[:-1]
        elif why == rt.FinishReason.Length:
            assert len(got) == m or n + len(got) >= max_seq
            assert ignore or stop not in got


def test_a_step_that_could_not_be_built_is_rolled_back():
    """Nothing of the step ran: the requests that the plan admitted give back their promise and stand at the head
    of the queue again in their old order; the running ones are untouched and the next plan is the same plan
    (reference: src/scheduler/prefill.rs:65-71, :119-129)."""
    cache, s = make(pages=32, budget=8)
    a = s.add_request([1, 2, 3], params())
    run_step(cache, s)                                         # a runs
    b = s.add_request([4, 5], params())
    c = s.add_request([6, 7, 8], params())
    d = s.add_request([9] * 20, params())
    free = cache.free_pages(0)
    unpromised = cache.unpromised_pages(0)
    plan = s.plan_step()
    assert shape(plan) == [(a, 3, 1, True), (b, 0, 2, True), (c, 0, 3, True), (d, 0, 3, False)]
    assert s.num_pending() == 0 and cache.unpromised_pages(0) < unpromised
    assert s.rollback_step(plan) == 3
    assert s.num_pending() == 3 and s.num_running() == 1 and cache.check() == ""
    assert cache.free_pages(0) == free and cache.unpromised_pages(0) == unpromised
    assert s.status_of(b) == rt.Status.Waiting and s.status_of(a) == rt.Status.Decoding
    again = s.plan_step()
    assert shape(again) == shape(plan)                         # arrival order is kept
    assert s.rollback_step(again) == 3
    plan, out = run_step(cache, s)
    assert [o.uid for o in out] == [a, b, c]
    # a request whose prompt is already partly through is not sent back
    plan = s.plan_step()
    assert (d, 3, 8, False) in shape(plan) and s.rollback_step(plan) == 0 and s.num_running() == 4
