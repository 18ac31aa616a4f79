"""The scheduler's decisions, on the CPU with a stand-in for the model: admission,
portions under the token budget, decoding, finishing and freeing, and what happens
when pages run out (the request admitted last is preempted and recomputed)."""
import numpy as np
import pytest

from ai_engine_b200.cache import host


def make(pages=16, page=4, max_seqs=4, budget=8, max_len=64, window=0):
    h = host()
    cache = h.CacheManager([h.GroupSpec(page, pages, window)], max_seqs, (max_len + page - 1) // page)
    return h, cache, h.Scheduler(cache, max_seqs, budget, max_len)


def run(sched, cache, lens, max_new, eos_at=None, max_steps=10000):
    """Drive the scheduler with fake tokens: token value = (request id, index)."""
    total = {i: n for i, n in lens.items()}
    out = {i: [] for i in lens}
    log = []
    for _ in range(max_steps):
        if not sched.has_work():
            break
        plan = sched.schedule()
        cache.check_invariants()
        log.append(plan)
        assert plan.entries, "a step with work must schedule something"
        sched.commit(plan)
        for e in plan.entries:
            if e.sample:
                tok = (e.id, total[e.id])
                total[e.id] += 1
                stop = eos_at is not None and len(out[e.id]) + 1 == eos_at.get(e.id, -1)
                out[e.id].append(tok)
                sched.on_token(e.id, stop)
        cache.check_invariants()
    assert not sched.has_work()
    return out, log


def test_prompt_is_cut_into_portions_under_the_budget():
    h, cache, s = make(budget=8)
    assert s.add(0, 21, 2) == ""
    plans = []
    while s.has_work():
        p = s.schedule()
        plans.append([(e.start, e.n_tokens, e.sample) for e in p.entries])
        s.commit(p)
        for e in p.entries:
            if e.sample:
                s.on_token(e.id, False)
    assert plans == [[(0, 8, False)], [(8, 8, False)], [(16, 5, True)], [(21, 1, True)]]
    assert cache.free_pages(0) == 16 and cache.free_slots == 4


def test_decodes_come_first_and_share_the_step_with_a_prompt_portion():
    h, cache, s = make(budget=8, pages=32)
    s.add(0, 3, 10)
    p = s.schedule(); s.commit(p); s.on_token(0, False)
    s.add(1, 20, 2)
    p = s.schedule()
    got = [(e.id, e.start, e.n_tokens, e.sample) for e in p.entries]
    assert got == [(0, 3, 1, True), (1, 0, 7, False)]       # 1 decode + 7 of the budget of 8
    assert sum(e.n_tokens for e in p.entries) <= 8


def test_max_num_seqs_bounds_admission_fifo():
    h, cache, s = make(max_seqs=2, budget=64, pages=64)
    for i in range(4):
        s.add(i, 2, 3)
    p = s.schedule()
    assert [e.id for e in p.entries] == [0, 1] and s.num_waiting == 2
    out, _ = run(s, cache, {i: 2 for i in range(4)}, 3)
    assert all(len(v) == 3 for v in out.values())


def test_finish_on_eos_max_tokens_and_context_limit():
    h, cache, s = make(max_len=10, pages=16)
    s.add(0, 4, 100)      # runs into the context limit
    s.add(1, 4, 3)        # max_tokens
    s.add(2, 4, 100)      # EOS on its 2nd token
    out, _ = run(s, cache, {0: 4, 1: 4, 2: 4}, None, eos_at={2: 2})
    assert len(out[1]) == 3 and len(out[2]) == 2
    assert len(out[0]) == 7            # 4 + 7 = 11 known tokens > 10: the last one is still returned
    assert cache.free_pages(0) == 16 and cache.free_slots == 4
    assert s.stats()["finished"] == 3


def test_requests_that_can_never_run_are_rejected_with_a_reason():
    h, cache, s = make(pages=4, page=4, max_len=64)
    assert "max context" in s.add(0, 65, 1)
    assert "never fit" in s.add(1, 20, 1)           # 20 tokens need 5 pages of 4
    assert "max_tokens" in s.add(2, 3, 0)
    assert "empty" in s.add(3, 0, 5)
    assert s.add(4, 12, 5) == "" and "already" in s.add(4, 3, 3)


def test_pages_run_out_last_admitted_is_preempted_and_recomputed():
    # 6 pages of 4 tokens; three requests of 6 + 10 tokens each cannot all finish side by side
    h, cache, s = make(pages=6, page=4, budget=16, max_len=32)
    lens = {0: 6, 1: 6, 2: 6}
    for i, n in lens.items():
        assert s.add(i, n, 10) == ""
    out, log = run(s, cache, lens, 10)
    st = s.stats()
    assert st["preemptions"] >= 1
    pre = [i for p in log for i in p.preempted]
    assert 0 not in pre                      # the first admitted is never the victim while others run
    for i in lens:                           # every request still gets all its tokens, in order
        assert out[i] == [(i, lens[i] + k) for k in range(10)]
    # a preempted request starts again from its first token with everything known so far
    seen_restart = False
    for p in log:
        for e in p.entries:
            if e.id in pre and e.start == 0 and e.n_tokens > lens[e.id]:
                seen_restart = True
    assert seen_restart
    assert cache.free_pages(0) == 6 and cache.free_slots == 4


def test_a_preempted_step_entry_is_withdrawn_from_the_plan():
    h, cache, s = make(pages=4, page=4, budget=16, max_len=16)
    s.add(0, 7, 8)
    s.add(1, 7, 8)
    out, log = run(s, cache, {0: 7, 1: 7}, 8)
    for p in log:
        ids = [e.id for e in p.entries]
        assert len(ids) == len(set(ids))
        assert not (set(ids) & set(p.preempted))
    assert out[0] == [(0, 7 + k) for k in range(8)] and out[1] == [(1, 7 + k) for k in range(8)]


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_and_free_everything(seed):
    rng = np.random.RandomState(seed)
    h, cache, s = make(pages=int(rng.randint(10, 30)), page=int(rng.choice([2, 4, 8])),
                       max_seqs=int(rng.randint(1, 5)), budget=int(rng.randint(2, 20)), max_len=64,
                       window=int(rng.choice([0, 0, 12])))
    lens, news = {}, {}
    for i in range(12):
        n, m = int(rng.randint(1, 30)), int(rng.randint(1, 12))
        if s.add(i, n, m) == "":
            lens[i], news[i] = n, m
    assert lens
    out, log = run(s, cache, lens, None)
    for i in lens:
        want = min(news[i], 64 - lens[i] + 1)
        assert out[i] == [(i, lens[i] + k) for k in range(want)], i
    for p in log:
        assert sum(e.n_tokens for e in p.entries) <= 20
    assert cache.pages_in_use(0) == 0 and cache.free_slots == cache.max_seqs
