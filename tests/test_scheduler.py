"""The scheduler's decisions with a fake model (a constant token instead of a forward pass), as
the reference tests its scheduler (tests/test_scheduler.cpp:19-87), plus what is new here:
prompts cut into portions under the token budget.  No GPU."""
import random

import pytest

from kvcm.cache import core


def make(num_blocks=64, block_size=4, max_seq_len=256, prefix=False, watermark=0, policy="paged",
         **sched):
    if policy == "paged":
        kv = core.PagedManager(num_blocks, block_size, max_seq_len, prefix, watermark)
    else:
        kv = core.ContiguousManager(num_blocks, block_size, max_seq_len)
    c = core.SchedulerConfig()
    for k, v in sched.items():
        setattr(c, k, v)
    return kv, core.Scheduler(kv, c)


def run_to_completion(s, kv, token=42, max_steps=100000, check=None):
    """schedule -> check the plan -> update with a constant token, until idle."""
    steps, finished = 0, []
    while not s.idle():
        plan = s.schedule(float(steps))
        rows = 0
        for p in plan:
            q = p.seq
            assert p.start == q.num_computed and p.num_tokens >= 1
            assert p.start + p.num_tokens <= q.length()
            assert p.wants_logits == (p.start + p.num_tokens == q.length())
            need = (p.start + p.num_tokens + kv.block_size() - 1) // kv.block_size()
            assert len(q.table(0)) >= need, "scheduled without pages"
            assert q.state_slot >= 0
            rows += p.num_tokens
        if check:
            check(plan, rows)
        s.update([token] * sum(1 for p in plan if p.wants_logits), float(steps))
        finished += s.take_finished()
        steps += 1
        assert steps < max_steps, "scheduler does not terminate"
    return steps, finished


def test_completes_without_pressure():
    kv, s = make(num_blocks=256)
    for i in range(20):
        s.add_request(i, [1] * (5 + i), 10)
    steps, fin = run_to_completion(s, kv)
    assert len(fin) == 20 and all(f.num_generated() == 10 and not f.rejected for f in fin)
    assert kv.blocks_in_use() == 0 and s.slots_taken() == 0
    c = s.counters()
    assert c.preemptions == 0 and c.admissions == 20 and c.rejected == 0


def test_token_budget_cuts_prompts_into_portions():
    kv, s = make(num_blocks=256, max_batched_tokens=16)
    s.add_request(0, [1] * 50, 3)
    s.add_request(1, [2] * 7, 3)
    seen = []

    def check(plan, rows):
        assert rows <= 16
        seen.append([(p.seq.id, p.start, p.num_tokens, p.wants_logits) for p in plan])
    run_to_completion(s, kv, check=check)
    assert seen[0] == [(0, 0, 16, False)]
    assert seen[1] == [(0, 16, 16, False)]
    assert seen[2] == [(0, 32, 16, False)]
    assert seen[3] == [(0, 48, 2, True), (1, 0, 7, True)]      # the rest of the budget admits request 1
    assert seen[4] == [(0, 50, 1, True), (1, 7, 1, True)]      # both decode


def test_prefill_chunk_caps_a_portion_and_mixes_with_decodes():
    kv, s = make(num_blocks=256, max_batched_tokens=64, prefill_chunk=24)
    s.add_request(0, [1] * 5, 40)
    plans = []
    s.schedule(0.0); s.update([9], 0.0)                        # request 0 is decoding now
    s.add_request(1, [2] * 60, 2)
    for step in range(1, 4):
        plan = s.schedule(float(step))
        plans.append([(p.seq.id, p.start, p.num_tokens) for p in plan])
        s.update([9] * sum(1 for p in plan if p.wants_logits), float(step))
    assert plans[0] == [(0, 5, 1), (1, 0, 24)]                 # a decode beside a portion
    assert plans[1] == [(0, 6, 1), (1, 24, 24)]
    assert plans[2] == [(0, 7, 1), (1, 48, 12)]


def test_unchunked_mode_schedules_prompts_whole():
    kv, s = make(num_blocks=256, max_batched_tokens=16, chunked_prefill=False)
    s.add_request(0, [1] * 50, 2)        # larger than the budget: still taken when alone
    s.add_request(1, [1] * 10, 2)

    def check(plan, rows):
        for p in plan:
            if p.is_prefill:
                assert p.start == 0 and p.num_tokens == p.seq.prompt_len
    steps, fin = run_to_completion(s, kv, check=check)
    assert len(fin) == 2


def test_max_num_seqs_caps_the_running_batch():
    kv, s = make(num_blocks=256, max_num_seqs=3)
    for i in range(8):
        s.add_request(i, [1] * 4, 5)

    def check(plan, rows):
        assert len(plan) <= 3
    run_to_completion(s, kv, check=check)
    assert s.counters().max_running == 3


def test_preemption_by_recomputation_when_pages_run_out():
    # 8 requests of 32 + 64 tokens need 8 * 24 = 192 pages of 4; the pool has 24 * 4 = 96.
    kv, s = make(num_blocks=96, block_size=4, max_seq_len=128)
    for i in range(8):
        s.add_request(i, [i + 1] * 32, 64)
    steps, fin = run_to_completion(s, kv)
    c = s.counters()
    assert c.preemptions > 0
    assert len(fin) == 8 and all(f.num_generated() == 64 and not f.rejected for f in fin)
    assert any(f.num_preemptions > 0 for f in fin)
    assert kv.blocks_in_use() == 0 and s.slots_taken() == 0     # nothing leaks


def test_evicted_request_is_the_youngest_and_returns_to_the_front():
    kv, s = make(num_blocks=4, block_size=4, max_seq_len=64)
    s.add_request(0, [1] * 8, 20)
    s.add_request(1, [2] * 8, 20)
    s.add_request(2, [3] * 3, 20)
    s.schedule(0.0)                         # 0 and 1 take all four pages; 2 waits
    assert s.num_running() == 2 and s.num_waiting() == 1
    s.update([9, 9], 0.0)                   # both now have 9 tokens: the next one needs a third page
    plan = s.schedule(1.0)                  # the oldest needs a third page: the youngest (1) goes
    assert [p.seq.id for p in plan] == [0]
    assert s.counters().preemptions == 1 and s.num_waiting() == 2
    s.update([9], 1.0)
    # the evicted request is ahead of request 2 in the queue and is computed again from token 0
    seen = []
    for step in range(2, 200):
        if s.idle():
            break
        plan = s.schedule(float(step))
        seen += [(p.seq.id, p.start) for p in plan if p.start == 0]
        s.update([9] * sum(1 for p in plan if p.wants_logits), float(step))
    assert seen[0][0] == 1, seen


def test_no_admission_in_a_step_that_evicted():
    kv, s = make(num_blocks=4, block_size=4, max_seq_len=64)
    s.add_request(0, [1] * 8, 20)
    s.add_request(1, [2] * 8, 20)
    s.schedule(0.0); s.update([9, 9], 0.0)
    plan = s.schedule(1.0)
    assert [p.seq.id for p in plan] == [0] and s.num_running() == 1


def test_request_that_can_never_fit_is_rejected():
    kv, s = make(num_blocks=4, block_size=4, max_seq_len=64)
    s.add_request(0, [1] * 100, 4)          # longer than max_seq_len
    s.add_request(1, [1] * 20, 4)           # more pages than the pool
    s.add_request(2, [1] * 5, 4)
    steps, fin = run_to_completion(s, kv)
    by_id = {f.id: f for f in fin}
    assert by_id[0].rejected and by_id[1].rejected and by_id[0].num_generated() == 0
    assert not by_id[2].rejected and by_id[2].num_generated() == 4
    assert s.counters().rejected == 2


def test_blocked_head_waits_and_nothing_overtakes_it():
    kv, s = make(num_blocks=8, block_size=4, max_seq_len=64)
    s.add_request(0, [1] * 20, 3)           # 5 pages (6 with its outputs)
    s.add_request(1, [2] * 20, 3)           # does not fit beside request 0
    s.add_request(2, [3] * 2, 3)            # would fit, but must not overtake request 1
    order = []
    while not s.idle():
        plan = s.schedule(0.0)
        order += [p.seq.id for p in plan if p.start == 0]
        s.update([9] * sum(1 for p in plan if p.wants_logits), 0.0)
    assert order == [0, 1, 2]
    assert s.counters().admission_blocked_steps > 0


def test_stops_at_max_seq_len_and_at_eos():
    kv, s = make(num_blocks=64, block_size=4, max_seq_len=12)
    s.add_request(0, [1] * 10, 100)
    _, fin = run_to_completion(s, kv)
    assert fin[0].length() == 12
    kv, s = make(num_blocks=64, eos_token_id=42)
    s.add_request(0, [1] * 10, 100)
    _, fin = run_to_completion(s, kv, token=42)
    assert fin[0].num_generated() == 1


def test_prefix_cache_resumes_after_the_cached_pages():
    kv, s = make(num_blocks=64, block_size=16, max_seq_len=256, prefix=True)
    prompt = list(range(100))
    s.add_request(0, prompt, 2)
    run_to_completion(s, kv)
    s.add_request(1, prompt, 2)
    plan = s.schedule(0.0)
    assert plan[0].start == 96 and plan[0].num_tokens == 4      # 6 full pages of 16 are reused
    assert s.counters().prefill_tokens_saved == 96


def test_contiguous_policy_runs_the_same_loop():
    kv, s = make(num_blocks=32, block_size=4, max_seq_len=32, policy="contiguous")
    for i in range(6):
        s.add_request(i, [1] * 6, 8)        # 8 pages reserved each: 4 fit at a time
    steps, fin = run_to_completion(s, kv)
    assert len(fin) == 6 and s.counters().max_running == 4 and kv.blocks_in_use() == 0


def test_random_workloads_finish_and_leak_nothing():
    rng = random.Random(3)
    for trial in range(10):
        kv, s = make(num_blocks=rng.randint(12, 40), block_size=4, max_seq_len=64,
                     max_num_seqs=rng.randint(2, 8), max_batched_tokens=rng.randint(8, 48),
                     prefill_chunk=rng.choice([0, 5, 16]), prefix=rng.random() < 0.5)
        n = rng.randint(5, 25)
        for i in range(n):
            s.add_request(i, [rng.randint(0, 3) for _ in range(rng.randint(1, 40))], rng.randint(1, 20))
        steps, fin = run_to_completion(s, kv)
        assert len(fin) == n
        for f in fin:
            assert f.rejected or f.num_generated() == min(f.max_new_tokens, 64 - f.prompt_len) \
                or f.length() == 64
        assert kv.blocks_in_use() == 0 and s.slots_taken() == 0


def test_update_wants_exactly_one_token_per_sampling_entry():
    kv, s = make()
    s.add_request(0, [1] * 4, 2)
    s.schedule(0.0)
    with pytest.raises(Exception):
        s.update([], 0.0)
    with pytest.raises(Exception):
        s.update([1, 2], 0.0)


def test_empty_request_is_refused():
    kv, s = make()
    with pytest.raises(Exception):
        s.add_request(0, [], 2)
