"""The request loop in C++ (``csrc/core/native_engine.cpp``) on a stand-in device that runs on the
CPU: "device" memory is host memory, the forward pass writes logits whose maximum is a fixed function
of (token, position), and a recorded graph replays the calls made while it was recorded.  So every
request's tokens are known in advance, whatever the batching, and the loop's own decisions show:
portions under the token budget, decode steps replayed from graphs per shape, the step that records
a graph running exactly once, eviction when pages run out, limits."""
import pytest

from kvcm.cache import core

V = 97


def make(num_blocks=64, block_size=4, max_seq_len=64, max_num_seqs=4, max_batched_tokens=16, graphs=True,
         prefill_chunk=0, eos=-1, lookahead=True):
    kv = core.PagedManager(num_blocks, block_size, max_seq_len, False, 0)
    sc = core.SchedulerConfig()
    sc.max_num_seqs, sc.max_batched_tokens, sc.prefill_chunk, sc.eos_token_id = max_num_seqs, max_batched_tokens, prefill_chunk, eos
    sched = core.Scheduler(kv, sc)
    layer = dict(w_qkv=0, w_o=0, w_gate_up=0, w_down=0, norm1=0, norm2=0, k_cache=0, v_cache=0, eps1=1e-5, eps2=1e-5,
                 group=0, window=0, writes=1, num_pages=num_blocks)
    model = dict(embed=0, final_norm=0, lm_head=0, inv_freq=0, f32=0, H=8, I=16, nh=2, nkv=1, hd=4, V=V, sm_count=1,
                 final_eps=1e-5, scale=0.5, layers=[layer, layer])
    cfg = dict(block_size=block_size, max_seq_len=max_seq_len, num_groups=1, max_rows=max(max_batched_tokens, max_seq_len),
               max_seqs=max_num_seqs, graphs=graphs, lookahead=lookahead)
    return kv, sched, core.NativeEngine(kv, sched, model, cfg, 0)


def expected(prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(core.fake_next_token(toks[-1], len(toks) - 1, V))
    return toks[len(prompt):]


def run(sched, eng, prompts, max_new, arrive_every=0):
    done, infos, i = {}, [], 0
    while i < len(prompts) or not sched.idle():
        if i < len(prompts) and (arrive_every == 0 or len(infos) % arrive_every == 0):
            for j in range(i, len(prompts) if arrive_every == 0 else i + 1):
                sched.add_request(j, prompts[j], max_new)
            i = len(prompts) if arrive_every == 0 else i + 1
        infos.append(eng.step())
        for f in sched.take_finished():
            done[f.id] = f
        assert len(infos) < 10000
    return done, infos


@pytest.mark.parametrize("graphs,lookahead", [(True, True), (True, False), (False, False)])
def test_tokens_do_not_depend_on_batching_and_every_step_runs_once(graphs, lookahead):
    prompts = [[5, 9, 3], list(range(10, 33)), [7], [2] * 17, [11, 12, 13, 14, 15, 16, 17]]
    kv, sched, eng = make(graphs=graphs, lookahead=lookahead)
    before = core.fake_backend_forward_calls()
    done, infos = run(sched, eng, prompts, 12, arrive_every=3)
    for j, p in enumerate(prompts):
        assert not done[j].rejected and done[j].generated() == expected(p, 12), j
    steps = [i for i in infos if i.rows > 0]
    assert core.fake_backend_forward_calls() - before == len(steps)       # a recorded step ran once, not twice
    assert max(i.rows for i in steps) <= 16 and any(i.prefill_tokens and i.decode_seqs for i in steps)
    assert (eng.lookahead_steps() > 5) == lookahead and not eng.in_flight()
    if graphs:
        assert eng.graphs_captured() >= 2 and eng.graph_replays() > 5
        assert {b for b, _, _ in eng.graph_shapes()} <= {1, 2, 4}
        assert sum(i.graph for i in steps) == eng.graph_replays()
    else:
        assert eng.graphs_captured() == 0 and not any(i.graph for i in steps)
    assert kv.blocks_in_use() == 0 and sched.slots_taken() == 0
    c = sched.counters()
    assert c.prefill_tokens == sum(len(p) for p in prompts) and c.preemptions == 0


def test_lookahead_enqueues_the_next_step_before_this_one_is_read():
    """Steady greedy decoding: every call returns one step while the next is already on the device
    (the stand-in device runs a step when it is enqueued, so "on the device" shows as a forward call
    made one step early); a request that arrives, or ends, interrupts the chain and nothing is lost."""
    kv, sched, eng = make(max_num_seqs=4, max_batched_tokens=64)
    prompts = [[5, 9, 3], [8] * 6]
    for j, p in enumerate(prompts):
        sched.add_request(j, p, 30)
    infos = [eng.step(), eng.step()]                 # the prompts; the first decode step records its shape
    assert infos[0].prefill_tokens == 9 and not eng.in_flight()
    before = core.fake_backend_forward_calls()
    eng.step()                                       # a replayed decode step: the one after it is enqueued already
    assert eng.in_flight() and core.fake_backend_forward_calls() - before == 2
    eng.step()
    assert eng.in_flight() and core.fake_backend_forward_calls() - before == 3 and eng.lookahead_steps() == 2
    live = sched.live()
    assert [s.num_generated() for s in live] == [4, 4] and all(t != 0 for s in live for t in s.generated())
    sched.add_request(2, [4, 4, 4, 4], 5)            # a newcomer: the step in flight ends, then a mixed step
    a, b = eng.step(), eng.step()
    assert a.decode_seqs == 2 and a.prefill_tokens == 0 and b.prefill_tokens == 4 and b.decode_seqs == 2
    done = {}
    while not sched.idle():
        eng.step()
        for f in sched.take_finished():
            done[f.id] = f
    assert not eng.in_flight() and eng.step().rows == 0
    for j, (p, n) in enumerate([(prompts[0], 30), (prompts[1], 30), ([4, 4, 4, 4], 5)]):
        assert done[j].generated() == expected(p, n), j
    eng.drain()


def test_drain_finishes_a_step_in_flight_and_hands_its_result_out_later():
    kv, sched, eng = make(max_num_seqs=2, max_batched_tokens=64)
    sched.add_request(0, [5, 9, 3], 12)
    eng.step(); eng.step(); eng.step()
    assert eng.in_flight()
    n = sched.live()[0].num_generated()
    eng.drain()
    assert not eng.in_flight() and sched.live()[0].num_generated() == n + 1
    info = eng.step()                                # the drained step's result
    assert info.decode_seqs == 1 and info.graph and sched.live()[0].num_generated() == n + 1
    while not sched.idle():
        eng.step()
    assert sched.take_finished()[0].generated() == expected([5, 9, 3], 12)


def test_eviction_when_pages_run_out_keeps_the_tokens():
    prompts = [[3 + i] * 9 for i in range(4)]
    kv, sched, eng = make(num_blocks=12, block_size=4, max_seq_len=40, max_num_seqs=4, max_batched_tokens=64)
    done, infos = run(sched, eng, prompts, 20)
    assert sched.counters().preemptions > 0
    for j, p in enumerate(prompts):
        assert done[j].generated() == expected(p, 20), j
    assert kv.blocks_in_use() == 0


def test_limits_eos_and_rejection():
    kv, sched, eng = make(max_seq_len=16, eos=core.fake_next_token(5, 0, V))
    sched.add_request(0, [5], 10)                    # its first sampled token is the end-of-sequence token
    sched.add_request(1, [6] * 40, 3)                # longer than max_seq_len: can never fit
    sched.add_request(2, [9, 9], 50)                 # stops at max_seq_len
    done, _ = run(sched, eng, [], 0)
    assert done[0].generated() == [core.fake_next_token(5, 0, V)]
    assert done[1].rejected and done[1].generated() == []
    assert len(done[2].tokens) == 16 and done[2].generated() == expected([9, 9], 14)
    assert eng.step().rows == 0                      # nothing to do: an empty step
    assert core.NativeEngine.batch_bucket(3) == 4 and core.NativeEngine.batch_bucket(600) == 768
    assert core.NativeEngine.ctx_bucket(1) == 256 and core.NativeEngine.ctx_bucket(257) == 512


def test_a_step_beyond_the_limits_is_refused():
    kv = core.PagedManager(64, 4, 64, False, 0)
    sc = core.SchedulerConfig()
    sc.max_num_seqs, sc.max_batched_tokens = 8, 64
    sched = core.Scheduler(kv, sc)
    layer = dict(w_qkv=0, w_o=0, w_gate_up=0, w_down=0, norm1=0, norm2=0, k_cache=0, v_cache=0, eps1=1e-5, eps2=1e-5,
                 group=0, window=0, writes=1, num_pages=64)
    model = dict(embed=0, final_norm=0, lm_head=0, inv_freq=0, f32=0, H=8, I=16, nh=2, nkv=1, hd=4, V=V, sm_count=1,
                 final_eps=1e-5, scale=0.5, layers=[layer])
    eng = core.NativeEngine(kv, sched, model, dict(block_size=4, max_seq_len=64, num_groups=1, max_rows=8, max_seqs=2,
                                                  graphs=False), 0)
    sched.add_request(0, [4] * 30, 2)
    with pytest.raises(RuntimeError, match="exceeds the limits"):
        eng.step()
    with pytest.raises(ValueError, match="sizes are incomplete"):
        core.NativeEngine(kv, sched, dict(model, layers=[]), dict(block_size=4, max_seq_len=64, num_groups=1, max_rows=8,
                                                                 max_seqs=2, graphs=False), 0)
