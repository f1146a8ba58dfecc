"""kvsim: the scheduler and the cache manager without a model (after the reference's
``src/sim/simulator.cpp`` and ``src/main_sim.cpp``): a step "executes" by doing nothing and every
sampled token is a constant.  Answers what-if questions about policies, pool sizes and page sizes
on the CPU.  Time is counted in steps.

    kvsim --policy both --pool-gb 1 --requests 300 --bytes-per-token 22528

Flags as kvbench minus the model, plus --bytes-per-token (default: TinyLlama's 22,528),
--policy both, --trace CSV, --trace-every N; defaults --max-num-seqs 1024, --max-batched-tokens 8192.
"""
from __future__ import annotations

import sys


def simulate(policy: str, a, wl, num_blocks: int, block_size: int, max_seq_len: int, prefix: bool,
             watermark: int, max_num_seqs: int, max_batched_tokens: int, prefill_chunk: int, trace=None,
             trace_every: int = 1):
    from ..cache import core
    from ..engine.workload import generate_workload, make_prompt_tokens
    c = core.KVManagerConfig()
    c.policy, c.num_blocks, c.block_size, c.max_seq_len = policy, num_blocks, block_size, max_seq_len
    c.prefix_caching = prefix and policy == "paged"
    c.watermark_blocks = watermark
    kv = core.make_kv_manager(c)
    sc = core.SchedulerConfig()
    sc.max_num_seqs, sc.max_batched_tokens, sc.prefill_chunk = max_num_seqs, max_batched_tokens, prefill_chunk
    sched = core.Scheduler(kv, sc)
    reqs = generate_workload(wl)
    nxt, step, finished, rejected, peak, frag_sum, frag_n = 0, 0, 0, 0, 0, 0.0, 0
    while finished + rejected < len(reqs):
        while nxt < len(reqs) and reqs[nxt].arrival <= step:
            r = reqs[nxt]
            sched.add_request(r.id, make_prompt_tokens(r, wl), r.output_len, 0.0, 0, float(step))
            nxt += 1
        if sched.idle():
            step += 1
            continue
        sched.schedule(float(step))
        _, _, wants, _, _, _ = sched.plan_summary()
        sched.update([42] * wants, float(step))
        for f in sched.take_finished():
            if f.rejected:
                rejected += 1
            else:
                finished += 1
        peak = max(peak, kv.blocks_in_use())
        if step % 16 == 0:
            st = sched.kv_stats()
            frag_sum += st.fragmentation()
            frag_n += 1
        if trace and step % trace_every == 0:
            trace.write(f"{policy},{step},{sched.num_running()},{sched.num_waiting()},{kv.blocks_in_use()}\n")
        step += 1
    k = sched.counters()
    return dict(policy=kv.name(), steps=k.steps, preemptions=k.preemptions, max_running=k.max_running,
                mean_batch=k.batch_size_sum / max(k.steps, 1), finished=finished, rejected=rejected,
                peak_blocks=peak, mean_fragmentation=frag_sum / max(frag_n, 1),
                prefill_tokens=k.prefill_tokens, prefill_saved=k.prefill_tokens_saved)


def main(argv=None) -> int:
    from .args import Args
    from ..engine.workload import WorkloadConfig
    a = Args(argv)
    try:
        policy = a.str("policy", "both")
        block_size = a.i32("block-size", 16)
        max_seq_len = a.i32("max-seq-len", 2048)
        bpt = a.i64("bytes-per-token", 22528)
        num_blocks = a.i32("num-blocks", 0) or int(a.f64("pool-gb", 1.0) * 2**30 / (bpt * block_size))
        wm = a.i32("watermark", -1)
        watermark = wm if wm >= 0 else int(0.01 * num_blocks)
        wl = WorkloadConfig.from_args(a)
        wl.max_seq_len = max_seq_len
        trace_path = a.str("trace", "")
        trace_every = a.i32("trace-every", 1)
        kw = dict(num_blocks=num_blocks, block_size=block_size, max_seq_len=max_seq_len, prefix=a.flag("prefix"),
                  watermark=watermark, max_num_seqs=a.i32("max-num-seqs", 1024),
                  max_batched_tokens=a.i32("max-batched-tokens", 8192), prefill_chunk=a.i32("prefill-chunk", 0))
        a.warn_unused()
        trace = open(trace_path, "w") if trace_path else None
        if trace:
            trace.write("policy,step,running,waiting,blocks_in_use\n")
        print(f"pool {num_blocks} blocks of {block_size} tokens ({num_blocks * block_size * bpt / 2**30:.2f} GB), "
              f"{wl.describe()}")
        for pol in (["paged", "contiguous"] if policy == "both" else [policy]):
            r = simulate(pol, a, wl, trace=trace, trace_every=trace_every, **kw)
            print(f"[{r['policy']}] steps {r['steps']}  finished {r['finished']}  rejected {r['rejected']}  "
                  f"preemptions {r['preemptions']}  max running {r['max_running']}  mean batch {r['mean_batch']:.1f}  "
                  f"peak blocks {r['peak_blocks']}  mean waste {100 * r['mean_fragmentation']:.1f}%  "
                  f"prefill {r['prefill_tokens']} (saved {r['prefill_saved']})")
        if trace:
            trace.close()
    except Exception as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
