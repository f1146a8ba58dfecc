"""kvbench: end-to-end serving benchmark on the GPU (after the reference's ``src/main_bench.cpp``).

    kvbench --preset tinyllama-1.1b --policy paged --pool-gb 1 --requests 500 --rate 8 --summary out.csv

Requests arrive by a Poisson process in wall-clock time (``--rate`` req/s, 0 = all at once).  Token
contents are random.  Flags of the reference keep their names and meanings: --policy
paged|contiguous, --block-size, --max-seq-len, --prefix, --num-blocks, --watermark, --pool-gb,
--max-num-seqs, --max-batched-tokens, --attn v1|v2|auto, --warmup, --summary CSV, --step-log CSV,
--time-limit s, and the workload flags (--requests --rate --prompt-mu --prompt-sigma --output-mu
--output-sigma --min-prompt --max-prompt --min-output --max-output --shared-frac --shared-len
--num-prefixes --lengths-csv --seed --prompt-len --output-len).  Added: --model DIR | --preset NAME
[--random-seed S], --dtype, --temperature, --sampling-seed, --prefill-chunk, --no-chunked-prefill,
--no-graphs, --gemm auto|native|library|plain (native: only this engine's product kernels),
--profile (device time per kernel family, from an event after every launch; runs without CUDA graphs).
"""
from __future__ import annotations

import math
import sys
import time


def main(argv=None) -> int:
    from .args import Args
    from .common import engine_config_from_args, load_model_from_args
    a = Args(argv)
    try:
        import torch
        from ..engine.engine import Engine
        from ..engine.metrics import BenchSummary, MetricsCollector, append_bench_csv, print_summary
        from ..engine.workload import WorkloadConfig, generate_workload, make_prompt_tokens
        ec = engine_config_from_args(a)
        profile = a.flag("profile")
        if profile:
            ec.cuda_graphs = False           # events cannot be recorded into a graph
        wl = WorkloadConfig.from_args(a)
        wl.max_seq_len = ec.kv.max_seq_len
        warmup = a.i32("warmup", 8)
        summary_csv, step_log = a.str("summary", ""), a.str("step-log", "")
        time_limit = a.f64("time-limit", 1e9)
        temperature = a.f64("temperature", 0.0)
        spec = load_model_from_args(a, ec.dtype)
        a.warn_unused()
        wl.vocab = spec.lm_head.vocab
        eng = Engine(spec, ec)
        print(f"KV pool {ec.kv.num_blocks} blocks x {eng.runner.bytes_per_block()} B = "
              f"{eng.runner.pools.total_bytes() / 2**30:.2f} GB, dtype {ec.dtype}")

        if warmup > 0:                       # short requests: library heuristics, kernel attributes, graphs
            w = WorkloadConfig(**{**wl.__dict__, "num_requests": warmup, "arrival_rate": 0.0, "shared_frac": 0.0,
                                  "seed": wl.seed + 999, "min_output": 16, "max_output": 16, "output_sigma": 0.0,
                                  "output_mu": math.log(16.0)})
            for r in generate_workload(w):
                eng.add_request(make_prompt_tokens(r, w), r.output_len)
            eng.run_until_idle()
            eng.take_finished()
            eng.sched.reset_counters()
        ps0 = eng.kv.prefix_stats()
        if profile:
            from ..kernels import library as K
            K.profile_start()
        reqs = generate_workload(wl)
        log = open(step_log, "w") if step_log else None
        if log:
            log.write("t,rows,seqs,prefill_tokens,decode_seqs,ms,running,waiting,blocks_in_use\n")
        mc, s = MetricsCollector(), BenchSummary()
        nxt, step_ms_sum, done = 0, 0.0, 0
        eng.reset_clock()
        while done < len(reqs):
            now = eng.now()
            if now > time_limit:
                print("time limit reached")
                break
            while nxt < len(reqs) and reqs[nxt].arrival <= now:
                r = reqs[nxt]
                eng.add_request(make_prompt_tokens(r, wl), r.output_len, temperature, arrival=r.arrival)
                nxt += 1
            if eng.idle():
                if nxt < len(reqs):
                    time.sleep(max(0.0, reqs[nxt].arrival - eng.now()))
                continue
            si = eng.step()
            step_ms_sum += si.ms
            s.peak_blocks = max(s.peak_blocks, eng.kv.blocks_in_use())
            if log:
                log.write(f"{eng.now():.4f},{si.rows},{si.seqs},{si.prefill_tokens},{si.decode_seqs},{si.ms:.3f},"
                          f"{eng.sched.num_running()},{eng.sched.num_waiting()},{eng.kv.blocks_in_use()}\n")
            for f in eng.take_finished():
                mc.add_finished(f)
                done += 1
        wall = eng.now()
        if log:
            log.close()
        c = eng.sched.counters()
        s.policy, s.block_size, s.num_blocks = eng.kv.name(), ec.kv.block_size, ec.kv.num_blocks
        s.pool_gb = eng.runner.pools.total_bytes() / 2**30
        s.rate, s.shared_frac, s.requests = wl.arrival_rate, wl.shared_frac, len(reqs)
        mc.finalize(s, wall)
        s.mean_batch = c.batch_size_sum / c.steps if c.steps else 0.0
        s.max_batch, s.preemptions, s.steps = c.max_running, c.preemptions, c.steps
        s.mean_step_ms = step_ms_sum / c.steps if c.steps else 0.0
        s.prefill_tokens, s.prefill_saved = c.prefill_tokens, c.prefill_tokens_saved
        ps = eng.kv.prefix_stats()
        q = ps.queried_blocks - ps0.queried_blocks
        s.prefix_hit_rate = (ps.hit_blocks - ps0.hit_blocks) / q if q else 0.0
        s.evictions = ps.evictions - ps0.evictions
        s.peak_kv_gb = s.peak_blocks * eng.runner.bytes_per_block() / 2**30
        free_b, total_b = torch.cuda.mem_get_info()
        s.gpu_used_gb = (total_b - free_b) / 2**30
        print_summary(s)
        if profile:
            fam = K.profile_stop()
            total = sum(ms for _, ms in fam.values()) or 1.0
            print(f"profile: device time per kernel family ({total:.1f} ms in {sum(c for c, _ in fam.values())} launches)")
            for name, (calls, ms) in sorted(fam.items(), key=lambda kv: -kv[1][1]):
                print(f"profile: {name or 'other':<28} {calls:>8} launches {ms:>10.2f} ms {100 * ms / total:>6.1f} %")
        if summary_csv:
            append_bench_csv(summary_csv, s)
    except (Exception, SystemExit) as e:
        if isinstance(e, SystemExit) and e.code in (0, None):
            return 0
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
