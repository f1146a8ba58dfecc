"""Serving metrics as the reference reports them (``src/engine/metrics.cpp:11-96``):
TTFT = first token - arrival, E2E = finished - arrival, TPOT = (finished - first token) /
(outputs - 1); percentiles with linear interpolation; one CSV row per run."""
from __future__ import annotations

import math
import os
from dataclasses import asdict, dataclass, field
from typing import List


def percentile(values: List[float], p: float) -> float:
    if not values:
        return 0.0
    v = sorted(values)
    idx = p * (len(v) - 1)
    lo, hi = int(math.floor(idx)), int(math.ceil(idx))
    return v[lo] + (v[hi] - v[lo]) * (idx - lo)


@dataclass
class BenchSummary:
    policy: str = ""
    block_size: int = 0
    num_blocks: int = 0
    pool_gb: float = 0.0
    rate: float = 0.0
    shared_frac: float = 0.0
    requests: int = 0
    completed: int = 0
    rejected: int = 0
    wall_s: float = 0.0
    output_tokens: int = 0
    prompt_tokens: int = 0
    out_tok_s: float = 0.0
    total_tok_s: float = 0.0
    req_s: float = 0.0
    ttft_mean: float = 0.0
    ttft_p50: float = 0.0
    ttft_p95: float = 0.0
    ttft_p99: float = 0.0
    e2e_p50: float = 0.0
    e2e_p95: float = 0.0
    e2e_p99: float = 0.0
    tpot_mean_ms: float = 0.0
    mean_batch: float = 0.0
    max_batch: int = 0
    preemptions: int = 0
    steps: int = 0
    mean_step_ms: float = 0.0
    prefill_tokens: int = 0
    prefill_saved: int = 0
    prefix_hit_rate: float = 0.0
    evictions: int = 0
    peak_blocks: int = 0
    peak_kv_gb: float = 0.0
    gpu_used_gb: float = 0.0


class MetricsCollector:
    def __init__(self) -> None:
        self.ttft: List[float] = []
        self.e2e: List[float] = []
        self.tpot: List[float] = []
        self.out_tokens = 0
        self.prompt_tokens = 0
        self.rejected = 0

    def add_finished(self, s) -> None:
        if s.first_token < 0:
            self.rejected += 1
            return
        self.ttft.append(s.first_token - s.arrival)
        self.e2e.append(s.finished - s.arrival)
        out = s.num_generated()
        if out > 1:
            self.tpot.append((s.finished - s.first_token) / (out - 1))
        self.out_tokens += out
        self.prompt_tokens += s.prompt_len

    def count(self) -> int:
        return len(self.ttft)

    def finalize(self, o: BenchSummary, wall_s: float) -> None:
        mean = lambda v: sum(v) / len(v) if v else 0.0
        wall_s = max(wall_s, 1e-9)
        o.completed, o.rejected, o.wall_s = len(self.ttft), self.rejected, wall_s
        o.output_tokens, o.prompt_tokens = self.out_tokens, self.prompt_tokens
        o.out_tok_s = self.out_tokens / wall_s
        o.total_tok_s = (self.out_tokens + self.prompt_tokens) / wall_s
        o.req_s = o.completed / wall_s
        o.ttft_mean = mean(self.ttft)
        o.ttft_p50, o.ttft_p95, o.ttft_p99 = (percentile(self.ttft, p) for p in (0.5, 0.95, 0.99))
        o.e2e_p50, o.e2e_p95, o.e2e_p99 = (percentile(self.e2e, p) for p in (0.5, 0.95, 0.99))
        o.tpot_mean_ms = 1e3 * mean(self.tpot)


def print_summary(s: BenchSummary) -> None:
    print(f"[{s.policy}] B={s.block_size} blocks={s.num_blocks} ({s.pool_gb:.2f} GB) rate={s.rate:g} shared={s.shared_frac:g}")
    print(f"  completed {s.completed}/{s.requests} (rejected {s.rejected}) in {s.wall_s:.2f}s, "
          f"{s.steps} steps ({s.mean_step_ms:.2f} ms/step)")
    print(f"  throughput: {s.out_tok_s:.1f} out tok/s, {s.total_tok_s:.1f} total tok/s, {s.req_s:.2f} req/s")
    print(f"  TTFT p50/p95/p99 = {s.ttft_p50:.3f} / {s.ttft_p95:.3f} / {s.ttft_p99:.3f} s   "
          f"E2E p50/p95/p99 = {s.e2e_p50:.3f} / {s.e2e_p95:.3f} / {s.e2e_p99:.3f} s")
    print(f"  TPOT mean {s.tpot_mean_ms:.2f} ms   batch mean {s.mean_batch:.1f} max {s.max_batch}   "
          f"preemptions {s.preemptions}")
    print(f"  prefill tokens {s.prefill_tokens} (saved {s.prefill_saved}, block hit rate "
          f"{100 * s.prefix_hit_rate:.1f}%, evictions {s.evictions})")
    print(f"  peak KV blocks {s.peak_blocks} ({s.peak_kv_gb:.3f} GB), GPU memory used {s.gpu_used_gb:.2f} GB")


def append_bench_csv(path: str, s: BenchSummary) -> None:
    d = asdict(s)
    fresh = not os.path.exists(path) or os.path.getsize(path) == 0
    with open(path, "a") as f:
        if fresh:
            f.write(",".join(d) + "\n")
        f.write(",".join(f"{v:.4f}" if isinstance(v, float) else str(v) for v in d.values()) + "\n")
