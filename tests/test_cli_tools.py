"""Command-line pieces that need no GPU: the flag parser, the workload generator, the metrics,
and the scheduler/cache simulator (kvsim)."""
import io
import math
import os
import subprocess
import sys

import pytest

from kvcm.cli.args import Args
from kvcm.engine.metrics import BenchSummary, MetricsCollector, append_bench_csv, percentile
from kvcm.engine.workload import WorkloadConfig, generate_workload, make_prompt_tokens

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_args_forms_and_unused_warning(capsys):
    a = Args(["--policy=paged", "--block-size", "32", "--prefix", "--rate", "2.5", "--typo", "x"])
    assert a.str("policy", "contiguous") == "paged" and a.i32("block-size", 16) == 32
    assert a.flag("prefix") and not a.flag("absent") and a.f64("rate", 0) == 2.5
    assert a.i32("missing", 7) == 7 and a.has("rate") and not a.has("nothing")
    assert a.ints("ctx", "1,2,3") == [1, 2, 3]
    a.warn_unused()
    assert "unused flag --typo" in capsys.readouterr().err
    with pytest.raises(ValueError):
        Args(["positional"])


def test_workload_lengths_clamps_and_shared_prefixes():
    c = WorkloadConfig(num_requests=400, arrival_rate=8.0, shared_frac=0.6, shared_len=32, num_shared_prefixes=4,
                       max_seq_len=512, vocab=1000, seed=3)
    reqs = generate_workload(c)
    assert len(reqs) == 400 and all(b.arrival >= a.arrival for a, b in zip(reqs, reqs[1:]))
    assert all(1 <= r.prompt_len <= 511 and 1 <= r.output_len and r.prompt_len + r.output_len <= 512 for r in reqs)
    shared = [r for r in reqs if r.prefix_id >= 0]
    assert 0.45 < len(shared) / 400 < 0.75 and {r.prefix_id for r in shared} == {0, 1, 2, 3}
    a, b = [r for r in shared if r.prefix_id == 2][:2]
    ta, tb = make_prompt_tokens(a, c), make_prompt_tokens(b, c)
    assert ta[:32] == tb[:32] and ta[32:40] != tb[32:40] and len(ta) == a.prompt_len
    assert all(3 <= t < 1000 for t in ta)
    assert make_prompt_tokens(a, c) == ta                                  # deterministic
    mean_gap = reqs[-1].arrival / 400
    assert 0.08 < mean_gap < 0.18                                          # Poisson at 8 requests/s
    burst = generate_workload(WorkloadConfig(num_requests=5, arrival_rate=0))
    assert all(r.arrival == 0 for r in burst)


def test_workload_fixed_lengths_from_flags():
    c = WorkloadConfig.from_args(Args(["--prompt-len", "100", "--output-len", "20", "--requests", "3"]))
    assert [(r.prompt_len, r.output_len) for r in generate_workload(c)] == [(100, 20)] * 3


def test_percentile_and_metrics(tmp_path):
    assert percentile([], 0.5) == 0 and percentile([1, 2, 3, 4], 0.5) == 2.5 and percentile([5], 0.99) == 5

    class S:                      # what the collector reads of a finished request
        def __init__(self, arrival, first, fin, prompt, out):
            self.arrival, self.first_token, self.finished, self.prompt_len, self._out = arrival, first, fin, prompt, out

        def num_generated(self):
            return self._out
    mc = MetricsCollector()
    mc.add_finished(S(0.0, 0.1, 1.1, 10, 11))
    mc.add_finished(S(0.5, 0.7, 0.7, 5, 1))
    mc.add_finished(S(0.0, -1, 0.2, 99, 0))                                # rejected: no first token
    s = BenchSummary()
    mc.finalize(s, 2.0)
    assert (s.completed, s.rejected, s.output_tokens, s.prompt_tokens) == (2, 1, 12, 15)
    assert abs(s.ttft_mean - 0.15) < 1e-9 and abs(s.tpot_mean_ms - 100.0) < 1e-6 and s.out_tok_s == 6.0
    p = str(tmp_path / "s.csv")
    append_bench_csv(p, s)
    append_bench_csv(p, s)
    lines = open(p).read().splitlines()
    assert len(lines) == 3 and lines[0].startswith("policy,block_size") and lines[0].count(",") == lines[1].count(",")


def test_kvsim_paged_holds_more_requests_than_contiguous():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kvsim"), "--pool-gb", "1", "--requests", "200"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    rows = {l.split("]")[0][1:]: l for l in out.stdout.splitlines() if l.startswith("[")}
    get = lambda l, k: float(l.split(k)[1].split()[0].rstrip('%'))
    assert get(rows["paged"], "max running") > 4 * get(rows["contiguous"], "max running")
    assert get(rows["contiguous"], "max running") == 2978 // 128          # pool pages / pages reserved per request
    assert get(rows["paged"], "finished") == 200 and get(rows["contiguous"], "finished") == 200
    assert get(rows["contiguous"], "mean waste") > 50 > get(rows["paged"], "mean waste")
