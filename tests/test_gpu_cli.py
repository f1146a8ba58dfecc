"""The command-line tools as a user runs them, on a tiny random model: exit code and the lines
they promise (``bin/kvbench``, ``bin/kvcorrect``, ``bin/kvkernel``)."""
import os
import subprocess
import sys

import pytest

import helpers

pytestmark = pytest.mark.gpu


def run(tool, *args, timeout=900):
    p = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "bin", tool), *args], text=True,
                       stdout=subprocess.PIPE, stderr=subprocess.PIPE, timeout=timeout)
    return p.returncode, p.stdout, p.stderr


def test_kvbench_serves_a_workload_and_writes_its_files(tmp_path):
    summary, steps = str(tmp_path / "summary.csv"), str(tmp_path / "steps.csv")
    rc, out, err = run("kvbench", "--preset", "tiny-c", "--requests", "24", "--rate", "0", "--prompt-mu", "3.5",
                       "--prompt-sigma", "0.6", "--output-mu", "2.5", "--output-sigma", "0.5", "--max-prompt", "200",
                       "--max-output", "40", "--max-seq-len", "256", "--num-blocks", "96", "--max-num-seqs", "6",
                       "--max-batched-tokens", "128", "--prefix", "--shared-frac", "0.5", "--shared-len", "32",
                       "--warmup", "2", "--summary", summary, "--step-log", steps)
    assert rc == 0, err[-2000:]
    assert "KV pool 96 blocks" in out and "completed 24/24" in out
    rows = open(summary).read().strip().splitlines()
    assert len(rows) == 2 and rows[0].split(",")[0] == "policy" and rows[1].startswith("paged+prefix")
    log = open(steps).read().strip().splitlines()
    assert log[0] == "t,rows,seqs,prefill_tokens,decode_seqs,ms,running,waiting,blocks_in_use" and len(log) > 20
    assert "warning: unused flag" not in err


def test_kvbench_profile_mode_names_the_kernel_families(tmp_path):
    rc, out, err = run("kvbench", "--preset", "tiny-c", "--requests", "6", "--prompt-len", "40", "--output-len", "8",
                       "--max-seq-len", "128", "--num-blocks", "64", "--max-num-seqs", "4", "--warmup", "1", "--profile")
    assert rc == 0, err[-2000:]
    lines = [l for l in out.splitlines() if l.startswith("profile:")]
    names = " ".join(lines)
    assert len(lines) >= 6 and "rmsnorm" in names and "argmax" in names and "attention" in names
    shares = [float(l.split()[-2]) for l in lines[1:]]
    assert 99.0 < sum(shares) < 101.0


def test_kvcorrect_passes_on_a_tiny_model():
    rc, out, err = run("kvcorrect", "--preset", "tiny-c", "--steps", "12", "--prompts", "4", "--prompt-len", "48")
    assert rc == 0, out[-2000:] + err[-2000:]
    assert out.count("[PASS]") >= 5 and "[FAIL]" not in out and "all checks passed" in out


def test_kvkernel_families(tmp_path):
    csv = str(tmp_path / "attn.csv")
    rc, out, err = run("kvkernel", "--family", "attention", "--ctx", "256", "--batch", "2", "--iters", "5", "--out", csv)
    assert rc == 0, err[-2000:]
    assert "paged-v2" in out and "HBM peak" in out
    assert len(open(csv).read().strip().splitlines()) == 5
    rc, out, err = run("kvkernel", "--family", "gemm", "--batch", "4", "--hidden", "256", "--ffn", "512", "--vocab", "1000",
                       "--heads", "4", "--kv-heads", "2", "--head-dim", "64")
    assert rc == 0, err[-2000:]
    assert "gate_up" in out and "lm_head" in out
    rc, out, err = run("kvkernel", "--family", "nonsense")
    assert rc != 0
