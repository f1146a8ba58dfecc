"""The reference arm of bench.py: the unmodified reference, built by its own CMake project, driven
through its own serving benchmark ``kvbench`` (src/main_bench.cpp) on a random weight file.

Nothing of this repository's engine is imported here.  What this file does:

* ``ensure_built`` configures and builds the reference's CMake project (tests off, which is its only
  network fetch: CMakeLists.txt:11,70-77; architecture through CMAKE_CUDA_ARCHITECTURES: :17-19)
  into ``baseline/_ref/build`` when ``kvbench`` is not there yet and the source tree is present.
* ``write_weight_file`` writes a file in the reference's own weight format (src/model/weights.cpp:
  24-46 for the 64-byte header, :69-82 for the order of the flat fp16 tensors) with N(0, 0.02)
  matrices and norm weights of 1.
* ``decode_run`` / ``prefill_run`` start ``kvbench`` with fixed prompt and output lengths
  (src/sim/workload.cpp:31-38) and ``--step-log`` (src/main_bench.cpp:66-67,89-92) and read the
  per-step milliseconds of the rows that are pure decode steps of the whole batch, or the prefill
  steps of one 2,048-token prompt.  The reference times a step on the host, from before scheduling to
  after the stream synchronize that ends its forward pass (src/engine/engine.cpp:75-88): that is an
  end-to-end time, and the only one its public path gives.
"""
from __future__ import annotations

import csv
import json
import os
import shutil
import struct
import subprocess
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
BUILD = os.path.join(HERE, "_ref", "build")
KVBENCH = os.path.join(BUILD, "kvbench")


class ReferenceUnavailable(RuntimeError):
    pass


def reference_source() -> str | None:
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            p = json.load(f).get("reference_path")
    except (OSError, ValueError):
        return None
    return p if p and os.path.isfile(os.path.join(p, "CMakeLists.txt")) else None


def ensure_built() -> str:
    if os.path.isfile(KVBENCH) and os.access(KVBENCH, os.X_OK):
        return KVBENCH
    src = reference_source()
    if src is None:
        raise ReferenceUnavailable("baseline/_ref/build/kvbench is not built and the reference's source tree "
                                   "is not on this machine")
    if shutil.which("cmake") is None or shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        raise ReferenceUnavailable("cmake or nvcc is missing: the reference's CMake project cannot be built")
    os.makedirs(BUILD, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    for cmd in (["cmake", "-S", src, "-B", BUILD, "-DKVP_BUILD_TESTS=OFF", "-DCMAKE_BUILD_TYPE=Release",
                 "-DCMAKE_CUDA_ARCHITECTURES=100a", f"-DCMAKE_CUDA_COMPILER={nvcc}"],
                ["cmake", "--build", BUILD, "-j", "16", "--target", "kvbench", "kvkernel", "kvsim"]):
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise ReferenceUnavailable("building the reference failed: " + r.stdout.strip().splitlines()[-1][:200])
    return KVBENCH


def write_weight_file(path: str, m: dict, seed: int = 0, repeat_block: bool = False) -> int:
    """Random weights in the reference's file format; returns the bytes written.  ``repeat_block``:
    draw 16 Mi values once and write them over and over (for the 7B and 8B shapes, whose 13-16 GB of
    distinct normals would take minutes to draw; speed does not depend on the values)."""
    import numpy as np
    V, H, I, L = m["vocab_size"], m["hidden_size"], m["intermediate_size"], m["num_hidden_layers"]
    nh, nkv, hd = m["num_attention_heads"], m["num_key_value_heads"], m["head_dim"]
    if nh * hd != H:
        raise ReferenceUnavailable("the reference assumes hidden == heads * head_dim (src/model/weights.h:23)")
    hdr = b"KVPW" + struct.pack("<9i", 1, V, H, I, L, nh, nkv, hd, m["max_position_embeddings"]) \
        + struct.pack("<2f", m["rope_theta"], m["rms_norm_eps"])
    hdr += b"\0" * (64 - len(hdr))
    rng = np.random.default_rng(seed)
    block = (rng.standard_normal(1 << 24, dtype=np.float32) * 0.02).astype(np.float16) if repeat_block else None

    def matrix(f, rows, cols):
        left = rows * cols
        while left:
            n = min(left, 1 << 24)
            if block is not None:
                f.write(block[:n].tobytes())
            else:
                f.write((rng.standard_normal(n, dtype=np.float32) * 0.02).astype(np.float16).tobytes())
            left -= n

    ones = np.ones(H, dtype=np.float16).tobytes()
    with open(path, "wb") as f:
        f.write(hdr)
        matrix(f, V, H)                                   # embed
        for _ in range(L):
            f.write(ones)                                 # attn_norm
            matrix(f, (nh + 2 * nkv) * hd, H)             # wqkv
            matrix(f, H, H)                               # wo
            f.write(ones)                                 # ffn_norm
            matrix(f, 2 * I, H)                           # w_gate_up
            matrix(f, H, I)                               # w_down
        f.write(ones)                                     # final_norm
        matrix(f, V, H)                                   # lm_head
        return f.tell()


def _run_kvbench(args: list[str], log: str, timeout: float) -> list[dict]:
    cmd = [ensure_built()] + args + ["--step-log", log]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout)
    if r.returncode != 0:
        tail = " | ".join(r.stdout.strip().splitlines()[-3:])[:300]
        raise ReferenceUnavailable(f"kvbench exited with {r.returncode}: {tail}")
    with open(log) as f:
        return [dict(row) for row in csv.DictReader(f)]


def decode_run(weights: str, batch: int, prompt_len: int, steps: int, warmup: int, kv_bytes_per_token: int,
               max_seq_len: int, workdir: str, timeout: float = 900.0) -> dict:
    """`batch` requests of `prompt_len` tokens; skips `warmup` pure decode steps and averages the next
    `steps` (host milliseconds of the reference's own step log)."""
    # The reference takes whole prompts, a few a step, while the requests it took earlier decode:
    # the first must still run when the last is in (at most one step a request).
    outputs = min(warmup + steps + 8 + batch, max_seq_len - prompt_len)
    pool_gb = batch * (max_seq_len + 64) * kv_bytes_per_token / float(1 << 30) * 1.1 + 0.1
    rows = _run_kvbench(["--weights", weights, "--policy", "paged", "--block-size", "16",
                         "--max-seq-len", str(max_seq_len), "--pool-gb", f"{pool_gb:.3f}",
                         "--max-num-seqs", str(batch), "--requests", str(batch),
                         "--prompt-len", str(prompt_len), "--output-len", str(outputs), "--rate", "0"],
                        os.path.join(workdir, f"steps_b{batch}.csv"), timeout)
    pure = [r for r in rows if int(r["prefill_tokens"]) == 0 and int(r["decode_seqs"]) == batch]
    if len(pure) < warmup + steps:
        raise ReferenceUnavailable(f"kvbench logged {len(pure)} pure decode steps of {batch} requests, "
                                   f"{warmup + steps} needed")
    timed = pure[warmup:warmup + steps]
    ms = sum(float(r["ms"]) for r in timed) / steps
    # Context of the timed steps: every request holds its prompt and what it decoded so far; the
    # first timed pure decode step is warm-up steps after the first pure one.
    first_pure = rows.index(pure[0])
    decoded_before = sum(int(r["decode_seqs"]) for r in rows[:first_pure]) / batch
    mean_ctx = prompt_len + decoded_before + warmup + (steps + 1) / 2.0
    return dict(ms_per_step=ms, mean_ctx=mean_ctx, steps_logged=len(rows))


def prefill_run(weights: str, tokens: int, reps: int, workdir: str, timeout: float = 900.0) -> float:
    """Median host milliseconds of the steps that prefill one prompt of `tokens` tokens alone."""
    rows = _run_kvbench(["--weights", weights, "--policy", "paged", "--block-size", "16",
                         "--max-seq-len", str(2 * tokens), "--pool-gb", "1.0", "--max-num-seqs", "1",
                         "--max-batched-tokens", str(tokens), "--requests", str(reps),
                         "--prompt-len", str(tokens), "--output-len", "1", "--rate", "0", "--warmup", "2"],
                        os.path.join(workdir, "steps_prefill.csv"), timeout)
    ms = sorted(float(r["ms"]) for r in rows if int(r["prefill_tokens"]) == tokens)
    if not ms:
        raise ReferenceUnavailable("kvbench logged no step with the whole prompt as its prefill")
    return ms[len(ms) // 2]


def make_workdir() -> str:
    return tempfile.mkdtemp(prefix="kvref_")
