#!/usr/bin/env python3
"""The reference's own serving benchmark on a named shape with random weights, on this machine.

    python baseline/reference_workloads.py llama-2-7b [kvbench flags ...]

Writes a weight file of the shape in the reference's format into a temporary folder (values drawn
once and repeated: 13 GB of distinct normals take minutes and change nothing), starts the unmodified
``kvbench`` (built by ``baseline/reference_arm.py``) with the flags given, and prints what it prints.
The shapes are those of this repository's presets (``kv-cache-manager_b200/cli/common.py``); the
reference's attention kernels take head sizes 64 and 128 and 1, 4 or 8 query heads to a KV head.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import reference_arm as ra  # noqa: E402

SHAPES = {
    "tinyllama-1.1b": dict(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22,
                           num_attention_heads=32, num_key_value_heads=4, head_dim=64, max_position_embeddings=2048,
                           rope_theta=10000.0, rms_norm_eps=1e-5),
    "llama-2-7b": dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                       num_attention_heads=32, num_key_value_heads=32, head_dim=128, max_position_embeddings=4096,
                       rope_theta=10000.0, rms_norm_eps=1e-5),
    "llama-3-8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                       num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=8192,
                       rope_theta=500000.0, rms_norm_eps=1e-5),
}


def main() -> int:
    if len(sys.argv) < 2 or sys.argv[1] not in SHAPES:
        print("usage: reference_workloads.py " + "|".join(SHAPES) + " [kvbench flags]", file=sys.stderr)
        return 2
    exe = ra.ensure_built()
    work = ra.make_workdir()
    try:
        weights = os.path.join(work, "weights.bin")
        n = ra.write_weight_file(weights, SHAPES[sys.argv[1]], seed=0, repeat_block=True)
        print(f"reference weights: {n / 2**30:.2f} GB in {weights}", flush=True)
        return subprocess.run([exe, "--weights", weights, *sys.argv[2:]]).returncode
    finally:
        shutil.rmtree(work, ignore_errors=True)


if __name__ == "__main__":
    sys.exit(main())
