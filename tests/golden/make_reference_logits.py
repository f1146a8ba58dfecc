#!/usr/bin/env python3
"""Logits of the reference engine on the small random models of golden_models.py.

    python tests/golden/make_reference_logits.py --build            # where the reference's sources are
    python tests/golden/make_reference_logits.py --run --out DIR    # on a machine with a GPU

``--build`` compiles reference_score_dump.cpp (beside this file) against the reference's headers
and the static libraries of its CMake build in ``baseline/_ref/build`` (made by
``baseline/reference_arm.py``).  ``--run`` writes each model in the reference's weight format into a
temporary folder, runs the dump tool on it (the reference's ``Engine::score``: its kernels, cuBLAS,
fp16 storage) and stores ``reference_logits_<model>.npy`` ([kept rows, vocab] float32: the logits of
the last rows of the sequence).  The files committed under tests/golden/ were made this way on a
B200; tests/test_reference_logits.py compares the plain implementation with them.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
BUILD = os.path.join(ROOT, "baseline", "_ref", "build")
EXE = os.path.join(BUILD, "reference_score_dump")
sys.path.insert(0, HERE)
import golden_models as gm  # noqa: E402


def build() -> int:
    with open(os.path.join(ROOT, "BASELINE.json")) as f:
        ref = json.load(f)["reference_path"]
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-O2", "-I", os.path.join(ref, "src"), "-I", os.path.join(cuda, "include"),
           os.path.join(HERE, "reference_score_dump.cpp"), os.path.join(BUILD, "libkvp_gpu.a"),
           os.path.join(BUILD, "libkvp_core.a"), "-L", os.path.join(cuda, "lib64"), "-lcudart", "-lcublas",
           f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}", "-o", EXE]
    return subprocess.run(cmd).returncode


def run(out: str) -> int:
    os.makedirs(out, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        for name, m in gm.MODELS.items():
            w, t, o = (os.path.join(tmp, f"{name}.{e}") for e in ("bin", "txt", "f32"))
            gm.write_reference_weight_file(name, w)
            toks = gm.token_ids(m["seed"], m["tokens"], m["cfg"]["vocab_size"])
            with open(t, "w") as f:
                f.write(" ".join(map(str, toks)))
            r = subprocess.run([EXE, w, t, o, str(m["keep"]), str(m["block_size"])])
            if r.returncode != 0:
                return r.returncode
            logits = np.fromfile(o, dtype="<f4").reshape(m["keep"], m["cfg"]["vocab_size"])
            np.save(os.path.join(out, f"reference_logits_{name}.npy"), logits)
            print(name, logits.shape, float(logits.std()))
    return 0


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--build", action="store_true")
    ap.add_argument("--run", action="store_true")
    ap.add_argument("--out", default=HERE)
    a = ap.parse_args()
    rc = 0
    if a.build:
        rc = build()
    if rc == 0 and a.run:
        rc = run(a.out)
    sys.exit(rc)
