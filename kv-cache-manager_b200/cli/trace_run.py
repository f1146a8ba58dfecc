"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and owns no forward pass, cache or loader: it drives the engine's model
loader, cache manager, batch builder and step function, the ones generation uses.  The nearest
thing in the reference is ``Engine::score`` (``src/engine/engine.cpp:92-108``), which scores one
whole sequence; here the caller decides step by step which tokens of which request run.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
              [--policy paged|contiguous] [--prefix] [--block-size B] [--max-seq-len L]

Steps are read from standard input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, ``DIR/<step>.f32`` receives the logits at the wanted
places ([wanted, vocab], little-endian float32, in the order of the entries and of ``want``).
After every step ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", help="bfloat16 (serving kernels) | float32 (true 32-bit)")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (sizes the page pool)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--max-live", type=int, default=64, help="most requests live at a time")
    ap.add_argument("--policy", default="paged", choices=["paged", "contiguous"],
                    help="cache policy (the reference's two: src/core/kv_manager.h:64-72)")
    ap.add_argument("--prefix", action="store_true",
                    help="prefix caching: a new request takes over the cached pages that match its first "
                         "portion; those tokens are not computed and their places cannot be wanted")
    ap.add_argument("--max-seq-len", type=int, default=0,
                    help="longest request (0: the whole pool when paged, a quarter of it when contiguous, "
                         "where every request reserves this many tokens)")
    ap.add_argument("--attention", default="auto", choices=["auto", "plain"])
    ap.add_argument("--gemm", default="auto", choices=["auto", "plain", "library", "tcgen05", "native"])
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    print("trace_run: loading (the first call compiles the kernels; lines from [kvcm build] follow)",
          file=sys.stderr, flush=True)
    import torch
    from ..config import canonical_dtype
    from ..engine import load_model
    from ..engine.replay import ReplayError, ReplaySession
    from ..kernels import library as K

    dtype = canonical_dtype(args.dtype)
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this engine has no CPU path", file=sys.stderr)
        return 3
    os.makedirs(args.out, exist_ok=True)
    spec = load_model(args.model, dtype, args.device)
    session = ReplaySession(spec, dtype, args.max_tokens, block_size=args.block_size, max_live=args.max_live,
                            policy=args.policy, prefix_caching=args.prefix, max_seq_len=args.max_seq_len,
                            options={"attention": args.attention, "gemm": args.gemm}, device=args.device)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        tag = step["step"]
        try:
            logits = session.step(step.get("entries", []), step.get("end", []), tag=tag)
        except ReplayError as e:
            raise SystemExit(f"trace_run: {e}")
        torch.cuda.synchronize()
        K.check_errors()                            # a kernel that gave up a bounded wait: no logits are written
        if logits is not None:
            logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False).tofile(
                os.path.join(args.out, f"{tag}.f32"))
        print(f"done {tag}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
