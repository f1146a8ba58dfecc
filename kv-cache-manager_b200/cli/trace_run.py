"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and owns no forward pass, cache or loader: it drives the engine's model
loader, cache manager, batch builder and step function, the ones generation uses.  The nearest
thing in the reference is ``Engine::score`` (``src/engine/engine.cpp:92-108``), which scores one
whole sequence; here the caller decides step by step which tokens of which request run.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

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
    ap.add_argument("--attention", default="auto", choices=["auto", "plain"])
    ap.add_argument("--gemm", default="auto", choices=["auto", "plain", "library", "skinny", "tcgen05"])
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    print("trace_run: loading (the first call compiles the kernels; lines from [kvcm build] follow)",
          file=sys.stderr, flush=True)
    import torch
    from ..cache import core, manager_from_config
    from ..config import KVManagerConfig, canonical_dtype
    from ..engine import ModelRunner, load_model, torch_dtype

    dtype = canonical_dtype(args.dtype)
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this engine has no CPU path", file=sys.stderr)
        return 3
    os.makedirs(args.out, exist_ok=True)
    spec = load_model(args.model, dtype, args.device)
    B = args.block_size
    num_blocks = (args.max_tokens + B - 1) // B
    max_seq_len = num_blocks * B
    runner = ModelRunner(spec, torch_dtype(dtype), args.device, num_blocks=num_blocks, block_size=B,
                         max_seq_len=max_seq_len, num_slots=args.max_live, max_rows=max_seq_len,
                         max_seqs=args.max_live, max_logit_rows=max_seq_len,
                         options={"attention": args.attention, "gemm": args.gemm})
    kv = manager_from_config(KVManagerConfig(policy="paged", num_blocks=num_blocks, block_size=B,
                                             max_seq_len=max_seq_len, prefix_caching=False,
                                             watermark_blocks=0), runner.windows)
    slots = core.StateSlots(args.max_live)
    vocab = spec.lm_head.vocab
    live = {}
    next_id = 0

    def release(rid):
        seq = live.pop(rid)
        kv.release(seq)
        if seq.state_slot >= 0:
            slots.give_back(seq.state_slot)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        tag = step["step"]
        entries = []
        for e in step.get("entries", []):
            rid, toks = e["id"], [int(t) for t in e["tokens"]]
            want = [int(w) for w in e.get("want", [])]
            if not toks:
                raise SystemExit(f"trace_run: step {tag}: request {rid!r} brings no tokens")
            bad = [t for t in toks if t < 0 or t >= vocab]
            if bad:
                raise SystemExit(f"trace_run: step {tag}: token {bad[0]} outside the vocabulary of {vocab}")
            bad = [w for w in want if w < 0 or w >= len(toks)]
            if bad:
                raise SystemExit(f"trace_run: step {tag}: request {rid!r} wants place {bad[0]} of a portion of "
                                 f"{len(toks)} tokens")
            seq = live.get(rid)
            if seq is None:
                seq = core.Sequence()
                seq.id = next_id
                next_id += 1
                seq.state_slot = slots.take()
                if seq.state_slot < 0:
                    raise SystemExit(f"trace_run: step {tag}: more than {args.max_live} live requests")
                kv.admit(seq)                       # empty token list: starts the page tables
                runner.pools.reset_slot(seq.state_slot)
                live[rid] = seq
            start = seq.length()
            seq.extend_tokens(toks)
            if not kv.ensure(seq, seq.length()):
                raise SystemExit(f"trace_run: step {tag}: out of cache pages for request {rid!r} "
                                 f"({seq.length()} tokens; pool made for --max-tokens {args.max_tokens})")
            entries.append((seq, start, len(toks), want))
        if entries:
            logits = runner.step(entries)
            for seq, start, n, _ in entries:
                seq.num_computed = start + n
                kv.commit(seq)
            if logits is not None:
                logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False).tofile(
                    os.path.join(args.out, f"{tag}.f32"))
            else:
                torch.cuda.synchronize()
        for rid in step.get("end", []):
            if rid in live:
                release(rid)
        print(f"done {tag}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
