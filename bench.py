#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second at TinyLlama-1.1B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A *step* is one decode step of the whole batch.  The default run has the layer sizes of the
reference's benchmark model (TinyLlama 1.1B: 22 layers, hidden 2048, 32 query / 4 KV heads of
64, FFN 5632, vocabulary 32000) with random bfloat16 weights, a batch of 8 requests with
1,024-token prompts that are decoded towards 2,048 tokens.  It prints ONE JSON line:

* ``value``     decoded tokens per second, from CUDA events around the device work of each of
                the K timed steps (kernels of the step, without the host's batch building);
* ``e2e``       the same K steps through the Python entry point (``Engine.step``): host tokens in
                through one pinned host-to-device copy per step, sampled tokens read back;
* ``prefill``   one 2,048-token prompt in one step: tokens/s, ms and fraction of the bf16 peak;
* ``roofline``  bytes the decode step must read (every weight once, the cache of the live
                requests) over its time, against the HBM copy bandwidth;
* ``points``    decode tokens/s at batch 1 and 64, each with the same roofline fraction
                (``decode_b1_hbm_frac``, ``decode_b64_hbm_frac``).

The timed decode window is centred on a context of 1,536 tokens (the middle of 1,024 -> 2,048)
whatever K is: prompts have ``1536 - W - K/2`` tokens, which is 1,020 for the default K = 1,000.

This engine is single-GPU: for ``--gpus N`` with N > 1 it says so and exits with 2.  The
reference arm (``--impl reference``) runs the unmodified reference, built by its own CMake project
under ``baseline/_ref``, through its serving benchmark ``kvbench`` on a random weight file of the
same shape, with the same prompts lengths, batch and steps (``baseline/reference_arm.py``); it
prints the same JSON line with ``"impl": "reference"``, or one ``unavailable`` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Layer sizes of the benchmark model (the reference's TinyLlama-1.1B, docs/design.md:3-7).
MODEL = dict(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22,
             num_attention_heads=32, num_key_value_heads=4, head_dim=64,
             max_position_embeddings=2048, rope_theta=10000.0, rms_norm_eps=1e-5,
             tie_word_embeddings=False)
PROMPT_LEN = 1024          # of the metric; the run's own prompt length centres the timed window
MID_CONTEXT = 1536         # middle of 1,024 -> 2,048
CONTEXT = 2048
PREFILL_TOKENS = 2048
BLOCK_SIZE = 16
# Reference numbers (RTX 4080, its own trace): decode tokens/s at batch 1 / 8 / 64.
PUBLISHED = {1: 222.0, 8: 1643.0, 64: 9257.0}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    try:
        with open(p) as f:
            d = json.load(f)
        for k in FALLBACK_PEAKS:
            if isinstance(d.get(k), (int, float)) and d[k] > 0:
                out[k] = float(d[k])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6
                          for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": int(statistics.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


def model_bytes_and_flops(cfg, layers):
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = (cfg.qkv_dim * H + H * cfg.q_dim + 2 * I * H + H * I)
    weights = per_layer * layers + V * H                       # matrices read by a decode step
    norms = (2 * layers + 1) * H
    kv_per_token = 2 * layers * cfg.kv_dim
    return dict(matrix_params=weights, weight_bytes=2 * (weights + norms),
                kv_bytes_per_token=2 * kv_per_token, per_layer_params=per_layer)


def build_engine(layers, batch, max_len, graphs=True, max_batched=4096):
    import torch
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, LlamaConfig, SchedulerConfig
    from kvcm.engine import Engine, model_from_tensors
    from kvcm.weights import random_tensors
    cfg = LlamaConfig(architecture="LlamaForCausalLM", **dict(MODEL, num_hidden_layers=layers))
    tensors = dict(random_tensors(cfg, 0, torch.bfloat16, device="cuda:0"))
    spec = model_from_tensors(cfg, tensors, "bfloat16", "cuda:0")
    del tensors
    pages = batch * ((max_len + BLOCK_SIZE - 1) // BLOCK_SIZE + 1) + 8
    ec = EngineConfig(kv=KVManagerConfig(num_blocks=pages, block_size=BLOCK_SIZE, max_seq_len=max_len,
                                         watermark_blocks=0),
                      sched=SchedulerConfig(max_num_seqs=max(batch, 8), max_batched_tokens=max_batched),
                      dtype="bfloat16", cuda_graphs=graphs)
    return cfg, spec, ec


def window_prompt_len(steps, warmup):
    """Prompt length that puts the middle of the timed steps at a context of MID_CONTEXT tokens."""
    return max(16, MID_CONTEXT - warmup - steps // 2)


def decode_run(spec, ec, vocab, batch, steps, warmup, prompt_len, sample_clocks=False):
    """Prefills `batch` prompts of `prompt_len` tokens, runs `warmup` untimed and `steps` timed decode
    steps through Engine.step().  Returns device ms, wall ms, copies per step, launches per step."""
    import torch
    from kvcm.engine.engine import DeviceTimer, Engine
    from kvcm.kernels import launch_count
    eng = Engine(spec, ec)
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(3, vocab, (batch, prompt_len), generator=g).tolist()
    for p in prompts:
        eng.add_request(p, max_new_tokens=1 << 30)   # ends only at max_seq_len, sized with headroom
    while eng.sched.num_waiting() or eng.sched.counters().prefill_tokens < batch * prompt_len:
        eng.step()                                   # prompt portions (and the first tokens)
    for _ in range(warmup):
        info = eng.step()
    assert info.decode_seqs == batch and info.prefill_tokens == 0, "warm-up must end in pure decoding"
    torch.cuda.synchronize()
    clocks = ClockSampler()
    if sample_clocks:
        clocks.start()
        time.sleep(0.25)
    timer = DeviceTimer()
    eng.device_timer = timer
    h2d = d2h = 0
    launches0 = launch_count()
    graph_kernels = 0
    ctx_sum = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        info = eng.step()
        h2d += info.h2d_bytes
        d2h += info.d2h_bytes
        if info.graph and eng.native is None:
            graph_kernels += eng.graphs.kernels_last       # (the C++ loop reports its launches itself)
        ctx_sum += eng.sched.cached_tokens_total()
    wall_ms = (time.perf_counter() - t0) * 1e3     # the host holds the tokens of `steps` steps
    dev_ms = timer.total_ms()                      # device time of exactly these steps
    if eng.native is not None:
        eng.native.drain()                         # (a step enqueued ahead ends outside the timed region)
    torch.cuda.synchronize()
    eager_kernels = launch_count() - launches0
    eng.device_timer = None
    clk = clocks.stop() if sample_clocks else None
    assert info.decode_seqs == batch, f"a request ended inside the timed region: {info}"
    res = dict(dev_ms=dev_ms, wall_ms=wall_ms, h2d=h2d / steps, d2h=d2h / steps,
               launches=graph_kernels + eager_kernels, mean_ctx=ctx_sum / (steps * batch), clocks=clk,
               graph_steps=eng.graphs.replays if eng.graphs else 0)
    del eng
    torch.cuda.empty_cache()
    return res


def prefill_run(spec, ec, vocab, cfg, layers, reps=5):
    """One prompt of PREFILL_TOKENS tokens in one step.  Returns (device ms, flops, end-to-end ms): the
    device time of the step's kernels from CUDA events, and the wall time of the same step through
    ``Engine.add_request`` + ``Engine.step`` (host tokens in, the first sampled token out)."""
    import torch
    from kvcm.engine.engine import DeviceTimer, Engine
    eng = Engine(spec, ec)
    g = torch.Generator().manual_seed(2)
    dev, wall = [], []
    for r in range(reps + 2):
        toks = torch.randint(3, vocab, (PREFILL_TOKENS,), generator=g).tolist()
        timer = DeviceTimer()
        eng.device_timer = timer
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.add_request(toks, max_new_tokens=1)
        info = eng.step()
        t1 = time.perf_counter()
        assert info.prefill_tokens == PREFILL_TOKENS and info.sampled == 1, info
        eng.take_finished()
        ms = timer.total_ms()
        eng.device_timer = None
        if r >= 2:
            dev.append(ms)
            wall.append((t1 - t0) * 1e3)
    m = model_bytes_and_flops(cfg, layers)
    T = PREFILL_TOKENS
    gemm_flops = 2.0 * m["per_layer_params"] * layers * T + 2.0 * cfg.vocab_size * cfg.hidden_size
    attn_flops = 4.0 * cfg.head_dim * cfg.num_attention_heads * (T * (T + 1) / 2) * layers
    del eng
    torch.cuda.empty_cache()
    return statistics.median(dev), gemm_flops + attn_flops, statistics.median(wall)

def reference_main(args) -> int:
    """The same metric and shape through the unmodified reference (fp16, its own kvbench)."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ra
    if args.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a single-GPU engine"}))
        return 0
    steps, warmup, B = args.steps, max(args.warmup, 3), args.batch
    layers = MODEL["num_hidden_layers"]
    prompt_len = window_prompt_len(steps, warmup)
    kv_per_token = 2 * 2 * layers * MODEL["num_key_value_heads"] * MODEL["head_dim"]
    max_len = max(CONTEXT, prompt_len + warmup + steps + 64 + 16)
    pk = peaks()
    work = None
    try:
        ra.ensure_built()
        work = ra.make_workdir()
        wfile = os.path.join(work, "weights.bin")
        ra.write_weight_file(wfile, MODEL, seed=0)
        clocks = ClockSampler()
        clocks.start()
        main_run = ra.decode_run(wfile, B, prompt_len, steps, warmup, kv_per_token, max_len, work)
        clk = clocks.stop()
        pts, prefill = {}, None
        if not args.no_points:
            for b in (1, 64):
                r = ra.decode_run(wfile, b, prompt_len, steps, warmup, kv_per_token, max_len, work)
                pts[f"decode_b{b}"] = round(b * 1e3 / r["ms_per_step"], 1)
            prefill = ra.prefill_run(wfile, PREFILL_TOKENS, 7, work)
    except ra.ReferenceUnavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return 0
    except subprocess.TimeoutExpired:
        print(json.dumps({"impl": "reference", "unavailable": "the reference's kvbench did not end in time"}))
        return 0
    finally:
        if work:
            import shutil
            shutil.rmtree(work, ignore_errors=True)
    H, I, V = MODEL["hidden_size"], MODEL["intermediate_size"], MODEL["vocab_size"]
    qkv = (MODEL["num_attention_heads"] + 2 * MODEL["num_key_value_heads"]) * MODEL["head_dim"]
    per_layer = qkv * H + H * H + 2 * I * H + H * I
    weight_bytes = 2 * (per_layer * layers + V * H + (2 * layers + 1) * H)
    ms = main_run["ms_per_step"]
    value = B * 1e3 / ms
    achieved = (weight_bytes + B * main_run["mean_ctx"] * kv_per_token) / (ms * 1e-3) / 1e9
    out = {
        "metric": "decode tokens/s (TinyLlama-1.1B shape, batch 8, 1,024-token prompts decoded towards 2,048)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / PUBLISHED[B], 2) if B in PUBLISHED else None,
        "dtype": "fp16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "impl": "reference",
        "config": {"model": "TinyLlama-1.1B shape (Llama dense decoder)", "layers": layers,
                   "layers_full": layers, "hidden": H, "heads": MODEL["num_attention_heads"],
                   "kv_heads": MODEL["num_key_value_heads"], "head_dim": MODEL["head_dim"], "ffn": I,
                   "vocab": V, "global_batch": B, "seq_len": CONTEXT, "prompt_len": prompt_len,
                   "mean_context": round(main_run["mean_ctx"], 1), "kv_block": BLOCK_SIZE,
                   "parallelism": "single GPU", "cuda_graphs": False, "gemm": "cuBLAS",
                   "l2": "inputs larger than L2 (2.2 GB of weights read per step)",
                   "peaks": pk["source"],
                   "timing": "host clock of the reference's own step log (schedule, copies, forward, synchronize)"},
        # The reference has one clock, around its whole step on the host: both figures are that one.
        "e2e": {"value": round(value, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(4 * (6 * B + B * ((max_len + BLOCK_SIZE - 1) // BLOCK_SIZE))),
                "d2h_bytes_per_step": 4 * B},
        "gpu_launches": 13 * layers + 4 + 2 * layers,   # src/model/llama.cpp:104-129, attention v2 adds its merge
        "clocks": clk,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]},
    }
    if pts:
        out["points"] = pts
    if prefill:
        flops = 2.0 * per_layer * layers * PREFILL_TOKENS + 2.0 * V * H \
            + 4.0 * MODEL["head_dim"] * MODEL["num_attention_heads"] * (PREFILL_TOKENS * (PREFILL_TOKENS + 1) / 2) * layers
        out["prefill"] = {"value": round(PREFILL_TOKENS * 1e3 / prefill, 1), "tokens": PREFILL_TOKENS,
                          "ms": round(prefill, 3),
                          "frac": round(flops / (prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"])
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64 and the prefill")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--gemm", default="auto", choices=["auto", "native", "library"],
                    help="bfloat16 products: 'auto' the fastest measured (this engine's kernels or the library), "
                         "'native' this engine's kernels only, 'library' the library wherever it can stand")
    ap.add_argument("--only", default="all", choices=["all", "prefill"],
                    help="'prefill': run only the 2,048-token prefill step and print its numbers (for profiling)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_main(args)
    if args.gpus != 1:
        print(f"bench.py: this engine is single-GPU by design; --gpus {args.gpus} is not supported "
              f"(run with --gpus 1)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    if not torch.cuda.is_available():
        print("bench.py: no CUDA device", file=sys.stderr)
        return 1
    steps, warmup, layers = args.steps, args.warmup, args.layers
    # Requests admitted first already decode while later prompts are still being prefilled.
    prompt_len = window_prompt_len(steps, warmup)
    head = 64 * prompt_len // 4096 + 32
    max_len = max(CONTEXT, prompt_len + warmup + steps + head)
    pk = peaks()

    cfg, spec, ec = build_engine(layers, max(args.batch, 64 if not args.no_points else args.batch),
                                 max_len, graphs=not args.no_graphs)
    ec.gemm = args.gemm
    vocab = cfg.vocab_size
    m = model_bytes_and_flops(cfg, layers)
    if args.only == "prefill":
        ms, flops, wall = prefill_run(spec, ec, vocab, cfg, layers, reps=3)
        print(json.dumps({"prefill": {"value": round(PREFILL_TOKENS * 1e3 / ms, 1), "tokens": PREFILL_TOKENS,
                                      "ms": round(ms, 3), "layers": layers, "e2e_ms": round(wall, 3),
                                      "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}}))
        return 0

    main_run = decode_run(spec, ec, vocab, args.batch, steps, warmup, prompt_len, sample_clocks=True)
    B = args.batch
    ms_per_step = main_run["dev_ms"] / steps
    value = B * 1e3 / ms_per_step
    e2e_value = B * steps * 1e3 / main_run["wall_ms"]
    step_bytes = m["weight_bytes"] + B * main_run["mean_ctx"] * m["kv_bytes_per_token"]
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9

    out = {
        "metric": "decode tokens/s (TinyLlama-1.1B shape, batch 8, 1,024-token prompts decoded towards 2,048)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / PUBLISHED[B], 2) if B in PUBLISHED else None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "impl": "ours",
        "config": {"model": "TinyLlama-1.1B shape (Llama dense decoder)", "layers": layers,
                   "layers_full": MODEL["num_hidden_layers"], "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "ffn": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": B, "seq_len": CONTEXT, "prompt_len": prompt_len,
                   "mean_context": round(main_run["mean_ctx"], 1), "kv_block": BLOCK_SIZE,
                   "parallelism": "single GPU", "cuda_graphs": not args.no_graphs, "gemm": args.gemm,
                   "l2": "inputs larger than L2 (2.2 GB of weights read per step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(main_run["h2d"]), "d2h_bytes_per_step": int(main_run["d2h"])},
        "gpu_launches": int(main_run["launches"]),
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                     "of": pk["source"]},
    }
    if not args.no_points:
        pts = {}
        for b in (1, 64):
            r = decode_run(spec, ec, vocab, b, steps, warmup, prompt_len)
            pts[f"decode_b{b}"] = round(b * steps * 1e3 / r["dev_ms"], 1)
            # the same roofline fraction as above: bytes the step has to read over its time, of the copy rate
            need = m["weight_bytes"] + b * r["mean_ctx"] * m["kv_bytes_per_token"]
            pts[f"decode_b{b}_hbm_frac"] = round(need / (r["dev_ms"] / steps * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        out["points"] = pts
        ms, flops, wall = prefill_run(spec, ec, vocab, cfg, layers)
        out["prefill"] = {"value": round(PREFILL_TOKENS * 1e3 / ms, 1), "tokens": PREFILL_TOKENS,
                          "ms": round(ms, 3), "e2e_ms": round(wall, 3),
                          "e2e_value": round(PREFILL_TOKENS * 1e3 / wall, 1),
                          "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
