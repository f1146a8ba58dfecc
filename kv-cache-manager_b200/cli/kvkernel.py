"""kvkernel: kernel microbenchmarks (after the reference's ``src/main_kernel_bench.cpp``, which
times decode attention only; here also the decode matrix products).

    kvkernel --family attention --ctx 512,2048 --batch 1,8,64 --block-size 16 --out attn.csv
    kvkernel --family gemm --batch 1,8 --hidden 2048 --ffn 5632 --vocab 32000
    kvkernel --family gemm-large --rows 512,2048

attention: for every (block size, batch, context): zero-filled K/V/Q, a sequential and a shuffled
page table, variants paged/contiguous x v1/v2; 5 warm-up runs, ``--iters`` timed runs recorded in
one CUDA graph and replayed between two events; bytes = 2 * batch * ctx * kv_heads * head_dim * 2
(``src/main_kernel_bench.cpp:102``).  "contiguous" is the same kernel on consecutive pages (the
layout baseline).  gemm: the weight-streaming kernel against the library product for the decode
shapes of a model of the given sizes, weights rotated so that every call reads cold weights.
Flags: --ctx --batch --block-size (lists), --heads 32 --kv-heads 4 --head-dim 64 --iters 100 --out CSV.
"""
from __future__ import annotations

import sys
import types


def graph_time_us(fns, reps: int = 5) -> float:
    """Mean microseconds per call of the callables, recorded once each into one CUDA graph."""
    import torch
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for f in fns:
            f()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(fns))


def bench_attention(a, out) -> None:
    import torch
    from ..kernels import library as K
    ctxs, batches = a.ints("ctx", "128,256,512,1024,2048"), a.ints("batch", "1,8,32,128")
    blocks = a.ints("block-size", "16")
    nh, nkv, hd, iters = a.i32("heads", 32), a.i32("kv-heads", 4), a.i32("head-dim", 64), a.i32("iters", 100)
    a.warn_unused()
    from ..engine.peaks import measured_peaks
    pk = measured_peaks()
    peak = pk["hbm_gbs"]
    print(f"HBM peak {peak:.0f} GB/s ({pk['source']})")
    print(f"{'B':>4} {'batch':>6} {'ctx':>6} {'variant':<16} {'us/call':>9} {'GB/s':>9} {'of peak':>8}")
    if out:
        out.write("block_size,batch,ctx,variant,us,gbps\n")
    dev = "cuda:0"
    g = torch.Generator().manual_seed(0)
    for B in blocks:
        for batch in batches:
            for ctx in ctxs:
                mb = (ctx + B - 1) // B
                nb = batch * mb
                kc = torch.zeros(nb, nkv, B, hd, dtype=torch.bfloat16, device=dev)
                vc = torch.zeros_like(kc)
                q = torch.zeros(batch, nh * hd, dtype=torch.bfloat16, device=dev)
                o = torch.zeros_like(q)
                seq_tab = torch.arange(nb, dtype=torch.int32).reshape(batch, mb)
                shuf_tab = seq_tab.flatten()[torch.randperm(nb, generator=g)].reshape(batch, mb).contiguous()
                lens = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
                nbytes = 2.0 * batch * ctx * nkv * hd * 2
                for name, table, version in (("paged-v1", shuf_tab, "v1"), ("contiguous-v1", seq_tab, "v1"),
                                             ("paged-v2", shuf_tab, "v2"), ("contiguous-v2", seq_tab, "v2")):
                    t = table.to(dev)
                    c = types.SimpleNamespace(max_decode_ctx=ctx, seq_ctx_len=lens, options={"attn_version": version})
                    us = graph_time_us([lambda: K.attention_decode(q, o, kc, vc, t, c, nh, nkv, hd, hd ** -0.5)] * iters)
                    gbs = nbytes / (us * 1e-6) / 1e9
                    print(f"{B:>4} {batch:>6} {ctx:>6} {name:<16} {us:>9.2f} {gbs:>9.1f} {gbs / peak:>8.3f}")
                    if out:
                        out.write(f"{B},{batch},{ctx},{name},{us:.3f},{gbs:.2f}\n")


def bench_gemm(a, out) -> None:
    import torch
    from ..kernels import library as K
    H, I, V = a.i32("hidden", 2048), a.i32("ffn", 5632), a.i32("vocab", 32000)
    nh, nkv, hd = a.i32("heads", 32), a.i32("kv-heads", 4), a.i32("head-dim", 64)
    batches = a.ints("batch", "1,8,16")
    a.warn_unused()
    shapes = [("qkv", (nh + 2 * nkv) * hd, H), ("o", H, nh * hd), ("gate_up", 2 * I, H), ("down", H, I), ("lm_head", V, H)]
    dev = "cuda:0"
    if out:
        out.write("rows,product,n,k,variant,us,gbps\n")
    for M in batches:
        for name, N, Kd in shapes:
            copies = max(4, int(600e6 // (N * Kd * 2)))             # more than L2 between repeats
            ws = [torch.randn(N, Kd, device=dev).to(torch.bfloat16) for _ in range(copies)]
            x = torch.randn(M, Kd, device=dev).to(torch.bfloat16)
            y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            res = {"library": graph_time_us([(lambda w=w: torch.mm(x, w.t(), out=y)) for w in ws])}
            if K.stream_gemm_supported(M, N, Kd):
                res["stream"] = graph_time_us([(lambda w=w: K.gemm_stream(x, w, y)) for w in ws])
            if K.splitk_gemm_supported(x, ws[0]):
                res["splitk"] = graph_time_us([(lambda w=w: K.gemm_tcgen05_splitk(x, w, y)) for w in ws])
            gb = N * Kd * 2 / 1e9
            print(f"M={M:<3} {name:<8} [{N} x {Kd}] " +
                  "  ".join(f"{k} {v:.1f} us ({gb / (v * 1e-6) / 1e3:.2f} TB/s)" for k, v in res.items()))
            if out:
                for k, v in res.items():
                    out.write(f"{M},{name},{N},{Kd},{k},{v:.3f},{gb / (v * 1e-6):.1f}\n")
            del ws
    for what, err in (("streaming", K.stream_error()), ("split-K tcgen05", K.splitk_error())):
        if err:
            raise RuntimeError(f"a bounded wait of the {what} kernel ran out (code {err >> 16}, block {err & 0xffff})")


def bench_gemm_large(a, out) -> None:
    """Prefill products (many rows): this engine's tcgen05 kernels (one SM or a pair of SMs to a
    tile) against the library product."""
    import torch
    from ..kernels import library as K
    H, I, V = a.i32("hidden", 2048), a.i32("ffn", 5632), a.i32("vocab", 32000)
    nh, nkv, hd = a.i32("heads", 32), a.i32("kv-heads", 4), a.i32("head-dim", 64)
    rows = a.ints("rows", "2048")
    a.warn_unused()
    shapes = [("qkv", (nh + 2 * nkv) * hd, H), ("o", H, nh * hd), ("gate_up", 2 * I, H), ("down", H, I)]
    dev = "cuda:0"
    if out:
        out.write("rows,product,n,k,variant,us,tflops\n")
    for M in rows:
        for name, N, Kd in shapes:
            w = (torch.randn(N, Kd, device=dev) * 0.05).to(torch.bfloat16)
            x = torch.randn(M, Kd, device=dev).to(torch.bfloat16)
            y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            res = {"library": graph_time_us([lambda: torch.mm(x, w.t(), out=y)] * 10),
                   "tcgen05": graph_time_us([lambda: K.gemm_tcgen05(x, w, y)] * 10),
                   "pair": graph_time_us([lambda: K.gemm_tcgen05_pair(x, w, y)] * 10)}
            if name == "gate_up":                # the same product with the activation in its epilogue
                act = torch.empty(M, N // 2, dtype=torch.bfloat16, device=dev)
                res["tcgen05+silu"] = graph_time_us([lambda: K.gate_up_silu_tcgen05(x, w, act)] * 10)
                res["pair+silu"] = graph_time_us([lambda: K.gate_up_silu_tcgen05_pair(x, w, act)] * 10)
            fl = 2.0 * M * N * Kd
            print(f"M={M:<5} {name:<8} [{N} x {Kd}] " +
                  "  ".join(f"{k} {v:.1f} us ({fl / (v * 1e-6) / 1e12:.0f} TFLOP/s)" for k, v in res.items()))
            if out:
                for k, v in res.items():
                    out.write(f"{M},{name},{N},{Kd},{k},{v:.3f},{fl / (v * 1e-6) / 1e12:.1f}\n")
    for what, err in (("tcgen05", K.tcgen05_error()), ("two-SM tcgen05", K.pair_error())):
        if err:
            raise RuntimeError(f"a bounded wait of the {what} kernel ran out (code {err >> 16}, block {err & 0xffff})")


def main(argv=None) -> int:
    from .args import Args
    a = Args(argv)
    try:
        family = a.str("family", "attention")
        path = a.str("out", "")
        out = open(path, "w") if path else None
        if family == "attention":
            bench_attention(a, out)
        elif family == "gemm":
            bench_gemm(a, out)
        elif family == "gemm-large":
            bench_gemm_large(a, out)
        else:
            raise ValueError(f"unknown --family '{family}' (attention | gemm | gemm-large)")
        if out:
            out.close()
    except Exception as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
