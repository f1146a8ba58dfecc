"""Each kernel alone against a plain PyTorch reference of the same operation (float64 on the
CPU), at sizes other than the engine's: head sizes in steps of 16, odd numbers of heads and
groups, widths and vocabularies that are no power of two, several page sizes.  Where random
inputs would hide a fault (a far key among hundreds, a window's edge, a page's edge) the
inputs are made so that it shows."""
import math
import types

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def K():
    from kvcm.kernels import library
    return library


def tol(dtype, ref):
    return 1e-5 * max(1.0, ref.abs().max().item()) if dtype == "float32" else 0.02 * max(ref.abs().max().item(), 1e-3)


def close(got, ref, dtype, what=""):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert torch.isfinite(got).all(), what
    d = (got - ref).abs().max().item()
    assert d <= tol(dtype, ref), f"{what}: max diff {d:.3e} > {tol(dtype, ref):.3e}"


# ------------------------------------------------------------------------- small kernels

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [70, 72, 2048, 1028])                # (70: the scalar form; the others four elements a thread)
def test_embedding(dtype, H):
    V = 301
    table = torch.randn(V, H).to(DT[dtype]).to(DEV)
    ids = torch.tensor([0, 300, 5, 5, 17], dtype=torch.int32, device=DEV)
    x = torch.empty(5, H, dtype=torch.float32, device=DEV)
    K().embed(ids, table, x)
    assert torch.equal(x.cpu(), table.float().cpu()[ids.cpu().long()])
    bad = torch.tensor([V], dtype=torch.int32, device=DEV)
    y = torch.zeros(1, H, dtype=torch.float32, device=DEV)
    K().embed(bad, table, y)
    assert torch.isnan(y).all()                       # out of range: loud, not wrong


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,eps", [(70, 1e-5), (2048, 1e-6), (5000, 1e-3)])
def test_rmsnorm_with_residual_and_gather(dtype, H, eps):
    T = 9
    dt = DT[dtype]
    x = torch.randn(T, H) * 3
    delta = torch.randn(T, H).to(dt)
    w = (1 + 0.2 * torch.randn(H)).to(dt)
    xd = x.clone().to(DEV)
    out = torch.empty(T, H, dtype=dt, device=DEV)
    K().rmsnorm(xd, delta.to(DEV), w.to(DEV), out, eps)
    x_new = x.double() + delta.double()
    close(xd, x_new, "float32", "residual written back")
    normed = x_new * torch.rsqrt((x_new ** 2).mean(-1, keepdim=True) + eps)
    if dtype == "bfloat16":
        normed = normed.to(dt).double()
    close(out, w.double() * normed, dtype, "rmsnorm")
    # gather: only rows 7 and 2, nothing written back, weight kept in float32
    xg = x.clone().to(DEV)
    rows = torch.tensor([7, 2], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, H, dtype=dt, device=DEV)
    K().rmsnorm(xg, delta.to(DEV), w.float().to(DEV), out2, eps, rows)
    assert torch.equal(xg.cpu(), x)
    close(out2, (w.double() * normed)[[7, 2]], dtype, "rmsnorm gather")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul_and_add_residual(dtype):
    dt = DT[dtype]
    T, I = 5, 173
    gu = (torch.randn(T, 2 * I) * 2).to(dt)
    out = torch.empty(T, I, dtype=dt, device=DEV)
    K().silu_mul(gu.to(DEV), out)
    g, u = gu[:, :I].double(), gu[:, I:].double()
    close(out, g * torch.sigmoid(g) * u, dtype, "silu_mul")
    x = torch.randn(T, I)
    xd = x.clone().to(DEV)
    K().add_residual(xd, gu[:, :I].contiguous().to(DEV))
    close(xd, x.double() + g, "float32", "add_residual")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hd,rot,inter,theta", [(16, 16, False, 1e4), (48, 48, False, 5e5),
                                                (64, 32, False, 1e4), (32, 32, True, 1e4)])
def test_rope_and_cache_write(dtype, hd, rot, inter, theta):
    dt = DT[dtype]
    nh, nkv, B, T = 5, 3, 8, 11
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, width + 16).to(dt)[:, :width]          # padded row stride
    pos = torch.tensor([0, 1, 7, 8, 1999, 3, 100, 15, 16, 17, 2], dtype=torch.int32)
    pages = 6
    perm = torch.randperm(pages * B)[:T].to(torch.int32)
    perm[4] = -1                                                # a row that writes nothing
    kc = torch.zeros(pages, nkv, B, hd, dtype=dt, device=DEV)
    vc = torch.zeros_like(kc)
    inv = (1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64),
                           2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float()
    qd = qkv.to(DEV)
    K().rope_cache(qd, pos.to(DEV), inv.to(DEV), rot, inter, perm.to(DEV), kc, vc, nh, nkv, hd, B)
    # reference
    x = qkv.double().reshape(T, nh + 2 * nkv, hd).clone()
    # the angle is formed in float32 (position * frequency), as the engine and the reference do
    ang = (pos.float()[:, None] * inv[None, :]).double()
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    heads = x[:, :nh + nkv]
    if inter:
        a, b = heads[..., 0:rot:2].clone(), heads[..., 1:rot:2].clone()
        heads[..., 0:rot:2], heads[..., 1:rot:2] = a * c - b * s, b * c + a * s
    else:
        a, b = heads[..., :rot // 2].clone(), heads[..., rot // 2:rot].clone()
        heads[..., :rot // 2], heads[..., rot // 2:rot] = a * c - b * s, b * c + a * s
    close(qd.reshape(T, -1, hd)[:, :nh + nkv], heads, dtype, "rotated q and k")
    assert torch.equal(qd.cpu().reshape(T, -1, hd)[:, nh + nkv:], qkv.reshape(T, -1, hd)[:, nh + nkv:])  # v untouched
    got_k, got_v = kc.cpu(), vc.cpu()
    rotated = qd.cpu().reshape(T, -1, hd)
    expect_k, expect_v = torch.zeros_like(got_k), torch.zeros_like(got_v)
    for t in range(T):
        sl = int(perm[t])
        if sl < 0:
            continue
        expect_k[sl // B, :, sl % B] = rotated[t, nh:nh + nkv]
        expect_v[sl // B, :, sl % B] = rotated[t, nh + nkv:]
    assert torch.equal(got_k, expect_k) and torch.equal(got_v, expect_v)      # exact copies, nothing else touched


@pytest.mark.parametrize("M,N,Kd", [(1, 7, 5), (3, 100, 172), (70, 130, 96), (64, 64, 64), (129, 33, 250)])
def test_plain_gemm(M, N, Kd):
    for dtype in ("float32", "bfloat16"):
        dt = DT[dtype]
        x, w = torch.randn(M, Kd).to(dt), torch.randn(N, Kd).to(dt)
        y = torch.empty(M, N, dtype=dt, device=DEV)
        K().gemm_plain(x.to(DEV), w.to(DEV), y)
        close(y, x.double() @ w.double().T, dtype, f"gemm {M}x{N}x{Kd} {dtype}")
    y32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    K().gemm_plain(x.to(DEV), w.to(DEV), y32)
    close(y32, x.double() @ w.double().T, "float32", "bf16 operands, float result")


def test_plain_gemm_rows_do_not_depend_on_the_batch():
    x, w = torch.randn(37, 300, device=DEV), torch.randn(90, 300, device=DEV)
    full = torch.empty(37, 90, device=DEV)
    K().gemm_plain(x, w, full)
    one = torch.empty(1, 90, device=DEV)
    K().gemm_plain(x[20:21].contiguous(), w, one)
    assert torch.equal(full[20:21], one)


@pytest.mark.parametrize("M,N,Kd", [(1, 2048, 2048), (8, 2560, 2048), (3, 100, 176), (16, 37, 2048), (8, 37, 5632),
                                    (9, 515, 96), (8, 32003, 256), (5, 16, 8), (8, 11264, 2048),
                                    (7, 4096, 1032), (2, 33, 520),
                                    # one tile per block and a long K: X comes straight from L2
                                    (8, 2048, 5632), (16, 2048, 5632), (11, 2368, 2120), (1, 520, 4104),
                                    (8, 2400, 5632)])                # a tile too many for that: X is staged
def test_streaming_gemm(M, N, Kd):
    lib = K()
    assert lib.stream_gemm_supported(M, N, Kd)
    x = torch.randn(M, Kd + 8).to(torch.bfloat16)[:, :Kd]           # strided rows
    w = torch.randn(N, Kd).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    for out_dt in (torch.bfloat16, torch.float32):
        y = torch.full((M, N), float("nan"), dtype=out_dt, device=DEV)
        lib.gemm_stream(x.to(DEV), w.to(DEV), y)
        assert lib.stream_error() == 0
        d = (y.double().cpu() - ref).abs().max().item()
        bound = (0.02 if out_dt == torch.bfloat16 else 2e-3) * ref.abs().max().item()
        assert d <= bound, f"{out_dt}: {d} > {bound}"
    y2 = torch.empty_like(y)
    lib.gemm_stream(x.to(DEV), w.to(DEV), y2)
    assert torch.equal(y, y2)                                       # fixed summation order


@pytest.mark.parametrize("T,nh,nkv,hd,B,write", [(2048, 32, 4, 64, 16, True), (77, 3, 1, 16, 8, True), (300, 6, 3, 48, 4, True),
                                                  (65, 2, 2, 128, 32, False), (1, 5, 5, 32, 1, True)])
def test_rope_with_the_angles_of_a_step_from_a_table(T, nh, nkv, hd, B, write):
    """The cosines and sines of a step computed once, and the rotary + cache-write kernel that reads
    them: the bits of the kernel that computes its angles itself."""
    lib = K()
    g = torch.Generator().manual_seed(T + hd)
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, width + 8, generator=g).to(torch.bfloat16).to(DEV)[:, :width]       # strided rows
    pos = torch.randint(0, 100000, (T,), generator=g).to(torch.int32).to(DEV)
    pages = (T + B - 1) // B + 3
    slots = torch.randperm(pages * B, generator=g)[:T].to(torch.int32)
    if T > 2:
        slots[1] = -1                                                # a row that writes nothing
    slots = slots.to(DEV)
    inv = (1.0 / torch.pow(torch.tensor(500000.0, dtype=torch.float64),
                           2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().to(DEV)
    a, b = qkv.clone(), qkv.clone()
    k1 = torch.zeros(pages, nkv, B, hd, dtype=torch.bfloat16, device=DEV)
    v1, k2, v2 = torch.zeros_like(k1), torch.zeros_like(k1), torch.zeros_like(k1)
    lib.rope_cache(a, pos, inv, hd, False, slots, k1, v1, nh, nkv, hd, B, write)
    table = torch.full((T, hd), float("nan"), device=DEV)
    lib.rope_table(pos, inv, table)
    ang = (pos.float().cpu()[:, None] * inv.cpu()[None, :]).double()        # the angle itself is a float product
    assert torch.allclose(table.double().cpu(), torch.cat([torch.cos(ang), torch.sin(ang)], 1), atol=2e-6)
    lib.rope_cache_table(b, table, slots, k2, v2, nh, nkv, hd, B, write)
    assert torch.equal(a, b) and torch.equal(k1, k2) and torch.equal(v1, v2)
    if not write:
        assert torch.equal(b[:, nh * hd:], qkv[:, nh * hd:]) and not k2.any()


@pytest.mark.parametrize("M,H,nh,nkv,hd,B", [(1, 64, 4, 2, 16, 16), (8, 2048, 32, 4, 64, 16), (5, 96, 3, 1, 32, 8),
                                              (16, 256, 6, 3, 48, 4), (3, 512, 2, 2, 128, 32)])
def test_fused_qkv_rope_cache_gives_the_bits_of_the_separate_kernels(M, H, nh, nkv, hd, B):
    lib = K()
    assert lib.qkv_rope_cache_supported(M, H, nh, nkv, hd)
    g = torch.Generator().manual_seed(M * 7 + hd)
    x = torch.randn(M, H, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn((nh + 2 * nkv) * hd, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    pos = torch.randint(0, 3000, (M,), generator=g).to(torch.int32).to(DEV)
    pages = 9
    slots = torch.randperm(pages * B, generator=g)[:M].to(torch.int32)
    if M > 2:
        slots[1] = -1                                                # a row that writes nothing
    slots = slots.to(DEV)
    inv = (1.0 / torch.pow(torch.tensor(10000.0, dtype=torch.float64),
                           2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().to(DEV)
    # separate kernels
    qkv = torch.empty(M, (nh + 2 * nkv) * hd, dtype=torch.bfloat16, device=DEV)
    lib.gemm_stream(x, w, qkv)
    k1 = torch.zeros(pages, nkv, B, hd, dtype=torch.bfloat16, device=DEV)
    v1 = torch.zeros_like(k1)
    lib.rope_cache(qkv, pos, inv, hd, False, slots, k1, v1, nh, nkv, hd, B)
    # fused
    q2 = torch.full((M, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    k2, v2 = torch.zeros_like(k1), torch.zeros_like(v1)
    lib.qkv_rope_cache(x, w, q2, pos, inv, slots, k2, v2, nh, nkv, hd)
    assert lib.stream_error() == 0
    assert torch.equal(q2, qkv[:, :nh * hd]) and torch.equal(k2, k1) and torch.equal(v2, v1)
    # and against float64
    ref = (x.double().cpu() @ w.double().cpu().T)
    close(qkv[:, (nh + nkv) * hd:], ref[:, (nh + nkv) * hd:], "bfloat16", "v part of the product")


@pytest.mark.parametrize("M,H,I", [(1, 64, 24), (8, 2048, 5632), (5, 96, 256), (16, 128, 1000)])
def test_fused_gate_up_silu_gives_the_bits_of_the_separate_kernels(M, H, I):
    lib = K()
    assert lib.gate_up_silu_supported(M, I, H) and not lib.gate_up_silu_supported(M, 172, H)
    g = torch.Generator().manual_seed(I)
    x = torch.randn(M, H, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * I, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    gu = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=DEV)
    lib.gemm_stream(x, w, gu)
    a1 = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    lib.silu_mul(gu, a1)
    a2 = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    lib.gate_up_silu(x, w, a2)
    assert lib.stream_error() == 0
    assert torch.equal(a1, a2)
    gg = (x.double().cpu() @ w.double().cpu().T)
    close(a2, gg[:, :I] * torch.sigmoid(gg[:, :I]) * gg[:, I:], "bfloat16", "against float64")


@pytest.mark.parametrize("M,H,Kd,I,eps", [(8, 2048, 2048, 5632, 1e-5), (1, 64, 48, 24, 1e-6), (5, 96, 256, 256, 1e-5),
                                          (16, 264, 1000, 128, 1e-3), (8, 2048, 5632, 64, 1e-5), (11, 2120, 2368, 40, 1e-5)])
def test_residual_and_norm_ride_in_the_streaming_products(M, H, Kd, I, eps):
    """The product that ends a sublayer adds into the float residual, leaves partial sums of squares
    and the next norm's row before its scale; the product that begins the next sublayer scales its
    sums by the norm's 1/rms.  Against the separate kernels: the residual bit for bit, the products
    within bfloat16 rounding (the normed row is rounded once instead of twice); against float64;
    twice the same bits."""
    lib = K()
    g = torch.Generator().manual_seed(M + H + Kd)
    y = torch.randn(M, Kd, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(H, Kd, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    resid0 = (3.0 * torch.randn(M, H, generator=g)).to(DEV)              # (not of unit scale: the norm has work to do)
    norm_w = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).to(DEV)
    # separate kernels: product, then residual add + norm
    proj = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
    lib.gemm_stream(y, w, proj)
    resid1 = resid0.clone()
    x1 = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
    lib.rmsnorm(resid1, proj, norm_w, x1, eps)
    # riding along
    resid2 = resid0.clone()
    tiles = (H + 15) // 16
    partials = torch.full((tiles, 16), float("nan"), device=DEV)
    h = torch.full((M, H), float("nan"), dtype=torch.bfloat16, device=DEV)
    lib.gemm_stream_residual(y, w, resid2, partials, h, norm_w)
    assert lib.stream_error() == 0
    assert torch.equal(resid1, resid2)
    assert torch.equal(h, (norm_w.float() * resid2).to(torch.bfloat16))
    ss = partials[:, :M].double().sum(0).cpu()
    want = (resid2.double().cpu() ** 2).sum(1)
    assert torch.allclose(ss, want, rtol=1e-5), "partial sums of squares"
    resid3, partials3 = resid0.clone(), torch.zeros_like(partials)
    lib.gemm_stream_residual(y, w, resid3, partials3)                     # nothing handed on: the residual alone
    assert torch.equal(resid3, resid2) and torch.equal(partials3[:, :M], partials[:, :M])
    # ... into a gate/up product
    wg = (torch.randn(2 * I, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    a1 = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    lib.gate_up_silu(x1, wg, a1)
    a2 = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    lib.gate_up_silu(h, wg, a2, partials, eps)
    a3 = torch.full_like(a2, float("nan"))
    lib.gate_up_silu(h, wg, a3, partials, eps)
    assert lib.stream_error() == 0 and torch.equal(a2, a3)
    xr = resid2.double().cpu()
    xn = norm_w.double().cpu() * (xr * torch.rsqrt((xr ** 2).mean(1, keepdim=True) + eps))
    gg = xn @ wg.double().cpu().T
    ref = gg[:, :I] * torch.sigmoid(gg[:, :I]) * gg[:, I:]
    close(a2, ref, "bfloat16", "scaled gate/up against float64")
    close(a2, a1.double().cpu(), "bfloat16", "scaled gate/up against the separate kernels")
    # ... and into a qkv product with rotary encoding and cache write
    nh, nkv, hd, B, pages = 4, 2, 16, 8, 5
    wq = (torch.randn((nh + 2 * nkv) * hd, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    pos = torch.randint(0, 3000, (M,), generator=g).to(torch.int32).to(DEV)
    slots = torch.randperm(pages * B, generator=g)[:M].to(torch.int32).to(DEV)
    inv = (1.0 / torch.pow(torch.tensor(10000.0, dtype=torch.float64),
                           2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().to(DEV)
    q1 = torch.empty(M, nh * hd, dtype=torch.bfloat16, device=DEV)
    k1 = torch.zeros(pages, nkv, B, hd, dtype=torch.bfloat16, device=DEV)
    v1 = torch.zeros_like(k1)
    lib.qkv_rope_cache(x1, wq, q1, pos, inv, slots, k1, v1, nh, nkv, hd)
    q2 = torch.full_like(q1, float("nan"))
    k2, v2 = torch.zeros_like(k1), torch.zeros_like(v1)
    lib.qkv_rope_cache(h, wq, q2, pos, inv, slots, k2, v2, nh, nkv, hd, partials, eps)
    assert lib.stream_error() == 0
    for got, sep, what in ((q2, q1, "q"), (k2, k1, "k pages"), (v2, v1, "v pages")):
        close(got, sep.double().cpu(), "bfloat16", f"scaled qkv against the separate kernels: {what}")
    vref = (xn @ wq.double().cpu().T)[:, (nh + nkv) * hd:].reshape(M, nkv, hd)
    sl = slots.cpu().long()
    close(v2.cpu()[sl // B, :, sl % B], vref, "bfloat16", "v rows against float64")


@pytest.mark.parametrize("M,N,Kd", [(64, 2560, 2048), (64, 2048, 5632), (17, 100, 136), (256, 515, 96), (33, 32003, 256),
                                    (100, 11264, 2048), (1, 8, 8), (48, 2048, 2048), (200, 130, 4104), (24, 129, 72)])
def test_tcgen05_splitk_gemm(M, N, Kd):
    """Swap-AB tcgen05 product with K split over a cluster, against float64; ragged edges in every
    dimension; the same bits on a second run (the partial sums are added in a fixed order)."""
    lib = K()
    g = torch.Generator().manual_seed(M * 3 + N)
    x = torch.randn(M, Kd + 8, generator=g).to(torch.bfloat16).to(DEV)[:, :Kd]        # strided rows
    w = (torch.randn(N, Kd, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    assert lib.splitk_gemm_supported(x, w)
    ref = x.double().cpu() @ w.double().cpu().T
    for out_dt in (torch.bfloat16, torch.float32):
        y = torch.full((M, N), float("nan"), dtype=out_dt, device=DEV)
        lib.gemm_tcgen05_splitk(x, w, y)
        assert lib.splitk_error() == 0
        d = (y.double().cpu() - ref).abs().max().item()
        bound = (0.02 if out_dt == torch.bfloat16 else 2e-3) * ref.abs().max().item()
        assert d <= bound, f"{out_dt}: {d} > {bound}"
    y2 = torch.empty_like(y)
    lib.gemm_tcgen05_splitk(x, w, y2)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("M,H,I", [(2048, 2048, 5632), (300, 96, 1000), (129, 64, 24), (640, 256, 128)])
def test_tcgen05_gate_up_with_the_activation_in_its_epilogue(M, H, I):
    """Bit for bit the tcgen05 product followed by the activation kernel, and close to float64."""
    lib = K()
    g = torch.Generator().manual_seed(M + I)
    x = torch.randn(M, H, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * I, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    gu = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=DEV)
    lib.gemm_tcgen05(x, w, gu)
    a1 = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    lib.silu_mul(gu, a1)
    a2 = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    lib.gate_up_silu_tcgen05(x, w, a2)
    assert lib.tcgen05_error() == 0
    assert torch.equal(a1, a2)
    gg = (x.double().cpu() @ w.double().cpu().T)
    close(a2, gg[:, :I] * torch.sigmoid(gg[:, :I]) * gg[:, I:], "bfloat16", "against float64")


@pytest.mark.parametrize("M,N,Kd", [(128, 256, 64), (1, 8, 8), (100, 300, 136), (257, 129, 1000), (2048, 2560, 2048),
                                    (640, 11264, 2048), (300, 2048, 5632), (17, 32003, 96)])
def test_tcgen05_gemm(M, N, Kd):
    """TMA tensor maps + tcgen05.mma + tensor memory against float64; ragged edges are zero-filled by
    the TMA unit, so sizes need not be multiples of the 128 x 256 x 64 tile."""
    lib = K()
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, Kd + 8, generator=g).to(torch.bfloat16).to(DEV)[:, :Kd]        # strided rows
    w = (torch.randn(N, Kd, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    assert lib.tcgen05_gemm_supported(x, w)
    ref = x.double().cpu() @ w.double().cpu().T
    for out_dt in (torch.bfloat16, torch.float32):
        y = torch.full((M, N), float("nan"), dtype=out_dt, device=DEV)
        lib.gemm_tcgen05(x, w, y)
        assert lib.tcgen05_error() == 0
        d = (y.double().cpu() - ref).abs().max().item()
        bound = (0.01 if out_dt == torch.bfloat16 else 1e-3) * max(ref.abs().max().item(), 1e-3)
        assert d <= bound, f"{out_dt}: {d} > {bound}"
    assert not lib.tcgen05_gemm_supported(x[:, :Kd - 4], w[:, :Kd - 4])               # K not a multiple of 8


@pytest.mark.parametrize("M,N,Kd,bn", [(256, 256, 64, 0), (1, 8, 8, 0), (100, 300, 136, 0), (257, 129, 1000, 0),
                                       (2048, 2560, 2048, 0), (640, 11264, 2048, 0), (300, 2048, 5632, 0),
                                       (17, 32003, 96, 0), (513, 700, 264, 32), (513, 700, 264, 96), (900, 2048, 2048, 160),
                                       (2048, 2048, 2048, 224), (2048, 2560, 2048, 288), (700, 1000, 520, 512),
                                       (5000, 4100, 264, 352), (2304, 700, 64, 0)])
def test_tcgen05_pair_gemm(M, N, Kd, bn):
    """The two-SM kernel (tcgen05.mma.cta_group::2, tiles of 256 x bn over a pair of blocks) against
    float64 at every tile width; ragged edges in every dimension; many tiles per pair."""
    lib = K()
    g = torch.Generator().manual_seed(M + N + bn)
    x = torch.randn(M, Kd + 8, generator=g).to(torch.bfloat16).to(DEV)[:, :Kd]        # strided rows
    w = (torch.randn(N, Kd, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    assert lib.pair_gemm_supported(x, w)
    ref = x.double().cpu() @ w.double().cpu().T
    for out_dt in (torch.bfloat16, torch.float32):
        y = torch.full((M, N), float("nan"), dtype=out_dt, device=DEV)
        lib.gemm_tcgen05_pair(x, w, y, bn)
        assert lib.pair_error() == 0
        d = (y.double().cpu() - ref).abs().max().item()
        bound = (0.01 if out_dt == torch.bfloat16 else 1e-3) * max(ref.abs().max().item(), 1e-3)
        assert d <= bound, f"{out_dt}: {d} > {bound}"
    assert not lib.pair_gemm_supported(x[:, :Kd - 4], w[:, :Kd - 4])                  # K not a multiple of 8
    with pytest.raises(lib.KernelError):
        lib.gemm_tcgen05_pair(x, w, y, 48)                                            # no such tile width


@pytest.mark.parametrize("M,H,I,bn", [(2048, 2048, 5632, 0), (300, 96, 1000, 0), (129, 64, 24, 0), (640, 256, 128, 64),
                                      (700, 136, 344, 128), (512, 2048, 1000, 192), (700, 136, 344, 320),
                                      (1100, 264, 1000, 512)])
def test_tcgen05_pair_gate_up_with_the_activation_in_its_epilogue(M, H, I, bn):
    """Bit for bit the two-SM product followed by the activation kernel, and close to float64."""
    lib = K()
    g = torch.Generator().manual_seed(M + I + bn)
    x = torch.randn(M, H, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * I, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    gu = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=DEV)
    lib.gemm_tcgen05_pair(x, w, gu, 0, 0, 0)           # whole tiles: the same order of sums
    a1 = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    lib.silu_mul(gu, a1)
    a2 = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    lib.gate_up_silu_tcgen05_pair(x, w, a2, bn)
    assert lib.pair_error() == 0
    assert torch.equal(a1, a2)
    gg = (x.double().cpu() @ w.double().cpu().T)
    close(a2, gg[:, :I] * torch.sigmoid(gg[:, :I]) * gg[:, I:], "bfloat16", "against float64")


@pytest.mark.parametrize("M,N,Kd", [(2048, 2560, 2048), (2048, 2048, 2048), (300, 700, 136), (256, 256, 64), (1, 8, 8),
                                    (5000, 4100, 264), (700, 515, 4104), (257, 129, 1000), (640, 11264, 2048)])
def test_tcgen05_pair_gemm_with_split_k_ranges(M, N, Kd):
    """The pairs take equal shares of all (tile, k-step) units; a tile whose k range is cut is summed
    from partial sums in a fixed order: against float64, the same bits on every run (the flags are
    put back by their readers), and again after a launch without the split."""
    lib = K()
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, Kd + 8, generator=g).to(torch.bfloat16).to(DEV)[:, :Kd]
    w = (torch.randn(N, Kd, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    ref = x.double().cpu() @ w.double().cpu().T
    for out_dt in (torch.bfloat16, torch.float32):
        runs = []
        for i in range(3):
            y = torch.full((M, N), float("nan"), dtype=out_dt, device=DEV)
            lib.gemm_tcgen05_pair(x, w, y, 0, 0, 1)
            runs.append(y)
            if i == 1:
                lib.gemm_tcgen05_pair(x, w, torch.empty_like(y), 0, 0, 0)
        assert lib.pair_error() == 0
        d = (runs[0].double().cpu() - ref).abs().max().item()
        bound = (0.01 if out_dt == torch.bfloat16 else 1e-3) * max(ref.abs().max().item(), 1e-3)
        assert d <= bound, f"{out_dt}: {d} > {bound}"
        assert torch.equal(runs[0], runs[1]) and torch.equal(runs[0], runs[2])


@pytest.mark.parametrize("M,H,I", [(2048, 2048, 5632), (300, 96, 1000), (700, 4104, 344)])
def test_tcgen05_pair_gate_up_with_split_k_ranges(M, H, I):
    lib = K()
    g = torch.Generator().manual_seed(M + I)
    x = torch.randn(M, H, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * I, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    a1 = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    a2 = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    lib.gate_up_silu_tcgen05_pair(x, w, a1, 0, 0, 1)
    lib.gate_up_silu_tcgen05_pair(x, w, a2, 0, 0, 1)
    assert lib.pair_error() == 0
    assert torch.equal(a1, a2)
    gg = (x.double().cpu() @ w.double().cpu().T)
    close(a1, gg[:, :I] * torch.sigmoid(gg[:, :I]) * gg[:, I:], "bfloat16", "against float64")


def test_streaming_gemm_refuses_what_it_cannot_run():
    lib = K()
    assert not lib.stream_gemm_supported(17, 64, 64)                # too many rows
    assert not lib.stream_gemm_supported(4, 64, 60)                 # K not a multiple of 8
    x = torch.zeros(4, 60, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(64, 60, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(lib.KernelError, match="not supported"):
        lib.gemm_stream(x, w, torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV))


def test_argmax_ties_and_edges():
    V = 1000
    lg = torch.randn(5, V)
    lg[0, 17] = lg[0, 900] = 50.0          # tie: lowest index
    lg[1, V - 1] = 60.0                    # last index
    lg[2, 0] = 60.0
    lg[3] = -5.0                           # all equal
    out = torch.zeros(5, dtype=torch.int32, device=DEV)
    K().argmax(lg.to(DEV), out)
    assert out.cpu().tolist()[:4] == [17, V - 1, 0, 0] and out[4].item() == int(lg[4].argmax())


@pytest.mark.parametrize("V", [257, 1000, 32003])
def test_temperature_sampling_matches_the_inverse_cdf(V):
    from kvcm.sampling import uniform_for
    R = 16
    lg = (torch.randn(R, V) * 3)
    temp = torch.tensor([0.8, 1.0, 0.3, 2.0] * 4)
    temp[5] = 0.0                                                # greedy row
    seed = torch.arange(R, dtype=torch.int64) * 7919 + 3
    rid = torch.arange(R, dtype=torch.int64) + 100
    pos = torch.arange(R, dtype=torch.int32) * 13
    out = torch.zeros(R, dtype=torch.int32, device=DEV)
    K().sample(lg.to(DEV), temp.to(DEV), seed.to(DEV), rid.to(DEV), pos.to(DEV), out)
    got = out.cpu().tolist()
    assert got[5] == int(lg[5].argmax())
    for r in range(R):
        if temp[r] == 0:
            continue
        p = torch.softmax(lg[r].double() / float(temp[r]), 0)
        c = torch.cumsum(p, 0)
        u = uniform_for(int(seed[r]), int(rid[r]), int(pos[r]))
        t = got[r]
        lo = float(c[t - 1]) if t else 0.0
        assert lo - 1e-5 <= u <= float(c[t]) + 1e-5, (r, t, u, lo, float(c[t]))
    out2 = torch.zeros(R, dtype=torch.int32, device=DEV)
    K().sample(lg.to(DEV), temp.to(DEV), seed.to(DEV), rid.to(DEV), pos.to(DEV), out2)
    assert torch.equal(out, out2)                                 # the same draw every time


def test_sampling_distribution_is_right():
    V, R = 50, 4096
    row = torch.randn(V) * 2
    lg = row.repeat(R, 1).to(DEV)
    out = torch.zeros(R, dtype=torch.int32, device=DEV)
    K().sample(lg, torch.full((R,), 0.7, device=DEV), torch.zeros(R, dtype=torch.int64, device=DEV),
               torch.arange(R, dtype=torch.int64, device=DEV), torch.zeros(R, dtype=torch.int32, device=DEV), out)
    freq = torch.bincount(out.cpu().long(), minlength=V).double() / R
    p = torch.softmax(row.double() / 0.7, 0)
    assert (freq - p).abs().max().item() < 4 * math.sqrt(0.25 / R)


# ----------------------------------------------------------------------------- attention

def paged_case(seq_lens, q_lens, nh, nkv, hd, B, dtype, seed=0, spare=7):
    """Random requests in a shuffled page pool with unreferenced spare pages (as the reference's
    attention test does, tests/test_paged_attention.cu:41,56).  Returns device tensors, a context
    object and the dense K/V per request for the reference."""
    g = torch.Generator().manual_seed(seed)
    dt = DT[dtype]
    need = [(n + B - 1) // B for n in seq_lens]
    pages = sum(need) + spare
    perm = torch.randperm(pages, generator=g).tolist()
    max_blocks = max(need) + 1
    kc = torch.randn(pages, nkv, B, hd, generator=g).to(dt)      # spare pages hold junk, not zeros
    vc = torch.randn(pages, nkv, B, hd, generator=g).to(dt)
    tables = torch.full((len(seq_lens), max_blocks), -1, dtype=torch.int32)
    dense = []
    at = 0
    for i, n in enumerate(seq_lens):
        ids = perm[at:at + need[i]]
        at += need[i]
        tables[i, :need[i]] = torch.tensor(ids, dtype=torch.int32)
        kd = torch.randn(n, nkv, hd, generator=g).to(dt)
        vd = torch.randn(n, nkv, hd, generator=g).to(dt)
        for t in range(n):
            kc[ids[t // B], :, t % B] = kd[t]
            vc[ids[t // B], :, t % B] = vd[t]
        dense.append((kd, vd))
    # rows: single-row entries first (the builder's order)
    order = sorted(range(len(seq_lens)), key=lambda i: q_lens[i] != 1)
    T = sum(q_lens)
    q = torch.randn(T, nh * hd + 32, generator=g).to(dt)[:, :nh * hd]      # strided rows
    row_seq, positions, q_start, tile_seq, tile_q0 = [], [], [], [], []
    for si, i in enumerate(order):
        q_start.append(len(row_seq))
        for j in range(q_lens[i]):
            row_seq.append(si)
            positions.append(seq_lens[i] - q_lens[i] + j)
        if q_lens[i] > 1:
            for q0 in range(0, q_lens[i], 64):
                tile_seq.append(si)
                tile_q0.append(q0)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    nd = sum(1 for x in q_lens if x == 1)
    ctx = types.SimpleNamespace(
        rows=T, seqs=len(seq_lens), decode_seqs=nd, prefill_tiles=len(tile_seq), tile_rows=64,
        max_ctx=max(seq_lens), max_decode_ctx=max([seq_lens[i] for i in order[:nd]] or [1]),
        row_seq=i32(row_seq), positions=i32(positions), seq_q_start=i32(q_start),
        seq_q_len=i32([q_lens[i] for i in order]), seq_ctx_len=i32([seq_lens[i] for i in order]),
        tile_seq=i32(tile_seq or [0]), tile_q0=i32(tile_q0 or [0]), options={})
    return dict(q=q.to(DEV), kc=kc.to(DEV), vc=vc.to(DEV), tables=tables[order].contiguous().to(DEV), ctx=ctx,
                dense=[dense[i] for i in order], order=order, q_cpu=q, row_seq=row_seq, positions=positions)


def reference_attention(case, nh, nkv, hd, scale, window):
    q = case["q_cpu"].double().reshape(-1, nh, hd)
    out = torch.zeros(q.shape[0], nh, hd, dtype=torch.float64)
    G = nh // nkv
    for r, (si, pos) in enumerate(zip(case["row_seq"], case["positions"])):
        kd, vd = case["dense"][si]
        lo = max(0, pos + 1 - window) if window else 0
        for h in range(nh):
            k, v = kd[lo:pos + 1, h // G].double(), vd[lo:pos + 1, h // G].double()
            p = torch.softmax((q[r, h] * scale) @ k.T, 0)
            out[r, h] = p @ v
    return out.reshape(q.shape[0], nh * hd)


SHAPES = [(4, 2, 16, 16), (3, 1, 32, 8), (5, 5, 48, 16), (8, 2, 64, 32), (6, 3, 80, 16),
          (32, 4, 64, 16), (20, 1, 64, 16), (4, 4, 128, 64), (2, 1, 256, 16), (9, 3, 112, 4)]


@pytest.mark.parametrize("nh,nkv,hd,B", SHAPES)
@pytest.mark.parametrize("window", [0, 37])
def test_attention_kernels_on_a_mixed_batch(nh, nkv, hd, B, window):
    """Decode rows at contexts around page and tile edges beside portions that start anywhere."""
    seq_lens = [1, 15, 16, 17, 63, 64, 65, 300, 129, 200, 70]
    q_lens = [1, 1, 1, 1, 1, 1, 1, 1, 129, 2, 70]
    scale = 1.0 / math.sqrt(hd)
    for dtype in ("float32", "bfloat16"):
        case = paged_case(seq_lens, q_lens, nh, nkv, hd, B, dtype, seed=nh * 100 + hd)
        ref = reference_attention(case, nh, nkv, hd, scale, window)
        out = torch.zeros(case["ctx"].rows, nh * hd, dtype=DT[dtype], device=DEV)
        K().attention_plain(case["q"], out, case["kc"], case["vc"], case["tables"], case["ctx"].row_seq,
                            case["ctx"].positions, nh, nkv, hd, scale, window)
        close(out, ref, dtype, f"plain {dtype}")
        if dtype == "bfloat16":
            assert K().fast_attention_supported(nh, nkv, hd, B)
            got = {}
            for version in ("v1", "v2", "v2 merge kernel"):
                case["ctx"].options = {"attn_version": version[:2],
                                       "attn_merge": "kernel" if "kernel" in version else "cluster"}
                fast = torch.zeros_like(out)
                K().paged_attention(case["q"], fast, case["kc"], case["vc"], case["tables"], case["ctx"],
                                    nh, nkv, hd, scale, window)
                close(fast, ref, dtype, f"fast {version}")
                got[version] = fast
            # merging inside the cluster and merging in a kernel of its own give the same bits
            assert torch.equal(got["v2"], got["v2 merge kernel"])


@pytest.mark.parametrize("B", [8, 16, 32, 64, 128])
@pytest.mark.parametrize("window,hd", [(0, 64), (150, 64), (0, 128), (90, 128)])
def test_prefill_attention_on_tcgen05(B, window, hd):
    """The tcgen05 prefill kernel (head_dim 64 and 128) against float64 and against the mma.sync
    kernel: portions that start anywhere, end anywhere, are shorter than a tile, span several key
    tiles, with pages of every supported size, beside decode rows."""
    nh, nkv = (8, 2) if hd == 64 else (6, 3)
    lib = K()
    assert lib.prefill_tcgen05_supported(hd, B) and not lib.prefill_tcgen05_supported(96, B)
    seq_lens = [300, 129, 128, 640, 70, 2, 513, 1]
    q_lens = [300, 129, 1, 131, 64, 2, 257, 1]
    scale = 1.0 / math.sqrt(hd)
    case = paged_case(seq_lens, q_lens, nh, nkv, hd, B, "bfloat16", seed=B + window + hd)
    ref = reference_attention(case, nh, nkv, hd, scale, window)
    got = {}
    for mode in ("tcgen05", "mma"):
        case["ctx"].options = {"attn_prefill": mode}
        out = torch.zeros(case["ctx"].rows, nh * hd, dtype=torch.bfloat16, device=DEV)
        lib.paged_attention(case["q"], out, case["kc"], case["vc"], case["tables"], case["ctx"], nh, nkv, hd,
                            scale, window)
        assert lib.attention_tcgen05_error() == 0
        close(out, ref, "bfloat16", f"prefill {mode}, pages of {B}")
        got[mode] = out
    close(got["tcgen05"], got["mma"].double(), "bfloat16", "tcgen05 against mma.sync")


def test_prefill_attention_on_tcgen05_finds_one_far_key():
    """Each query row points at one key of its own; a kernel that misses a key (a page's or a
    tile's edge, the first or the last key of the row) returns an average instead of that value."""
    nh, nkv, hd, B, n = 2, 1, 64, 16, 700
    lib = K()
    case = paged_case([n], [n], nh, nkv, hd, B, "bfloat16", seed=5)
    kd, vd = case["dense"][0]
    q = case["q_cpu"].clone()
    g = torch.Generator().manual_seed(9)
    needles = [int(torch.randint(0, i + 1, (1,), generator=g)) for i in range(n)]
    for i in (0, 127, 128, 129, 255, 256, 511, 512, 699):
        needles[i] = i                                              # the row's own (last) key
    for i in (130, 300, 600):
        needles[i] = 0                                              # the first key
    for i in range(n):
        unit = kd[needles[i], 0].float() / kd[needles[i], 0].float().norm()
        for h in range(nh):
            q[i, h * hd:(h + 1) * hd] = (6.0 * math.sqrt(hd) * unit).to(torch.bfloat16)
    case["q"], case["q_cpu"] = q.to(DEV), q
    ref = reference_attention(case, nh, nkv, hd, 1 / math.sqrt(hd), 0)
    want = torch.stack([torch.cat([vd[needles[i], 0]] * nh) for i in range(n)]).double()
    assert (ref - want).abs().max() < 0.1                           # the reference itself picks the needles
    case["ctx"].options = {"attn_prefill": "tcgen05"}
    out = torch.zeros(n, nh * hd, dtype=torch.bfloat16, device=DEV)
    lib.paged_attention(case["q"], out, case["kc"], case["vc"], case["tables"], case["ctx"], nh, nkv, hd,
                        1 / math.sqrt(hd), 0)
    assert lib.attention_tcgen05_error() == 0
    close(out, ref, "bfloat16", "needles")


def test_decode_attention_long_contexts_and_many_partitions():
    nh, nkv, hd, B = 32, 4, 64, 16
    seq_lens = [2047, 2048, 1, 4097, 513]
    case = paged_case(seq_lens, [1] * 5, nh, nkv, hd, B, "bfloat16", seed=3)
    ref = reference_attention(case, nh, nkv, hd, 0.125, 0)
    for version in ("v1", "v2", "v2 merge kernel"):
        case["ctx"].options = {"attn_version": version[:2], "attn_merge": "kernel" if "kernel" in version else "cluster"}
        out = torch.zeros(5, nh * hd, dtype=torch.bfloat16, device=DEV)
        K().paged_attention(case["q"], out, case["kc"], case["vc"], case["tables"], case["ctx"], nh, nkv, hd, 0.125, 0)
        close(out, ref, "bfloat16", version)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("needle", [0, 15, 16, 63, 64, 255, 256, 700, 998])
def test_one_far_key_among_hundreds_decides_the_output(dtype, needle):
    """One key is made to match the query so strongly that the output must be its value; a kernel
    that misses it (a page's edge, a partition's edge, the first or last key) returns an average."""
    nh, nkv, hd, B, n = 4, 2, 64, 16, 999
    case = paged_case([n], [1], nh, nkv, hd, B, dtype, seed=needle)
    q = case["q_cpu"].clone()
    kd, vd = case["dense"][0]
    for h in range(nh):
        q[0, h * hd:(h + 1) * hd] = 6.0 * kd[needle, h // 2] / kd[needle, h // 2].float().norm() * math.sqrt(hd)
    case["q"], case["q_cpu"] = q.to(DEV), q
    ref = reference_attention(case, nh, nkv, hd, 1 / math.sqrt(hd), 0)
    want = torch.cat([vd[needle, h // 2] for h in range(nh)]).double()
    assert (ref[0] - want).abs().max() < 0.05                      # the reference itself picks the needle
    for mode in (["plain"] if dtype == "float32" else ["plain", "v1", "v2"]):
        case["ctx"].options = {"attention": "plain"} if mode == "plain" else {"attn_version": mode}
        out = torch.zeros(1, nh * hd, dtype=DT[dtype], device=DEV)
        K().paged_attention(case["q"], out, case["kc"], case["vc"], case["tables"], case["ctx"],
                            nh, nkv, hd, 1 / math.sqrt(hd), 0)
        close(out, ref, dtype, f"{mode} needle at {needle}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_edge_is_exact(dtype):
    """The key just outside the window would dominate if it were read; the key just inside must
    be read.  Checked for decode rows and for rows of a portion."""
    nh, nkv, hd, B, W = 2, 1, 32, 8, 40
    for q_len in (1, 50):
        n = 200
        case = paged_case([n], [q_len], nh, nkv, hd, B, dtype, seed=q_len)
        kd, vd = case["dense"][0]
        q = case["q_cpu"].clone()
        last = len(case["positions"]) - 1
        pos = case["positions"][last]
        outside, inside = pos - W, pos - W + 1
        # the last row's query points at the key just outside the window
        for h in range(nh):
            q[last, h * hd:(h + 1) * hd] = 6.0 * kd[outside, 0] / kd[outside, 0].float().norm() * math.sqrt(hd)
        case["q"], case["q_cpu"] = q.to(DEV), q
        ref_w = reference_attention(case, nh, nkv, hd, 1 / math.sqrt(hd), W)
        ref_all = reference_attention(case, nh, nkv, hd, 1 / math.sqrt(hd), 0)
        assert (ref_w[last] - ref_all[last]).abs().max() > 0.3       # reading it would show
        for mode in (["plain"] if dtype == "float32" else ["plain", "v2"]):
            case["ctx"].options = {"attention": "plain"} if mode == "plain" else {"attn_version": mode}
            out = torch.zeros(case["ctx"].rows, nh * hd, dtype=DT[dtype], device=DEV)
            K().paged_attention(case["q"], out, case["kc"], case["vc"], case["tables"], case["ctx"],
                                nh, nkv, hd, 1 / math.sqrt(hd), W)
            close(out, ref_w, dtype, f"{mode} window edge q_len={q_len}")


def test_layout_does_not_change_bits():
    """Shuffled pages and sequential pages give equal bits (the reference checks the same,
    tests/test_paged_attention.cu:208-228)."""
    nh, nkv, hd, B = 8, 2, 64, 16
    a = paged_case([300, 77], [1, 77], nh, nkv, hd, B, "bfloat16", seed=5, spare=9)
    b = paged_case([300, 77], [1, 77], nh, nkv, hd, B, "bfloat16", seed=5, spare=9)
    # rebuild b's pool in sequential order
    pages = b["kc"].shape[0]
    kc, vc = torch.zeros_like(b["kc"]), torch.zeros_like(b["vc"])
    tables = b["tables"].clone().cpu()
    nxt = 0
    for i in range(tables.shape[0]):
        for j in range(tables.shape[1]):
            if tables[i, j] >= 0:
                kc[nxt], vc[nxt] = b["kc"][tables[i, j]], b["vc"][tables[i, j]]
                tables[i, j] = nxt
                nxt += 1
    outs = []
    for case, k_, v_, t_ in ((a, a["kc"], a["vc"], a["tables"]), (b, kc, vc, tables.to(DEV))):
        out = torch.zeros(case["ctx"].rows, nh * hd, dtype=torch.bfloat16, device=DEV)
        K().paged_attention(case["q"], out, k_, v_, t_, case["ctx"], nh, nkv, hd, 0.125, 0)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])


def test_unsupported_sizes_are_refused_not_miscomputed():
    lib = K()
    assert not lib.fast_attention_supported(4, 2, 24, 16)        # head_dim not a multiple of 16
    assert not lib.fast_attention_supported(5, 2, 64, 16)        # heads not a multiple of KV heads
    case = paged_case([40], [1], 4, 2, 24, 8, "bfloat16")
    out = torch.zeros(1, 96, dtype=torch.bfloat16, device=DEV)
    # the dispatcher falls back to the plain kernel, which takes any head_dim
    lib.paged_attention(case["q"], out, case["kc"], case["vc"], case["tables"], case["ctx"], 4, 2, 24, 0.2, 0)
    close(out, reference_attention(case, 4, 2, 24, 0.2, 0), "bfloat16", "hd=24 through the plain kernel")
    with pytest.raises(lib.KernelError):
        lib.attention_plain(case["q"], out, case["kc"], case["vc"], case["tables"], case["ctx"].row_seq,
                            case["ctx"].positions, 5, 2, 24, 0.2, 0)
    with pytest.raises(lib.KernelError):
        lib.rmsnorm(torch.zeros(2, 8), None, torch.ones(8), torch.zeros(2, 8), 1e-5)     # CPU tensors


@pytest.mark.parametrize("hd,B,window", [(64, 16, 150), (128, 32, 90), (64, 8, 40)])
def test_prefill_attention_on_tcgen05_with_pages_given_back(hd, B, window):
    """A windowed layer group gives pages back once every key on them lies below the window: their
    table entries are -1 while later portions of the same prompt still run.  The kernel must not
    read through such an entry (its key tiles start at multiples of 64 keys, below the window's
    first key).  Entries of pages that no row of the step may see are set to -1 here, as the cache
    manager leaves them, and the result is compared with float64."""
    nh, nkv = (8, 2) if hd == 64 else (6, 3)
    lib = K()
    seq_lens = [700, 333, 520, 64]
    q_lens = [131, 70, 257, 2]
    scale = 1.0 / math.sqrt(hd)
    case = paged_case(seq_lens, q_lens, nh, nkv, hd, B, "bfloat16", seed=hd + B + window)
    ref = reference_attention(case, nh, nkv, hd, scale, window)
    tables = case["tables"].cpu()
    gone = 0
    for si, i in enumerate(case["order"]):
        first_key = max(0, (seq_lens[i] - q_lens[i]) + 1 - window)      # of the portion's first row
        dead = first_key // B
        tables[si, :dead] = -1
        gone += dead
    assert gone > 20
    for mode in ("tcgen05", "mma"):
        case["ctx"].options = {"attn_prefill": mode}
        out = torch.zeros(case["ctx"].rows, nh * hd, dtype=torch.bfloat16, device=DEV)
        lib.paged_attention(case["q"], out, case["kc"], case["vc"], tables.to(DEV), case["ctx"], nh, nkv, hd,
                            scale, window)
        torch.cuda.synchronize()
        assert lib.attention_tcgen05_error() == 0
        close(out, ref, "bfloat16", f"prefill {mode} with pages given back")


def test_a_wait_that_runs_out_is_reported_and_the_kernel_returns():
    """Failure path of the bounded waits, without a fault: a test hook leaves out one copy of the
    streaming product, so its consumers wait for bytes that never come.  The wait gives up after the
    (shortened) limit, the kernel returns, the error word is set, the sampling kernel copies it out
    beside the tokens, and the host turns it into an exception.  Afterwards the same call works."""
    lib = K()
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(8, 2048, generator=g) * 0.5).bfloat16().to(DEV)
    w = (torch.randn(2560, 2048, generator=g) * 0.05).bfloat16().to(DEV)
    ref = x.double().cpu() @ w.double().cpu().T
    y = torch.zeros(8, 2560, dtype=torch.bfloat16, device=DEV)
    logits = torch.randn(8, 300, generator=g).to(DEV)
    packed = torch.zeros(2 + 8, dtype=torch.int32, device=DEV)
    lib.clear_errors()
    try:
        lib.stream_test_hooks(wait_limit_ns=3_000_000, skip_stage=0)
        lib.gemm_stream(x, w, y)
        lib.argmax(logits, packed[2:], packed[:2])
        torch.cuda.synchronize()                                   # returns: nothing spins for ever
        first, word = packed[:2].tolist()
        assert first == 1 and (word >> 16) in (1, 2), (first, word)
        with pytest.raises(lib.KernelError, match="gemm_stream: a bounded wait ran out"):
            lib.raise_on_status(first, word)
        assert lib.stream_error() == 0                              # cleared by raise_on_status
    finally:
        lib.stream_test_hooks(0, -1)
        lib.clear_errors()
    lib.gemm_stream(x, w, y)
    lib.argmax(logits, packed[2:], packed[:2])
    torch.cuda.synchronize()
    assert packed[:2].tolist() == [0, 0]
    close(y, ref, "bfloat16", "streaming product after the hooks were taken out")
    assert packed[2:].tolist() == logits.argmax(-1).tolist()


def test_the_engine_raises_when_a_kernel_gave_up_a_wait(tmp_path):
    """The same through generation: the step whose decode products could not finish raises instead
    of handing out tokens sampled from unfinished logits."""
    import kvcm
    import helpers
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    lib = K()
    folder = helpers.write_tiny("tiny-c", "bfloat16", str(tmp_path / "m"))
    ec = EngineConfig(kv=KVManagerConfig(num_blocks=32, block_size=16, max_seq_len=128, watermark_blocks=0),
                      sched=SchedulerConfig(max_num_seqs=2, max_batched_tokens=64), dtype="bfloat16", cuda_graphs=False)
    eng = kvcm.Engine.from_folder(folder, ec)
    eng.add_request(helpers.random_tokens(20, 320, 1), max_new_tokens=8)
    eng.step()                                                     # the prompt
    eng.step()                                                     # a healthy decode step
    lib.clear_errors()
    try:
        lib.stream_test_hooks(wait_limit_ns=3_000_000, skip_stage=0)
        with pytest.raises(lib.KernelError, match="gemm_stream: a bounded wait ran out"):
            eng.step()
    finally:
        lib.stream_test_hooks(0, -1)
        lib.clear_errors()
