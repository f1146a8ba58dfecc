"""Python face of ``libkvcm_cuda.so``: one function per exported launcher.

Every function checks what the kernel assumes (device, dtype, contiguity, shapes), passes raw
pointers and the current torch CUDA stream, and raises ``KernelError`` on a non-zero return.
There is no fallback of any kind: without the compiled library, or with tensors that are not
on a CUDA device, these functions raise.  ``launch_count()`` counts launches of this library's
kernels (used by the benchmark's ``gpu_launches``).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc.build import load_cuda

_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}
_ERR_UNSUPPORTED = 10001
_launches = 0


class KernelError(RuntimeError):
    pass


def launch_count() -> int:
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def add_launches(n: int) -> None:
    """Launches made by the C++ request loop, which calls the launchers without passing here."""
    global _launches
    _launches += int(n)


def profiling() -> bool:
    return _profile is not None


class DeviceBackend(ctypes.Structure):
    """Opaque room for the table of device functions that the kernel library fills for the C++
    request loop (csrc/include/device_backend.h): 23 function pointers."""
    _fields_ = [("slots", ctypes.c_void_p * 23)]


_backend = None


def device_backend_address() -> int:
    """Address of the filled table (kept alive for the life of the process)."""
    global _backend
    if _backend is None:
        b = DeviceBackend()
        size = int(_lib().kvcm_device_backend(ctypes.byref(b)))
        if size != ctypes.sizeof(DeviceBackend):
            raise KernelError("device backend: the table of the library has another layout")
        _backend = b
    return ctypes.addressof(_backend)


def _lib():
    return load_cuda()


def _suffix(t: torch.Tensor) -> str:
    try:
        return _SUFFIX[t.dtype]
    except KeyError:
        raise KernelError(f"kernels exist for float32 and bfloat16 storage, not {t.dtype}") from None


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    # (the raw handle of the current stream, without building a Stream object: a launch of a small
    # kernel costs about 10 us of host time, and a third of it was this)
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel called with a tensor that is not on a CUDA device "
                              "(this engine has no CPU path)")


_profile = None          # while profiling: [(kernel family, event recorded after its launch)]


def profile_start() -> None:
    """Starts per-family timing: from now on an event is recorded after every launch of this
    library's kernels (and after library products, which call ``profile_mark``).  The stream runs
    in order, so the time between two consecutive events is the time of the later launch (its
    launch gap included).  For eager steps only: events cannot be recorded into a CUDA graph."""
    global _profile
    first = torch.cuda.Event(enable_timing=True)
    first.record()
    _profile = [("", first)]


def profile_mark(name: str) -> None:
    if _profile is not None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        _profile.append((name, e))


def profile_stop() -> dict:
    """Ends profiling; {family: (launches, device milliseconds)}."""
    global _profile
    marks, _profile = _profile or [], None
    torch.cuda.synchronize()
    out: dict = {}
    for (_, before), (name, after) in zip(marks, marks[1:]):
        calls, ms = out.get(name, (0, 0.0))
        out[name] = (calls + 1, ms + before.elapsed_time(after))
    return out


def _check(rc: int, name: str, detail: str = "") -> None:
    global _launches
    _launches += 1
    if _profile is not None:
        profile_mark(name)
    if rc == 0:
        return
    if rc == _ERR_UNSUPPORTED:
        raise KernelError(f"{name}: sizes not supported by this kernel {detail}")
    raise KernelError(f"{name}: CUDA error {rc} at launch {detail}")


_I32 = torch.int32


def embed(ids: torch.Tensor, table: torch.Tensor, x: torch.Tensor) -> None:
    """x[t,:] = float(table[ids[t],:]); x is float32 [T, H]."""
    _cuda(ids, table, x)
    T, H = x.shape
    _need(ids.dtype == _I32 and ids.numel() >= T, "embed: ids must be int32 [T]")
    _need(x.dtype == torch.float32 and x.is_contiguous() and table.is_contiguous(), "embed: layout")
    _need(table.shape[1] == H, "embed: table width != hidden")
    fn = getattr(_lib(), "kvcm_embed_" + _suffix(table))
    _check(fn(_p(ids), _p(table), _p(x), T, H, table.shape[0], _stream()), "embed")


def rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
            out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """Optional x += delta, then out = weight * round(x * rsqrt(mean(x^2)+eps)).

    x float32 [T,H] (updated in place unless ``rows`` gathers); delta/out in the storage dtype;
    weight in the storage dtype or float32."""
    _cuda(x, delta, weight, out, rows)
    H = x.shape[1]
    n = out.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous(), "rmsnorm: x must be contiguous float32")
    _need(out.is_contiguous() and out.shape[1] == H and weight.numel() == H, "rmsnorm: shapes")
    _need(delta is None or (delta.dtype == out.dtype and delta.is_contiguous()
                            and delta.shape == x.shape), "rmsnorm: delta must match x in shape")
    _need(weight.dtype in (torch.float32, out.dtype), "rmsnorm: weight dtype")
    if rows is None:
        _need(n == x.shape[0], "rmsnorm: out rows != x rows")
    else:
        _need(rows.dtype == _I32 and rows.numel() >= n, "rmsnorm: rows must be int32 [n]")
    fn = getattr(_lib(), "kvcm_rmsnorm_" + _suffix(out))
    wf32 = int(weight.dtype == torch.float32)
    _check(fn(_p(x), _p(delta), _p(weight), wf32, _p(out), _p(rows), n, H,
              ctypes.c_float(eps), _stream()), "rmsnorm", f"(hidden={H})")


def add_residual(x: torch.Tensor, delta: torch.Tensor) -> None:
    _cuda(x, delta)
    _need(x.dtype == torch.float32 and x.is_contiguous() and delta.is_contiguous()
          and x.shape == delta.shape, "add_residual: shapes")
    fn = getattr(_lib(), "kvcm_add_residual_" + _suffix(delta))
    _check(fn(_p(x), _p(delta), ctypes.c_longlong(x.numel()), _stream()), "add_residual")


def rope_cache(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
               rotary_dim: int, interleaved: bool, slot_mapping: Optional[torch.Tensor],
               k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
               nh: int, nkv: int, hd: int, block_size: int, write_cache: bool = True) -> None:
    """Rotary encoding of the q and k heads of the fused rows in place, then K and V of each row
    are written to its page slot.  k_cache/v_cache: one layer, [pages, nkv, block, hd]."""
    _cuda(qkv, positions, inv_freq, slot_mapping, k_cache, v_cache)
    T = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] >= (nh + 2 * nkv) * hd, "rope_cache: qkv row too short")
    _need(positions.dtype == _I32 and positions.numel() >= T, "rope_cache: positions int32 [T]")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 >= rotary_dim,
              "rope_cache: inv_freq must be float32 [rotary_dim/2]")
    if write_cache:
        _need(slot_mapping is not None and slot_mapping.dtype == _I32 and slot_mapping.numel() >= T,
              "rope_cache: slot_mapping int32 [T]")
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype and k_cache.is_contiguous()
              and v_cache.is_contiguous(), "rope_cache: cache dtype/layout")
        _need(tuple(k_cache.shape[1:]) == (nkv, block_size, hd), "rope_cache: cache page shape")
    fn = getattr(_lib(), "kvcm_rope_cache_" + _suffix(qkv))
    _check(fn(_p(qkv), qkv.stride(0), _p(positions), _p(inv_freq), rotary_dim, int(interleaved),
              _p(slot_mapping), _p(k_cache), _p(v_cache), T, nh, nkv, hd, block_size,
              int(write_cache), _stream()), "rope_cache", f"(rotary_dim={rotary_dim}, hd={hd})")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, table: torch.Tensor) -> None:
    """table[t] = [cos(positions[t] * inv_freq) | sin(...)] (float32 [T, 2 * len(inv_freq)]): the
    angles of a step, which are the same in every layer."""
    _cuda(positions, inv_freq, table)
    T, width = table.shape
    _need(positions.dtype == _I32 and positions.numel() >= T, "rope_table: positions int32 [T]")
    _need(inv_freq.dtype == torch.float32 and table.dtype == torch.float32 and table.is_contiguous()
          and width == 2 * inv_freq.numel(), "rope_table: float32 inv_freq [hd/2] and table [T, hd]")
    _check(_lib().kvcm_rope_table_f32(_p(positions), _p(inv_freq), T, width // 2, _p(table), _stream()), "rope_table")


def rope_cache_table(qkv: torch.Tensor, table: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                     k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], nh: int, nkv: int, hd: int,
                     block_size: int, write_cache: bool = True) -> None:
    """``rope_cache`` for bfloat16 rows rotated over the whole head in rotate-half pairs, with the
    cosines and sines read from ``table`` (``rope_table``): the same bits."""
    _cuda(qkv, table, slot_mapping, k_cache, v_cache)
    T = qkv.shape[0]
    _need(qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape[1] >= (nh + 2 * nkv) * hd,
          "rope_cache_table: bfloat16 rows of q, k and v heads")
    _need(table.dtype == torch.float32 and table.is_contiguous() and tuple(table.shape) == (T, hd),
          "rope_cache_table: table float32 [T, hd]")
    if write_cache:
        _need(slot_mapping is not None and slot_mapping.dtype == _I32 and slot_mapping.numel() >= T,
              "rope_cache_table: slot_mapping int32 [T]")
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype and k_cache.is_contiguous()
              and v_cache.is_contiguous() and tuple(k_cache.shape[1:]) == (nkv, block_size, hd),
              "rope_cache_table: cache dtype/layout")
    rc = _lib().kvcm_rope_cache_table_bf16(_p(qkv), qkv.stride(0), _p(table), _p(slot_mapping), _p(k_cache), _p(v_cache),
                                           T, nh, nkv, hd, block_size, int(write_cache), _stream())
    _check(rc, "rope_cache_table", f"(hd={hd}, row stride {qkv.stride(0)})")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(gate_up, out)
    T, I = out.shape
    _need(gate_up.is_contiguous() and out.is_contiguous() and gate_up.shape == (T, 2 * I)
          and gate_up.dtype == out.dtype, "silu_mul: gate_up must be [T, 2I]")
    fn = getattr(_lib(), "kvcm_silu_mul_" + _suffix(out))
    _check(fn(_p(gate_up), _p(out), T, I, _stream()), "silu_mul")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, dst: torch.Tensor) -> None:
    _cuda(src, rows, dst)
    n, W = dst.shape
    _need(src.is_contiguous() and dst.is_contiguous() and src.shape[1] == W and src.dtype == dst.dtype
          and rows.dtype == _I32 and rows.numel() >= n, "gather_rows: shapes")
    fn = getattr(_lib(), "kvcm_gather_rows_" + _suffix(dst))
    _check(fn(_p(src), _p(rows), _p(dst), n, W, _stream()), "gather_rows")


def gemm_plain(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y[M,N] = x[M,K] @ w[N,K]^T with float accumulation in a fixed k order (plain kernel)."""
    _cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and y.shape == (M, N), "gemm_plain: shapes")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1, "gemm_plain: rows must be dense")
    _need(x.dtype == w.dtype, "gemm_plain: operand dtypes differ")
    if x.dtype == torch.float32:
        _need(y.dtype == torch.float32, "gemm_plain: float32 operands need a float32 result")
        name = "kvcm_gemm_plain_f32"
    elif x.dtype == torch.bfloat16:
        name = "kvcm_gemm_plain_bf16" if y.dtype == torch.bfloat16 else "kvcm_gemm_plain_bf16_f32out"
        _need(y.dtype in (torch.bfloat16, torch.float32), "gemm_plain: result dtype")
    else:
        raise KernelError(f"gemm_plain: dtype {x.dtype}")
    _check(getattr(_lib(), name)(_p(x), _p(w), _p(y), M, N, K, x.stride(0), w.stride(0), y.stride(0),
                                 _stream()), "gemm_plain")


def attention_plain(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_tables: torch.Tensor, row_seq: torch.Tensor, positions: torch.Tensor,
                    nh: int, nkv: int, hd: int, scale: float, window: int = 0) -> None:
    """Row-per-query paged attention.  q: [T, >= nh*hd] (row stride free), out: [T, nh*hd];
    caches [pages, nkv, block, hd]; block_tables int32 [S, max_blocks]."""
    _cuda(q, out, k_cache, v_cache, block_tables, row_seq, positions)
    T = out.shape[0]
    _need(q.stride(1) == 1 and out.stride(1) == 1, "attention: rows must be dense")
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype, "attention: dtypes differ")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape[1] == nkv
          and k_cache.shape[3] == hd, "attention: cache page shape")
    _need(block_tables.dtype == _I32 and block_tables.is_contiguous() and block_tables.dim() == 2,
          "attention: block_tables int32 [S, max_blocks]")
    _need(row_seq.dtype == _I32 and positions.dtype == _I32 and row_seq.numel() >= T
          and positions.numel() >= T, "attention: row_seq/positions int32 [T]")
    fn = getattr(_lib(), "kvcm_attention_plain_" + _suffix(q))
    _check(fn(_p(q), q.stride(0), _p(out), out.stride(0), _p(k_cache), _p(v_cache), _p(block_tables),
              block_tables.shape[1], _p(row_seq), _p(positions), T, nh, nkv, hd, k_cache.shape[2],
              ctypes.c_float(scale), int(window), _stream()), "attention_plain", f"(hd={hd}, nh={nh}, nkv={nkv})")


# Kernel families whose bounded waits report through an error word, in the order of the status
# index that the sampling kernels write (csrc/cuda/sampling.cu: status_words).
STATUS_FAMILIES = ("gemm_stream", "gemm_tcgen05", "gemm_tcgen05_pair", "gemm_tcgen05_splitk", "attention_tcgen05")


def describe_status(first: int, word: int) -> str:
    """Text for a status pair written by the sampling kernels: ``first`` = 1 + index of the kernel
    family whose error word was set (0 = none), ``word`` = (code << 16) | block."""
    name = STATUS_FAMILIES[first - 1] if 1 <= first <= len(STATUS_FAMILIES) else f"family {first}"
    return (f"{name}: a bounded wait ran out on the device (code {(word >> 16) & 0xffff}, block {word & 0xffff}); "
            f"the outputs of this step are not valid")


def raise_on_status(first: int, word: int) -> None:
    """Raises ``KernelError`` when the status pair of a step names a kernel family; clears the
    device's error words first so that the next step starts clean."""
    if not first:
        return
    clear_errors()
    raise KernelError(describe_status(int(first), int(word)))


def clear_errors() -> None:
    """Reads and clears every family's error word (synchronises with the device)."""
    for fn in (stream_error, tcgen05_error, pair_error, splitk_error, attention_tcgen05_error):
        fn()


def check_errors() -> None:
    """Host-side read of every family's error word (synchronises); raises if one is set.  For paths
    that synchronise anyway (scoring, replay); generation reads the status pair beside its tokens."""
    for i, fn in enumerate((stream_error, tcgen05_error, pair_error, splitk_error, attention_tcgen05_error)):
        word = fn()
        if word:
            clear_errors()
            raise KernelError(describe_status(i + 1, word))


def _status_ptr(status: Optional[torch.Tensor]):
    if status is None:
        return None
    _cuda(status)
    _need(status.dtype == _I32 and status.numel() >= 2 and status.is_contiguous(), "status: int32 [2]")
    return _p(status)


def argmax(logits: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """out[r] = first index of the row's maximum.  ``status`` (int32 [2], optional) receives the
    first error word that a kernel of this step has set (see ``describe_status``)."""
    _cuda(logits, out)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous() and out.dtype == _I32
          and out.numel() >= R, "argmax: logits float32 [R,V], out int32 [R]")
    _check(_lib().kvcm_argmax_status_f32(_p(logits), _p(out), R, V, _status_ptr(status), _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor,
           request_id: torch.Tensor, position: torch.Tensor, out: torch.Tensor,
           status: Optional[torch.Tensor] = None) -> None:
    """Per row: temperature <= 0 -> argmax; else one draw from softmax(logits / temperature) with a
    uniform number that depends only on (seed, request id, position).  ``status`` as in ``argmax``."""
    _cuda(logits, temperature, seed, request_id, position, out)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: logits float32 [R,V]")
    _need(temperature.dtype == torch.float32 and seed.dtype == torch.int64
          and request_id.dtype == torch.int64 and position.dtype == _I32 and out.dtype == _I32,
          "sample: temperature f32, seed/request_id i64, position/out i32")
    _need(min(temperature.numel(), seed.numel(), request_id.numel(), position.numel(),
              out.numel()) >= R, "sample: per-row arrays shorter than the number of rows")
    _check(_lib().kvcm_sample_status_f32(_p(logits), _p(temperature), _p(seed), _p(request_id),
                                         _p(position), _p(out), R, V, _status_ptr(status), _stream()), "sample")


# ------------------------------------------------------------------ dispatch of attention

def paged_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_tables: torch.Tensor, ctx, nh: int, nkv: int, hd: int, scale: float,
                    window: int = 0) -> None:
    """Attention of all rows of a step.  Rows [0, ctx.decode_seqs) are single-row entries, the
    rest are the rows of longer portions.  ``ctx.options['attention']``: 'plain' forces the plain
    kernel for every row; float32 storage always uses it (the true 32-bit path)."""
    mode = ctx.options.get("attention", "auto")
    if mode == "plain" or q.dtype == torch.float32 or not fast_attention_supported(nh, nkv, hd, k_cache.shape[2]):
        attention_plain(q, out, k_cache, v_cache, block_tables, ctx.row_seq, ctx.positions,
                        nh, nkv, hd, scale, window)
        return
    nd = ctx.decode_seqs
    if nd > 0:
        attention_decode(q[:nd], out[:nd], k_cache, v_cache, block_tables, ctx, nh, nkv, hd, scale, window)
    if ctx.rows > nd:
        attention_prefill(q, out, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, scale, window)


def fast_attention_supported(nh: int, nkv: int, hd: int, block_size: int) -> bool:
    return nkv > 0 and nh % nkv == 0 and bool(_lib().kvcm_attention_fast_supports(int(hd)))


_SM_COUNT = {}


def sm_count(device) -> int:
    d = torch.device(device)
    if d not in _SM_COUNT:
        _SM_COUNT[d] = torch.cuda.get_device_properties(d).multi_processor_count
    return _SM_COUNT[d]


KEY_TILE = 64
CLUSTER_PARTS = 8           # kvcm_attention_decode_cluster_parts()


_RESIDENT = {}


def _decode_resident_blocks(hd: int, device) -> int:
    key = (int(hd), torch.device(device))
    if key not in _RESIDENT:
        n = int(_lib().kvcm_attention_decode_resident_blocks(int(hd)))
        _RESIDENT[key] = n if n > 0 else 3 * sm_count(device)
    return _RESIDENT[key]


def decode_partitions(seqs: int, nh: int, nkv: int, hd: int, max_ctx: int, device, version: str = "auto",
                      force_parts: int = 0):
    """How the decode kernel splits the context: (keys per partition, number of partitions).

    'v1': the whole context in one block per (request, KV head).  'v2'/'auto': as many partitions
    as keep the whole grid resident at once (a second wave of blocks costs more than longer
    partitions), each at least 128 keys long, and no more than the 8 that merge inside one cluster
    unless that would leave partitions of more than 512 keys.  Measured on a B200 over batches
    1..128 and contexts 512..8192.  (The reference fixes 512 keys per partition,
    src/cuda/paged_attention.cu:22.)  ``force_parts`` > 0 asks for that many partitions (tuning
    and tests)."""
    max_ctx = max(int(max_ctx), 1)
    whole = (max_ctx + KEY_TILE - 1) // KEY_TILE * KEY_TILE
    if version == "v1":
        return whole, 1
    G = nh // nkv
    blocks = max(1, seqs * nkv * ((G + 15) // 16))
    if force_parts > 0:
        parts = min(int(force_parts), max(1, whole // KEY_TILE))
    else:
        parts = max(1, min(_decode_resident_blocks(hd, device) // blocks, max_ctx // 128))
        if parts > CLUSTER_PARTS:
            parts = max(CLUSTER_PARTS, min(parts, (max_ctx + 511) // 512))
    size = ((max_ctx + parts - 1) // parts + KEY_TILE - 1) // KEY_TILE * KEY_TILE
    parts = (max_ctx + size - 1) // size
    return size, parts


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_tables: torch.Tensor, ctx, nh: int, nkv: int, hd: int, scale: float,
                     window: int = 0) -> None:
    """Single-row entries: q/out hold one row per request, in the order of the batch's entries."""
    _cuda(q, out, k_cache, v_cache, block_tables)
    S = q.shape[0]
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16,
          "attention_decode: bfloat16 only")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous(),
          "attention_decode: layout")
    _need(q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0, "attention_decode: q rows must be 16-byte aligned")
    size, parts = decode_partitions(S, nh, nkv, hd, ctx.max_decode_ctx, q.device,
                                    ctx.options.get("attn_version", "auto"), int(ctx.options.get("attn_parts", 0)))
    scratch = None
    # Up to 8 partitions merge inside a thread-block cluster; more go through scratch memory
    # and a merge kernel ('attn_merge': 'kernel' forces that path).
    in_cluster = 1 < parts <= CLUSTER_PARTS and ctx.options.get("attn_merge", "cluster") == "cluster"
    if parts > 1 and not in_cluster:
        n = S * nh * parts * (hd + 2)          # partial outputs + (max, sum) per partition
        scratch = torch.empty(n, dtype=torch.float32, device=q.device)
    rc = _lib().kvcm_attention_decode_bf16(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_cache), _p(v_cache), _p(block_tables),
        block_tables.shape[1], _p(ctx.seq_ctx_len), S, nh, nkv, hd, k_cache.shape[2],
        ctypes.c_float(scale), int(window), size, parts, _p(scratch), int(in_cluster), _stream())
    _check(rc, "attention_decode", f"(hd={hd}, nh={nh}, nkv={nkv})")
    if parts > 1 and not in_cluster:
        global _launches
        _launches += 1                      # the merge kernel


def attention_prefill(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      block_tables: torch.Tensor, ctx, nh: int, nkv: int, hd: int, scale: float,
                      window: int = 0) -> None:
    """Rows of portions longer than one token; q/out are the step's full row arrays.
    ``ctx.options['attn_prefill']``: 'tcgen05' | 'mma' force a kernel; 'auto' takes the tcgen05
    kernel where it supports the sizes (head_dim 64 or 128; pages of 8 to 64 keys dividing 64, or multiples of 64)."""
    _cuda(q, out, k_cache, v_cache, block_tables)
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16,
          "attention_prefill: bfloat16 only")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous(),
          "attention_prefill: layout")
    _need(q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0, "attention_prefill: q rows must be 16-byte aligned")
    _need(ctx.tile_rows == 64, "attention_prefill: the batch must be tiled in 64 query rows")
    mode = ctx.options.get("attn_prefill", "auto")
    B = k_cache.shape[2]
    if mode != "mma" and (mode == "tcgen05" or prefill_tcgen05_supported(hd, B)):
        _need(out.data_ptr() % 16 == 0 and out.stride(0) % 8 == 0, "attention_prefill: out rows must be 16-byte aligned")
        rc = _lib().kvcm_attention_prefill_tcgen05_bf16(
            _p(q), q.stride(0), q.shape[0], _p(out), out.stride(0), _p(k_cache), _p(v_cache), k_cache.shape[0],
            _p(block_tables), block_tables.shape[1], _p(ctx.tile_seq), _p(ctx.tile_q0), _p(ctx.seq_q_start),
            _p(ctx.seq_q_len), _p(ctx.seq_ctx_len), ctx.prefill_tiles, nh, nkv, hd, B, ctypes.c_float(scale),
            int(window), _stream())
        _check(rc, "attention_prefill_tcgen05", f"(hd={hd}, nh={nh}, nkv={nkv}, block={B})")
        return
    rc = _lib().kvcm_attention_prefill_bf16(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_cache), _p(v_cache), _p(block_tables),
        block_tables.shape[1], _p(ctx.tile_seq), _p(ctx.tile_q0), _p(ctx.seq_q_start), _p(ctx.seq_q_len),
        _p(ctx.seq_ctx_len), ctx.prefill_tiles, nh, nkv, hd, B, ctypes.c_float(scale),
        int(window), _stream())
    _check(rc, "attention_prefill", f"(hd={hd}, nh={nh}, nkv={nkv})")


def prefill_tcgen05_supported(hd: int, block_size: int) -> bool:
    return bool(_lib().kvcm_attention_tcgen05_supports(int(hd), int(block_size)))


def attention_tcgen05_error() -> int:
    """Error word of the tcgen05 attention kernel: 0, or (code << 16 | block) of a bounded wait that
    ran out.  Reading clears it.  Synchronises the device."""
    return int(_lib().kvcm_attention_tcgen05_error())

def stream_gemm_supported(M: int, N: int, K: int) -> bool:
    """True when the TMA-pipelined weight-streaming kernel takes this product."""
    return bool(_lib().kvcm_gemm_stream_supports(int(M), int(N), int(K)))


def gemm_stream(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y[M,N] = x[M,K] @ w[N,K]^T for M <= 16 with W streamed through a shared-memory ring by bulk
    asynchronous copies (bfloat16 operands, float accumulation, bfloat16 or float result)."""
    _cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and y.shape == (M, N), "gemm_stream: shapes")
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and y.dtype in (torch.bfloat16, torch.float32),
          "gemm_stream: bfloat16 operands, bfloat16 or float32 result")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1, "gemm_stream: rows must be dense")
    rc = _lib().kvcm_gemm_stream_bf16(_p(x), _p(w), _p(y), M, N, K, x.stride(0), w.stride(0), y.stride(0),
                                      int(y.dtype == torch.float32), sm_count(x.device), _stream())
    _check(rc, "gemm_stream", f"(M={M}, N={N}, K={K})")


def stream_test_hooks(wait_limit_ns: int = 0, skip_stage: int = -1) -> None:
    """For tests of the failure path: the streaming product's wait limit (0 = its default) and a
    stage of every block whose copy is left out (-1 = none), so that a wait runs out."""
    rc = _lib().kvcm_stream_test_hooks(ctypes.c_uint64(int(wait_limit_ns)), int(skip_stage))
    if rc != 0:
        raise KernelError("stream_test_hooks: could not set the device words")


def stream_error() -> int:
    """Error word of the streaming kernels: 0, or (code << 16 | block) of a bounded wait that ran
    out (1: the producer waited for a free stage, 2: a consumer waited for data).  Reading clears it.
    Synchronises the device."""
    return int(_lib().kvcm_stream_error())


def qkv_rope_cache(x: torch.Tensor, w_qkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                   inv_freq: torch.Tensor, slot_mapping: torch.Tensor, k_cache: torch.Tensor,
                   v_cache: torch.Tensor, nh: int, nkv: int, hd: int,
                   partials: Optional[torch.Tensor] = None, eps: float = 0.0) -> None:
    """Fused decode kernel: qkv product (M <= 16), rotate-half rotary encoding over the whole head,
    q into ``q_out`` [M, nh*hd], k (rotated) and v into the rows' cache page slots.  Gives the same
    bits as ``gemm_stream`` followed by ``rope_cache``.  With ``partials`` (float32 [tiles, 16] as
    ``gemm_stream_residual`` leaves them) row m of the product is first scaled by
    rsqrt(sum(partials[:, m]) / K + eps): ``x`` is then a normed row before its scale."""
    _cuda(x, w_qkv, q_out, positions, inv_freq, slot_mapping, k_cache, v_cache, partials)
    _need(partials is None or (partials.dtype == torch.float32 and partials.is_contiguous() and partials.dim() == 2
                               and partials.shape[1] == 16), "qkv_rope_cache: partials float32 [tiles, 16]")
    M, K = x.shape
    _need(w_qkv.shape == ((nh + 2 * nkv) * hd, K) and q_out.shape[0] == M and q_out.shape[1] >= nh * hd,
          "qkv_rope_cache: shapes")
    _need(x.dtype == w_qkv.dtype == q_out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16,
          "qkv_rope_cache: bfloat16 only")
    _need(x.stride(1) == 1 and w_qkv.stride(1) == 1 and q_out.stride(1) == 1 and k_cache.is_contiguous()
          and v_cache.is_contiguous(), "qkv_rope_cache: layout")
    _need(tuple(k_cache.shape[1:]) == (nkv, k_cache.shape[2], hd), "qkv_rope_cache: cache page shape")
    _need(positions.dtype == _I32 and slot_mapping.dtype == _I32 and positions.numel() >= M
          and slot_mapping.numel() >= M, "qkv_rope_cache: positions/slot_mapping int32 [M]")
    _need(inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == hd, "qkv_rope_cache: inv_freq float32 [hd/2]")
    rc = _lib().kvcm_qkv_rope_cache_scaled_bf16(_p(x), _p(partials) if partials is not None else None,
                                                partials.shape[0] if partials is not None else 0, ctypes.c_float(eps),
                                                _p(w_qkv), _p(q_out), M, K, x.stride(0), w_qkv.stride(0),
                                                q_out.stride(0), _p(positions), _p(inv_freq), _p(slot_mapping),
                                                _p(k_cache), _p(v_cache), nh, nkv, hd, k_cache.shape[2],
                                                sm_count(x.device), _stream())
    _check(rc, "qkv_rope_cache", f"(M={M}, K={K}, nh={nh}, nkv={nkv}, hd={hd})")


def gemm_stream_residual(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, partials: torch.Tensor,
                         h_out: Optional[torch.Tensor] = None, next_w: Optional[torch.Tensor] = None) -> None:
    """The product that ends a sublayer (M <= 16): resid[M,N] (float32, in place) += bfloat16(x @ w^T);
    partials[t, m] = the sum over columns 16t..16t+15 of the new resid[m]^2 (``partials`` float32
    [ceil(N/16), 16]); and with ``next_w`` (bfloat16 [N]) h_out[M,N] = bfloat16(next_w * resid): the row
    the next norm hands on before its scale, which the ``partials`` argument of ``qkv_rope_cache`` and
    ``gate_up_silu`` applies."""
    _cuda(x, w, resid, partials, h_out, next_w)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and resid.shape == (M, N), "gemm_stream_residual: shapes")
    _need(x.dtype == w.dtype == torch.bfloat16 and resid.dtype == partials.dtype == torch.float32,
          "gemm_stream_residual: bfloat16 operands, float32 residual and partial sums")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and resid.stride(1) == 1, "gemm_stream_residual: rows must be dense")
    _need(partials.is_contiguous() and tuple(partials.shape) == ((N + 15) // 16, 16), "gemm_stream_residual: partials [ceil(N/16), 16]")
    _need((h_out is None) == (next_w is None), "gemm_stream_residual: h_out and next_w go together")
    if next_w is not None:
        _need(h_out.dtype == next_w.dtype == torch.bfloat16 and h_out.shape == (M, N) and h_out.stride(1) == 1
              and next_w.numel() == N and next_w.is_contiguous(), "gemm_stream_residual: h_out [M,N], next_w [N] bfloat16")
    rc = _lib().kvcm_gemm_stream_residual_bf16(_p(x), _p(w), _p(resid), _p(partials),
                                               _p(h_out) if h_out is not None else None,
                                               _p(next_w) if next_w is not None else None, M, N, K, x.stride(0),
                                               w.stride(0), resid.stride(0), h_out.stride(0) if h_out is not None else 0,
                                               sm_count(x.device), _stream())
    _check(rc, "gemm_stream_residual", f"(M={M}, N={N}, K={K})")


def qkv_rope_cache_supported(M: int, K: int, nh: int, nkv: int, hd: int) -> bool:
    return hd % 16 == 0 and bool(_lib().kvcm_gemm_stream_fused_supports(int(M), int((nh + 2 * nkv) * hd), int(K)))


def gate_up_silu(x: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor,
                 partials: Optional[torch.Tensor] = None, eps: float = 0.0) -> None:
    """Fused decode kernel: act[M, I] = silu(x Wg^T) * (x Wu^T), Wg/Wu the halves of w [2I, K].
    ``partials``: both products scaled per row first, as in ``qkv_rope_cache``."""
    _cuda(x, w_gate_up, act, partials)
    _need(partials is None or (partials.dtype == torch.float32 and partials.is_contiguous() and partials.dim() == 2
                               and partials.shape[1] == 16), "gate_up_silu: partials float32 [tiles, 16]")
    M, K = x.shape
    I = act.shape[1]
    _need(w_gate_up.shape == (2 * I, K) and act.shape[0] == M, "gate_up_silu: shapes")
    _need(x.dtype == w_gate_up.dtype == act.dtype == torch.bfloat16, "gate_up_silu: bfloat16 only")
    _need(x.stride(1) == 1 and w_gate_up.stride(1) == 1 and act.stride(1) == 1, "gate_up_silu: layout")
    rc = _lib().kvcm_gate_up_silu_scaled_bf16(_p(x), _p(partials) if partials is not None else None,
                                              partials.shape[0] if partials is not None else 0, ctypes.c_float(eps),
                                              _p(w_gate_up), _p(act), M, I, K, x.stride(0), w_gate_up.stride(0),
                                              act.stride(0), sm_count(x.device), _stream())
    _check(rc, "gate_up_silu", f"(M={M}, I={I}, K={K})")


def gate_up_silu_supported(M: int, I: int, K: int) -> bool:
    return I % 8 == 0 and bool(_lib().kvcm_gemm_stream_fused_supports(int(M), int(2 * I), int(K)))


def gate_up_silu_tcgen05(x: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor) -> None:
    """act[M, I] = silu(x Wg^T) * (x Wu^T) for many rows: the tcgen05 product with the activation in
    its epilogue (the roundings of the separate product and activation kernels); the [M, 2I]
    intermediate never goes to memory."""
    _cuda(x, w_gate_up, act)
    M, K = x.shape
    I = act.shape[1]
    _need(w_gate_up.shape == (2 * I, K) and act.shape[0] == M, "gate_up_silu_tcgen05: shapes")
    _need(x.dtype == w_gate_up.dtype == act.dtype == torch.bfloat16, "gate_up_silu_tcgen05: bfloat16 only")
    _need(x.stride(1) == 1 and w_gate_up.stride(1) == 1 and act.stride(1) == 1, "gate_up_silu_tcgen05: rows must be dense")
    rc = _lib().kvcm_gate_up_silu_tcgen05_bf16(_p(x), _p(w_gate_up), _p(act), M, I, K, x.stride(0),
                                               w_gate_up.stride(0), act.stride(0), _stream())
    _check(rc, "gate_up_silu_tcgen05", f"(M={M}, I={I}, K={K})")


def tcgen05_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """True when the tcgen05 kernel takes this product (bfloat16, K and row strides multiples of 8)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(_lib().kvcm_gemm_tcgen05_supports(x.shape[0], w.shape[0], x.shape[1], x.stride(0), w.stride(0))))


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y[M,N] = x[M,K] @ w[N,K]^T on the fifth-generation tensor cores (TMA tensor maps, tcgen05.mma
    with the accumulator in tensor memory).  bfloat16 operands; bfloat16 or float32 result."""
    _cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and y.shape == (M, N), "gemm_tcgen05: shapes")
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and y.dtype in (torch.bfloat16, torch.float32),
          "gemm_tcgen05: bfloat16 operands, bfloat16 or float32 result")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1, "gemm_tcgen05: rows must be dense")
    rc = _lib().kvcm_gemm_tcgen05_bf16(_p(x), _p(w), _p(y), M, N, K, x.stride(0), w.stride(0), y.stride(0),
                                       int(y.dtype == torch.float32), _stream())
    _check(rc, "gemm_tcgen05", f"(M={M}, N={N}, K={K})")


def splitk_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """True when the split-K tcgen05 kernel takes this product (up to 256 rows, bfloat16, K and row
    strides multiples of 8)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(_lib().kvcm_gemm_tcgen05_splitk_supports(x.shape[0], w.shape[0], x.shape[1], x.stride(0), w.stride(0))))


def gemm_tcgen05_splitk(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y[M,N] = x[M,K] @ w[N,K]^T for M <= 256 on the fifth-generation tensor cores with the operands
    swapped (128 weight rows are the tall operand) and K split over a thread-block cluster whose
    blocks add their partial sums through distributed shared memory.  bfloat16 operands; bfloat16 or
    float32 result."""
    _cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and y.shape == (M, N), "gemm_tcgen05_splitk: shapes")
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and y.dtype in (torch.bfloat16, torch.float32),
          "gemm_tcgen05_splitk: bfloat16 operands, bfloat16 or float32 result")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1, "gemm_tcgen05_splitk: rows must be dense")
    rc = _lib().kvcm_gemm_tcgen05_splitk_bf16(_p(x), _p(w), _p(y), M, N, K, x.stride(0), w.stride(0), y.stride(0),
                                              int(y.dtype == torch.float32), _stream())
    _check(rc, "gemm_tcgen05_splitk", f"(M={M}, N={N}, K={K})")


def splitk_error() -> int:
    """Error word of the split-K tcgen05 kernel: 0, or (code << 16 | block) of a bounded wait that
    ran out.  Reading clears it.  Synchronises the device."""
    return int(_lib().kvcm_gemm_tcgen05_splitk_error())


def pair_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """True when the two-SM tcgen05 kernel takes this product (bfloat16, K and row strides multiples of 8)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(_lib().kvcm_gemm_tcgen05_pair_supports(x.shape[0], w.shape[0], x.shape[1], x.stride(0), w.stride(0))))


_pair_workspaces: dict = {}


def _pair_workspace(device: torch.device, split: int):
    """Partial sums and flags of the two-SM kernel's split walk, one set per device (the kernel's
    launches on a device are expected on one stream at a time).  (None, None, 0) without it."""
    if split == 0:
        return None, None, 0
    key = torch.device(device).index or 0
    ws = _pair_workspaces.get(key)
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            return None, None, 0
        slots = int(_lib().kvcm_gemm_tcgen05_pair_capacity())
        if slots <= 0:
            return None, None, 0
        part = torch.empty(slots * int(_lib().kvcm_gemm_tcgen05_pair_slot_floats()), dtype=torch.float32, device=device)
        flag = torch.zeros(slots * int(_lib().kvcm_gemm_tcgen05_pair_slot_flags()), dtype=torch.int32, device=device)
        ws = _pair_workspaces[key] = (part, flag, slots)
    return ws


def gemm_tcgen05_pair(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, bn: int = 0, band: int = 0,
                      split: int = -1) -> None:
    """y[M,N] = x[M,K] @ w[N,K]^T with 256 x bn tiles computed by pairs of SMs (tcgen05.mma.cta_group::2:
    each block of a pair loads half of the tile's rows of w).  bn: tile width, band: row tiles walked
    together; 0 = chosen by the kernel's host side.  split: 1 = equal shares of k-steps for every
    pair (partial sums through a workspace), 0 = whole tiles, -1 = chosen by the host side.
    bfloat16 operands; bfloat16 or float32 result."""
    _cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and y.shape == (M, N), "gemm_tcgen05_pair: shapes")
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and y.dtype in (torch.bfloat16, torch.float32),
          "gemm_tcgen05_pair: bfloat16 operands, bfloat16 or float32 result")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1, "gemm_tcgen05_pair: rows must be dense")
    part, flag, slots = _pair_workspace(x.device, split)
    rc = _lib().kvcm_gemm_tcgen05_pair_bf16(_p(x), _p(w), _p(y), M, N, K, x.stride(0), w.stride(0), y.stride(0),
                                            int(y.dtype == torch.float32), int(bn), int(band), int(split),
                                            _p(part) if part is not None else None,
                                            _p(flag) if flag is not None else None, slots, _stream())
    _check(rc, "gemm_tcgen05_pair", f"(M={M}, N={N}, K={K}, bn={bn}, split={split})")


def gate_up_silu_tcgen05_pair(x: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor, bn: int = 0,
                              band: int = 0, split: int = -1) -> None:
    """act[M, I] = silu(x Wg^T) * (x Wu^T) on pairs of SMs: one block of a pair loads the tile's gate
    rows, the other its up rows, and the epilogue applies the activation (the roundings of the
    separate product and activation kernels)."""
    _cuda(x, w_gate_up, act)
    M, K = x.shape
    I = act.shape[1]
    _need(w_gate_up.shape == (2 * I, K) and act.shape[0] == M, "gate_up_silu_tcgen05_pair: shapes")
    _need(x.dtype == w_gate_up.dtype == act.dtype == torch.bfloat16, "gate_up_silu_tcgen05_pair: bfloat16 only")
    _need(x.stride(1) == 1 and w_gate_up.stride(1) == 1 and act.stride(1) == 1, "gate_up_silu_tcgen05_pair: rows must be dense")
    part, flag, slots = _pair_workspace(x.device, split)
    rc = _lib().kvcm_gate_up_silu_tcgen05_pair_bf16(_p(x), _p(w_gate_up), _p(act), M, I, K, x.stride(0),
                                                    w_gate_up.stride(0), act.stride(0), int(bn), int(band), int(split),
                                                    _p(part) if part is not None else None,
                                                    _p(flag) if flag is not None else None, slots, _stream())
    _check(rc, "gate_up_silu_tcgen05_pair", f"(M={M}, I={I}, K={K}, bn={bn}, split={split})")


def pair_error() -> int:
    """Error word of the two-SM tcgen05 kernel: 0, or (code << 16 | block) of a bounded wait that ran
    out (1: a TMA thread waited for a free stage, 2: the MMA thread waited for data, 3: an epilogue
    waited for the accumulator, 4: the MMA thread waited for the epilogues, 5: an epilogue waited for
    another pair's partial sums).  Reading clears it.
    Synchronises the device."""
    return int(_lib().kvcm_gemm_tcgen05_pair_error())


def tcgen05_error() -> int:
    """Error word of the tcgen05 kernel: 0, or (code << 16 | block) of a bounded wait that ran out
    (1: the TMA thread waited for a free stage, 2: the MMA thread waited for data, 3: the epilogue
    waited for the accumulator).  Reading clears it.  Synchronises the device."""
    return int(_lib().kvcm_tcgen05_error())


# ------------------------------------------------------------------ the step's forward pass from C++

FORWARD_MAX_GROUPS = 4


class ForwardLayer(ctypes.Structure):
    """One call site of the run order (csrc/cuda/step_forward.cu: KvcmForwardLayer)."""
    _fields_ = [("w_qkv", ctypes.c_void_p), ("w_o", ctypes.c_void_p), ("w_gate_up", ctypes.c_void_p),
                ("w_down", ctypes.c_void_p), ("norm1", ctypes.c_void_p), ("norm2", ctypes.c_void_p),
                ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
                ("eps1", ctypes.c_float), ("eps2", ctypes.c_float),
                ("group", ctypes.c_int), ("window", ctypes.c_int), ("writes", ctypes.c_int), ("num_pages", ctypes.c_int)]


class ForwardArgs(ctypes.Structure):
    """The argument block of ``kvcm_forward`` (csrc/cuda/step_forward.cu: KvcmForwardArgs)."""
    _fields_ = [
        ("layers", ctypes.c_void_p), ("embed", ctypes.c_void_p), ("final_norm", ctypes.c_void_p),
        ("lm_head", ctypes.c_void_p), ("inv_freq", ctypes.c_void_p),
        ("tokens", ctypes.c_void_p), ("positions", ctypes.c_void_p), ("row_seq", ctypes.c_void_p),
        ("seq_q_start", ctypes.c_void_p), ("seq_q_len", ctypes.c_void_p), ("seq_ctx_len", ctypes.c_void_p),
        ("tile_seq", ctypes.c_void_p), ("tile_q0", ctypes.c_void_p), ("logit_rows", ctypes.c_void_p),
        ("group_tables", ctypes.c_void_p * FORWARD_MAX_GROUPS), ("group_slots", ctypes.c_void_p * FORWARD_MAX_GROUPS),
        ("x", ctypes.c_void_p), ("h", ctypes.c_void_p), ("qkv", ctypes.c_void_p), ("attn", ctypes.c_void_p),
        ("proj", ctypes.c_void_p), ("gate_up", ctypes.c_void_p), ("act", ctypes.c_void_p), ("h_last", ctypes.c_void_p),
        ("logits", ctypes.c_void_p), ("attn_scratch", ctypes.c_void_p), ("lib_workspace", ctypes.c_void_p),
        ("norm_partials", ctypes.c_void_p), ("rope_table", ctypes.c_void_p),
        ("attn_scratch_floats", ctypes.c_longlong), ("lib_workspace_bytes", ctypes.c_longlong),
        ("norm_partials_floats", ctypes.c_longlong), ("rope_table_floats", ctypes.c_longlong),
        ("num_layers", ctypes.c_int), ("f32", ctypes.c_int), ("H", ctypes.c_int), ("I", ctypes.c_int),
        ("nh", ctypes.c_int), ("nkv", ctypes.c_int), ("hd", ctypes.c_int), ("V", ctypes.c_int),
        ("block_size", ctypes.c_int), ("max_blocks", ctypes.c_int), ("sm_count", ctypes.c_int),
        ("rows", ctypes.c_int), ("seqs", ctypes.c_int), ("decode_seqs", ctypes.c_int), ("prefill_tiles", ctypes.c_int),
        ("tile_rows", ctypes.c_int), ("max_decode_ctx", ctypes.c_int), ("num_logits", ctypes.c_int),
        ("reserved", ctypes.c_int),
        ("final_eps", ctypes.c_float), ("scale", ctypes.c_float),
    ]


def forward_layouts_match() -> bool:
    lib = _lib()
    return (ctypes.sizeof(ForwardArgs) == int(lib.kvcm_forward_args_bytes())
            and ctypes.sizeof(ForwardLayer) == int(lib.kvcm_forward_layer_bytes()))


_forward_launches = ctypes.c_int(0)


def forward(args: ForwardArgs) -> int:
    """The whole forward pass of a step launched from C++ (csrc/cuda/step_forward.cu); returns the
    number of kernel launches it made.  The caller owns every buffer the block names."""
    global _launches
    rc = _lib().kvcm_forward(ctypes.byref(args), ctypes.byref(_forward_launches), _stream())
    n = int(_forward_launches.value)
    _launches += n
    if _profile is not None:
        profile_mark("forward (whole step)")
    if rc == 0:
        return n
    if rc == _ERR_UNSUPPORTED:
        raise KernelError(f"forward: sizes not supported (rows {args.rows}, hidden {args.H}, heads {args.nh}/{args.nkv} "
                          f"of {args.hd})")
    raise KernelError(f"forward: error {rc} at a launch (rows {args.rows})")
