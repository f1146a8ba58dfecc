"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some callers cannot call cudaMalloc while they run a step: a step being captured into a CUDA graph
by a host framework, a real-time loop that must not take the allocator's lock, a plugin that may
not touch its host's memory pool.  For them the library keeps the split-context partial results in
a built-in device array.  The test calls ``kvcm_attention_decode_bf16_noalloc`` twice in a row on
different inputs and compares each result with the ordinary entry point (whose scratch the caller
allocates) and with a float64 reference, and checks that a request beyond the built-in array is
refused with a clear message.  The file sorts last so that a run stopping at the first failure has
already run every other test; it passes alone in a fresh process as well as after the others.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from kvcm.csrc.build import load_cuda
    lib = load_cuda()
    lib.kvcm_attention_decode_noalloc_error.restype = ctypes.c_char_p
    lib.kvcm_attention_decode_noalloc_capacity.restype = ctypes.c_longlong
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _call(lib, symbol, case, out, nh, nkv, hd, scale, part_size, parts, scratch=None):
    args = [_p(case["q"]), case["q"].stride(0), _p(out), out.stride(0), _p(case["kc"]), _p(case["vc"]),
            _p(case["tables"]), case["tables"].shape[1], _p(case["ctx"].seq_ctx_len), out.shape[0], nh, nkv,
            hd, case["kc"].shape[2], ctypes.c_float(scale), 0, part_size, parts]
    if scratch is not None:
        args += [_p(scratch), 0]             # the merge through scratch memory, not inside a cluster
    args.append(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return getattr(lib, symbol)(*args)


def test_decode_attention_without_allocation_matches_the_ordinary_entry_point():
    from test_gpu_kernels import close, paged_case, reference_attention
    lib = _lib()
    nh, nkv, hd, B = 16, 4, 64, 16
    scale = 1.0 / math.sqrt(hd)
    part_size, parts = 256, 5
    assert lib.kvcm_attention_decode_noalloc_capacity() == 2 * 1024 * 1024
    for round_no, lens in enumerate(([1200, 700, 64, 1], [33, 1279, 513, 900])):      # two calls in a row
        case = paged_case(lens, [1] * len(lens), nh, nkv, hd, B, "bfloat16", seed=40 + round_no)
        S = len(lens)
        ref = reference_attention(case, nh, nkv, hd, scale, 0)
        scratch = torch.empty(S * nh * parts * (hd + 2), dtype=torch.float32, device="cuda:0")
        want = torch.zeros(S, nh * hd, dtype=torch.bfloat16, device="cuda:0")
        assert _call(lib, "kvcm_attention_decode_bf16", case, want, nh, nkv, hd, scale, part_size, parts, scratch) == 0
        got = torch.full_like(want, float("nan"))
        if round_no == 0:
            # The first call on a device looks up the array's address; it stays outside the measured
            # region (the runtime may set up its own bookkeeping then).
            warm = torch.empty_like(got)
            assert _call(lib, "kvcm_attention_decode_bf16_noalloc", case, warm, nh, nkv, hd, scale, part_size, parts) == 0
        torch.cuda.synchronize()
        # Free device memory as the DRIVER counts it: torch's own counters only see torch's allocator
        # and could not notice a cudaMalloc made inside the library.
        free_before = torch.cuda.mem_get_info()[0]
        rc = _call(lib, "kvcm_attention_decode_bf16_noalloc", case, got, nh, nkv, hd, scale, part_size, parts)
        torch.cuda.synchronize()
        assert rc == 0, lib.kvcm_attention_decode_noalloc_error().decode()
        assert torch.cuda.mem_get_info()[0] == free_before
        close(got, ref, "bfloat16", f"no-alloc call {round_no} vs reference")
        close(got, want.double(), "bfloat16", f"no-alloc call {round_no} vs ordinary entry point")
        assert torch.equal(got, want)             # the same kernels on the same partitions: equal bits


def test_sizes_beyond_the_built_in_scratch_are_refused_with_a_clear_error():
    from test_gpu_kernels import paged_case
    lib = _lib()
    nh, nkv, hd = 64, 8, 128
    case = paged_case([40, 40], [1, 1], nh, nkv, hd, 16, "bfloat16", seed=1)
    out = torch.zeros(2, nh * hd, dtype=torch.bfloat16, device="cuda:0")
    # pretend there are 4096 requests: 4096 * 64 * 8 * 130 floats is far beyond the array
    args = [_p(case["q"]), case["q"].stride(0), _p(out), out.stride(0), _p(case["kc"]), _p(case["vc"]),
            _p(case["tables"]), case["tables"].shape[1], _p(case["ctx"].seq_ctx_len), 4096, nh, nkv, hd, 16,
            ctypes.c_float(0.1), 0, 64, 8, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)]
    rc = lib.kvcm_attention_decode_bf16_noalloc(*args)
    assert rc == 10002
    msg = lib.kvcm_attention_decode_noalloc_error().decode()
    assert "exceed" in msg and "2097152" in msg and str(4096 * nh * 8 * (hd + 2)) in msg
    torch.cuda.synchronize()
    assert torch.count_nonzero(out) == 0          # nothing was launched
