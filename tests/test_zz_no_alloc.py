"""The library's one entry point that allocates nothing, hymt2_attention_decode_noalloc,
called through its exported C symbol as a program without torch's allocator would call it,
against the ordinary entry point that takes its scratch from the caller.

The split-key decode attention needs room for its partial results.  Callers that cannot
allocate (a C host program without an allocator at hand, a serving loop that has given all
free GPU memory to the cache and must not meet cudaMalloc in mid-request) get that room from
a fixed device array inside the library.  Two calls in a row must both be right: the array
keeps the first call's contents, and the second call has other lengths, so stale partials
would show.  The file's name makes pytest collect it last.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_FLOATS = 1 << 20


def _call(lib, out, q, kp, vp, table, cu, slots, kv, nh, nkv, d, scale, window, split, max_splits):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    fn = lib.hymt2_attention_decode_noalloc
    fn.restype = ctypes.c_int
    return fn(p(out), p(q), p(kp), p(vp), ctypes.c_int(0 if out.dtype == torch.float32 else 1), p(table),
              ctypes.c_int(table.stride(0)), ctypes.c_int(kp.shape[2]), p(cu), p(slots), p(kv),
              ctypes.c_int(out.shape[0]), ctypes.c_int(nh), ctypes.c_int(nkv), ctypes.c_int(d), ctypes.c_float(scale),
              ctypes.c_int(window), ctypes.c_int(split), ctypes.c_int(max_splits),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_entry_matches_the_ordinary_one_twice(dtype):
    from hymt2sharp_b200.kernels import ops
    from hymt2sharp_b200.kernels.build import load_library
    from test_gpu_kernels import _paged, _tol
    lib = load_library()
    nh, nkv, d, window = 8, 2, 64, 0
    scale = 1 / math.sqrt(d)
    torch.manual_seed(7)
    for call, lens in enumerate([[700, 1, 257, 64, 300], [90, 513, 2, 1024]]):   # two calls in a row
        rows = len(lens)
        keys = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
        vals = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
        q = torch.randn(rows, nh * d, device=DEV).to(dtype)
        kp, vp, table = _paged(keys, vals, 64, dtype, shuffle_seed=call)
        cu = torch.arange(rows + 1, dtype=torch.int32, device=DEV)
        slots = torch.arange(rows, dtype=torch.int32, device=DEV)
        kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
        splits = -(-max(lens) // 256)
        na, nm = ops.attention_simt_scratch(rows, nh, d, splits)
        want = torch.zeros(rows, nh * d, dtype=dtype, device=DEV)
        ops.attention_simt(want, q, kp, vp, table, cu, slots, kv, rows, 1, nh, nkv, d, scale, window, 256, splits,
                           torch.empty(na, device=DEV), torch.empty(nm, device=DEV))
        torch.cuda.synchronize()
        got = torch.full((rows, nh * d), 3.0, dtype=dtype, device=DEV)
        after_out = torch.cuda.memory_allocated()
        rc = _call(lib, got, q, kp, vp, table, cu, slots, kv, nh, nkv, d, scale, window, 256, splits)
        assert rc == 0, lib.hymt2_last_error().decode()
        torch.cuda.synchronize()
        now = torch.cuda.memory_allocated()
        assert now == after_out, (after_out, now)   # nothing was taken from torch's allocator
        assert torch.allclose(got.float(), want.float(), **_tol(dtype)), f"call {call}"


def test_noalloc_entry_refuses_what_does_not_fit():
    from hymt2sharp_b200.kernels.build import load_library
    lib = load_library()
    rows, nh, nkv, d, splits = 64, 32, 8, 128, 8            # 64*32*8*130 floats > 2^20
    assert rows * nh * splits * (d + 2) > SCRATCH_FLOATS
    z = torch.zeros(8, dtype=torch.int32, device=DEV)
    buf = torch.zeros(16, device=DEV)
    kp = torch.zeros(1, nkv, 64, d, device=DEV)
    out = torch.zeros(rows, nh * d, device=DEV)
    table = torch.zeros(1, 1, dtype=torch.int32, device=DEV)
    rc = _call(lib, out, buf, kp, kp, table, z, z, z, nh, nkv, d, 1.0, 0, 256, splits)
    assert rc == -1
    msg = lib.hymt2_last_error().decode()
    assert "exceed the built-in scratch" in msg and str(SCRATCH_FLOATS) in msg
    assert float(out.abs().sum()) == 0.0   # nothing ran
