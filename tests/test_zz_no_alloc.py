"""The library's one entry point that allocates nothing, hymt2_attention_decode_noalloc,
called through its exported C symbol as a program without torch's allocator would call it.

The split-key decode attention needs room for its partial results.  Callers that cannot
allocate (a C host program without an allocator at hand, a serving loop that has given all
free GPU memory to the cache and must not meet cudaMalloc in mid-request) get that room from
a fixed device array inside the library.  Two calls in a row must both be right: the array
keeps the first call's contents, and the second call has other lengths, so stale partials
would show.  Its output is compared with a float64 restatement of the formula and with the
ordinary entry point (scratch from the caller).  The file's name makes pytest collect it last.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_FLOATS = 1 << 20


def _call(lib, out, q, kp, vp, table, cu, slots, kv, nh, nkv, d, scale, window, split, max_splits, status):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    fn = lib.hymt2_attention_decode_noalloc
    fn.restype = ctypes.c_int
    return fn(p(out), p(q), p(kp), p(vp), ctypes.c_int(0 if out.dtype == torch.float32 else 1), p(table),
              ctypes.c_int(table.stride(0)), ctypes.c_int(kp.shape[2]), p(cu), p(slots), p(kv),
              ctypes.c_int(out.shape[0]), ctypes.c_int(nh), ctypes.c_int(nkv), ctypes.c_int(d), ctypes.c_float(scale),
              ctypes.c_int(window), ctypes.c_int(split), ctypes.c_int(max_splits), p(status),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _case(lens, nh, nkv, d, dtype, seed, padding_row=None):
    from test_gpu_kernels import _paged
    rows = len(lens)
    keys = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    vals = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    q = torch.randn(rows, nh * d, device=DEV).to(dtype)
    kp, vp, table = _paged(keys, vals, 64, dtype, shuffle_seed=seed)
    cu = torch.arange(rows + 1, dtype=torch.int32, device=DEV)
    slots = torch.arange(rows, dtype=torch.int32, device=DEV)
    if padding_row is not None:
        slots[padding_row] = -1
    kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
    return keys, vals, q, kp, vp, table, cu, slots, kv


@pytest.mark.parametrize("window", [0, 300])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_entry_is_right_twice_in_a_row(dtype, window):
    from hymt2sharp_b200.kernels import ops
    from hymt2sharp_b200.kernels.build import load_library
    from test_gpu_kernels import _ref_attention, _tol
    lib = load_library()
    nh, nkv, d = 8, 2, 64
    scale = 1 / math.sqrt(d)
    torch.manual_seed(7)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    # the second call has other lengths and a padding row (slot -1) in the middle
    for call, (lens, pad) in enumerate([([700, 1, 257, 64, 300], None), ([90, 513, 2, 1024], 2)]):
        rows = len(lens)
        keys, vals, q, kp, vp, table, cu, slots, kv = _case(lens, nh, nkv, d, dtype, call, pad)
        splits = -(-max(lens) // 256)
        ref = torch.stack([_ref_attention(q[b].view(1, nh, d), keys[b], vals[b], 1, window, scale)[0] for b in range(rows)])
        na, nm = ops.attention_simt_scratch(rows, nh, d, splits)
        ordinary = torch.full((rows, nh * d), 3.0, dtype=dtype, device=DEV)
        ops.attention_simt(ordinary, q, kp, vp, table, cu, slots, kv, rows, 1, nh, nkv, d, scale, window, 256, splits,
                           torch.empty(na, device=DEV), torch.empty(nm, device=DEV), status=status)
        got = torch.full((rows, nh * d), 3.0, dtype=dtype, device=DEV)
        torch.cuda.synchronize()
        # by the second call the array's address is known: nothing may come out of the device's free memory, whoever
        # allocates it (torch's own counters would not see a cudaMalloc inside the library)
        free_before = torch.cuda.mem_get_info()[0]
        torch_before = torch.cuda.memory_allocated()
        rc = _call(lib, got, q, kp, vp, table, cu, slots, kv, nh, nkv, d, scale, window, 256, splits, status)
        assert rc == 0, lib.hymt2_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == torch_before
        if call > 0:
            assert torch.cuda.mem_get_info()[0] == free_before
        live = [b for b in range(rows) if b != pad]
        assert torch.allclose(got[live].double(), ref[live], **_tol(dtype)), f"call {call}: against the formula"
        assert torch.equal(got, ordinary), f"call {call}: against the ordinary entry point"
        if pad is not None:
            assert float((got[pad].float() - 3.0).abs().max()) == 0.0   # a padding row is left alone
    assert int(status[0].item()) == 0


def test_noalloc_entry_flags_a_row_longer_than_its_splits_cover():
    """max_splits * split_keys must cover the longest row; the lengths are on the device, so only the
    kernels can tell.  The row is left as it was, the others are right, and the status word says 2."""
    from hymt2sharp_b200.kernels.build import load_library
    from test_gpu_kernels import _ref_attention, _tol
    lib = load_library()
    nh, nkv, d, dtype = 4, 2, 32, torch.float32
    scale = 1 / math.sqrt(d)
    torch.manual_seed(11)
    lens = [100, 600, 256]                      # 600 > 2 * 256
    keys, vals, q, kp, vp, table, cu, slots, kv = _case(lens, nh, nkv, d, dtype, 5)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    got = torch.full((3, nh * d), 3.0, dtype=dtype, device=DEV)
    rc = _call(lib, got, q, kp, vp, table, cu, slots, kv, nh, nkv, d, scale, 0, 256, 2, status)
    assert rc == 0, lib.hymt2_last_error().decode()
    torch.cuda.synchronize()
    assert int(status[0].item()) == 2
    assert float((got[1] - 3.0).abs().max()) == 0.0
    for b in (0, 2):
        ref = _ref_attention(q[b].view(1, nh, d), keys[b], vals[b], 1, 0, scale)[0]
        assert torch.allclose(got[b].double(), ref, **_tol(dtype))


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
    rc = _call(lib, out, buf, kp, kp, table, z, z, z, nh, nkv, d, 1.0, 0, 256, splits, z)
    assert rc == -1
    msg = lib.hymt2_last_error().decode()
    assert "exceed the built-in scratch" in msg and str(SCRATCH_FLOATS) in msg
    assert float(out.abs().sum()) == 0.0   # nothing ran
