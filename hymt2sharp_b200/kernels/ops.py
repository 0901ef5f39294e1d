"""Python face of the CUDA library: every function checks its tensors, passes raw
pointers and the current torch stream to one exported C function and raises
KernelError when that function refuses.  Nothing here computes; there is no
fallback to torch operators."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from .build import load_library

F32, BF16 = 0, 1
EPILOGUE_STORE, EPILOGUE_ACCUMULATE, EPILOGUE_SWIGLU = 0, 1, 2


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.dtype) -> int:
    if t == torch.float32:
        return F32
    if t == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {t} is not supported by the kernels (float32 and bfloat16 are)")


_library = None


def _lib():
    global _library
    if _library is None:
        _library = load_library()
    return _library


def _stream() -> c_void_p:
    # (the raw handle: torch.cuda.current_stream() builds a Stream object for it, ten times the cost, once per launch)
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


launches = 0  # kernels of this library launched (or captured into a graph) so far

# The profiling switch (the counterpart of HunyuanDenseModel.ProfileEnabled and its tick counters,
# src/HyMT2Sharp/HunyuanDenseModel.cs:48-78): between profile_begin() and profile_end() every launch on the current
# stream is followed by a CUDA event, and the time between two events is booked under the launch's name, or under
# `tag` where a caller set one (a Linear names the product it is: "qkv", "o_proj", ...).  Kernels then run one after
# the other (an event between two launches keeps the second from starting early), so the sum is more than an
# unprofiled step takes; the shares are what it is for.  A step that is launched kernel by kernel from the host is
# timed truly only where its kernels outlast the host's work per launch (prompts); a decode step is therefore captured
# with a kernel between every two of its kernels that writes the device's clock (capture_begin/capture_end), and the
# stamps are read after each replay.
tag: str | None = None
_profile: list | None = None      # (name, event) in launch order, eager launches
_booked: dict | None = None       # {name: ms} already read from captured steps
_capturing: list | None = None    # the capture that is being made: [stamps, None, name, name, ...]
_suspended = False


def profile_begin() -> None:
    global _profile, _booked
    e = torch.cuda.Event(enable_timing=True)
    e.record()
    _profile = [(None, e)]
    _booked = {}


def profile_active() -> bool:
    return _profile is not None


def profile_end() -> dict:
    """{name: milliseconds} of everything launched since profile_begin(), in the order of first appearance."""
    global _profile, _booked
    events, _profile = _profile or [], None
    booked, _booked = _booked or {}, None
    torch.cuda.synchronize()
    out: dict = {}
    for (_, before), (name, after) in zip(events, events[1:]):
        if name is not None:
            out[name] = out.get(name, 0.0) + before.elapsed_time(after)
    for name, ms in booked.items():
        out[name] = out.get(name, 0.0) + ms
    return out


class profile_suspended:
    """Launches inside are not timed (a warm-up step in front of a capture)."""

    def __enter__(self):
        global _suspended
        self.was, _suspended = _suspended, True

    def __exit__(self, *exc):
        global _suspended
        _suspended = self.was
        if _profile is not None:   # what ran meanwhile is not booked to the next launch
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            _profile.append((None, e))


STAMPS = 8192   # kernels of one captured step that can be timed


def _stamp(stamps: torch.Tensor, index: int) -> None:
    rc = _lib().hymt2_stamp(ctypes.c_void_p(stamps.data_ptr() + 8 * index), _stream())
    if rc != 0:
        raise KernelError(f"stamp failed ({rc}): {_lib().hymt2_last_error().decode(errors='replace')}")


def capture_begin(device) -> None:
    """Inside a graph capture: from here on every launch is followed by a kernel that writes the device's clock."""
    global _capturing
    stamps = torch.zeros(STAMPS, dtype=torch.int64, device=device)
    _capturing = [stamps, None]
    _stamp(stamps, STAMPS - 2)   # two stamps with nothing between them: what a stamp itself costs
    _stamp(stamps, STAMPS - 1)
    _stamp(stamps, 0)


def capture_end() -> list:
    """[the stamps' tensor, None, name of launch 1, name of launch 2, ...]: what book_captured() wants."""
    global _capturing
    record, _capturing = _capturing or [], None
    return record


def book_captured(record: list) -> None:
    """After a replay of a graph captured between capture_begin() and capture_end(): waits for it and adds its kernels'
    times to the running profile (the time from the stamp in front of a kernel to the stamp behind it, less what a
    stamp costs)."""
    torch.cuda.synchronize()
    if _booked is None or not record:
        return
    names = record[2:]
    at = record[0].cpu().tolist()
    own = max(0, at[STAMPS - 1] - at[STAMPS - 2])
    for i, name in enumerate(names):
        _booked[name] = _booked.get(name, 0.0) + max(0, at[i + 1] - at[i] - own) * 1e-6


def profile_line(phase: str, times: dict) -> str:
    """One line in the manner of src/HyMT2Sharp.Benchmark/Program.cs:243-261."""
    body = " ".join(f"{k}={v:.2f}ms" for k, v in times.items())
    return f"profile {phase}: {body} accounted={sum(times.values()):.2f}ms"


def _check(rc: int, what: str, kernels: int = 1, timed: bool = True) -> None:
    global launches
    launches += kernels
    if rc != 0:
        msg = _lib().hymt2_last_error().decode(errors="replace")
        raise KernelError(f"{what} failed ({rc}): {msg}")
    if timed and kernels > 0 and not _suspended:
        if _capturing is not None:
            if len(_capturing) - 1 >= STAMPS - 2:
                raise KernelError(f"a captured step of more than {STAMPS - 3} kernels cannot be timed")
            _stamp(_capturing[0], len(_capturing) - 1)
            _capturing.append(tag or what)
        elif _profile is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            _profile.append((tag or what, e))


def _need(t: torch.Tensor, name: str, dtype=None, dims=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got {t.dim()}")


# ---------------------------------------------------------------------------
def embed(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = float32(table[ids[t]]) * scale; out is [T, hidden] float32."""
    _need(out, "out", torch.float32, 2); _need(table, "table", None, 2); _need(ids, "ids", torch.int32, 1)
    T, H = out.shape
    if table.shape[1] != H or ids.shape[0] < T:
        raise KernelError(f"embed: shapes out {tuple(out.shape)} table {tuple(table.shape)} ids {tuple(ids.shape)}")
    _check(_lib().hymt2_embed(_ptr(out), _ptr(table), c_int(dtype_code(table.dtype)), _ptr(ids), c_int(T),
                              c_int(H), c_int(table.shape[0]), c_float(scale), _ptr(status), _stream()), "embed")


def advance_decode(token_pos: torch.Tensor, kv_lens: torch.Tensor, slot_ids: torch.Tensor) -> None:
    """After a decode step: positions and lengths of the live rows (slot >= 0) grow by one."""
    _need(token_pos, "token_pos", torch.int32, 1); _need(kv_lens, "kv_lens", torch.int32, 1)
    _need(slot_ids, "slot_ids", torch.int32, 1)
    _check(_lib().hymt2_advance_decode(_ptr(token_pos), _ptr(kv_lens), _ptr(slot_ids), c_int(slot_ids.shape[0]),
                                       _stream()), "advance_decode")


PREFETCH_MAX_BYTES = 48 << 20   # of a larger tensor only the beginning is asked for: more would push too much else out of L2
_side = {}   # device index -> (side stream, event, whether the side stream has work that the main stream has not joined)


def prefetch_beside(t: torch.Tensor) -> None:
    """Asks for the beginning of `t` (at most PREFETCH_MAX_BYTES) to be brought into L2 by a small kernel on a
    stream BESIDE the current one, ordered after everything launched on the current stream so far.  The current
    stream does not wait for it (join_beside does, once, at the end of a step), so kernels that follow run while
    the memory fetches; in a captured step this is a branch of the graph."""
    if t is None or not t.is_contiguous() or t.data_ptr() % 16:
        return
    nbytes = min(t.numel() * t.element_size(), PREFETCH_MAX_BYTES)
    key = t.device.index if t.device.index is not None else torch.cuda.current_device()
    if key not in _side:
        _side[key] = [torch.cuda.Stream(device=t.device), torch.cuda.Event(), False]
    side, event, _ = _side[key]
    main = torch.cuda.current_stream(t.device)
    event.record(main)
    side.wait_event(event)
    with torch.cuda.stream(side):
        _check(_lib().hymt2_l2_prefetch(_ptr(t), c_long(nbytes), _stream()), "l2_prefetch", timed=False)
    _side[key][2] = True


def join_beside(device) -> None:
    """The current stream waits for what prefetch_beside put on the side stream (a step calls it at its end)."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _side.get(key)
    if st and st[2]:
        torch.cuda.current_stream(device).wait_stream(st[0])
        st[2] = False


def rmsnorm(out: torch.Tensor, x: torch.Tensor, gain: torch.Tensor, eps: float,
            rows_index: torch.Tensor | None = None, out_scale: float = 1.0) -> None:
    """out[r] = rmsnorm(x[rows_index[r]] or x[r]) * gain * out_scale, computed in float32."""
    _need(out, "out", None, 2); _need(x, "x", None, 2); _need(gain, "gain", None, 1)
    rows, dim = out.shape
    if x.shape[1] != dim or gain.shape[0] != dim:
        raise KernelError(f"rmsnorm: shapes out {tuple(out.shape)} x {tuple(x.shape)} gain {tuple(gain.shape)}")
    if rows_index is not None:
        _need(rows_index, "rows_index", torch.int32, 1)
        if rows_index.shape[0] < rows:
            raise KernelError("rmsnorm: rows_index is shorter than out")
    elif x.shape[0] < rows:
        raise KernelError("rmsnorm: x has fewer rows than out")
    _check(_lib().hymt2_rmsnorm(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(x), c_int(dtype_code(x.dtype)),
                                _ptr(gain), c_int(dtype_code(gain.dtype)), _ptr(rows_index), c_int(rows),
                                c_int(dim), c_float(eps), c_float(out_scale), _stream()), "rmsnorm")


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor) -> None:
    """out[r, c] = silu(gate_up[r, c]) * gate_up[r, width + c]."""
    _need(out, "out", None, 2); _need(gate_up, "gate_up", out.dtype, 2)
    rows, width = out.shape
    if gate_up.shape != (rows, 2 * width):
        raise KernelError(f"silu_mul: shapes out {tuple(out.shape)} gate_up {tuple(gate_up.shape)}")
    _check(_lib().hymt2_silu_mul(_ptr(out), _ptr(gate_up), c_int(dtype_code(out.dtype)), c_int(rows), c_int(width),
                                 _stream()), "silu_mul")


def gemm_simt(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int = EPILOGUE_STORE) -> None:
    """out[M, N] = epilogue(a[M, K] @ w[N, K]^T) on CUDA cores, float32 accumulation in K order.
    With EPILOGUE_SWIGLU w has 2N rows (gate rows, then up rows)."""
    for t, n in ((out, "out"), (a, "a"), (w, "w")):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm: {n} must be a CUDA matrix with contiguous rows")
    M, N = out.shape
    K = a.shape[1]
    rows_w = 2 * N if epilogue == EPILOGUE_SWIGLU else N
    if a.shape[0] != M or w.shape != (rows_w, K):
        raise KernelError(f"gemm: shapes out {tuple(out.shape)} a {tuple(a.shape)} w {tuple(w.shape)} epilogue {epilogue}")
    _check(_lib().hymt2_gemm_simt(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(a), c_int(dtype_code(a.dtype)),
                                  _ptr(w), c_int(dtype_code(w.dtype)), c_int(M), c_int(N), c_int(K),
                                  c_long(a.stride(0)), c_long(w.stride(0)), c_long(out.stride(0)),
                                  c_int(epilogue), _stream()), "gemm_simt")


_status: dict = {}
_status_of: dict = {}   # the same by what callers pass (a torch.device with an index)


def device_status(device) -> torch.Tensor:
    """The int32[4] status word of a device: kernels set [0] when a device-side check fails or a
    bounded wait gives up (1: token id outside the table; 2: a sequence longer than the split attention was given
    room for; 101-106: a wait of the tensor-core GEMM (106: for the partial sums of a tile's other CTAs); 108-119: of the prompt attention; 120-129: of the decode
    attention)."""
    hit = _status_of.get(device)
    if hit is not None:
        return hit
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(4, dtype=torch.int32, device=dev)
    if dev.index is not None:          # ("cuda" without an index means the current device, which may change)
        _status_of[device] = _status[key]
    return _status[key]


_tc_scratch: dict = {}   # device index -> (workspace float32, counters int32, earlier tensors kept alive)


def _tc_workspace(device: torch.device, floats: int, counters: int):
    """Scratch of the split-K tensor-core GEMM: partial tiles and per-tile arrival counters.  One
    pair per device, shared by all calls (they run in stream order); it only ever grows, and what it
    replaced stays alive because captured graphs may still point at it."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws, cnt, old = _tc_scratch.get(key, (None, None, []))
    if ws is None or ws.numel() < floats or cnt.numel() < counters:
        if ws is not None:
            old = old + [ws, cnt]
        ws = torch.empty(max(floats, 8 << 20), dtype=torch.float32, device=device)
        cnt = torch.zeros(max(counters, 1 << 14), dtype=torch.int32, device=device)
        _tc_scratch[key] = (ws, cnt, old)
    return ws, cnt


def gemm_tc_supported(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int) -> bool:
    """Whether the tcgen05 kernel takes these operands (types, alignment, the epilogue's output type)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    if a.dim() != 2 or w.dim() != 2 or out.dim() != 2 or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        return False
    K = a.shape[1]
    if K % 8 or a.stride(0) % 8 or w.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    if epilogue == EPILOGUE_STORE:
        return out.dtype in (torch.bfloat16, torch.float32)
    if epilogue == EPILOGUE_ACCUMULATE:
        return out.dtype == torch.float32
    return out.dtype == torch.bfloat16


def gemm_tc_norm_tiles(tokens: int, out_features: int, inner: int, epilogue: int) -> int:
    """How many partial sums of squares per token gemm_tc leaves behind when it is asked to prepare the norm that follows it
    (`norm_after`); 0: this shape's plan cannot, and the norm runs as a kernel of its own."""
    key = (tokens, out_features, inner, epilogue)
    hit = _norm_tiles.get(key)
    if hit is None:
        hit = _norm_tiles[key] = int(_lib().hymt2_gemm_tc_norm_tiles(c_int(tokens), c_int(out_features), c_int(inner), c_int(epilogue)))
    return hit


# What the library answered about a shape (its plan depends on the sizes and the device's SMs only): asked once a shape,
# since a step asks the same questions layer after layer.
_norm_tiles: dict = {}
_plans: dict = {}
_rope_plans: dict = {}


def _plan_scratch(T: int, N: int, K: int, epilogue: int) -> tuple:
    """(floats of workspace, counters) that the tensor-core product of this shape wants."""
    key = (T, N, K, epilogue)
    hit = _plans.get(key)
    if hit is None:
        floats, counters = ctypes.c_long(0), c_int(0)
        _check(_lib().hymt2_gemm_tc_plan(c_int(T), c_int(N), c_int(K), c_int(epilogue), ctypes.byref(floats),
                                         ctypes.byref(counters)), "gemm_tc_plan", 0)
        hit = _plans[key] = (floats.value, counters.value)
    return hit


def gemm_tc(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int, status: torch.Tensor,
            row_scale: tuple | None = None, norm_after: tuple | None = None, checked: bool = False) -> None:
    """out[T, N] = epilogue(a[T, K] @ w[N, K]^T) on the tcgen05 tensor cores (bfloat16 operands,
    float32 accumulation in tensor memory).  With EPILOGUE_SWIGLU w has 2N rows.

    An RMSNorm can be folded into the products around it.  `row_scale` = (ss [T, tiles] float32, width, eps): `a` holds
    bf16(x * gain) and the sums are multiplied by 1 / sqrt(sum(ss[t]) / width + eps) (store and SwiGLU epilogues).
    `norm_after` = (normed [T, N] bfloat16, gain [N], ss [T, gemm_tc_norm_tiles(...)] float32), accumulate epilogue only:
    bf16(out_new * gain) and the partial sums of squares of the new rows are written for the product that comes next.
    `checked`: the caller has just asked gemm_tc_supported about these very operands."""
    T, N = out.shape
    K = a.shape[1]
    rows_w = 2 * N if epilogue == EPILOGUE_SWIGLU else N
    if a.shape[0] != T or w.shape != (rows_w, K) or not (checked or gemm_tc_supported(out, a, w, epilogue)):
        raise KernelError(f"gemm_tc: operands out {tuple(out.shape)} {out.dtype} a {tuple(a.shape)} {a.dtype} "
                          f"w {tuple(w.shape)} {w.dtype} epilogue {epilogue} are not taken")
    floats, counters = _plan_scratch(T, N, K, epilogue)
    ws = cnt = None
    if floats:
        ws, cnt = _tc_workspace(out.device, floats, counters)
    ss_in = normed = gain = ss_out = None
    tiles_in, width, eps = 0, 0, 0.0
    if row_scale is not None:
        ss_in, width, eps = row_scale
        _need(ss_in, "row_scale sums", torch.float32, 2)
        if ss_in.shape[0] < T or epilogue == EPILOGUE_ACCUMULATE:
            raise KernelError("gemm_tc: row_scale needs sums for every token and a store or SwiGLU epilogue")
        tiles_in = ss_in.shape[1]
    if norm_after is not None:
        normed, gain, ss_out = norm_after
        tiles = gemm_tc_norm_tiles(T, N, K, epilogue)
        _need(normed, "normed", torch.bfloat16, 2); _need(gain, "gain", None, 1); _need(ss_out, "ss_out", torch.float32, 2)
        if tiles == 0 or normed.shape != (T, N) or gain.shape[0] != N or ss_out.shape != (T, tiles) or out.dtype != torch.float32:
            raise KernelError(f"gemm_tc: norm_after does not fit T={T} N={N} K={K} epilogue {epilogue} (tiles {tiles})")
    _check(_lib().hymt2_gemm_tc_norm(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(a), _ptr(w), c_int(T), c_int(N), c_int(K),
                                     c_long(a.stride(0)), c_long(w.stride(0)), c_long(out.stride(0)), c_int(epilogue),
                                     _ptr(ws), c_long(ws.numel() if ws is not None else 0), _ptr(cnt),
                                     c_int(cnt.numel() if cnt is not None else 0), _ptr(status), _stream(),
                                     _ptr(ss_in), c_int(tiles_in), c_int(width), c_float(eps), _ptr(normed), _ptr(gain),
                                     c_int(dtype_code(gain.dtype) if gain is not None else F32), _ptr(ss_out)), "gemm_tc")


def gemm_tc_debug(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int, status: torch.Tensor,
                  wait_limit: int, withhold_block: int) -> None:
    """gemm_tc with a fault put in on purpose: the copies of k block `withhold_block` are announced and never made,
    and every wait gives up after `wait_limit` tries.  The kernel must set status[0] = 102, free what it holds and
    return; `out` is then not a product.  Only products of few tokens whose K is not cut are taken."""
    T, N = out.shape
    K = a.shape[1]
    if a.shape[0] != T or w.shape != (N, K) or not gemm_tc_supported(out, a, w, epilogue):
        raise KernelError("gemm_tc_debug: operands are not taken")
    _check(_lib().hymt2_gemm_tc_debug(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(a), _ptr(w), c_int(T), c_int(N), c_int(K),
                                      c_long(a.stride(0)), c_long(w.stride(0)), c_long(out.stride(0)), c_int(epilogue),
                                      _ptr(status), _stream(), c_int(wait_limit), c_int(withhold_block)), "gemm_tc_debug")


def gemm_tc_rope_kv_supported(x: torch.Tensor, w: torch.Tensor, nh: int, nkv: int, d: int, cache_dtype, rope_dim: int) -> bool:
    """Whether the fused projection + rotation + cache append takes these operands: bfloat16, head_dim 128, and
    either few enough tokens that the product is cut over K among clusters (any even rope_dim), or more than 128
    tokens, which are the accumulator's rows (rope_dim 0 or 128)."""
    if d != 128 or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or cache_dtype != torch.bfloat16:
        return False
    if x.dim() != 2 or w.dim() != 2 or x.stride(1) != 1 or w.stride(1) != 1 or w.shape != ((nh + 2 * nkv) * d, x.shape[1]):
        return False
    K = x.shape[1]
    if K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    key = (x.shape[0], w.shape[0], K, rope_dim)
    hit = _rope_plans.get(key)
    if hit is None:
        hit = _rope_plans[key] = bool(_lib().hymt2_gemm_tc_rope_kv_supported(c_int(key[0]), c_int(key[1]), c_int(K), c_int(rope_dim)))
    return hit


def gemm_tc_rope_kv(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, k_plane: torch.Tensor | None,
                    v_plane: torch.Tensor | None, block_table: torch.Tensor, block_tokens: int, token_seq: torch.Tensor,
                    token_pos: torch.Tensor, slot_ids: torch.Tensor, inv_freq: torch.Tensor | None, rope_dim: int,
                    q_gain: torch.Tensor | None, k_gain: torch.Tensor | None, eps: float, nh: int, nkv: int,
                    status: torch.Tensor, angles: torch.Tensor | None = None, row_scale: tuple | None = None,
                    checked: bool = False) -> None:
    """q_out[T, nh*128] = rotation and per-head norm of the query part of x @ w^T; the key part, rotated and
    normed, and the value part go to the rows of the cache planes that (slot, position) of every token name
    (k_plane None: nothing is written).  One tcgen05 kernel; head_dim 128; see rope_kv for the arguments.
    `angles`: what rope_angles(token_pos, inv_freq) gave, where gemm_tc_rope_kv_wants_angles says so.
    `row_scale` = (ss [T, tiles] float32, width, eps): x holds bf16(h * gain) of an RMSNorm whose row scale is applied to the
    projection's sums here (see gemm_tc).  `checked`: the caller has just asked gemm_tc_rope_kv_supported about these operands."""
    d = 128
    T = x.shape[0]
    if gemm_tc_rope_kv_wants_angles(T, rope_dim):
        if angles is None:
            raise KernelError(f"gemm_tc_rope_kv: {T} tokens need the table of their angles (rope_angles)")
        _need(angles, "angles", torch.float32, 3)
        if angles.shape != (T, rope_dim // 2, 2) or not angles.is_contiguous():
            raise KernelError(f"gemm_tc_rope_kv: angles is {tuple(angles.shape)}, expected {(T, rope_dim // 2, 2)}")
    else:
        angles = None
    if not (checked or gemm_tc_rope_kv_supported(x, w, nh, nkv, d, (k_plane if k_plane is not None else q_out).dtype, rope_dim)):
        raise KernelError(f"gemm_tc_rope_kv: operands x {tuple(x.shape)} {x.dtype} w {tuple(w.shape)} {w.dtype} are not taken")
    _need(q_out, "q_out", torch.bfloat16, 2)
    if q_out.shape != (T, nh * d) or not q_out.is_contiguous():
        raise KernelError(f"gemm_tc_rope_kv: q_out is {tuple(q_out.shape)}, expected {(T, nh * d)}")
    write = k_plane is not None
    if write:
        for t, n in ((k_plane, "k_plane"), (v_plane, "v_plane")):
            _need(t, n, torch.bfloat16, 4)
            if t.shape[1:] != (nkv, block_tokens, d):
                raise KernelError(f"gemm_tc_rope_kv: {n} is {tuple(t.shape)}, expected [blocks, {nkv}, {block_tokens}, {d}]")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((token_seq, "token_seq"), (token_pos, "token_pos"), (slot_ids, "slot_ids")):
        _need(t, n, torch.int32, 1)
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rope_dim // 2:
            raise KernelError("gemm_tc_rope_kv: inv_freq must hold rope_dim/2 values")
    gain_dtype = F32
    if q_gain is not None:
        _need(q_gain, "q_gain", None, 1); _need(k_gain, "k_gain", q_gain.dtype, 1)
        if q_gain.shape[0] != d or k_gain.shape[0] != d:
            raise KernelError("gemm_tc_rope_kv: the gains must hold head_dim values")
        gain_dtype = dtype_code(q_gain.dtype)
    _check(_lib().hymt2_gemm_tc_rope_kv(_ptr(x), _ptr(w), c_int(T), c_int(x.shape[1]), c_long(x.stride(0)), c_long(w.stride(0)),
                                        _ptr(q_out), _ptr(k_plane), _ptr(v_plane), _ptr(block_table),
                                        c_int(block_table.stride(0)), c_int(block_tokens), _ptr(token_seq), _ptr(token_pos),
                                        _ptr(slot_ids), _ptr(inv_freq), _ptr(angles), c_int(rope_dim), _ptr(q_gain), _ptr(k_gain),
                                        c_int(gain_dtype), c_float(eps), c_int(nh), c_int(nkv), c_int(1 if write else 0),
                                        _ptr(status), _stream(), _ptr(row_scale[0] if row_scale else None),
                                        c_int(row_scale[0].shape[1] if row_scale else 0), c_int(row_scale[1] if row_scale else 0),
                                        c_float(row_scale[2] if row_scale else 0.0)), "gemm_tc_rope_kv")


def gemm_tc_describe(tokens: int, out_features: int, inner: int, epilogue: int, sm_count: int = 0) -> dict:
    """How the tensor-core kernel would run this product (nothing is launched; works without a GPU when sm_count
    is given): orientation, kernel, tile width, ring depth, splits of K and how they fold, tiles and CTAs.
    epilogue: EPILOGUE_STORE / _ACCUMULATE / _SWIGLU, or 3 for the q/k/v projection with rotation."""
    out = (ctypes.c_int * 8)()
    rc = _lib().hymt2_gemm_tc_describe(c_int(tokens), c_int(out_features), c_int(inner), c_int(epilogue), c_int(sm_count), out)
    if rc != 0:
        raise KernelError(f"gemm_tc_describe failed ({rc}): {_lib().hymt2_last_error().decode(errors='replace')}")
    keys = ("swapped", "persistent", "tile_width", "stages", "k_splits", "cluster", "tiles", "ctas")
    return {k: (bool(v) if k in ("swapped", "persistent", "cluster") else int(v)) for k, v in zip(keys, out)}


def protocol_numbers() -> dict:
    """The numbers that the barrier protocols of the tcgen05 kernels are built on, as compiled (stages, slots, barriers
    per purpose, issuers): what an exploration of the protocols has to be run with.  Works without a GPU."""
    def ask(fn, names):
        out = (ctypes.c_int * 8)()
        getattr(_lib(), fn)(out)
        return dict(zip(names, out))
    return {"prefill": ask("hymt2_attention_prefill_tc_protocol", ("kv_stages", "k_slots", "p_bars", "o_bars", "stage_holders", "s_buffers")),
            "decode": ask("hymt2_attention_decode_tc_protocol", ("stages", "accumulators")),
            "gemm": ask("hymt2_gemm_tc_protocol", ("max_stages", "accumulators", "issuers", "issuers_own_stages", "epilogue_groups"))}


def gemm_tc_rope_kv_wants_angles(tokens: int, rope_dim: int) -> bool:
    """Whether gemm_tc_rope_kv of this many tokens wants the table of their angles: where tokens are the
    accumulator's rows, a thread owns a whole token and would compute every angle once per head."""
    key = ("angles", tokens, rope_dim)
    hit = _rope_plans.get(key)
    if hit is None:
        hit = _rope_plans[key] = bool(_lib().hymt2_gemm_tc_rope_kv_wants_angles(c_int(tokens), c_int(rope_dim)))
    return hit


def rope_angles(token_pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """[T, rope_dim/2, 2] float32: (cos, sin) of float32(position) * inv_freq, the product and the functions of
    the rotation kernels; once per step and frequency table, for every layer that uses that table."""
    _need(token_pos, "token_pos", torch.int32, 1)
    _need(inv_freq, "inv_freq", torch.float32, 1)
    out = torch.empty((token_pos.shape[0], inv_freq.shape[0], 2), dtype=torch.float32, device=token_pos.device)
    _check(_lib().hymt2_rope_angles(_ptr(out), _ptr(token_pos), _ptr(inv_freq), c_int(token_pos.shape[0]),
                                    c_int(inv_freq.shape[0]), _stream()), "rope_angles")
    return out


def rope_kv(qkv: torch.Tensor, q_out: torch.Tensor, k_plane: torch.Tensor | None, v_plane: torch.Tensor | None,
            block_table: torch.Tensor, block_tokens: int, token_seq: torch.Tensor, token_pos: torch.Tensor,
            slot_ids: torch.Tensor, inv_freq: torch.Tensor | None, rope_dim: int, q_gain: torch.Tensor | None,
            k_gain: torch.Tensor | None, eps: float, nh: int, nkv: int, d: int) -> None:
    """Rotation, per-head norm and cache append for the fused projection qkv[T, (nh+2nkv)*d].
    k_plane/v_plane are one layer's cache planes [blocks, nkv, block_tokens, d], or None to
    write no keys and values (a layer that reads another layer's cache)."""
    _need(qkv, "qkv", None, 2); _need(q_out, "q_out", qkv.dtype, 2)
    T = q_out.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * d or q_out.shape[1] != nh * d or qkv.shape[0] < T:
        raise KernelError(f"rope_kv: shapes qkv {tuple(qkv.shape)} q_out {tuple(q_out.shape)} for nh={nh} nkv={nkv} d={d}")
    write = k_plane is not None
    if write:
        for t, n in ((k_plane, "k_plane"), (v_plane, "v_plane")):
            _need(t, n, qkv.dtype, 4)
            if t.shape[1:] != (nkv, block_tokens, d):
                raise KernelError(f"rope_kv: {n} is {tuple(t.shape)}, expected [blocks, {nkv}, {block_tokens}, {d}]")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((token_seq, "token_seq"), (token_pos, "token_pos"), (slot_ids, "slot_ids")):
        _need(t, n, torch.int32, 1)
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rope_dim // 2:
            raise KernelError("rope_kv: inv_freq must hold rope_dim/2 values")
    gain_dtype = F32
    if q_gain is not None:
        _need(q_gain, "q_gain", None, 1); _need(k_gain, "k_gain", q_gain.dtype, 1)
        if q_gain.shape[0] != d or k_gain.shape[0] != d:
            raise KernelError("rope_kv: the q and k gains must have head_dim entries")
        gain_dtype = dtype_code(q_gain.dtype)
    _check(_lib().hymt2_rope_kv(_ptr(qkv), _ptr(q_out), _ptr(k_plane), _ptr(v_plane), c_int(dtype_code(qkv.dtype)),
                                _ptr(block_table), c_int(block_table.stride(0)), c_int(block_tokens),
                                _ptr(token_seq), _ptr(token_pos), _ptr(slot_ids), _ptr(inv_freq), c_int(rope_dim),
                                _ptr(q_gain), _ptr(k_gain), c_int(gain_dtype), c_float(eps), c_int(T), c_int(nh),
                                c_int(nkv), c_int(d), c_int(1 if write else 0), _stream()), "rope_kv")


def attention_simt_scratch(tokens: int, nh: int, d: int, max_splits: int) -> tuple[int, int]:
    """Floats of scratch (partial outputs, partial max/sum) that a split run needs."""
    return tokens * nh * max_splits * d, tokens * nh * max_splits * 2


def attention_simt(out: torch.Tensor, q: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                   block_table: torch.Tensor, cu_seqlens: torch.Tensor, slot_ids: torch.Tensor,
                   kv_lens: torch.Tensor, batch: int, max_new_tokens: int, nh: int, nkv: int, d: int,
                   scale: float, window: int = 0, split_keys: int = 0, max_splits: int = 0,
                   part_acc: torch.Tensor | None = None, part_ml: torch.Tensor | None = None,
                   status: torch.Tensor | None = None) -> None:
    """Causal grouped-query attention of the new tokens over the paged cache (CUDA cores).  With a split, a row
    longer than max_splits * split_keys is left as it was and status[0] (the device's status word unless another is
    given) becomes 2."""
    if status is None:
        status = device_status(out.device)
    _need(out, "out", None, 2); _need(q, "q", out.dtype, 2)
    _need(k_plane, "k_plane", out.dtype, 4); _need(v_plane, "v_plane", out.dtype, 4)
    T = out.shape[0]
    block_tokens = k_plane.shape[2]
    if out.shape[1] != nh * d or q.shape[1] != nh * d or q.shape[0] < T or k_plane.shape[1] != nkv \
            or k_plane.shape[3] != d or v_plane.shape != k_plane.shape:
        raise KernelError(f"attention: shapes out {tuple(out.shape)} q {tuple(q.shape)} k {tuple(k_plane.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    if split_keys > 0:
        need_acc, need_ml = attention_simt_scratch(T, nh, d, max_splits)
        _need(part_acc, "part_acc", torch.float32); _need(part_ml, "part_ml", torch.float32)
        if part_acc.numel() < need_acc or part_ml.numel() < need_ml:
            raise KernelError("attention: the split scratch is too small")
    _check(_lib().hymt2_attention_simt(_ptr(out), _ptr(q), _ptr(k_plane), _ptr(v_plane), c_int(dtype_code(out.dtype)),
                                       _ptr(block_table), c_int(block_table.stride(0)), c_int(block_tokens),
                                       _ptr(cu_seqlens), _ptr(slot_ids), _ptr(kv_lens), c_int(batch), c_int(T),
                                       c_int(max_new_tokens), c_int(nh), c_int(nkv), c_int(d), c_float(scale),
                                       c_int(window), c_int(split_keys), c_int(max_splits), _ptr(part_acc),
                                       _ptr(part_ml), _stream(), _ptr(status)), "attention_simt", 2 if split_keys > 0 else 1)


def attention_decode_tc_scratch(rows: int, nh: int, nkv: int, d: int, max_splits: int) -> tuple[int, int, int]:
    """What attention_decode_tc needs: floats of partial outputs, floats of partial (maximum, sum), one
    copy for each quarter of d, and zeroed int32 counters."""
    return rows * nh * max_splits * d, rows * nh * max_splits * 8, rows * nkv * 4


def attention_decode_tc(out: torch.Tensor, q: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                        block_table: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor, nh: int, nkv: int,
                        d: int, scale: float, window: int, max_splits: int, part_acc: torch.Tensor,
                        part_ml: torch.Tensor, counters: torch.Tensor, status: torch.Tensor) -> None:
    """bfloat16 decode attention on the tcgen05 tensor cores with the keys on the 128-row side;
    head_dim 128, cache blocks of 64 tokens, at most 16 heads per kv head.  Chunks of 128 keys:
    max_splits >= ceil(longest length / 128); scratch and counters as attention_decode_tc_scratch
    says, the counters zeroed (the kernel leaves them zeroed)."""
    _need(out, "out", torch.bfloat16, 2); _need(q, "q", torch.bfloat16, 2)
    _need(k_plane, "k_plane", torch.bfloat16, 4); _need(v_plane, "v_plane", torch.bfloat16, 4)
    rows = out.shape[0]
    if out.shape[1] != nh * d or q.shape != out.shape or k_plane.shape[1] != nkv or k_plane.shape[3] != d \
            or v_plane.shape != k_plane.shape:
        raise KernelError(f"attention_decode_tc: shapes out {tuple(out.shape)} q {tuple(q.shape)} k {tuple(k_plane.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    _need(slot_ids, "slot_ids", torch.int32, 1); _need(kv_lens, "kv_lens", torch.int32, 1)
    need_acc, need_ml, need_counters = attention_decode_tc_scratch(rows, nh, nkv, d, max_splits)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml or counters.numel() < need_counters:
        raise KernelError("attention_decode_tc: the scratch for the partials is too small")
    _check(_lib().hymt2_attention_decode_tc(_ptr(out), _ptr(q), _ptr(k_plane), _ptr(v_plane), c_long(k_plane.shape[0]),
                                            _ptr(block_table), c_int(block_table.stride(0)), c_int(k_plane.shape[2]),
                                            _ptr(slot_ids), _ptr(kv_lens), c_int(rows), c_int(nh), c_int(nkv), c_int(d),
                                            c_float(scale), c_int(window), c_int(max_splits), _ptr(part_acc),
                                            _ptr(part_ml), _ptr(counters), _ptr(status), _stream()), "attention_decode_tc")


def attention_prefill_tc(out: torch.Tensor, q: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                         block_table: torch.Tensor, cu_seqlens: torch.Tensor, slot_ids: torch.Tensor,
                         kv_lens: torch.Tensor, batch: int, max_new_tokens: int, nh: int, nkv: int, d: int,
                         scale: float, window: int, status: torch.Tensor) -> None:
    """bfloat16 causal attention of the new tokens over the paged cache on the tcgen05 tensor cores
    (flash attention with S and O in tensor memory); head_dim 64 or 128, cache blocks of 64 tokens."""
    _need(out, "out", torch.bfloat16, 2); _need(q, "q", torch.bfloat16, 2)
    _need(k_plane, "k_plane", torch.bfloat16, 4); _need(v_plane, "v_plane", torch.bfloat16, 4)
    T = out.shape[0]
    if out.shape[1] != nh * d or q.shape != out.shape or k_plane.shape[1] != nkv or k_plane.shape[3] != d \
            or v_plane.shape != k_plane.shape:
        raise KernelError(f"attention_prefill_tc: shapes out {tuple(out.shape)} q {tuple(q.shape)} k {tuple(k_plane.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    _check(_lib().hymt2_attention_prefill_tc(_ptr(out), _ptr(q), _ptr(k_plane), _ptr(v_plane), c_long(k_plane.shape[0]),
                                             _ptr(block_table), c_int(block_table.stride(0)), c_int(k_plane.shape[2]),
                                             _ptr(cu_seqlens), _ptr(slot_ids), _ptr(kv_lens), c_int(batch), c_int(T),
                                             c_int(max_new_tokens), c_int(nh), c_int(nkv), c_int(d), c_float(scale),
                                             c_int(window), _ptr(status), _stream()), "attention_prefill_tc")


_counters: dict = {}


def zeroed_counters(device, n: int) -> torch.Tensor:
    """A per-device int32 array that is zero between kernels: arrival counters of kernels whose
    last-arriving block finishes the work (each such kernel leaves its counters at zero)."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    old = _counters.get(key)
    if old is None or old[-1].numel() < n:
        _counters[key] = (old or []) + [torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)]
    return _counters[key][-1]


def reset_counters(device) -> None:
    """Zeroes every arrival counter that kernels of this device share between launches (the split products'
    and the attention kernels'), on the current stream: after a kernel gave up in mid-count."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    for t in _counters.get(key) or []:
        t.zero_()
    ws, cnt, old = _tc_scratch.get(key, (None, None, []))
    for t in [cnt] + [o for o in old if o.dtype == torch.int32]:
        if t is not None:
            t.zero_()


def attention_decode(out: torch.Tensor, q: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                     block_table: torch.Tensor, cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor,
                     nh: int, nkv: int, d: int, scale: float, window: int, max_splits: int,
                     part_acc: torch.Tensor, part_ml: torch.Tensor, counters: torch.Tensor) -> None:
    """bfloat16 decode attention (one new token per row) that streams the cache once per kv head;
    head_dim 64 or 128.  The partials go through part_acc / part_ml (sizes as attention_simt_scratch);
    `counters` holds rows*nh zeroed ints (the kernel leaves them zero)."""
    _need(out, "out", torch.bfloat16, 2); _need(q, "q", torch.bfloat16, 2)
    _need(k_plane, "k_plane", torch.bfloat16, 4); _need(v_plane, "v_plane", torch.bfloat16, 4)
    rows = out.shape[0]
    if out.shape[1] != nh * d or q.shape[1] != nh * d or q.shape[0] < rows or k_plane.shape[1] != nkv \
            or k_plane.shape[3] != d or v_plane.shape != k_plane.shape:
        raise KernelError(f"attention_decode: shapes out {tuple(out.shape)} q {tuple(q.shape)} k {tuple(k_plane.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    need_acc, need_ml = attention_simt_scratch(rows, nh, d, max_splits)
    _need(part_acc, "part_acc", torch.float32); _need(part_ml, "part_ml", torch.float32)
    _need(counters, "counters", torch.int32, 1)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml or counters.numel() < rows * nh:
        raise KernelError("attention_decode: the scratch for the partials is too small")
    _check(_lib().hymt2_attention_decode(_ptr(out), _ptr(q), _ptr(k_plane), _ptr(v_plane), _ptr(block_table),
                                         c_int(block_table.stride(0)), c_int(k_plane.shape[2]), _ptr(cu_seqlens),
                                         _ptr(slot_ids), _ptr(kv_lens), c_int(rows), c_int(nh), c_int(nkv), c_int(d),
                                         c_float(scale), c_int(window), c_int(max_splits), _ptr(part_acc),
                                         _ptr(part_ml), _ptr(counters), _stream()), "attention_decode")


# ---------------------------------------------------------------------------
def _logits_ok(logits: torch.Tensor, what: str) -> None:
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError(f"{what}: logits must be a float32 CUDA matrix with contiguous rows")


ARGMAX_PIECE = 4096


def argmax(out: torch.Tensor, logits: torch.Tensor, row_map: torch.Tensor | None = None,
           scratch: tuple | None = None) -> None:
    """out[r] = first index of the maximum of logits[r]; rows with row_map[r] < 0 are skipped.
    `scratch` = (float32, int32) tensors of rows * ceil(vocab / 4096) entries lets a wide
    vocabulary be scanned by many blocks per row."""
    _need(out, "out", torch.int32, 1)
    _logits_ok(logits, "argmax")
    rows, vocab = logits.shape
    val = idx = None
    if scratch is not None:
        val, idx = scratch
        need = rows * (-(-vocab // ARGMAX_PIECE))
        _need(val, "scratch values", torch.float32); _need(idx, "scratch indices", torch.int32)
        if val.numel() < need or idx.numel() < need:
            raise KernelError("argmax: the scratch is too small")
    two_stage = scratch is not None and vocab > 2 * ARGMAX_PIECE
    _check(_lib().hymt2_argmax(_ptr(out), _ptr(logits), c_long(logits.stride(0)), c_int(rows), c_int(vocab),
                               _ptr(row_map), _ptr(val), _ptr(idx), _stream()), "argmax", 2 if two_stage else 1)


def seed_rng(states: torch.Tensor, rows: torch.Tensor, seeds: torch.Tensor) -> None:
    """states[rows[i]] = xoshiro256** state seeded with seeds[i] through SplitMix64."""
    _need(states, "states", torch.int64, 2); _need(rows, "rows", torch.int32, 1); _need(seeds, "seeds", torch.int64, 1)
    _check(_lib().hymt2_seed_rng(_ptr(states), _ptr(rows), _ptr(seeds), c_int(rows.shape[0]), _stream()), "seed_rng")


def sample(out: torch.Tensor, logits: torch.Tensor, inv_temperature: torch.Tensor, rng_states: torch.Tensor,
           row_map: torch.Tensor | None = None) -> None:
    """Temperature sampling of one token for every logits row whose sequence has a temperature
    above 0; advances that sequence's random stream by one draw.  row_map[r] is the row of the
    per-sequence arrays (inv_temperature, rng_states) that logits row r belongs to; < 0 skips."""
    _need(out, "out", torch.int32, 1); _need(inv_temperature, "inv_temperature", torch.float32, 1)
    _need(rng_states, "rng_states", torch.int64, 2)
    _logits_ok(logits, "sample")
    rows, vocab = logits.shape
    _check(_lib().hymt2_sample(_ptr(out), _ptr(logits), c_long(logits.stride(0)), c_int(rows), c_int(vocab),
                               _ptr(inv_temperature), _ptr(rng_states), _ptr(row_map), _stream()), "sample")


def filter_logits(logits: torch.Tensor, inv_temperature: torch.Tensor, top_k: torch.Tensor | None,
                  top_p: torch.Tensor | None, min_p: torch.Tensor | None, penalty: torch.Tensor | None,
                  history: torch.Tensor | None, row_map: torch.Tensor | None = None) -> None:
    """In place: repetition penalty, then (temperature > 0 only) top-k / min-p / top-p drops;
    dropped entries become -inf."""
    _logits_ok(logits, "filter")
    rows, vocab = logits.shape
    hs = 0
    if history is not None:
        _need(history, "history", torch.int32, 2)
        hs = history.shape[1]
    _check(_lib().hymt2_filter_logits(_ptr(logits), c_long(logits.stride(0)), c_int(rows), c_int(vocab),
                                      _ptr(inv_temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(penalty),
                                      _ptr(history), c_int(hs), _ptr(row_map), _stream()), "filter_logits")


def record_history(history: torch.Tensor, counts: torch.Tensor, tokens: torch.Tensor,
                   row_map: torch.Tensor | None, rows: int) -> None:
    """history[sequence, count % width] = tokens[r]; count += 1, for every logits row r."""
    _need(history, "history", torch.int32, 2); _need(counts, "counts", torch.int32, 1)
    _need(tokens, "tokens", torch.int32, 1)
    _check(_lib().hymt2_record_history(_ptr(history), _ptr(counts), c_int(history.shape[1]), _ptr(tokens),
                                       _ptr(row_map), c_int(rows), _stream()), "record_history")
