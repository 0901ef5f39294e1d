"""Runs ONE kernel of the library at a given shape a few times and prints its time: the small
cases that profiles are taken on, and a quick way to see what a change did to a kernel.

    python -m hymt2sharp_b200.kernels.microbench gemm --tokens 8 --out 6144 --inner 2048 --epilogue swiglu
    python -m hymt2sharp_b200.kernels.microbench attention-decode --batch 8 --context 2100
    python -m hymt2sharp_b200.kernels.microbench attention-prefill --tokens 2048
    python -m hymt2sharp_b200.kernels.microbench rmsnorm | rope | argmax ...

Weights rotate through `--copies` buffers so that a repeated call streams from memory, not from
the L2 cache.  Times come from CUDA events around `--iters` calls after `--warmup` calls; with
`--graph` the calls are captured into one CUDA graph first (what a decode step does), which
takes the Python launch cost out of the number.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from . import ops

DEV = "cuda:0"
BF = torch.bfloat16


def _time(fn, warmup: int, iters: int, graph: bool) -> float:
    """Microseconds per call."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(g, stream=side):
            for _ in range(iters):
                fn()
        g.replay()
        torch.cuda.synchronize()
        run = g.replay
        calls = iters
    else:
        def run():
            for _ in range(iters):
                fn()
        calls = iters
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / calls * 1000.0


def measure_qkv_rope(tokens: int, heads: int, kv_heads: int, inner: int, copies: int = 8, warmup: int = 3, iters: int = 20,
                     graph: bool = True) -> dict:
    """The fused q/k/v projection with rotation, per-head norm and cache append alone (heads of 128).  Up to 128 tokens
    are one token each of as many sequences (a decode step), more are one prompt."""
    d, bt = 128, 64
    N = (heads + 2 * kv_heads) * d
    ws = [(torch.randn(N, inner, device=DEV) / math.sqrt(inner)).to(BF) for _ in range(copies)]
    x = torch.randn(tokens, inner, device=DEV).to(BF)
    decode = tokens <= 128
    seqs, per_seq = (tokens, 1) if decode else (1, tokens)
    first = 2100 if decode else 0                                   # a decode step appends at position 2,100
    blocks_per_seq = (first + per_seq + bt - 1) // bt
    table = torch.arange(seqs * blocks_per_seq, dtype=torch.int32, device=DEV).view(seqs, blocks_per_seq).contiguous()
    kp = torch.zeros(seqs * blocks_per_seq, kv_heads, bt, d, dtype=BF, device=DEV)
    vp = torch.zeros_like(kp)
    token_seq = torch.arange(tokens, dtype=torch.int32, device=DEV) // per_seq
    token_pos = (first + torch.arange(tokens, dtype=torch.int32, device=DEV) % per_seq).to(torch.int32)
    slots = torch.arange(seqs, dtype=torch.int32, device=DEV)
    inv = (1.0 / (10000.0 ** (torch.arange(d // 2, dtype=torch.float32) / (d // 2)))).to(DEV)
    gain = torch.ones(d, device=DEV, dtype=BF)
    q_out = torch.empty(tokens, heads * d, dtype=BF, device=DEV)
    status = ops.device_status(DEV)
    angles = ops.rope_angles(token_pos, inv) if ops.gemm_tc_rope_kv_wants_angles(tokens, d) else None
    i = [0]

    def fn():
        ops.gemm_tc_rope_kv(x, ws[i[0] % copies], q_out, kp, vp, table, bt, token_seq, token_pos, slots, inv, d, gain, gain, 1e-5,
                            heads, kv_heads, status, angles=angles)
        i[0] += 1
    us = _time(fn, warmup, iters, graph)
    return {"us": us, "flops": 2.0 * tokens * N * inner, "bytes": N * inner * 2.0}


def measure_gemm(tokens: int, out_features: int, inner: int, epilogue: str = "store", float_out: bool = False,
                 copies: int = 8, warmup: int = 3, iters: int = 20, graph: bool = True) -> dict:
    """One tensor-core product alone: microseconds a call, its flops and the bytes of weights it streams."""
    epi = {"store": ops.EPILOGUE_STORE, "accumulate": ops.EPILOGUE_ACCUMULATE, "swiglu": ops.EPILOGUE_SWIGLU}[epilogue]
    rows = 2 * out_features if epi == ops.EPILOGUE_SWIGLU else out_features
    ws = [(torch.randn(rows, inner, device=DEV) / math.sqrt(inner)).to(BF) for _ in range(copies)]
    x = torch.randn(tokens, inner, device=DEV).to(BF)
    cdt = torch.float32 if (epi == ops.EPILOGUE_ACCUMULATE or float_out) else BF
    out = torch.zeros(tokens, out_features, device=DEV, dtype=cdt)
    status = ops.device_status(DEV)
    i = [0]

    def fn():
        ops.gemm_tc(out, x, ws[i[0] % copies], epi, status)
        i[0] += 1
    us = _time(fn, warmup, iters, graph)
    return {"us": us, "flops": 2.0 * tokens * rows * inner, "bytes": rows * inner * 2.0}


def gemm(a) -> None:
    if a.epilogue == "rope":   # --out is (heads + 2 kv heads) * 128
        m = measure_qkv_rope(a.tokens, a.heads, a.kv_heads, a.inner, a.copies, a.warmup, a.iters, a.graph)
        a.out = (a.heads + 2 * a.kv_heads) * 128
    else:
        m = measure_gemm(a.tokens, a.out, a.inner, a.epilogue, a.float_out, a.copies, a.warmup, a.iters, a.graph)
    print(f"gemm_tc tokens={a.tokens} out={a.out} inner={a.inner} epilogue={a.epilogue}: {m['us']:.1f} us  "
          f"{m['flops'] / m['us'] / 1e6:.1f} TFLOP/s  weights {m['bytes'] / m['us'] / 1e3:.0f} GB/s")


def _cache(batch: int, context: int, nkv: int, d: int):
    nblk = -(-context // 64) + 1
    kp = torch.randn(batch * nblk, nkv, 64, d, device=DEV).to(BF)
    vp = torch.randn_like(kp)
    table = torch.arange(batch * nblk, dtype=torch.int32, device=DEV).reshape(batch, nblk)
    return kp, vp, table


def measure_attention_decode(batch: int, context: int, heads: int, kv_heads: int, head_dim: int = 128, kernel: str = "tc",
                             copies: int = 8, warmup: int = 3, iters: int = 20, graph: bool = True) -> dict:
    """The decode attention alone over `batch` sequences of `context` cached tokens: microseconds a call and the
    bytes of keys and values it has to read."""
    from types import SimpleNamespace
    a = SimpleNamespace(batch=batch, context=context, heads=heads, kv_heads=kv_heads, head_dim=head_dim, kernel=kernel,
                        copies=copies, warmup=warmup, iters=iters, graph=graph)
    return _attention_decode(a)


def attention_decode(a) -> None:
    m = _attention_decode(a)
    print(f"attention_decode[{a.kernel}] batch={a.batch} context={a.context} heads={a.heads}/{a.kv_heads} d={a.head_dim}: "
          f"{m['us']:.1f} us  cache {m['bytes'] / m['us'] / 1e3:.0f} GB/s ({m['bytes'] / 1e6:.1f} MB)")


def _attention_decode(a) -> dict:
    B, nh, nkv, d = a.batch, a.heads, a.kv_heads, a.head_dim
    caches = [_cache(B, a.context, nkv, d) for _ in range(a.copies)]
    table = caches[0][2]
    q = torch.randn(B, nh * d, device=DEV).to(BF)
    out = torch.empty_like(q)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    kv = torch.full((B,), a.context, dtype=torch.int32, device=DEV)
    i = [0]
    chunk = 128 if a.kernel == "tc" else 256
    splits = -(-a.context // chunk)
    na, nm, nc = ops.attention_decode_tc_scratch(B, nh, nkv, d, splits)
    acc, ml = torch.empty(na, device=DEV), torch.empty(nm, device=DEV)
    cnt = torch.zeros(max(nc, B * nh), dtype=torch.int32, device=DEV)
    status = ops.device_status(DEV)
    scale = 1 / math.sqrt(d)

    def fn():
        kp, vp, _ = caches[i[0] % a.copies]
        i[0] += 1
        if a.kernel == "tc":
            ops.attention_decode_tc(out, q, kp, vp, table, slots, kv, nh, nkv, d, scale, 0, splits, acc, ml, cnt, status)
        else:
            ops.attention_decode(out, q, kp, vp, table, cu, slots, kv, nh, nkv, d, scale, 0, splits, acc, ml, cnt)
    us = _time(fn, a.warmup, a.iters, a.graph)
    return {"us": us, "bytes": B * a.context * nkv * d * 2 * 2.0, "flops": 4.0 * B * a.context * nh * d}


def measure_attention_prefill(tokens: int, heads: int, kv_heads: int, head_dim: int = 128, batch: int = 1,
                              warmup: int = 3, iters: int = 20, graph: bool = True) -> dict:
    """The prompt attention alone over `batch` prompts of `tokens` tokens: microseconds a call and its (causal) flops."""
    from types import SimpleNamespace
    return _attention_prefill(SimpleNamespace(tokens=tokens, heads=heads, kv_heads=kv_heads, head_dim=head_dim, batch=batch,
                                              warmup=warmup, iters=iters, graph=graph))


def attention_prefill(a) -> None:
    m = _attention_prefill(a)
    print(f"attention_prefill_tc batch={a.batch} tokens={a.tokens} heads={a.heads}/{a.kv_heads} d={a.head_dim}: {m['us']:.1f} us  "
          f"{m['flops'] / m['us'] / 1e6:.1f} TFLOP/s (causal)")


def _attention_prefill(a) -> dict:
    nh, nkv, d, T = a.heads, a.kv_heads, a.head_dim, a.tokens
    kp, vp, table = _cache(a.batch, T, nkv, d)
    q = torch.randn(a.batch * T, nh * d, device=DEV).to(BF)
    out = torch.empty_like(q)
    slots = torch.arange(a.batch, dtype=torch.int32, device=DEV)
    cu = (torch.arange(a.batch + 1, dtype=torch.int32, device=DEV) * T).contiguous()
    kv = torch.full((a.batch,), T, dtype=torch.int32, device=DEV)
    status = ops.device_status(DEV)
    fn = lambda: ops.attention_prefill_tc(out, q, kp, vp, table, cu, slots, kv, a.batch, T, nh, nkv, d, 1 / math.sqrt(d), 0, status)
    us = _time(fn, a.warmup, a.iters, a.graph)
    return {"us": us, "flops": 4.0 * nh * d * (T * (T + 1) / 2) * a.batch, "bytes": a.batch * T * (2 * nh + 2 * nkv) * d * 2.0}


def small(a) -> None:
    B, H, nh, nkv, d, V = a.tokens, a.hidden, a.heads, a.kv_heads, a.head_dim, a.vocab
    if a.op == "rmsnorm":
        x = torch.randn(B, H, device=DEV)
        gain = torch.ones(H, device=DEV, dtype=BF)
        y = torch.empty(B, H, device=DEV, dtype=BF)
        fn = lambda: ops.rmsnorm(y, x, gain, 1e-5)
        nbytes = B * H * 6
    elif a.op == "rope":
        kp, vp, table = _cache(B, a.context, nkv, d)
        qkv = torch.randn(B, (nh + 2 * nkv) * d, device=DEV).to(BF)
        qo = torch.empty(B, nh * d, device=DEV, dtype=BF)
        inv = torch.rand(d // 2, device=DEV)
        seq = torch.arange(B, dtype=torch.int32, device=DEV)
        pos = torch.full((B,), a.context - 1, dtype=torch.int32, device=DEV)
        gain = torch.ones(d, device=DEV, dtype=BF)
        fn = lambda: ops.rope_kv(qkv, qo, kp, vp, table, 64, seq, pos, seq, inv, d, gain, gain, 1e-5, nh, nkv, d)
        nbytes = B * (nh + 2 * nkv) * d * 4
    else:
        lg = torch.randn(B, V, device=DEV)
        o = torch.empty(B, dtype=torch.int32, device=DEV)
        pieces = B * (-(-V // ops.ARGMAX_PIECE))
        sc = (torch.empty(pieces, device=DEV), torch.empty(pieces, dtype=torch.int32, device=DEV))
        fn = lambda: ops.argmax(o, lg, None, sc)
        nbytes = B * V * 4
    us = _time(fn, a.warmup, a.iters, a.graph)
    print(f"{a.op} rows={B}: {us:.1f} us  {nbytes / us / 1e3:.0f} GB/s")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="op", required=True)

    def common(p):
        p.add_argument("--warmup", type=int, default=3)
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--graph", action="store_true")
        p.add_argument("--heads", type=int, default=16)
        p.add_argument("--kv-heads", type=int, default=4)
        p.add_argument("--head-dim", type=int, default=128)
    g = sub.add_parser("gemm")
    common(g)
    g.add_argument("--tokens", type=int, default=8)
    g.add_argument("--out", type=int, default=6144)
    g.add_argument("--inner", type=int, default=2048)
    g.add_argument("--epilogue", default="store", choices=["store", "accumulate", "swiglu", "rope"],
                   help="rope: the fused q/k/v projection with rotation, norm and cache append (--heads, --kv-heads; --out is not used)")
    g.add_argument("--float-out", action="store_true")
    g.add_argument("--copies", type=int, default=8)
    d = sub.add_parser("attention-decode")
    common(d)
    d.add_argument("--batch", type=int, default=8)
    d.add_argument("--context", type=int, default=2100)
    d.add_argument("--kernel", default="tc", choices=["tc", "stream"])
    d.add_argument("--copies", type=int, default=8, help="caches that the calls rotate through, so that keys come from memory")
    pf = sub.add_parser("attention-prefill")
    common(pf)
    pf.add_argument("--batch", type=int, default=1)
    pf.add_argument("--tokens", type=int, default=2048)
    for name in ("rmsnorm", "rope", "argmax"):
        s = sub.add_parser(name)
        common(s)
        s.add_argument("--tokens", type=int, default=8)
        s.add_argument("--hidden", type=int, default=2048)
        s.add_argument("--vocab", type=int, default=120818)
        s.add_argument("--context", type=int, default=2100)
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("microbench needs a CUDA device", file=sys.stderr)
        return 1
    {"gemm": gemm, "attention-decode": attention_decode, "attention-prefill": attention_prefill}.get(a.op, small)(a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
