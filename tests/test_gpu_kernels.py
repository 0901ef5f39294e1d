"""Each kernel alone against a plain torch float32 reference of the same formula, at sizes
other than the engine's tiny configurations (odd widths, tails, many heads and groups)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _ops():
    from hymt2sharp_b200.kernels import ops
    return ops


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    ops = _ops()
    table = torch.randn(301, 70, device=DEV).to(dtype)
    ids = torch.tensor([0, 300, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 70, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.embed(out, table, ids, status)
    assert torch.equal(out, table.float()[ids.long()]) and status[0].item() == 0
    bad = torch.tensor([3, 301], dtype=torch.int32, device=DEV)
    out2 = torch.full((2, 70), 9.0, device=DEV)
    ops.embed(out2, table, bad, status)
    assert status[0].item() == 1 and torch.equal(out2[1], torch.zeros(70, device=DEV))  # flagged, nothing read outside


@pytest.mark.parametrize("xdt, gdt, ydt", [(torch.float32, torch.float32, torch.float32),
                                           (torch.float32, torch.bfloat16, torch.bfloat16),
                                           (torch.float32, torch.float32, torch.bfloat16),
                                           (torch.bfloat16, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("dim", [70, 1000, 2052, 768, 2048])
def test_rmsnorm(xdt, gdt, ydt, dim):
    ops = _ops()
    x = (torch.randn(37, dim, device=DEV) * 3).to(xdt)
    g = (1 + 0.1 * torch.randn(dim, device=DEV)).to(gdt)
    eps = 1e-3
    ref = x.float() * torch.rsqrt((x.float() ** 2).mean(-1, keepdim=True) + eps) * g.float()
    out = torch.empty(37, dim, dtype=ydt, device=DEV)
    ops.rmsnorm(out, x, g, eps)
    assert torch.allclose(out.float(), ref, **_tol(ydt))
    idx = torch.tensor([36, 0, 5], dtype=torch.int32, device=DEV)
    out3 = torch.empty(3, dim, dtype=ydt, device=DEV)
    ops.rmsnorm(out3, x, g, eps, idx)
    assert torch.equal(out3, out[idx.long()])


@pytest.mark.parametrize("adt, wdt, cdt", [(torch.float32, torch.float32, torch.float32),
                                           (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                           (torch.bfloat16, torch.bfloat16, torch.float32),
                                           (torch.bfloat16, torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("M, N, K", [(1, 67, 70), (5, 64, 64), (130, 131, 257), (64, 1000, 33)])
def test_gemm_simt_epilogues(adt, wdt, cdt, M, N, K):
    ops = _ops()
    a = torch.randn(M, K, device=DEV).to(adt)
    w = (torch.randn(2 * N, K, device=DEV) / math.sqrt(K)).to(wdt)
    ref = a.double() @ w.double().T
    tol = _tol(cdt)
    out = torch.empty(M, N, dtype=cdt, device=DEV)
    ops.gemm_simt(out, a, w[:N], ops.EPILOGUE_STORE)
    assert torch.allclose(out.double(), ref[:, :N], **tol)
    base = torch.randn(M, N, device=DEV).to(cdt)
    acc = base.clone()
    ops.gemm_simt(acc, a, w[:N], ops.EPILOGUE_ACCUMULATE)
    assert torch.allclose(acc.double(), base.double() + ref[:, :N], **tol)
    glu = torch.empty(M, N, dtype=cdt, device=DEV)
    ops.gemm_simt(glu, a, w, ops.EPILOGUE_SWIGLU)
    g, u = ref[:, :N], ref[:, N:]
    assert torch.allclose(glu.double(), g / (1 + torch.exp(-g)) * u, **tol)
    # row strides larger than the rows (a view into a wider matrix)
    wide = torch.zeros(M, K + 8, device=DEV).to(adt)
    wide[:, :K] = a
    out2 = torch.empty(M, N, dtype=cdt, device=DEV)
    ops.gemm_simt(out2, wide[:, :K], w[:N], ops.EPILOGUE_STORE)
    assert torch.equal(out2, out)


def test_gemm_rows_do_not_depend_on_the_batch():
    ops = _ops()
    a = torch.randn(200, 300, device=DEV)
    w = torch.randn(77, 300, device=DEV)
    full = torch.empty(200, 77, device=DEV)
    ops.gemm_simt(full, a, w)
    one = torch.empty(1, 77, device=DEV)
    ops.gemm_simt(one, a[131:132].contiguous(), w)
    assert torch.equal(one[0], full[131])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(dtype):
    ops = _ops()
    gu = torch.randn(9, 2 * 35, device=DEV).to(dtype)
    out = torch.empty(9, 35, dtype=dtype, device=DEV)
    ops.silu_mul(out, gu)
    g, u = gu.float()[:, :35], gu.float()[:, 35:]
    assert torch.allclose(out.float(), g / (1 + torch.exp(-g)) * u, **_tol(dtype))


def _paged(keys, values, block_tokens, dtype, shuffle_seed=0):
    """keys/values: list per sequence of [len, nkv, d] → cache planes with shuffled blocks, table."""
    nkv, d = keys[0].shape[1:]
    need = [-(-k.shape[0] // block_tokens) for k in keys]
    total = sum(need) + 3
    perm = np.random.default_rng(shuffle_seed).permutation(total)
    kp = torch.full((total, nkv, block_tokens, d), 99.0, device=DEV).to(dtype)  # unused rows would poison a sum
    vp = torch.full((total, nkv, block_tokens, d), -99.0, device=DEV).to(dtype)
    table = torch.full((len(keys), max(need) + 1), -1, dtype=torch.int32)
    nxt = 0
    for s, (k, v) in enumerate(zip(keys, values)):
        for b in range(need[s]):
            phys = int(perm[nxt]); nxt += 1
            table[s, b] = phys
            chunk = slice(b * block_tokens, min((b + 1) * block_tokens, k.shape[0]))
            n = chunk.stop - chunk.start
            kp[phys, :, :n] = k[chunk].transpose(0, 1).to(dtype)
            vp[phys, :, :n] = v[chunk].transpose(0, 1).to(dtype)
    return kp, vp, table.to(DEV)


def _ref_attention(q, k, v, new, window, scale):
    """q [new, nh, d] are the last `new` positions of a sequence with keys k [len, nkv, d]."""
    L, nkv, d = k.shape
    nh = q.shape[1]
    g = nh // nkv
    out = torch.empty(new, nh, d, dtype=torch.float64, device=q.device)
    for i in range(new):
        p = L - new + i
        lo = max(0, p - window + 1) if window > 0 else 0
        for h in range(nh):
            s = (k[lo:p + 1, h // g].double() @ q[i, h].double()) * scale
            w = torch.softmax(s, dim=0)
            out[i, h] = w @ v[lo:p + 1, h // g].double()
    return out.reshape(new, nh * d)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, d, window", [(8, 2, 64, 0), (5, 5, 16, 0), (20, 1, 48, 0), (6, 3, 128, 37),
                                                (4, 2, 256, 0), (12, 4, 80, 100)])
def test_attention_prefill_and_decode(dtype, nh, nkv, d, window):
    ops = _ops()
    torch.manual_seed(nh * 100 + d)
    lens, news = [70, 1, 200, 33], [70, 1, 45, 2]   # whole prompt, single token, chunk after a prefix, 2 tokens
    keys = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    vals = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    qs = [torch.randn(n, nh, d, device=DEV).to(dtype) for n in news]
    kp, vp, table = _paged(keys, vals, 64, dtype)
    scale = 1 / math.sqrt(d)
    q = torch.cat([x.reshape(x.shape[0], nh * d) for x in qs])
    cu = torch.tensor(np.concatenate([[0], np.cumsum(news)]), dtype=torch.int32, device=DEV)
    slots = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = torch.zeros(sum(news), nh * d, dtype=dtype, device=DEV)
    ops.attention_simt(out, q, kp, vp, table, cu, slots, kv, len(lens), max(news), nh, nkv, d, scale, window)
    ref = torch.cat([_ref_attention(qs[i].float(), keys[i].float(), vals[i].float(), news[i], window, scale)
                     for i in range(len(lens))])
    assert torch.allclose(out.double(), ref, **_tol(dtype))

    # decode with split keys: one token per sequence, partials merged in order
    lens2 = [700, 1, 257, 64]
    keys = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens2]
    vals = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens2]
    qs = [torch.randn(1, nh, d, device=DEV).to(dtype) for _ in lens2]
    kp, vp, table = _paged(keys, vals, 64, dtype, shuffle_seed=1)
    q = torch.cat([x.reshape(1, nh * d) for x in qs])
    cu = torch.arange(5, dtype=torch.int32, device=DEV)
    kv = torch.tensor(lens2, dtype=torch.int32, device=DEV)
    splits = -(-max(lens2) // 256)
    na, nm = ops.attention_simt_scratch(4, nh, d, splits)
    acc = torch.full((na,), float("nan"), device=DEV)
    ml = torch.full((nm,), float("nan"), device=DEV)
    out = torch.zeros(4, nh * d, dtype=dtype, device=DEV)
    ops.attention_simt(out, q, kp, vp, table, cu, slots, kv, 4, 1, nh, nkv, d, scale, window, 256, splits, acc, ml)
    ref = torch.cat([_ref_attention(qs[i].float(), keys[i].float(), vals[i].float(), 1, window, scale) for i in range(4)])
    assert torch.allclose(out.double(), ref, **_tol(dtype))
    # a padding row (slot -1) is left alone
    slots2 = torch.tensor([0, -1, 2, 3], dtype=torch.int32, device=DEV)
    out2 = torch.full((4, nh * d), 5.0, dtype=dtype, device=DEV)
    ops.attention_simt(out2, q, kp, vp, table, cu, slots2, kv, 4, 1, nh, nkv, d, scale, window, 256, splits, acc, ml)
    assert torch.equal(out2[0], out[0]) and torch.equal(out2[2:], out[2:]) and (out2[1] == 5.0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, d, rope_dim, norm", [(8, 2, 64, 64, True), (3, 3, 16, 16, False),
                                                        (6, 1, 48, 16, True), (4, 2, 128, 0, True),
                                                        (4, 2, 128, 128, True), (2, 1, 256, 256, False)])
def test_rope_qknorm_kv_append(dtype, nh, nkv, d, rope_dim, norm):
    ops = _ops()
    torch.manual_seed(d)
    T, bt = 11, 64
    pos = torch.tensor([0, 1, 2, 63, 64, 65, 500, 7000, 3, 4, 127], dtype=torch.int32)
    seq = torch.tensor([0, 0, 0, 1, 1, 1, 2, 3, 4, 4, 5], dtype=torch.int32)
    slots = torch.tensor([2, 0, 3, 1, -1, 4], dtype=torch.int32)  # batch row 4 is padding
    qkv = torch.randn(T, (nh + 2 * nkv) * d, device=DEV).to(dtype)
    table = torch.full((5, 120), -1, dtype=torch.int32)
    nblocks = 0
    for t in range(T):
        s = int(slots[seq[t]])
        if s >= 0 and table[s, pos[t] // bt] < 0:
            table[s, pos[t] // bt] = nblocks
            nblocks += 1
    kp = torch.zeros(nblocks, nkv, bt, d, dtype=dtype, device=DEV)
    vp = torch.zeros(nblocks, nkv, bt, d, dtype=dtype, device=DEV)
    inv = (1.0 / (10000.0 ** (torch.arange(rope_dim // 2, dtype=torch.float32) / max(1, rope_dim // 2)))).to(DEV) \
        if rope_dim else None
    qg = (1 + 0.1 * torch.randn(d, device=DEV)).to(dtype) if norm else None
    kg = (1 + 0.1 * torch.randn(d, device=DEV)).to(dtype) if norm else None
    q_out = torch.empty(T, nh * d, dtype=dtype, device=DEV)
    eps = 1e-5
    ops.rope_kv(qkv, q_out, kp, vp, table.to(DEV), bt, seq.to(DEV), pos.to(DEV), slots.to(DEV), inv, rope_dim,
                qg, kg, eps, nh, nkv, d)

    x = qkv.float().reshape(T, nh + 2 * nkv, d)

    def rotate(h):
        if not rope_dim:
            return h
        half = rope_dim // 2
        ang = pos.to(DEV).float()[:, None] * inv[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        out = h.clone()
        out[..., :half] = h[..., :half] * c - h[..., half:rope_dim] * s
        out[..., half:rope_dim] = h[..., :half] * s + h[..., half:rope_dim] * c
        return out

    def normed(h, g):
        return h if g is None else h * torch.rsqrt((h ** 2).mean(-1, keepdim=True) + eps) * g.float()

    q_ref = normed(rotate(x[:, :nh]), qg).reshape(T, nh * d)
    k_ref = normed(rotate(x[:, nh:nh + nkv]), kg)
    v_ref = x[:, nh + nkv:]
    tol = _tol(dtype)
    assert torch.allclose(q_out.float(), q_ref, **tol)
    for t in range(T):
        s = int(slots[seq[t]])
        if s < 0:
            continue
        b, o = int(table[s, pos[t] // bt]), int(pos[t]) % bt
        assert torch.allclose(kp[b, :, o].float(), k_ref[t], **tol), f"key of token {t}"
        assert torch.allclose(vp[b, :, o].float(), v_ref[t], atol=0, rtol=0), f"value of token {t}"
    written = sum(1 for t in range(T) if int(slots[seq[t]]) >= 0)
    assert int((kp.float().abs().sum(-1) > 0).sum()) == written * nkv  # nothing else was touched
    # a run that reads another layer's cache writes only q
    q2 = torch.empty_like(q_out)
    ops.rope_kv(qkv, q2, None, None, table.to(DEV), bt, seq.to(DEV), pos.to(DEV), slots.to(DEV), inv, rope_dim,
                qg, kg, eps, nh, nkv, d)
    assert torch.equal(q2, q_out)


@pytest.mark.parametrize("T, nh, nkv, K, rope_dim, norm, gain_dtype", [
    (11, 16, 4, 2048, 128, True, torch.bfloat16), (1, 4, 2, 1024, 128, False, torch.bfloat16),
    (11, 6, 1, 1096, 48, True, torch.float32), (8, 16, 4, 2048, 0, True, torch.bfloat16), (40, 8, 2, 2048, 128, True, torch.bfloat16),
    # more than 128 tokens: tokens are the accumulator's rows; tiles of one head (300, 700 tokens) and the
    # persistent kernel's tiles of two heads (2,500 tokens; 4,800 with 7 heads: the last tile holds one)
    (300, 8, 2, 512, 128, True, torch.bfloat16), (700, 3, 1, 264, 0, True, torch.float32), (300, 4, 2, 512, 128, False, torch.bfloat16),
    (2500, 16, 4, 512, 128, True, torch.bfloat16), (4800, 5, 1, 256, 128, True, torch.float32), (2500, 16, 4, 256, 0, False, torch.bfloat16)])
def test_projection_with_rotation_and_cache_append_in_one_kernel(T, nh, nkv, K, rope_dim, norm, gain_dtype):
    """The fused kernel (q/k/v projection, rotation, per-head norm, cache append; head_dim 128) against the
    kernels it replaces: the plain projection followed by rope_kv.  Positions across block borders, a padding
    row, a rotation of part of the head, no rotation, gains of both types, and a run that writes no keys."""
    ops = _ops()
    torch.manual_seed(T + nh + K)
    d, bt, dtype = 128, 64, torch.bfloat16
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    base_pos = [0, 1, 2, 63, 64, 65, 500, 7000, 3, 4, 127]
    base_seq = [0, 0, 0, 1, 1, 1, 2, 3, 4, 4, 5]
    if T <= 11:
        pos, seq = base_pos[:T], base_seq[:T]
    elif T <= 128:
        pos, seq = list(range(100, 100 + T)), [0] * T
    else:
        # several prompts in one step: two long ones, five tokens of a padding row, one that starts inside a block
        a, b = T // 2, T // 4
        rest = T - a - b - 5
        pos = list(range(100, 100 + a)) + list(range(b)) + list(range(5)) + list(range(60, 60 + rest))
        seq = [0] * a + [2] * b + [4] * 5 + [5] * rest
    pos_t, seq_t = torch.tensor(pos, dtype=torch.int32), torch.tensor(seq, dtype=torch.int32)
    slots = torch.tensor([2, 0, 3, 1, -1, 4], dtype=torch.int32)   # batch row 4 is padding
    table = torch.full((5, 120), -1, dtype=torch.int32)
    nblocks = 0
    for t in range(T):
        s = int(slots[seq[t]])
        if s >= 0 and table[s, pos[t] // bt] < 0:
            table[s, pos[t] // bt] = nblocks
            nblocks += 1
    x = torch.randn(T, K, device=DEV).to(dtype)
    w = (torch.randn((nh + 2 * nkv) * d, K, device=DEV) / math.sqrt(K)).to(dtype)
    inv = (1.0 / (10000.0 ** (torch.arange(rope_dim // 2, dtype=torch.float32) / max(1, rope_dim // 2)))).to(DEV) \
        if rope_dim else None
    qg = (1 + 0.1 * torch.randn(d, device=DEV)).to(gain_dtype) if norm else None
    kg = (1 + 0.1 * torch.randn(d, device=DEV)).to(gain_dtype) if norm else None
    eps = 1e-5
    assert ops.gemm_tc_rope_kv_supported(x, w, nh, nkv, d, dtype, rope_dim)
    dev = lambda t: t.to(DEV)
    # the two kernels
    qkv = torch.empty(T, (nh + 2 * nkv) * d, dtype=dtype, device=DEV)
    ops.gemm_tc(qkv, x, w, ops.EPILOGUE_STORE, status)
    kp2, vp2 = (torch.zeros(nblocks, nkv, bt, d, dtype=dtype, device=DEV) for _ in range(2))
    q2 = torch.empty(T, nh * d, dtype=dtype, device=DEV)
    ops.rope_kv(qkv, q2, kp2, vp2, dev(table), bt, dev(seq_t), dev(pos_t), dev(slots), inv, rope_dim, qg, kg, eps, nh, nkv, d)
    # the one kernel
    kp1, vp1 = (torch.zeros(nblocks, nkv, bt, d, dtype=dtype, device=DEV) for _ in range(2))
    q1 = torch.full((T, nh * d), 9.0, dtype=dtype, device=DEV)
    angles = ops.rope_angles(dev(pos_t), inv) if ops.gemm_tc_rope_kv_wants_angles(T, rope_dim) else None
    if angles is not None:   # the table holds the angles that the rotation kernels compute in place
        want = dev(pos_t).float()[:, None] * inv[None, :]
        assert torch.allclose(angles[..., 0], torch.cos(want), atol=2e-6) and torch.allclose(angles[..., 1], torch.sin(want), atol=2e-6)
    ops.gemm_tc_rope_kv(x, w, q1, kp1, vp1, dev(table), bt, dev(seq_t), dev(pos_t), dev(slots), inv, rope_dim, qg, kg, eps,
                        nh, nkv, status, angles=angles)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    assert torch.equal(vp1, vp2)                                   # values are copied: the same bits
    # rotation and norm round once more: at most the last bit of a bfloat16 differs
    for one, two, what in ((q1, q2, "q"), (kp1, kp2, "k")):
        diff = (one.float() - two.float()).abs()
        assert float((diff / two.float().abs().clamp_min(1e-2)).max()) <= 2 ** -7, what
        assert float((diff > 0).float().mean()) < 0.02, what
    # a run that reads another layer's cache writes only q
    q3 = torch.empty_like(q1)
    ops.gemm_tc_rope_kv(x, w, q3, None, None, dev(table), bt, dev(seq_t), dev(pos_t), dev(slots), inv, rope_dim, qg, kg, eps,
                        nh, nkv, status, angles=angles)
    assert torch.equal(q3, q1)
    # what it does not take: another head size; a prompt's worth of tokens whose heads are rotated in part
    assert not ops.gemm_tc_rope_kv_supported(x, w, nh * 2, nkv * 2, 64, dtype, rope_dim)
    big = torch.randn(300, K, device=DEV).to(dtype)
    assert not ops.gemm_tc_rope_kv_supported(big, w, nh, nkv, d, dtype, 48)


def test_argmax_takes_the_first_maximum():
    ops = _ops()
    x = torch.randn(7, 120818, device=DEV)
    x[2, 100000] = x[2, 55] = 50.0
    x[3, :] = -1.0
    x[5, 120817] = 60.0
    out = torch.full((7,), -5, dtype=torch.int32, device=DEV)
    row_map = torch.tensor([0, 1, 2, 3, -1, 5, 6], dtype=torch.int32, device=DEV)
    ops.argmax(out, x, row_map)
    want = x.argmax(dim=1).tolist()
    want[2], want[3], want[4], want[5] = 55, 0, -5, 120817
    assert out.tolist() == want
    # the wide-vocabulary path: pieces of 4096 logits scanned by a block each, then one pick per row
    pieces = 7 * (-(-120818 // ops.ARGMAX_PIECE))
    scratch = (torch.full((pieces,), float("nan"), device=DEV), torch.full((pieces,), -3, dtype=torch.int32, device=DEV))
    out2 = torch.full((7,), -5, dtype=torch.int32, device=DEV)
    ops.argmax(out2, x, row_map, scratch)
    assert out2.tolist() == want
    wide = torch.randn(3, 1000, device=DEV)
    view = wide[:, :509]  # rows with a stride larger than the vocabulary
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    ops.argmax(out, view)
    assert out.tolist() == view.argmax(dim=1).tolist()


def test_sampling_distribution_and_stream():
    ops = _ops()
    import sys, os
    from plain.hunyuan_plain import Xoshiro256StarStar
    vocab = 509
    logits = torch.randn(1, vocab, device=DEV) * 2
    probs = torch.softmax(logits[0].double() / 0.7, dim=0).cpu().numpy()
    states = torch.zeros(3, 4, dtype=torch.int64, device=DEV)
    seeds = torch.tensor([5, 6, 7], dtype=torch.int64, device=DEV)
    ops.seed_rng(states, torch.arange(3, dtype=torch.int32, device=DEV), seeds)
    ref = Xoshiro256StarStar(6)
    assert [x & ((1 << 64) - 1) for x in states[1].tolist()] == ref.s
    inv_t = torch.tensor([0.0, 1 / 0.7, 0.0], device=DEV)
    row_map = torch.tensor([1], dtype=torch.int32, device=DEV)
    out = torch.empty(1, dtype=torch.int32, device=DEV)
    cdf = np.cumsum(probs)
    counts = np.zeros(vocab)
    for i in range(3000):
        ops.sample(out, logits, inv_t, states, row_map)
        tok = out.item()
        u = float(ref.next_single())
        lo = cdf[tok - 1] if tok else 0.0
        assert lo - 1e-5 <= u <= cdf[tok] + 1e-5, f"draw {i}: u={u} token {tok} interval [{lo}, {cdf[tok]}]"
        counts[tok] += 1
    top = np.argsort(-probs)[:5]
    assert np.allclose(counts[top] / 3000, probs[top], atol=0.03)
    assert states[0].tolist() != [0, 0, 0, 0] and [x & ((1 << 64) - 1) for x in states[1].tolist()] == ref.s


# T <= 128 runs swapped (weights on the 128-row side, split K when there are few tiles), larger T runs
# normal, and with many tiles (the last two cases) the persistent kernel with two accumulators;
# sizes with tails in T, N and K (K only needs to be a multiple of 8)
@pytest.mark.parametrize("T, N, K", [(1, 1000, 200), (8, 256, 128), (16, 2048, 2048), (33, 130, 72), (64, 384, 6144),
                                     (100, 3072, 512), (128, 128, 64), (129, 1000, 200), (300, 384, 256),
                                     (1000, 520, 1032), (3000, 4000, 136), (2100, 5000, 72)])
def test_gemm_tcgen05_epilogues(T, N, K):
    ops = _ops()
    torch.manual_seed(T + N)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    a = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    ref = a.double() @ w.double().T
    for cdt in (torch.float32, torch.bfloat16):
        out = torch.full((T, N), 7.0, dtype=cdt, device=DEV)
        ops.gemm_tc(out, a, w[:N], ops.EPILOGUE_STORE, status)
        assert torch.allclose(out.double(), ref[:, :N], **_tol(cdt)), f"store {cdt}"
    base = torch.randn(T, N, device=DEV)
    acc = base.clone()
    ops.gemm_tc(acc, a, w[:N], ops.EPILOGUE_ACCUMULATE, status)
    assert torch.allclose(acc.double(), base.double() + ref[:, :N], rtol=2e-5, atol=2e-5)
    glu = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(glu, a, w, ops.EPILOGUE_SWIGLU, status)
    g, u = ref[:, :N], ref[:, N:]
    assert torch.allclose(glu.double(), g / (1 + torch.exp(-g)) * u, **_tol(torch.bfloat16))
    # twice the same call gives the same bits (the split sum does not depend on arrival order)
    acc2 = base.clone()
    ops.gemm_tc(acc2, a, w[:N], ops.EPILOGUE_ACCUMULATE, status)
    assert torch.equal(acc, acc2)
    # a view with a larger row stride; an output with a larger row stride
    wide = torch.zeros(T, K + 16, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = a
    big = torch.zeros(T, N + 5, device=DEV)
    ops.gemm_tc(big[:, :N], wide[:, :K], w[:N], ops.EPILOGUE_STORE, status)
    assert torch.allclose(big[:, :N].double(), ref[:, :N], rtol=2e-5, atol=2e-5) and float(big[:, N:].abs().sum()) == 0
    assert status.tolist() == [0, 0, 0, 0]


# the shapes of the full-size models' products: few tokens (weight rows on the 128-row side, K cut over clusters or through the
# global workspace, the vocabulary's last tile of 114 rows) and a prompt's worth (the persistent kernel with its chosen tile width,
# 128-wide tiles where the product adds into the residual)
@pytest.mark.parametrize("T, N, K, epilogue, cdt", [
    (8, 120818, 2048, "store", torch.float32), (1, 120818, 2048, "store", torch.float32), (64, 128167, 4096, "store", torch.float32),
    (8, 6144, 2048, "swiglu", torch.bfloat16), (64, 6144, 2048, "swiglu", torch.bfloat16), (8, 14336, 4096, "swiglu", torch.bfloat16),
    (8, 2048, 6144, "add", torch.float32), (8, 2048, 2048, "add", torch.float32), (8, 3072, 2048, "store", torch.bfloat16),
    (2048, 6144, 2048, "swiglu", torch.bfloat16), (2048, 2048, 2048, "add", torch.float32), (2048, 2048, 6144, "add", torch.float32),
    (2048, 3072, 2048, "store", torch.bfloat16), (4096, 8192, 3072, "swiglu", torch.bfloat16)])
def test_gemm_tcgen05_at_full_size_shapes(T, N, K, epilogue, cdt):
    ops = _ops()
    torch.manual_seed(N % 1000 + T)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    a = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    rows_w = 2 * N if epilogue == "swiglu" else N
    w = (torch.randn(rows_w, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    ref = torch.empty(T, rows_w, dtype=torch.float64, device=DEV)
    for r0 in range(0, rows_w, 16384):   # in pieces: the float64 copy of a whole vocabulary table need not exist
        ref[:, r0:r0 + 16384] = a.double() @ w[r0:r0 + 16384].double().T
    if epilogue == "store":
        out = torch.full((T, N), 7.0, dtype=cdt, device=DEV)
        ops.gemm_tc(out, a, w, ops.EPILOGUE_STORE, status)
        want = ref
    elif epilogue == "add":
        base = torch.randn(T, N, device=DEV)
        out = base.clone()
        ops.gemm_tc(out, a, w, ops.EPILOGUE_ACCUMULATE, status)
        want = base.double() + ref
    else:
        out = torch.empty(T, N, dtype=cdt, device=DEV)
        ops.gemm_tc(out, a, w, ops.EPILOGUE_SWIGLU, status)
        g, u = ref[:, :N], ref[:, N:]
        want = g / (1 + torch.exp(-g)) * u
    tol = dict(rtol=1e-4, atol=1e-4) if cdt == torch.float32 else _tol(cdt)   # sums of thousands of bfloat16 products
    err = (out.double() - want).abs()
    worst = int(err.argmax())
    assert torch.allclose(out.double(), want, **tol), f"max error {float(err.max()):.3e} at {divmod(worst, N)}"
    assert status.tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("T, H, K_in, F, gain_dtype", [
    (8, 2048, 2048, 6144, torch.bfloat16),      # decode: the cluster's fold leaves the norm's input; gate/up through the workspace takes it
    (1, 256, 512, 392, torch.float32),          # one token, few tiles, 32-bit gain
    (40, 1000, 520, 520, torch.bfloat16),       # a last tile of features that is not full
    (300, 256, 512, 392, torch.bfloat16),       # a prompt: tiles of 128 x 128 leave it, the persistent kernel takes it
    (2048, 2048, 6144, 6144, torch.bfloat16),   # the full-size prompt
    (4500, 2048, 2048, 1024, torch.bfloat16)])  # many tokens: the persistent kernel leaves it too
def test_gemm_tcgen05_with_a_norm_folded_in(T, H, K_in, F, gain_dtype):
    """residual += a @ w^T leaves bf16(residual * gain) and the rows' sums of squares behind; the next product (SwiGLU or
    store) applies the row scale 1/rms to its sums.  Against the same products with the norm as a kernel of its own."""
    ops = _ops()
    torch.manual_seed(T + H)
    bf = torch.bfloat16
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    a = torch.randn(T, K_in, device=DEV).to(bf)
    w = (torch.randn(H, K_in, device=DEV) / math.sqrt(K_in)).to(bf)
    wgu = (torch.randn(2 * F, H, device=DEV) / math.sqrt(H)).to(bf)
    gain = (1 + 0.1 * torch.randn(H, device=DEV)).to(gain_dtype)
    res0 = torch.randn(T, H, device=DEV)
    eps = 1e-5
    # the norm as a kernel of its own
    res_ref = res0.clone()
    ops.gemm_tc(res_ref, a, w, ops.EPILOGUE_ACCUMULATE, status)
    x_ref = torch.empty(T, H, dtype=bf, device=DEV)
    ops.rmsnorm(x_ref, res_ref, gain, eps)
    act_ref = torch.empty(T, F, dtype=bf, device=DEV)
    ops.gemm_tc(act_ref, x_ref, wgu, ops.EPILOGUE_SWIGLU, status)
    plain_ref = torch.empty(T, F, device=DEV)
    ops.gemm_tc(plain_ref, x_ref, wgu[:F], ops.EPILOGUE_STORE, status)
    # folded
    tiles = ops.gemm_tc_norm_tiles(T, H, K_in, ops.EPILOGUE_ACCUMULATE)
    assert tiles > 0
    res = res0.clone()
    normed = torch.full((T, H), 7.0, dtype=bf, device=DEV)
    ss = torch.full((T, tiles), -1.0, device=DEV)
    ops.gemm_tc(res, a, w, ops.EPILOGUE_ACCUMULATE, status, norm_after=(normed, gain, ss))
    assert torch.equal(res, res_ref)                                             # the residual itself is what it was
    assert torch.equal(normed, (res * gain.float()).to(bf))                      # its rows times the gain, rounded once
    assert torch.allclose(ss.sum(1).double(), res.double().pow(2).sum(1), rtol=1e-5)
    act = torch.empty(T, F, dtype=bf, device=DEV)
    ops.gemm_tc(act, normed, wgu, ops.EPILOGUE_SWIGLU, status, row_scale=(ss, H, eps))
    plain = torch.empty(T, F, device=DEV)
    ops.gemm_tc(plain, normed, wgu[:F], ops.EPILOGUE_STORE, status, row_scale=(ss, H, eps))
    for got, ref, what in ((act, act_ref, "swiglu"), (plain, plain_ref, "store")):
        diff = (got.float() - ref.float()).abs()
        # the two ways round the activations at different places (x * gain against x * r * gain) and, for SwiGLU, round two
        # factors of the result: independent bfloat16 roundings (2^-9 relative each) of every input and output element
        rms = float(diff.pow(2).mean().sqrt()) / float(ref.float().pow(2).mean().sqrt())
        assert float(diff.max()) <= 3e-2 * float(ref.float().abs().max()), what
        assert rms <= 8e-3, (what, rms)
    assert status.tolist() == [0, 0, 0, 0]
    # what cannot leave a norm's input says so: a product that does not add, and one whose K is folded through the workspace
    assert ops.gemm_tc_norm_tiles(8, 6144, 2048, ops.EPILOGUE_SWIGLU) == 0


def test_gemm_tcgen05_sums_of_squares_do_not_depend_on_the_tile_width():
    """The product that adds into the residual leaves the rows' sums of squares behind in pieces; 300 rows alone and the
    same rows among 1,470 run with tiles of other widths.  The pieces are per 16 features, so the rows' pieces, their
    sums in the consumer and with them the consumer's results are the same bit for bit."""
    ops = _ops()
    torch.manual_seed(0)
    bf = torch.bfloat16
    N = K = 2048
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    x = torch.randn(1470, K, device=DEV).to(bf)
    w = (torch.randn(N, K, device=DEV) * 0.02).to(bf)
    res0 = torch.randn(1470, N, device=DEV)
    gain = (1 + 0.1 * torch.randn(N, device=DEV)).to(bf)
    w2 = (torch.randn(2 * 1024, N, device=DEV) * 0.02).to(bf)
    got = {}
    widths = set()
    for T in (300, 1470):
        widths.add(ops.gemm_tc_describe(T, N, K, ops.EPILOGUE_ACCUMULATE)["tile_width"])
        tiles = ops.gemm_tc_norm_tiles(T, N, K, ops.EPILOGUE_ACCUMULATE)
        assert tiles == N // 16
        res = res0[:T].clone()
        normed = torch.empty(T, N, dtype=bf, device=DEV)
        ss = torch.full((T, tiles), float("nan"), device=DEV)
        ops.gemm_tc(res, x[:T].contiguous(), w, ops.EPILOGUE_ACCUMULATE, status, norm_after=(normed, gain, ss))
        act = torch.empty(T, 1024, dtype=bf, device=DEV)
        ops.gemm_tc(act, normed, w2, ops.EPILOGUE_SWIGLU, status, row_scale=(ss, N, 1e-5))
        got[T] = (res[:300].clone(), normed[:300].clone(), ss[:300].clone(), act[:300].clone())
    assert len(widths) == 2, widths          # the case is about two tile widths
    for a, b in zip(got[300], got[1470]):
        assert torch.equal(a, b)
    assert torch.allclose(got[300][2].sum(1).double(), got[300][0].double().pow(2).sum(1), rtol=1e-5)
    assert status.tolist() == [0, 0, 0, 0]



def test_gemm_tcgen05_refuses_what_it_cannot_take():
    ops = _ops()
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    a = torch.randn(4, 100, device=DEV).to(torch.bfloat16)   # K = 100 is no multiple of 8
    w = torch.randn(16, 100, device=DEV).to(torch.bfloat16)
    out = torch.empty(4, 16, device=DEV)
    assert not ops.gemm_tc_supported(out, a, w, ops.EPILOGUE_STORE)
    with pytest.raises(ops.KernelError):
        ops.gemm_tc(out, a, w, ops.EPILOGUE_STORE, status)
    assert not ops.gemm_tc_supported(out, a.float(), w.float(), ops.EPILOGUE_STORE)   # the 32-bit path never goes here
    from hymt2sharp_b200.parts.linear import matmul
    matmul(out, a, w, ops.EPILOGUE_STORE)   # the general kernel takes it
    assert torch.allclose(out.double(), a.double() @ w.double().T, rtol=2e-5, atol=2e-5)


# (32 heads on one kv head is what the tcgen05 decode kernel refuses and this kernel takes over)
@pytest.mark.parametrize("nh, nkv, d, window", [(16, 4, 128, 0), (8, 2, 64, 0), (6, 2, 64, 300), (5, 5, 128, 0),
                                                (12, 2, 128, 0), (8, 8, 64, 70), (32, 1, 128, 0), (40, 2, 128, 90)])
def test_attention_decode_streaming(nh, nkv, d, window):
    """The bfloat16 decode kernel against the float64 reference, lengths around its chunks of 256
    keys and the cache's blocks of 64, a padding row, and a poisoned cache beyond the lengths."""
    ops = _ops()
    torch.manual_seed(nh + d)
    dtype = torch.bfloat16
    lens = [1, 64, 255, 256, 257, 700, 1025, 90]
    keys = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    vals = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    qs = [torch.randn(1, nh, d, device=DEV).to(dtype) for _ in lens]
    kp, vp, table = _paged(keys, vals, 64, dtype, shuffle_seed=3)   # rows past a length hold 99 / -99
    rows = len(lens)
    q = torch.cat([x.reshape(1, nh * d) for x in qs])
    cu = torch.arange(rows + 1, dtype=torch.int32, device=DEV)
    slots = torch.arange(rows, dtype=torch.int32, device=DEV)
    slots[7] = -1
    kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    splits = -(-max(lens) // 256) + 2   # more chunks than any row needs, as in a captured graph
    na, nm = ops.attention_simt_scratch(rows, nh, d, splits)
    acc = torch.full((na,), float("nan"), device=DEV)
    ml = torch.full((nm,), float("nan"), device=DEV)
    out = torch.full((rows, nh * d), 5.0, dtype=dtype, device=DEV)
    counters = torch.zeros(rows * nh, dtype=torch.int32, device=DEV)
    ops.attention_decode(out, q, kp, vp, table, cu, slots, kv, nh, nkv, d, scale, window, splits, acc, ml, counters)
    assert int(counters.abs().sum()) == 0   # left at zero for the next launch
    ref = torch.cat([_ref_attention(qs[i].float(), keys[i].float(), vals[i].float(), 1, window, scale) for i in range(rows)])
    assert torch.allclose(out[:7].double(), ref[:7], **_tol(dtype))
    assert (out[7] == 5.0).all()   # the padding row is left alone


def test_attention_decode_streaming_with_more_rows_than_the_tensor_core_kernel_takes():
    """600 sequences in one step: beyond the 512 rows of the tcgen05 decode kernel, the engine's choice
    (fast.try_attention) must go to the streaming kernel and give every row its own result."""
    from types import SimpleNamespace
    from hymt2sharp_b200.kernels import fast
    torch.manual_seed(9)
    nh, nkv, d, rows, dtype = 4, 2, 128, 600, torch.bfloat16
    rng = np.random.default_rng(4)
    lens = [int(x) for x in rng.integers(1, 300, rows)]
    keys = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    vals = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    q = torch.randn(rows, nh * d, device=DEV).to(dtype)
    kp, vp, table = _paged(keys, vals, 64, dtype, shuffle_seed=8)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    ctx = SimpleNamespace(decode=True, max_kv_len=max(lens), num_tokens=rows, num_seqs=rows, max_new_tokens=1,
                          cu_seqlens=torch.arange(rows + 1, dtype=torch.int32, device=DEV),
                          slot_ids=torch.arange(rows, dtype=torch.int32, device=DEV), kv_lens=i32(lens))
    out = torch.zeros(rows, nh * d, dtype=dtype, device=DEV)
    before = _ops().launches
    assert fast.try_attention(out, q, kp, vp, table, ctx, nh, nkv, d, 1 / math.sqrt(d), 0)
    assert _ops().launches - before == 1
    for b in range(0, rows, 37):
        ref = _ref_attention(q[b].view(1, nh, d), keys[b], vals[b], 1, 0, 1 / math.sqrt(d))
        assert torch.allclose(out[b:b + 1].double(), ref, **_tol(dtype)), f"row {b}"


@pytest.mark.parametrize("nh, nkv, d, window", [(4, 2, 128, 0), (8, 2, 64, 0), (3, 1, 128, 100), (6, 6, 64, 37)])
def test_attention_prefill_tcgen05(nh, nkv, d, window):
    """The tcgen05 flash-attention kernel against the float64 reference: whole prompts, a piece after
    a long prefix, single rows, lengths around its tiles of 128 queries and 64 keys."""
    ops = _ops()
    torch.manual_seed(nh * 7 + d)
    dtype = torch.bfloat16
    lens, news = [70, 1, 600, 33, 129, 256], [70, 1, 300, 2, 129, 128]
    keys = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    vals = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    qs = [torch.randn(n, nh, d, device=DEV).to(dtype) for n in news]
    kp, vp, table = _paged(keys, vals, 64, dtype, shuffle_seed=5)
    kp[kp == 99.0] = float("nan")    # rows that no sequence wrote
    vp[vp == -99.0] = float("nan")
    scale = 1 / math.sqrt(d)
    q = torch.cat([x.reshape(x.shape[0], nh * d) for x in qs])
    cu = torch.tensor(np.concatenate([[0], np.cumsum(news)]), dtype=torch.int32, device=DEV)
    slots = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    out = torch.full((sum(news), nh * d), 5.0, dtype=dtype, device=DEV)
    ops.attention_prefill_tc(out, q, kp, vp, table, cu, slots, kv, len(lens), max(news), nh, nkv, d, scale, window, status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    ref = torch.cat([_ref_attention(qs[i].float(), keys[i].float(), vals[i].float(), news[i], window, scale)
                     for i in range(len(lens))])
    assert torch.allclose(out.double(), ref, **_tol(dtype))
    # scores far apart (a maximum that rises late by much more than 2^8): the rescale of O in tensor memory
    big_q = [x * 6 for x in qs]
    q2 = torch.cat([x.reshape(x.shape[0], nh * d) for x in big_q])
    ops.attention_prefill_tc(out, q2, kp, vp, table, cu, slots, kv, len(lens), max(news), nh, nkv, d, scale, window, status)
    ref2 = torch.cat([_ref_attention(big_q[i].float(), keys[i].float(), vals[i].float(), news[i], window, scale)
                      for i in range(len(lens))])
    assert torch.allclose(out.double(), ref2, **_tol(dtype))


def test_attention_prefill_tcgen05_with_tens_of_thousands_of_ctas():
    """Eight prompts of 2,048 tokens with 32 heads: 4,096 CTAs of up to 32 key tiles, several times over.  One CTA
    in tens of thousands once waited for ever on a barrier that had run two phases ahead of a thread that was kept
    from running; the status word shows such a wait.  The result is compared with the general kernel."""
    ops = _ops()
    torch.manual_seed(3)
    dtype, nh, nkv, d, B, T = torch.bfloat16, 32, 8, 128, 8, 2048
    keys = [torch.randn(T, nkv, d, device=DEV).to(dtype) for _ in range(B)]
    vals = [torch.randn(T, nkv, d, device=DEV).to(dtype) for _ in range(B)]
    kp, vp, table = _paged(keys, vals, 64, dtype, shuffle_seed=9)
    q = torch.randn(B * T, nh * d, device=DEV).to(dtype)
    cu = (torch.arange(B + 1, dtype=torch.int32, device=DEV) * T).contiguous()
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    kv = torch.full((B,), T, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    out = torch.empty_like(q)
    for _ in range(6):
        ops.attention_prefill_tc(out, q, kp, vp, table, cu, slots, kv, B, T, nh, nkv, d, scale, 0, status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    ref = torch.empty_like(q)
    ops.attention_simt(ref, q, kp, vp, table, cu, slots, kv, B, T, nh, nkv, d, scale)
    assert torch.allclose(out.float(), ref.float(), **_tol(dtype))


def test_attention_decode_tcgen05_more_chunks_than_a_cta_holds():
    """Many long rows: more chunks of 128 keys than the CTAs hold at a time (they go through them in
    rounds), rows beyond 8,192 positions, and one far key that carries all the weight of its row."""
    ops = _ops()
    torch.manual_seed(11)
    dtype, d, nh, nkv = torch.bfloat16, 128, 8, 4
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rows = 40
    lens = [7700 + 13 * i for i in range(rows)]
    lens[3], lens[17] = 8300, 9001
    assert sum(-(-L // 128) for L in lens) * nkv > sms * 64
    keys = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    vals = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    qs = [torch.randn(1, nh, d, device=DEV).to(dtype) for _ in lens]
    # row 5, head 2 (kv head 1): key 37 is the query scaled up, so that it takes all the weight
    keys[5][37, 1] = (qs[5][0, 2].float() * 4).to(dtype)
    kp, vp, table = _paged(keys, vals, 64, dtype, shuffle_seed=9)
    q = torch.cat([x.reshape(1, nh * d) for x in qs])
    slots = torch.arange(rows, dtype=torch.int32, device=DEV)
    kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    splits = -(-max(lens) // 128)
    na, nm, nc = ops.attention_decode_tc_scratch(rows, nh, nkv, d, splits)
    acc = torch.full((na,), float("nan"), device=DEV)
    ml = torch.full((nm,), float("nan"), device=DEV)
    counters = torch.zeros(nc, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    out = torch.full((rows, nh * d), 5.0, dtype=dtype, device=DEV)
    for _ in range(2):
        ops.attention_decode_tc(out, q, kp, vp, table, slots, kv, nh, nkv, d, scale, 0, splits, acc, ml, counters, status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0] and int(counters.abs().sum()) == 0
    ref = torch.cat([_ref_attention(qs[i].float(), keys[i].float(), vals[i].float(), 1, 0, scale) for i in range(rows)])
    assert torch.allclose(out.double(), ref, **_tol(dtype))
    far = out[5].reshape(nh, d)[2].float()
    assert torch.allclose(far, vals[5][37, 1].float(), atol=0.05)


def test_attention_decode_tcgen05_rows_whose_chunks_fall_on_the_same_ctas():
    """Rows of 9 chunks each on a number of CTAs that 9 divides (or shares a divisor with): the chunk that folds a
    row then differs from row to row instead of being the last.  A key in the first chunk and one in the last chunk
    carry all the weight of their rows, so a fold that left a chunk out or took one twice shows."""
    ops = _ops()
    torch.manual_seed(21)
    dtype, d, nh, nkv = torch.bfloat16, 128, 8, 2
    rows = 16
    lens = [1030 + 7 * i for i in range(rows)]
    assert all(-(-L // 128) == 9 for L in lens)
    keys = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    vals = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    qs = [torch.randn(1, nh, d, device=DEV).to(dtype) for _ in lens]
    keys[4][5, 0] = (qs[4][0, 1].float() * 4).to(dtype)               # head 1 reads kv head 0
    keys[11][lens[11] - 2, 1] = (qs[11][0, 6].float() * 4).to(dtype)  # head 6 reads kv head 1
    kp, vp, table = _paged(keys, vals, 64, dtype, shuffle_seed=2)
    q = torch.cat([x.reshape(1, nh * d) for x in qs])
    slots = torch.arange(rows, dtype=torch.int32, device=DEV)
    kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    splits = 9
    na, nm, nc = ops.attention_decode_tc_scratch(rows, nh, nkv, d, splits)
    acc = torch.full((na,), float("nan"), device=DEV)
    ml = torch.full((nm,), float("nan"), device=DEV)
    counters = torch.zeros(nc, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    out = torch.full((rows, nh * d), 5.0, dtype=dtype, device=DEV)
    for _ in range(3):
        ops.attention_decode_tc(out, q, kp, vp, table, slots, kv, nh, nkv, d, scale, 0, splits, acc, ml, counters, status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0] and int(counters.abs().sum()) == 0
    ref = torch.cat([_ref_attention(qs[i].float(), keys[i].float(), vals[i].float(), 1, 0, scale) for i in range(rows)])
    assert torch.allclose(out.double(), ref, **_tol(dtype))
    assert torch.allclose(out[4].reshape(nh, d)[1].float(), vals[4][5, 0].float(), atol=0.05)
    assert torch.allclose(out[11].reshape(nh, d)[6].float(), vals[11][lens[11] - 2, 1].float(), atol=0.05)


@pytest.mark.parametrize("nh, nkv, window", [(16, 4, 0), (4, 4, 0), (32, 2, 0), (6, 2, 300), (10, 2, 70)])
def test_attention_decode_tcgen05(nh, nkv, window):
    """The tensor-core decode kernel (keys on the 128-row side, head_dim 128) against the float64
    reference: lengths around its chunks of 128 keys and the cache's blocks of 64, a padding row,
    and NaN in every cache row that no sequence has written."""
    ops = _ops()
    torch.manual_seed(nh)
    dtype, d = torch.bfloat16, 128
    lens = [1, 64, 65, 127, 128, 129, 700, 1025, 90]
    keys = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    vals = [torch.randn(L, nkv, d, device=DEV).to(dtype) for L in lens]
    qs = [torch.randn(1, nh, d, device=DEV).to(dtype) for _ in lens]
    kp, vp, table = _paged(keys, vals, 64, dtype, shuffle_seed=4)
    kp[kp == 99.0] = float("nan")    # rows that no sequence wrote
    vp[vp == -99.0] = float("nan")
    rows = len(lens)
    q = torch.cat([x.reshape(1, nh * d) for x in qs])
    slots = torch.arange(rows, dtype=torch.int32, device=DEV)
    slots[8] = -1
    kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    splits = -(-max(lens) // 128) + 2
    na, nm, nc = ops.attention_decode_tc_scratch(rows, nh, nkv, d, splits)
    acc = torch.full((na,), float("nan"), device=DEV)
    ml = torch.full((nm,), float("nan"), device=DEV)
    counters = torch.zeros(nc, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    out = torch.full((rows, nh * d), 5.0, dtype=dtype, device=DEV)
    for _ in range(2):   # twice: the counters are left at zero
        ops.attention_decode_tc(out, q, kp, vp, table, slots, kv, nh, nkv, d, scale, window, splits, acc, ml, counters, status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0] and int(counters.abs().sum()) == 0
    ref = torch.cat([_ref_attention(qs[i].float(), keys[i].float(), vals[i].float(), 1, window, scale) for i in range(rows)])
    assert torch.isfinite(out[:8].float()).all()
    assert torch.allclose(out[:8].double(), ref[:8], **_tol(dtype))
    assert (out[8] == 5.0).all()
