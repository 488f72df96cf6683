"""Each kernel alone against a plain PyTorch float32 statement of the same operation, at sizes other
than the engine's tiny models use (GPU)."""
import math
import random

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    from lucciola_b200 import ops
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    return ops, dev, torch.cuda.current_stream().cuda_stream


def rel(a, b):
    return ((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30)).item()


# ---- embedding ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [6, 100, 1030])
def test_embedding(env, dtype, hidden):
    ops, dev, st = env
    table = torch.randn(77, hidden, device=dev).to(dtype)
    ids = torch.tensor([0, 76, 5, 5, 33], dtype=torch.int32, device=dev)
    out = torch.empty(5, hidden, device=dev)
    ops.embedding(out, ids, table, st)
    assert torch.equal(out, table.float()[ids.long()])


# ---- residual add + RMSNorm ------------------------------------------------------------------------------
@pytest.mark.parametrize("hidden,eps", [(7, 1e-5), (100, 1e-6), (4100, 3e-3), (1024, 1e-6), (4096, 1e-6), (8192, 1e-5), (5120, 1e-6), (2560, 1e-6), (16384, 1e-6)])   # from 1024 on: rows held in registers
@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(env, hidden, eps, act):
    ops, dev, st = env
    T = 9
    res = torch.randn(T, hidden, device=dev) * 3
    delta = (torch.randn(T, hidden, device=dev)).to(act)
    w = 1 + 0.3 * torch.randn(hidden, device=dev)
    want_res = res + delta.float()
    want = plain.rms_norm(want_res.double(), w.double(), eps)
    r = res.clone()
    out = torch.empty(T, hidden, device=dev, dtype=act)
    ops.add_rmsnorm(out, r, delta, w, eps, st)
    assert torch.equal(r, want_res)                                   # the residual stream is updated in 32-bit
    assert rel(out, want) < (1e-6 if act == torch.float32 else 5e-3)
    # without a delta the residual stays and the norm is of the residual
    r2 = res.clone()
    ops.add_rmsnorm(out, r2, None, w, eps, st)
    assert torch.equal(r2, res) and rel(out, plain.rms_norm(res.double(), w.double(), eps)) < (1e-6 if act == torch.float32 else 5e-3)
    # on chosen rows: nothing is written back, the sum is formed on the fly
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=dev)
    r3 = res.clone()
    out3 = torch.empty(3, hidden, device=dev, dtype=act)
    ops.add_rmsnorm(out3, r3, delta, w, eps, st, rows=rows)
    assert torch.equal(r3, res) and rel(out3, want[rows.long()]) < (1e-6 if act == torch.float32 else 5e-3)


# ---- q/k norm + rotation + cache write ---------------------------------------------------------------------
def paged_setup(dev, seqs, nkv, d, ps, dtype, seed=0, fill=float("nan")):
    """seqs: (cached tokens, new tokens) per request.  Returns pools filled with `fill`, a shuffled block
    table, positions and the request index of each new token."""
    rnd = random.Random(seed)
    S = len(seqs)
    maxlen = max(s + n for s, n in seqs)
    P = -(-maxlen // ps) + 1
    npages = sum(-(-(s + n) // ps) for s, n in seqs) + 2
    perm = list(range(npages)); rnd.shuffle(perm)
    bt = torch.full((S, P), -1, dtype=torch.int32)
    pi = 0
    pos, seq = [], []
    for i, (s0, n) in enumerate(seqs):
        for j in range(-(-(s0 + n) // ps)):
            bt[i, j] = perm[pi]; pi += 1
        pos += list(range(s0, s0 + n)); seq += [i] * n
    kc = torch.full((npages, nkv, ps, d), fill, device=dev, dtype=dtype)
    vc = kc.clone()
    return kc, vc, bt.to(dev), torch.tensor(pos, dtype=torch.int32, device=dev), torch.tensor(seq, dtype=torch.int32, device=dev)


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,ps,theta", [(3, 1, 24, 4, 1e4), (8, 2, 64, 16, 5e5), (2, 2, 144, 32, 1e6), (6, 3, 128, 16, 1e6),
                                               (2, 1, 256, 8, 3e4)])
def test_rope_kv(env, act, nq, nkv, d, ps, theta):
    ops, dev, st = env
    seqs = [(0, 7), (37, 1), (1021, 3)]
    kc, vc, bt, pos, seq = paged_setup(dev, seqs, nkv, d, ps, act)
    T = pos.shape[0]
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=dev).to(act)
    qw, kw = 1 + 0.2 * torch.randn(d, device=dev), 1 + 0.2 * torch.randn(d, device=dev)
    eps = 1e-5
    inv = (1.0 / torch.pow(torch.tensor(theta), torch.arange(0, d, 2, dtype=torch.float32) / d)).to(dev)
    q_out = torch.empty(T, nq, d, device=dev, dtype=act)
    a, b = nq * d, (nq + nkv) * d
    ops.rope_kv(qkv[:, :a], qkv[:, a:b], qkv[:, b:], q_out, pos, nq, nkv, d, eps, st, q_norm_w=qw, k_norm_w=kw,
                inv_freq=inv, rot_dim=d, k_cache=kc, v_cache=vc, token_seq=seq, block_table=bt, page_size=ps)
    x = qkv.double().cpu()
    p = pos.cpu().tolist()
    q_ref = plain.rope(plain.rms_norm(x[:, :a].reshape(T, nq, d), qw.double().cpu(), eps), p, theta)
    k_ref = plain.rope(plain.rms_norm(x[:, a:b].reshape(T, nkv, d), kw.double().cpu(), eps), p, theta)
    v_ref = x[:, b:].reshape(T, nkv, d)
    tol = 2e-6 if act == torch.float32 else 6e-3
    assert rel(q_out.cpu(), q_ref) < tol
    btc, seqc = bt.cpu(), seq.cpu().tolist()
    written = torch.zeros(kc.shape[0], ps, dtype=torch.bool)
    for t in range(T):
        page, slot = int(btc[seqc[t], p[t] // ps]), p[t] % ps
        written[page, slot] = True
        assert rel(kc[page, :, slot].cpu(), k_ref[t]) < tol
        assert torch.equal(vc[page, :, slot].cpu().double(), v_ref[t])          # values are copied unchanged
    untouched = kc.cpu().float().permute(0, 2, 1, 3)[~written]
    assert torch.isnan(untouched).all()                                         # no other slot was written


@pytest.mark.parametrize("nq,nkv,ps,K,seqs,norm,rotate", [
    (8, 2, 16, 1024, [(0, 1), (37, 1), (1021, 1), (5, 1), (300, 1)], True, True),      # decoded tokens of five requests
    (4, 4, 8, 512, [(0, 7), (100, 3)], True, True),                                    # short portions
    (32, 8, 16, 4096, [(i * 11, 1) for i in range(8)], True, True),                    # the real head counts and width
    (6, 1, 32, 512, [(9, 30)], False, True), (2, 2, 64, 640, [(0, 20), (63, 2)], True, False),
    (3, 1, 16, 2048, [(0, 32)], True, True),                                           # the most tokens it takes
])
@pytest.mark.parametrize("scaled", [False, True])
def test_gemm_tcgen05_with_head_epilogue(env, nq, nkv, ps, K, seqs, norm, rotate, scaled):
    """The q|k|v product that finishes the heads itself against product, norm, rotation and cache write done plainly;
    `scaled`: its input rows lack a factor each, given as partial sums of squares, which the epilogue applies."""
    ops, dev, st = env
    d, theta, eps = 128, 1e6, 1e-6
    kc, vc, bt, pos, seq = paged_setup(dev, seqs, nkv, d, ps, torch.bfloat16)
    T = pos.shape[0]
    x = torch.randn(T, K, device=dev).bfloat16()
    w = (torch.randn((nq + 2 * nkv) * d, K, device=dev) / math.sqrt(K)).bfloat16()
    qw = (1 + 0.2 * torch.randn(d, device=dev)) if norm else None
    kw = (1 + 0.2 * torch.randn(d, device=dev)) if norm else None
    inv = (1.0 / torch.pow(torch.tensor(theta), torch.arange(0, d, 2, dtype=torch.float32) / d)).to(dev) if rotate else None
    assert ops.gemm_tcgen05_heads_ok(x, w, d, d if rotate else None)
    q_out = torch.full((T, nq, d), float("nan"), device=dev, dtype=torch.bfloat16)
    sumsq, row_eps, factor = None, 0.0, torch.ones(T, 1, dtype=torch.float64)
    if scaled:
        sumsq = (torch.rand(T, 5, device=dev) * K * 3).float()
        row_eps = 1e-3
        factor = torch.rsqrt(sumsq.double().sum(dim=1, keepdim=True) / K + row_eps).cpu()
    ops.gemm_tcgen05_heads(x, w, q_out, pos, seq, bt, kc, vc, nq, nkv, ps, eps, st, q_norm_w=qw, k_norm_w=kw, inv_freq=inv,
                           sumsq=sumsq, row_eps=row_eps)
    torch.cuda.synchronize()
    assert ops.device_error() == 0
    y = (x.double() @ w.double().t()).cpu() * factor
    a, b = nq * d, (nq + nkv) * d
    p = pos.cpu().tolist()
    q_ref, k_ref, v_ref = y[:, :a].reshape(T, nq, d), y[:, a:b].reshape(T, nkv, d), y[:, b:].reshape(T, nkv, d)
    if norm:
        q_ref, k_ref = plain.rms_norm(q_ref, qw.double().cpu(), eps), plain.rms_norm(k_ref, kw.double().cpu(), eps)
    if rotate:
        q_ref, k_ref = plain.rope(q_ref, p, theta), plain.rope(k_ref, p, theta)
    assert rel(q_out.cpu(), q_ref) < 6e-3
    btc, seqc = bt.cpu(), seq.cpu().tolist()
    written = torch.zeros(kc.shape[0], ps, dtype=torch.bool)
    for t in range(T):
        page, slot = int(btc[seqc[t], p[t] // ps]), p[t] % ps
        written[page, slot] = True
        assert rel(kc[page, :, slot].cpu(), k_ref[t]) < 6e-3 and rel(vc[page, :, slot].cpu(), v_ref[t]) < 6e-3
    assert torch.isnan(kc.cpu().float().permute(0, 2, 1, 3)[~written]).all()      # no other slot was written
    assert torch.isnan(vc.cpu().float().permute(0, 2, 1, 3)[~written]).all()
    # what it does not take: other head sizes, a rotation of part of the head, more than 32 tokens
    assert not ops.gemm_tcgen05_heads_ok(x, w, 64, 64) and not ops.gemm_tcgen05_heads_ok(x, w, d, 64)
    assert not ops.gemm_tcgen05_heads_ok(torch.empty(33, K, device=dev, dtype=torch.bfloat16), w, d, d)
    assert not ops.gemm_tcgen05_heads_ok(x[:, :192], w[:, :192].contiguous(), d, d)          # too short a k to split


# ---- attention ------------------------------------------------------------------------------------------------
def attention_reference(q, kc, vc, bt, pos, seq, nq, nkv, ps, window, scale):
    """Plain float64 attention of each query over the keys its request holds in the pages."""
    T, _, d = q.shape
    out = torch.zeros(T, nq, d, dtype=torch.float64)
    kcd, vcd, btc = kc.double().cpu(), vc.double().cpu(), bt.cpu()
    qd = q.double().cpu()
    for t in range(T):
        s, p = int(seq[t]), int(pos[t])
        lo = max(0, p - window + 1) if window else 0
        idx = list(range(lo, p + 1))
        k = torch.stack([kcd[int(btc[s, j // ps]), :, j % ps] for j in idx])        # [n, nkv, d]
        v = torch.stack([vcd[int(btc[s, j // ps]), :, j % ps] for j in idx])
        out[t] = plain.attention(qd[t:t + 1], k, v, [p], idx, scale, window)[0]
    return out


def fill_pages(kc, vc, bt, seqs, ps, seed=0, k_scale=1.0):
    g = torch.Generator().manual_seed(seed)
    nkv, d = kc.shape[1], kc.shape[3]
    for i, (s0, n) in enumerate(seqs):
        L = s0 + n
        k = torch.randn(L, nkv, d, generator=g) * k_scale
        v = torch.randn(L, nkv, d, generator=g)
        for j in range(L):
            kc[int(bt[i, j // ps]), :, j % ps] = k[j].to(kc.dtype).to(kc.device)
            vc[int(bt[i, j // ps]), :, j % ps] = v[j].to(vc.dtype).to(vc.device)


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,ps,window,seqs", [
    (6, 2, 24, 4, 0, [(0, 9), (30, 1), (5, 6)]),
    (4, 4, 72, 16, 11, [(0, 40), (100, 2)]),
    (8, 1, 160, 32, 0, [(63, 1), (64, 1), (0, 65)]),
])
def test_attention_plain(env, act, nq, nkv, d, ps, window, seqs):
    ops, dev, st = env
    kc, vc, bt, pos, seq = paged_setup(dev, seqs, nkv, d, ps, act)
    fill_pages(kc, vc, bt.cpu(), seqs, ps)
    q = torch.randn(pos.shape[0], nq, d, device=dev).to(act)
    out = torch.empty_like(q)
    ops.attention_plain(q, out, kc, vc, pos, seq, bt, nq, nkv, d, ps, window, 0.2, st)
    ref = attention_reference(q, kc, vc, bt, pos.cpu(), seq.cpu(), nq, nkv, ps, window, 0.2)
    assert torch.isfinite(out).all()                              # unused slots hold NaN and must not be read
    assert rel(out.cpu(), ref) < (3e-6 if act == torch.float32 else 6e-3)


def run_flash(ops, dev, st, nq, nkv, d, ps, window, seqs, splits=None, scale=None, k_scale=1.0, q=None, hook=None, tma=True):
    """splits < 0: that many key ranges, combined through the workspace even where a cluster could.  tma=False: decoded
    tokens, too, in the kernel that fetches with 16-byte copies."""
    kc, vc, bt, pos, seq = paged_setup(dev, seqs, nkv, d, ps, torch.bfloat16)
    fill_pages(kc, vc, bt.cpu(), seqs, ps, k_scale=k_scale)
    if hook:
        hook(kc, vc, bt.cpu())
    T = pos.shape[0]
    q = torch.randn(T, nq, d, device=dev).bfloat16() if q is None else q
    G, per = nq // nkv, 64 // (nq // nkv)
    tiles, t = [], 0
    for i, (_, n) in enumerate(seqs):
        for off in range(0, n, per):
            tiles.append((t + off, min(per, n - off), i, 0))
        t += n
    tl = torch.tensor(tiles, dtype=torch.int32, device=dev)
    scale = scale if scale is not None else 1 / math.sqrt(d)
    out = torch.full_like(q, float("nan"))
    rows = min(64, max(n for _, n, _, _ in tiles) * G)
    sp = abs(splits) if splits else ops.attention_splits(len(tiles), nkv, max(s + n for s, n in seqs), rows)
    ops.attention_flash(q, out, kc, vc, pos, bt, tl, rows, nq, nkv, d, ps, window, scale, sp, st,
                        force_workspace=bool(splits and splits < 0), tma=tma)
    torch.cuda.synchronize()
    assert ops.device_error() == 0
    ref = attention_reference(q, kc, vc, bt, pos.cpu(), seq.cpu(), nq, nkv, ps, window, scale)
    return out, ref


@pytest.mark.parametrize("nq,nkv,d,ps,window,seqs,splits", [
    (4, 2, 64, 16, 0, [(0, 5)], None),
    (8, 2, 128, 16, 0, [(0, 130), (37, 1), (0, 3)], None),
    (32, 8, 128, 16, 0, [(1000, 1), (17, 1), (2047, 1)], 8),
    (32, 8, 128, 16, 0, [(1000, 1), (17, 1), (2047, 1)], -8),
    (16, 8, 96, 16, 0, [(700, 1), (5, 1)], 4),
    (8, 2, 128, 8, 0, [(3000, 1)], 24),
    (4, 1, 64, 16, 100, [(500, 3), (90, 2)], 2),
    (8, 2, 128, 8, 77, [(1000, 1), (30, 1), (76, 1), (77, 1)], 4),      # a window that starts inside a page and a stage
    (32, 8, 128, 64, 0, [(63, 1), (64, 1), (65, 1), (700, 1)], None),   # a page as large as a stage
    (4, 4, 64, 32, 0, [(3999, 1)], 16),
    (6, 2, 48, 8, 0, [(5, 40), (63, 2)], None),
    (8, 1, 32, 8, 0, [(0, 100), (99, 1)], 2),
    (5, 5, 16, 16, 24, [(0, 33), (200, 7)], None),
    (4, 4, 80, 32, 64, [(300, 50)], 3),
    (3, 1, 104, 64, 0, [(0, 64), (64, 64), (127, 1)], None),
    (64, 1, 64, 16, 0, [(10, 3)], None),
    (4, 2, 48, 8, 0, [(300, 1), (17, 2)], 2),                           # decoded tokens with heads narrower than a TMA box
    (2, 2, 16, 16, 0, [(100, 1), (15, 1), (16, 1)], None),              # rows of 32 bytes
    (8, 2, 128, 128, 0, [(1000, 1), (130, 3), (127, 1), (128, 1)], 4),  # pages of two stages
    (8, 2, 112, 32, 50, [(1000, 2), (49, 1), (50, 1), (51, 1)], 2),     # a window over decoded tokens, head of 112
    (12, 4, 128, 16, 0, [(5000, 1)], 3),                                # three ranges: through the workspace
    (32, 8, 128, 16, 0, [(8191, 1)], 16),                               # sixteen ranges: one cluster of 16 a kv head
    (16, 2, 64, 32, 300, [(6000, 1), (5000, 2)], 16),
])
@pytest.mark.parametrize("tma", [True, False])
def test_attention_flash(env, nq, nkv, d, ps, window, seqs, splits, tma):
    ops, dev, st = env
    out, ref = run_flash(ops, dev, st, nq, nkv, d, ps, window, seqs, splits, tma=tma)
    assert torch.isfinite(out).all()
    assert rel(out.cpu(), ref) < 8e-3


def run_tc(ops, dev, st, nq, nkv, ps, window, seqs, hook=None, q=None, rows=256, splits=1):
    """The tensor-memory kernel for portions of prompts (head size 128) against the float64 statement; work items
    of up to `rows` query rows (256: two tiles in a CTA, 128: one), their keys cut into `splits` ranges (the workspace
    of the partial results holds NaN before: what a range did not write must not be read)."""
    d = 128
    kc, vc, bt, pos, seq = paged_setup(dev, seqs, nkv, d, ps, torch.bfloat16)
    fill_pages(kc, vc, bt.cpu(), seqs, ps)
    if hook:
        hook(kc, vc, bt.cpu())
    T = pos.shape[0]
    q = torch.randn(T, nq, d, device=dev).bfloat16() if q is None else q
    per = (rows // 128) * (128 // (nq // nkv))
    tiles, t = [], 0
    for i, (_, n) in enumerate(seqs):
        for off in range(0, n, per):
            tiles.append((t + off, min(per, n - off), i, 0))
        t += n
    tl = torch.tensor(tiles, dtype=torch.int32, device=dev)
    out = torch.full_like(q, float("nan"))
    if splits > 1:
        ops._attention_workspace(dev, len(tiles) * nkv * splits * 256 * (d + 2)).fill_(float("nan"))
    ops.attention_tcgen05(q, out, kc, vc, pos, bt, tl, nq, nkv, d, ps, window, 1 / math.sqrt(d), st, key_splits=splits)
    torch.cuda.synchronize()
    assert ops.device_error() == 0
    ref = attention_reference(q, kc, vc, bt, pos.cpu(), seq.cpu(), nq, nkv, ps, window, 1 / math.sqrt(d))
    return out, ref


@pytest.mark.parametrize("nq,nkv,ps,window,seqs", [
    (4, 1, 16, 0, [(0, 32)]),                       # one tile, one block, a quarter of the rows
    (4, 1, 16, 0, [(0, 128)]),                      # several tiles, the diagonal block only
    (32, 8, 16, 0, [(0, 300), (100, 17), (0, 1)]),  # the real head counts; a portion behind cached tokens; one token
    (8, 8, 8, 0, [(50, 70)]),                       # no grouping, pages of 8
    (4, 2, 32, 64, [(500, 100)]),                   # a window that leaves whole blocks and pages out
    (2, 2, 128, 0, [(0, 130)]),                     # a page as large as a block
    (16, 1, 64, 0, [(0, 40), (1000, 9)]),           # sixteen heads on one kv head; nine tokens after a thousand
    (8, 2, 16, 200, [(0, 700)]),                    # a window inside a long portion
    (40, 8, 16, 0, [(0, 260), (77, 30)]),           # five heads per kv head: tiles of 25 tokens, three rows unused
    (6, 2, 32, 90, [(10, 300)]), (7, 1, 16, 0, [(0, 150)]),      # three and seven heads per kv head
])
@pytest.mark.parametrize("rows", [256, 128])
def test_attention_tcgen05(env, nq, nkv, ps, window, seqs, rows):
    ops, dev, st = env
    out, ref = run_tc(ops, dev, st, nq, nkv, ps, window, seqs, rows=rows)
    assert torch.isfinite(out).all()                # unused slots and freed pages hold NaN and must not reach a sum
    assert rel(out.cpu(), ref) < 8e-3


@pytest.mark.parametrize("nq,nkv,ps,window,seqs", [
    (4, 1, 16, 0, [(0, 32)]),                       # one block: all ranges but one are empty
    (32, 8, 16, 0, [(0, 300), (100, 17), (0, 1)]),  # items of five, two and one blocks
    (32, 8, 16, 0, [(3000, 64), (1500, 40)]),       # portions behind long contexts, what the split is for
    (40, 8, 16, 0, [(2000, 100), (77, 30)]),        # five heads per kv head: rows of a tile unused
    (4, 2, 32, 64, [(500, 100)]),                   # a window: the ranges begin at its first block
    (2, 2, 128, 0, [(1000, 130)]),                  # a page of two blocks that a range's edge cuts
    (8, 2, 16, 200, [(0, 700)]),                    # rows that see no key of the later ranges
])
@pytest.mark.parametrize("splits", [2, 3, 8])
def test_attention_tcgen05_key_ranges(env, nq, nkv, ps, window, seqs, splits):
    ops, dev, st = env
    out, ref = run_tc(ops, dev, st, nq, nkv, ps, window, seqs, splits=splits)
    assert torch.isfinite(out).all()
    assert rel(out.cpu(), ref) < 8e-3


def test_attention_tcgen05_key_ranges_far_key_and_spike(env):
    """One key in the first range carries nearly all the weight of the last query, whose other ranges hold ordinary
    keys: the combination must weigh the ranges by their reference values, not add them up."""
    ops, dev, st = env
    nq, nkv, ps = 8, 2, 16
    q = torch.randn(1200, nq, 128, device=dev).bfloat16()

    def far(kc, vc, bt):
        for kvh in range(nkv):
            kc[int(bt[0, 1]), kvh, 3] = (q[-1, kvh * 4].float() * 3).bfloat16()      # key 19
            vc[int(bt[0, 1]), kvh, 3] = 7.0

    for splits in (2, 5):
        out, ref = run_tc(ops, dev, st, nq, nkv, ps, 0, [(0, 1200)], hook=far, q=q, splits=splits)
        assert rel(out.cpu(), ref) < 8e-3 and (out[-1, 0].float() - 7.0).abs().max() < 0.2


@pytest.mark.parametrize("order", ["growing", "shrinking", "late spike"])
def test_attention_tcgen05_moving_maximum(env, order):
    """The row's reference value moves only when the maximum has grown by 2^8: keys whose scores grow from block to
    block (many rescalings of O), shrink (none after the first block), or jump once at the end."""
    ops, dev, st = env
    nq, nkv, ps, n = 8, 2, 16, 1000

    def hook(kc, vc, bt):
        for j in range(n):
            if order == "growing":
                f = 0.2 + 6.0 * j / n
            elif order == "shrinking":
                f = 6.2 - 6.0 * j / n
            else:
                f = 8.0 if j >= n - 3 else 0.3
            page, slot = int(bt[0, j // ps]), j % ps
            kc[page, :, slot] = (kc[page, :, slot].float() * f).bfloat16()

    out, ref = run_tc(ops, dev, st, nq, nkv, ps, 0, [(0, n)], hook=hook)
    assert torch.isfinite(out).all()
    assert rel(out.cpu(), ref) < 8e-3


def test_attention_tcgen05_window_edge_and_far_key(env):
    ops, dev, st = env
    nq, nkv, ps = 8, 2, 16
    for window in (16, 17, 128, 129):
        pos_q = 400

        def hook(kc, vc, bt):
            j = pos_q - window                               # the last key that must NOT be seen by the query at pos_q
            vc[int(bt[0, j // ps]), :, j % ps] = 1000.0

        out, ref = run_tc(ops, dev, st, nq, nkv, ps, window, [(pos_q - 40, 41)], hook=hook)
        assert rel(out.cpu(), ref) < 8e-3 and out[-1].float().abs().max() < 50
    # one far key carries nearly all the weight of the last query
    q = torch.randn(300, nq, 128, device=dev).bfloat16()

    def far(kc, vc, bt):
        for kvh in range(nkv):
            kc[int(bt[0, 1]), kvh, 3] = (q[-1, kvh * 4].float() * 3).bfloat16()      # key 19
            vc[int(bt[0, 1]), kvh, 3] = 7.0

    out, ref = run_tc(ops, dev, st, nq, nkv, ps, 0, [(0, 300)], hook=far, q=q)
    assert rel(out.cpu(), ref) < 8e-3 and (out[-1, 0].float() - 7.0).abs().max() < 0.2


def test_attention_tcgen05_refuses_other_sizes(env):
    ops, dev, st = env
    q = torch.zeros(4, 4, 64, device=dev, dtype=torch.bfloat16)
    assert not ops.attention_tcgen05_ok(q, 4, 2, 64, 16)           # head size
    q = torch.zeros(4, 6, 128, device=dev, dtype=torch.bfloat16)
    assert ops.attention_tcgen05_ok(q, 6, 2, 128, 16)              # three heads per kv head: tiles of 42 tokens
    assert not ops.attention_tcgen05_ok(q, 258, 2, 128, 16)        # more than 128 heads per kv head
    assert not ops.attention_tcgen05_ok(q, 6, 6, 128, 24)          # page size
    assert ops.attention_tcgen05_ok(q, 6, 6, 128, 16)


def test_attention_flash_finds_a_far_key_among_hundreds(env):
    """Random keys make every score alike, so a key that is skipped changes little.  Here one key far back
    (at a page's first slot, in another split than the query) is made to carry nearly all the weight."""
    ops, dev, st = env
    nq, nkv, d, ps = 8, 2, 128, 16
    L, far = 900, 16 * 13                                      # first slot of page 13
    q = torch.randn(1, nq, d, device=dev).bfloat16()
    marks = {}

    def hook(kc, vc, bt):
        page, slot = int(bt[0, far // ps]), far % ps
        for kvh in range(nkv):
            kc[page, kvh, slot] = (q[0, kvh * 4].float() * 3).bfloat16()     # aligned with query head kvh*4
            vc[page, kvh, slot] = 7.0
        marks["v"] = vc[page, :, slot].clone()

    for splits, tma in ((1, True), (4, True), (-4, True), (7, True), (1, False), (4, False), (-4, False), (7, False)):
        out, ref = run_flash(ops, dev, st, nq, nkv, d, ps, 0, [(L - 1, 1)], splits, k_scale=0.05, q=q, hook=hook, tma=tma)
        assert rel(out.cpu(), ref) < 8e-3
        assert (out[0, 0].float() - 7.0).abs().max() < 0.1 and (out[0, 4].float() - 7.0).abs().max() < 0.1


@pytest.mark.parametrize("tma", [True, False])
@pytest.mark.parametrize("window", [1, 16, 17, 63, 64, 65])
def test_attention_flash_window_edge(env, window, tma):
    """The key just outside the window carries a huge value: if the edge is off by one it shows."""
    ops, dev, st = env
    nq, nkv, d, ps = 2, 1, 64, 16
    pos_q = 200

    def hook(kc, vc, bt):
        j = pos_q - window                                       # the last key that must NOT be seen
        vc[int(bt[0, j // ps]), :, j % ps] = 1000.0
        j = pos_q - window + 1                                   # the first key that must be seen
        vc[int(bt[0, j // ps]), :, j % ps] = -5.0

    out, ref = run_flash(ops, dev, st, nq, nkv, d, ps, window, [(pos_q, 1)], 1, hook=hook, tma=tma)
    assert out.float().abs().max() < 50 and rel(out.cpu(), ref) < 8e-3
    out, ref = run_flash(ops, dev, st, nq, nkv, d, ps, window, [(pos_q - 30, 31)], 1, hook=hook, tma=tma)
    assert rel(out.cpu(), ref) < 8e-3


# ---- SwiGLU ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("act,inter", [(torch.float32, 37), (torch.bfloat16, 37), (torch.bfloat16, 1000)])
def test_swiglu(env, act, inter):
    ops, dev, st = env
    gu = (torch.randn(5, 2 * inter, device=dev) * 3).to(act)
    out = torch.empty(5, inter, device=dev, dtype=act)
    ops.swiglu(out, gu[:, :inter], gu[:, inter:], st)
    want = plain.swiglu(gu[:, :inter].double(), gu[:, inter:].double())
    assert rel(out, want) < (1e-6 if act == torch.float32 else 5e-3)


# ---- matrix products --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (3, 70, 33), (65, 129, 100), (200, 64, 17)])
@pytest.mark.parametrize("tx,tw,ty", [(torch.float32,) * 3, (torch.bfloat16,) * 3, (torch.bfloat16, torch.float32, torch.float32)])
def test_gemm_plain(env, M, N, K, tx, tw, ty):
    ops, dev, st = env
    x, w = torch.randn(M, K, device=dev).to(tx), torch.randn(N, K, device=dev).to(tw)
    y = torch.empty(M, N, device=dev, dtype=ty)
    ops.gemm_plain(y, x, w, st)
    assert rel(y, x.double() @ w.double().t()) < (2e-6 if ty == torch.float32 else 5e-3)


def test_gemm_plain_is_true_32_bit(env):
    """No reduced-precision matrix mode: a product that needs all 24 bits of the inputs comes out right."""
    ops, dev, st = env
    x = torch.full((4, 8), 1.0 + 2.0 ** -20, device=dev)
    w = torch.full((4, 8), 1.0 + 2.0 ** -19, device=dev)
    y = torch.empty(4, 4, device=dev)
    ops.gemm_plain(y, x, w, st)
    exact = 8 * (1 + 2.0 ** -20) * (1 + 2.0 ** -19)
    assert abs(y[0, 0].item() - exact) < 2e-6 and abs(y[0, 0].item() - 8.0) > 1e-5     # tf32 would give 8.0


@pytest.mark.parametrize("M,N,K,bt,splits", [
    (16, 128, 64, 16, 1), (5, 100, 96, 0, 0), (1, 503, 96, 0, 0), (16, 128, 1024, 16, 4), (33, 384, 520, 64, 3),
    (128, 256, 512, 128, 1), (300, 1000, 776, 0, 0), (256, 384, 1024, 256, 1), (7, 1536, 2048, 0, 0), (70, 200, 4096, 0, 0),
    # splits > 0: through a cluster when the count is a power of two up to 8; < 0: through the workspace
    (16, 128, 1024, 16, -4), (9, 300, 2048, 16, 8), (40, 520, 1024, 64, 2), (100, 256, 4096, 128, 8), (64, 4096, 512, 64, -2),
    (200, 384, 2048, 256, 4), (3, 130, 8192, 16, 16),
    # more than 256 tokens: the persistent kernel (tokens on the lanes, two accumulators)
    (2048, 512, 4096, 0, 0), (1000, 300, 136, 0, 0), (257, 6144, 64, 0, 0), (5000, 260, 520, 0, 0), (640, 1030, 1024, 0, 0),
    # the same with a given feature width of the tiles (here `splits` stands for it): narrow, odd multiples of 16, the widest
    (2048, 512, 4096, 0, 128), (384, 4096, 1024, 0, 144), (1000, 300, 136, 0, 64), (640, 1030, 1024, 0, 240), (512, 4096, 512, 0, 16),
    (576, 4096, 1024, 0, 0), (512, 1000, 2048, 0, 256),
    # columns of tiles 256 wide, then narrower tiles for the rest of the features (-(columns * 1024 + width)); the last two
    # are sizes for which the kernel chooses such a plan itself
    (2048, 4096, 256, 0, -(9 * 1024 + 208)), (1024, 1030, 512, 0, -(2 * 1024 + 64)), (512, 700, 256, 0, -(0 * 1024 + 176)),
    (300, 2000, 128, 0, -(7 * 1024 + 16)), (2048, 6144, 128, 0, 0), (2048, 4096, 192, 0, 0),
    # pairs of CTAs on tiles of 256 tokens (bt -2; -1: one CTA a tile of 128 tokens): a token count that leaves the second
    # CTA of the last pair without tokens, partial tiles in both directions, given widths, the sizes that choose pairs themselves
    (512, 256, 64, -2, 0), (300, 1000, 136, -2, 0), (1000, 300, 520, -2, 64), (640, 1030, 1024, -2, 224),
    (2048, 4096, 256, -2, -(9 * 1024 + 192)), (1300, 520, 4096, -2, 0), (1024, 6144, 512, 0, 0), (1024, 6144, 512, -1, 0),
    # 129 to 256 tokens: tokens on the lanes when the product has more features than inner size, else the kernel that may cut K;
    # either asked for by name at a size where the other would be chosen
    (129, 1024, 512, 0, 0), (256, 2048, 1000, 0, 0), (200, 512, 1024, 0, 0), (200, 512, 1024, -1, 0), (65, 640, 256, -1, 0),
    (256, 2048, 1024, 256, 0), (40, 4096, 64, -1, 0),
])
@pytest.mark.parametrize("ty", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05(env, M, N, K, bt, splits, ty):
    ops, dev, st = env
    x, w = torch.randn(M, K, device=dev).bfloat16(), torch.randn(N, K, device=dev).bfloat16()
    y = torch.full((M, N), float("nan"), device=dev, dtype=ty)
    ops.gemm_tcgen05(y, x, w, st, bt, splits)
    torch.cuda.synchronize()
    assert ops.device_error() == 0
    # float32 out: what is left is the rounding of the 32-bit accumulation, which grows like sqrt(K)
    tol = 2e-6 * max(1.0, math.sqrt(K / 256)) if ty == torch.float32 else 5e-3
    assert rel(y, x.double() @ w.double().t()) < tol
    # a row-strided view of a wider matrix as input, as the q|k|v product's consumers use it
    wide = torch.randn(M, K + 64, device=dev).bfloat16()
    ops.gemm_tcgen05(y, wide[:, 32:32 + K] if (32 * 2) % 16 == 0 else wide[:, :K], w, st, bt, splits)
    assert rel(y, wide[:, 32:32 + K].double() @ w.double().t()) < tol


@pytest.mark.parametrize("M,I,K,bt,splits", [(5, 128, 96, 0, 0), (16, 256, 1024, 16, 4), (40, 640, 512, 64, 1), (8, 12288, 512, 0, 0),
                                             (64, 192, 2048, 0, 0), (300, 320, 264, 0, 0), (2048, 1024, 256, 0, 0), (700, 64, 4096, 0, 0),
                                             (700, 1024, 2048, 0, 128), (512, 2048, 512, 0, 0),
                                             (1024, 1536, 512, 0, -(8 * 1024 + 128)), (2048, 12288, 64, 0, 0),
                                             (1024, 1536, 512, -2, 0), (700, 512, 2048, -2, 128), (1100, 640, 256, -1, 0),
                                             # from 65 tokens on the kernel with tokens on the lanes; 64 stay with the other
                                             (65, 256, 512, 0, 0), (128, 384, 1024, 0, 0), (200, 1024, 2048, 0, 0), (200, 1024, 2048, 256, 0),
                                             (64, 384, 1024, -1, 0)])
@pytest.mark.parametrize("ty", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05_with_swiglu_epilogue(env, M, I, K, bt, splits, ty):
    """gate and up rows interleaved in blocks of 64; the product's epilogue forms silu(gate) * up."""
    ops, dev, st = env
    x = torch.randn(M, K, device=dev).bfloat16()
    gate, up = (torch.randn(I, K, device=dev) * 0.1).bfloat16(), (torch.randn(I, K, device=dev) * 0.1).bfloat16()
    w = ops.interleave_gate_up(gate, up)
    assert torch.equal(w[:64], gate[:64]) and torch.equal(w[64:128], up[:64])
    y = torch.full((M, I), float("nan"), device=dev, dtype=ty)
    ops.gemm_tcgen05(y, x, w, st, bt, splits, swiglu=True)
    torch.cuda.synchronize()
    assert ops.device_error() == 0
    want = plain.swiglu(x.double() @ gate.double().t(), x.double() @ up.double().t())
    # float32 out: the rounding of two 32-bit accumulations (it grows like sqrt(K)) meets in the product silu(gate) * up
    tol = 4e-6 * max(1.0, math.sqrt(K / 256)) if ty == torch.float32 else 5e-3
    assert rel(y, want) < tol


@pytest.mark.parametrize("M,N,K", [(8, 4096, 4096), (1, 4096, 12288), (3, 1000, 2048), (32, 512, 1024), (20, 5120, 5120), (64, 1024, 2048),
                                   (300, 16384, 512), (1024, 16384, 1024), (2048, 5000, 512), (900, 5004, 256), (2048, 4096, 12288)])
def test_gemm_tcgen05_that_adds_to_the_residual_stream(env, M, N, K):
    """residual += x . w^T; out = residual * norm weight (rounded, without the row's factor); partial sums of squares
    whose total is the row's sum of squares: against the same done plainly, and the factor formed from the partial
    sums against the norm's.  Few tokens (the epilogue of a product split over a cluster) and many (the persistent
    kernel with more tiles than CTAs: single CTAs and pairs, a width that is no multiple of 8)."""
    ops, dev, st = env
    x = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(N, K, device=dev) / math.sqrt(K)).bfloat16()
    assert ops.gemm_tcgen05_addnorm_ok(x, w)
    residual = torch.randn(M, N, device=dev)
    before = residual.double().cpu()
    nw = 1 + 0.2 * torch.randn(N, device=dev)
    tiles = ops.gemm_tcgen05_addnorm_tiles(M, N, K)
    assert tiles == -(-N // 128) if M <= 256 else 0 < tiles <= -(-N // 16)
    out = torch.full((M, N), float("nan"), device=dev, dtype=torch.bfloat16)
    sumsq = torch.full((M, tiles), float("nan"), device=dev)
    ops.gemm_tcgen05_addnorm(x, w, residual, nw, out, sumsq, st)
    torch.cuda.synchronize()
    assert ops.device_error() == 0
    want = before + (x.double() @ w.double().t()).cpu()
    tol32 = 2e-6 * max(1.0, math.sqrt(K / 256))                          # what the product itself keeps of 32-bit sums
    assert rel(residual.cpu(), want) < tol32
    assert rel(out.cpu(), want * nw.double().cpu()) < 5e-3
    assert torch.isfinite(sumsq).all()
    if M <= 256:                                                         # blocks of 128 features
        blocks = torch.nn.functional.pad(want * want, (0, tiles * 128 - N)).reshape(M, tiles, 128).sum(dim=2)
        assert rel(sumsq.cpu(), blocks) < 1e-5 + 2 * tol32
    assert rel(sumsq.double().sum(dim=1).cpu(), (want * want).sum(dim=1)) < 1e-5 + 2 * tol32
    eps = 1e-6
    normed = plain.rms_norm(want, nw.double().cpu(), eps)
    factor = torch.rsqrt(sumsq.double().sum(dim=1, keepdim=True) / N + eps).cpu()
    assert rel(out.double().cpu() * factor, normed) < 5e-3
    if M <= 256:   # what it does not take: few tokens in a product that is not split over a cluster (too many tiles, too short a k)
        assert not ops.gemm_tcgen05_addnorm_ok(x, torch.empty(24576, K, device=dev, dtype=torch.bfloat16))
        assert not ops.gemm_tcgen05_addnorm_ok(x[:, :192], w[:, :192].contiguous())
        with pytest.raises(ops.KernelError, match="columns of partial sums"):
            ops.gemm_tcgen05_addnorm(x, w, residual, nw, out, torch.empty(M, tiles + 1, device=dev), st)
    else:          # nor many tokens in a product of one round of tiles, whose epilogues no next tile would hide
        assert not ops.gemm_tcgen05_addnorm_ok(x[:300], w[:1024].contiguous())


@pytest.mark.parametrize("M,I,K", [(8, 12288, 4096), (1, 3072, 1024), (24, 512, 2048), (100, 1536, 512), (256, 12288, 1024),
                                   (600, 1536, 512), (1100, 2048, 1024)])
def test_gemm_tcgen05_swiglu_of_rows_that_lack_their_factor(env, M, I, K):
    """The gate|up product with the activation in its epilogue, given rows without their norm's factor: the factor is
    applied to the 32-bit sums before the activation (products that are not split, and ones split over a cluster)."""
    ops, dev, st = env
    x = torch.randn(M, K, device=dev).bfloat16()
    gate = (torch.randn(I, K, device=dev) / math.sqrt(K)).bfloat16()
    up = (torch.randn(I, K, device=dev) / math.sqrt(K)).bfloat16()
    w = ops.interleave_gate_up(gate, up)
    sumsq = (torch.rand(M, 7, device=dev) * K * 2).float()
    eps = 1e-5
    factor = torch.rsqrt(sumsq.double().sum(dim=1, keepdim=True) / K + eps).cpu()
    act = torch.full((M, I), float("nan"), device=dev, dtype=torch.bfloat16)
    ops.gemm_tcgen05(act, x, w, st, swiglu=True, sumsq=sumsq, eps=eps)
    torch.cuda.synchronize()
    assert ops.device_error() == 0
    g = (x.double() @ gate.double().t()).cpu() * factor
    u = (x.double() @ up.double().t()).cpu() * factor
    assert rel(act.cpu(), plain.swiglu(g, u)) < 6e-3
    # the product without the activation takes the factors too (few tokens: split over a cluster or not; many tokens)
    for out_dtype in (torch.bfloat16, torch.float32):
        y = torch.full((M, 2 * I), float("nan"), device=dev, dtype=out_dtype)
        ops.gemm_tcgen05(y, x, w, st, sumsq=sumsq, eps=eps)
        torch.cuda.synchronize()
        assert rel(y.cpu(), (x.double() @ w.double().t()).cpu() * factor) < 5e-3
    if M <= 256:
        with pytest.raises(ops.KernelError, match="through the workspace"):   # but not a product split through the workspace
            ops.gemm_tcgen05(torch.empty(M, 2 * I, device=dev, dtype=torch.bfloat16), x, w, st, force_splits=-2, sumsq=sumsq, eps=eps)


def test_gemm_tcgen05_refuses_what_it_cannot_do(env):
    ops, dev, st = env
    from lucciola_b200.ops import KernelError
    x, w = torch.randn(4, 100, device=dev).bfloat16(), torch.randn(8, 100, device=dev).bfloat16()
    y = torch.empty(4, 8, device=dev, dtype=torch.bfloat16)
    with pytest.raises(KernelError, match="multiple of 8"):
        ops.gemm_tcgen05(y, x, w, st)
    ops.linear(y, x, w, st, fast=True)                          # the dispatcher takes the plain kernel instead
    assert rel(y, x.double() @ w.double().t()) < 5e-3
    with pytest.raises(KernelError, match="do not fit"):
        ops.gemm_tcgen05(y, x, torch.randn(8, 96, device=dev).bfloat16(), st)


# ---- samplers ------------------------------------------------------------------------------------------------------
def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable(env):
    """The give-up path of the bounded waits, made to happen without anything in flight: one CTA of the smallest
    tensor-core product whose producer requests no tile, with a limit of 200 000 cycles (about 0.1 ms).  The kernel must
    return, leave its code in the device error flag, store nothing, and an ordinary product right after must be right."""
    import ctypes
    import time
    from lucciola_b200.csrc import library
    ops, dev, st = env
    fn = library().lb_gemm_tcgen05_wait_test
    fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3 + [ctypes.c_ulonglong, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    M, N, K = 8, 100, 256
    x, w = torch.randn(M, K, device=dev).bfloat16(), torch.randn(N, K, device=dev).bfloat16()
    y = torch.full((M, N), 7.0, device=dev, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    assert ops.device_error() == 0
    t0 = time.perf_counter()
    assert fn(y.data_ptr(), x.data_ptr(), w.data_ptr(), M, N, K, 200_000, st) == 0, library().lb_last_error().decode()
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0                     # it gave up after its limit, not after the ordinary two seconds
    assert ops.device_error() == 101                          # ERR_FULL_WAIT of csrc/gemm_tcgen05.cu
    assert ops.device_error() == 0                            # reading the flag clears it
    assert (y == 7.0).all()
    # sizes beyond one tile, and limits beyond the ordinary one, are refused
    assert fn(y.data_ptr(), x.data_ptr(), w.data_ptr(), 17, N, K, 200_000, st) != 0
    assert fn(y.data_ptr(), x.data_ptr(), w.data_ptr(), M, N, K, 1 << 40, st) != 0
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    ops.gemm_tcgen05(out, x, w, st)
    torch.cuda.synchronize()
    assert rel(out, x.double() @ w.double().t()) < 5e-3 and ops.device_error() == 0


def test_greedy_takes_the_lowest_index_among_equals(env):
    ops, dev, st = env
    logits = torch.zeros(3, 70001, device=dev)
    logits[0, [5, 69999]] = 2.0
    logits[1, 70000] = 1.0
    logits[2] = -1.0
    tokens = torch.empty(3, dtype=torch.int32, device=dev)
    ops.sample(tokens, logits, st)
    assert tokens.tolist() == [5, 70000, 0]


def test_temperature_sampler_equals_its_plain_restatement(env):
    ops, dev, st = env
    from lucciola_b200.sampling.sampler import sampling_key
    V, R = 503, 24
    logits = torch.randn(R, V, device=dev) * 2
    temps = torch.tensor([0.8] * 12 + [0.0] * 4 + [1.7] * 8, device=dev)
    seeds = [7] * 12 + [1] * 4 + [123456789] * 8
    keys = torch.from_numpy(np.array([sampling_key(s) for s in seeds], dtype=np.uint64).view(np.int64)).to(dev)
    counters = torch.arange(R, dtype=torch.int32, device=dev)
    tokens = torch.empty(R, dtype=torch.int32, device=dev)
    ops.sample(tokens, logits, st, temps, keys, counters)
    rows = logits.cpu().numpy()
    for r in range(R):
        want = plain.temperature_sample(rows[r], float(temps[r]), sampling_key(seeds[r]), r)
        assert int(tokens[r]) == want, r
    # the draw depends on the request's key and counter only: the same row alone gives the same token
    one = torch.empty(1, dtype=torch.int32, device=dev)
    ops.sample(one, logits[5:6].contiguous(), st, temps[5:6].contiguous(), keys[5:6].contiguous(), counters[5:6].contiguous())
    assert int(one[0]) == int(tokens[5])
    # and it follows the softmax
    l4 = torch.tensor([[2.0, 1.0, 0.0, -1.0]], device=dev).repeat(4000, 1)
    t4 = torch.full((4000,), 0.8, device=dev)
    k4 = keys[:1].repeat(4000)
    c4 = torch.arange(4000, dtype=torch.int32, device=dev)
    o4 = torch.empty(4000, dtype=torch.int32, device=dev)
    ops.sample(o4, l4, st, t4, k4, c4)
    p = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0]) / 0.8, 0)
    freq = torch.bincount(o4.cpu().long(), minlength=4).float() / 4000
    assert (freq - p).abs().max() < 0.03


@pytest.mark.gpu
def test_feature_tiles_of_the_many_token_product_cover_every_feature_once():
    """The plan of the many-token product (columns of tiles of one width, then tiles of a second width) is searched on
    the host: whatever it finds has to be launchable and must never cost more, by its own measure, than tiles of 256."""
    import ctypes
    from lucciola_b200.csrc import library
    lib = library()
    out = (ctypes.c_int * 3)()
    sms = 148

    def busiest(cols1, bn1, bn2, m_tiles, N):
        t1 = cols1 * m_tiles
        rest = N - cols1 * bn1
        tiles = t1 + (m_tiles * -(-rest // bn2) if rest > 0 else 0)
        G = min(tiles, sms)
        load = [0] * G
        for j in range(tiles):
            load[j % G] += (bn1 if j < t1 else bn2) + 64
        return max(load)

    for M in (257, 300, 512, 544, 1000, 2048, 4096, 5000, 16384):
        for N, swiglu in ((16, 0), (300, 0), (1024, 0), (4096, 0), (5120, 0), (6144, 0), (7168, 0), (151936, 0),
                          (128, 1), (2048, 1), (24576, 1), (34816, 1)):
            lib.lb_gemm_tcgen05_prefill_plan(M, N, swiglu, sms, out)
            cols1, bn1, bn2 = out[0], out[1], out[2]
            step = 128 if swiglu else 16
            assert cols1 >= 0 and 16 <= bn1 <= 256 and 16 <= bn2 <= 256 and bn1 % step == 0 and bn2 % step == 0, (M, N, list(out))
            if cols1 * bn1 < N:
                assert bn1 == 256, (M, N, list(out))          # a second width only behind columns of 256
            m_tiles = -(-M // 128)
            assert busiest(cols1, bn1, bn2, m_tiles, N) <= busiest(-(-N // 256), 256, 256, m_tiles, N), (M, N, list(out))
