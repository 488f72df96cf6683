"""The plain implementation against JunkuiZhang/lucciola's own kernels (GPU).

tests/plain_qwen3.py restates lucciola's formulas from reading its code.  Here lucciola's production kernel files
are compiled as they are (nvcc, lucciola's own flags, sm_100a; see baseline/reference_kernels.py) and each is run on
small bfloat16 inputs beside the matching function of the plain implementation.  They must agree to one rounding
of the bfloat16 output: what the other tests compare this engine with is then what lucciola's code computes.

Every call stays inside what the kernel indexes safely, as read from its source: hidden sizes that are multiples
of 4 (8-byte vector loads, src/kernels/rmsnorm.cu:62-66, linear.cu:36-41); pages of 16 tokens and heads of at most
128 for the prompt kernel (src/kernels/flash_attention.cu:33-34, 77-78) with at least 2 query tokens (:368); at most
1024 keys for the decode kernel (src/kernels/attention_paged.cu:80-81); kv heads x head size <= 1024 for the cache
append (:161-167).  Both attention kernels index the cache as [page][slot][kv head][d].

The sources are not part of this repository; where they are absent the tests are skipped.
"""
import math
import sys

import pytest
import torch

import plain_qwen3 as plain
from conftest import ROOT

pytestmark = pytest.mark.gpu
sys.path.insert(0, str(ROOT / "baseline"))
DEV = "cuda:0"
BF = torch.bfloat16


@pytest.fixture(scope="module")
def ref(tmp_path_factory):
    import reference_kernels as rk
    if rk.find_sources() is None:
        pytest.skip("lucciola's kernel sources are not here (python baseline/reference_kernels.py stage <lucciola checkout>)")
    return rk.build(tmp_path_factory.mktemp("lucciola_kernels"))


def stream():
    return torch.cuda.current_stream().cuda_stream


def rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, device=DEV, generator=g) * scale).to(BF)


def assert_one_rounding(got: torch.Tensor, want: torch.Tensor, what: str, floor: float = 2.0 ** -10):
    """|got - want| <= one spacing of bfloat16 at want (2^-7 relative at most), plus a floor of 2^-10 of the largest
    value for outputs that are small by cancellation (32-bit sums, fast-math functions)."""
    got, want = got.double().cpu(), want.double().cpu()
    assert torch.isfinite(got).all(), what
    tol = want.abs() * 2.0 ** -7 + floor * want.abs().max()
    bad = (got - want).abs() > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} values differ by more than one rounding; worst {((got - want).abs() / tol).max():.2f} x"


@pytest.mark.parametrize("rows,hidden,eps", [(7, 256, 1e-6), (3, 4096, 1e-6), (5, 1000, 1e-5), (64, 128, 1e-6)])
def test_rmsnorm(ref, rows, hidden, eps):
    x, w = rand(rows, hidden, scale=3.0), (1 + 0.2 * torch.randn(hidden, device=DEV)).to(BF)
    out = torch.full_like(x, float("nan"))
    ref.ref_rmsnorm(out.data_ptr(), x.data_ptr(), w.data_ptr(), rows, hidden, eps, stream())
    torch.cuda.synchronize()
    assert_one_rounding(out, plain.rms_norm(x.double().cpu(), w.double().cpu(), eps), "rmsnorm")


@pytest.mark.parametrize("heads,d,theta", [(4, 128, 1e6), (3, 64, 1e4), (8, 32, 1e6)])
def test_rope(ref, heads, d, theta):
    T = 40
    x = rand(T, heads, d, seed=1)
    pos = torch.tensor([0, 1, 2, 3, 17, 255, 256, 300] * 5, dtype=torch.int32, device=DEV)
    want = plain.rope(x.double().cpu(), pos.cpu(), theta)
    got = x.clone()
    ref.ref_rope(got.data_ptr(), pos.data_ptr(), T, heads, d, float(theta), stream())
    torch.cuda.synchronize()
    assert_one_rounding(got, want, "rope")
    assert not torch.equal(got[1:], x[1:])


@pytest.mark.parametrize("m,n,k", [(5, 48, 64), (33, 200, 1024), (2, 4096, 4096)])
def test_linear(ref, m, n, k):
    x, w = rand(m, k, seed=2), rand(n, k, scale=0.05, seed=3)
    y = torch.full((m, n), float("nan"), device=DEV, dtype=BF)
    ref.ref_linear(y.data_ptr(), x.data_ptr(), w.data_ptr(), m, n, k, stream())
    torch.cuda.synchronize()
    assert_one_rounding(y, plain.linear(x.double().cpu(), w.double().cpu()), "linear")


def test_swiglu_and_add(ref):
    T, inter = 6, 264
    g, u = rand(T, inter, scale=2.0, seed=4), rand(T, inter, seed=5)
    out = torch.full_like(g, float("nan"))
    ref.ref_swiglu(out.data_ptr(), g.data_ptr(), u.data_ptr(), T, inter, stream())
    torch.cuda.synchronize()
    assert_one_rounding(out, plain.swiglu(g.double().cpu(), u.double().cpu()), "swiglu")
    r, y = rand(T, inter, seed=6), rand(T, inter, seed=7)
    acc = r.clone()
    ref.ref_add(acc.data_ptr(), y.data_ptr(), T * inter, stream())                 # x = bf16(f32(r) + f32(y)), src/kernels/add.cu:11-14
    torch.cuda.synchronize()
    assert torch.equal(acc, (r.float() + y.float()).to(BF))


def test_embedding_and_argmax(ref):
    V, H = 300, 136
    table = rand(V, H, seed=8)
    ids = torch.tensor([0, 299, 7, 7, 150], dtype=torch.int32, device=DEV)
    out = torch.full((5, H), float("nan"), device=DEV, dtype=BF)
    ref.ref_embedding(out.data_ptr(), ids.data_ptr(), table.data_ptr(), 5, H, V, stream())
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), plain.embed(ids.cpu().tolist(), table.cpu()))     # a copy, unscaled
    logits = rand(4, 1003, seed=9)
    best = [5, 1002, 0, 777]
    for r, b in enumerate(best):
        logits[r, b] = 9.0                                                          # a single largest value: ties are undefined there
    tok = torch.full((4,), -1, dtype=torch.int32, device=DEV)
    ref.ref_argmax(tok.data_ptr(), logits.data_ptr(), 4, 1003, stream())
    torch.cuda.synchronize()
    assert tok.tolist() == best == [plain.greedy(logits[r].float().cpu()) for r in range(4)]


def paged(keys: torch.Tensor, values: torch.Tensor, lens, page=16, spare=3, seed=0):
    """Put keys/values [S][len, nkv, d] into NaN-filled pools [page][slot][kv head][d] under shuffled block tables."""
    nkv, d = keys[0].shape[1:]
    pages = [-(-n // page) for n in lens]
    order = torch.randperm(sum(pages) + spare, generator=torch.Generator().manual_seed(seed)).tolist()
    tables = torch.full((len(lens), max(pages) + 1), -1, dtype=torch.int32)
    kc = torch.full((sum(pages) + spare, page, nkv, d), float("nan"), dtype=BF, device=DEV)
    vc = torch.full_like(kc, float("nan"))
    o = 0
    for s, n in enumerate(lens):
        tables[s, :pages[s]] = torch.tensor(order[o:o + pages[s]], dtype=torch.int32)
        o += pages[s]
    return kc, vc, tables.to(DEV)


@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 128), (8, 1, 64), (6, 6, 32)])
def test_cache_append_and_decode_attention(ref, nq, nkv, d):
    """Keys and values go into the pages through lucciola's append kernel (a whole prompt, then one token), the decode
    kernel attends to them; against plain attention of the last position over all keys."""
    lens = [37, 100, 1000, 16]                                    # after the decoded token
    ks = [rand(n, nkv, d, seed=10 + i) for i, n in enumerate(lens)]
    vs = [rand(n, nkv, d, seed=20 + i) for i, n in enumerate(lens)]
    kc, vc, tables = paged(ks, vs, lens)
    P = tables.shape[1]
    for s, n in enumerate(lens):
        for a, b in ((0, n - 1), (n - 1, n)):                     # the prompt, then the decoded token
            if b > a:
                ctx = torch.tensor([b], dtype=torch.int32, device=DEV)
                kn, vn = ks[s][a:b].contiguous(), vs[s][a:b].contiguous()
                ref.ref_append_kv(kc.data_ptr(), vc.data_ptr(), kn.data_ptr(), vn.data_ptr(), ctx.data_ptr(),
                                  tables[s].data_ptr(), 1, b - a, nkv, d, 16, P, stream())
    q = rand(len(lens), nq, d, seed=30)
    out = torch.full_like(q, float("nan"))
    ctx = torch.tensor(lens, dtype=torch.int32, device=DEV)
    ref.ref_paged_attention(out.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ctx.data_ptr(), tables.data_ptr(),
                            len(lens), nq, nkv, d, 16, P, stream())
    torch.cuda.synchronize()
    for s, n in enumerate(lens):
        want = plain.attention(q[s:s + 1].double().cpu(), ks[s].double().cpu(), vs[s].double().cpu(), [n - 1], list(range(n)),
                               1.0 / math.sqrt(d))
        assert_one_rounding(out[s:s + 1], want, f"decode attention over {n} keys")
        page_of = tables[s, (n - 1) // 16].item()                 # where the append kernel put the last token
        assert torch.equal(kc[page_of, (n - 1) % 16], ks[s][n - 1])


@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 128), (2, 1, 64)])
@pytest.mark.parametrize("cached,q_len", [(0, 70), (80, 70), (45, 2), (0, 128)])
def test_prompt_attention(ref, nq, nkv, d, cached, q_len):
    """A portion of q_len tokens behind `cached` tokens of two requests, through lucciola's paged prompt kernel."""
    S, n = 2, cached + q_len
    ks = [rand(n, nkv, d, seed=40 + i) for i in range(S)]
    vs = [rand(n, nkv, d, seed=50 + i) for i in range(S)]
    kc, vc, tables = paged(ks, vs, [n] * S, seed=1)
    for s in range(S):
        for t in range(n):
            pg = tables[s, t // 16].item()
            kc[pg, t % 16], vc[pg, t % 16] = ks[s][t], vs[s][t]
    q = rand(S, q_len, nq, d, seed=60)
    out = torch.full_like(q, float("nan"))
    ctx = torch.tensor([n] * S, dtype=torch.int32, device=DEV)
    ref.ref_flash_attention(out.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), ctx.data_ptr(),
                            S, q_len, nq, nkv, d, tables.shape[1], stream())
    torch.cuda.synchronize()
    for s in range(S):
        want = plain.attention(q[s].double().cpu(), ks[s].double().cpu(), vs[s].double().cpu(), list(range(cached, n)),
                               list(range(n)), 1.0 / math.sqrt(d))
        assert_one_rounding(out[s], want, f"prompt attention, {q_len} tokens behind {cached}")
