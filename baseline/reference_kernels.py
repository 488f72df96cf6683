"""JunkuiZhang/lucciola's own CUDA kernels, compiled unchanged for sm_100a and callable from Python.

lucciola is a CMake project (C++23, dependencies fetched from the network at configure time), so its engine cannot
be installed offline; its ten kernel files, however, need nothing but the CUDA toolkit.  This module

  stage SRC    copies SRC/src/kernels/*.cu and SRC/include/ (nothing else, nothing changed) to baseline/_ref/lucciola,
               a folder that is not part of this repository's history;
  build(dir)   compiles those files with nvcc, with the flags of lucciola's CMakeLists.txt (--use_fast_math,
               --expt-relaxed-constexpr) but for sm_100a, together with a small file of `extern "C"` wrappers around
               lucciola's launch functions (which are C++ functions in namespace lucciola::kernels), and loads the
               result with ctypes.

Two users: tests/test_reference_kernels_gpu.py compares each kernel with the matching function of the plain
implementation (tests/plain_qwen3.py), which turns "formulas read from lucciola's code" into "formulas that
lucciola's code reproduces"; `python baseline/reference_kernels.py time` times each kernel beside this engine's
kernel for the same operation at the Qwen3-8B layer sizes, on the same GPU.

Where the sources are looked for: $LUCCIOLA_REFERENCE_DIR, then baseline/_ref/lucciola.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys
from ctypes import c_float, c_int, c_void_p
from pathlib import Path

HERE = Path(__file__).resolve().parent
STAGED = HERE / "_ref" / "lucciola"
KERNEL_FILES = ["rmsnorm", "rope", "linear", "swiglu", "add", "embedding", "argmax", "attention_paged", "flash_attention"]

# Wrappers with C linkage around lucciola's launch functions (include/kernels/*.h); nothing is computed here.
SHIM = r"""
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "kernels/add.h"
#include "kernels/argmax.h"
#include "kernels/attention.h"
#include "kernels/embedding.h"
#include "kernels/flash_attention.h"
#include "kernels/linear.h"
#include "kernels/rmsnorm.h"
#include "kernels/rope.h"
#include "kernels/swiglu.h"
namespace k = lucciola::kernels;
extern "C" {
void ref_rmsnorm(void* out, const void* in, const void* w, int rows, int hidden, float eps, cudaStream_t s) {
  k::rmsnorm_forward(out, in, w, rows, hidden, eps, s);
}
void ref_rope(void* x, const int* pos, int tokens, int heads, int head_dim, float theta, cudaStream_t s) {
  k::rope_forward(x, pos, tokens, heads, head_dim, theta, s);
}
void ref_linear(void* y, const void* x, const void* w, int m, int n, int kk, cudaStream_t s) { k::linear_forward(y, x, w, m, n, kk, s); }
void ref_swiglu(void* out, const void* gate, const void* up, int tokens, int inter, cudaStream_t s) {
  k::swiglu_forward(out, gate, up, tokens, inter, s);
}
void ref_add(void* in_out, const void* addend, int n, cudaStream_t s) { k::add_forward(in_out, addend, n, s); }
void ref_embedding(void* out, const int* ids, const void* table, int tokens, int hidden, int vocab, cudaStream_t s) {
  k::embedding_forward<__nv_bfloat16>(out, ids, table, tokens, hidden, vocab, s);
}
void ref_argmax(int* out, const void* logits, int rows, int vocab, cudaStream_t s) { k::argmax_forward(out, logits, rows, vocab, s); }
void ref_append_kv(void* k_cache, void* v_cache, const void* k_new, const void* v_new, const int* context_lens,
                   const int* block_tables, int seqs, int tokens_per_seq, int kv_heads, int head_dim, int block_size,
                   int max_blocks, cudaStream_t s) {
  k::append_paged_kv_cache(k_cache, v_cache, k_new, v_new, context_lens, block_tables, seqs, tokens_per_seq, kv_heads,
                           head_dim, block_size, max_blocks, s);
}
void ref_paged_attention(void* out, const void* q, void* k_cache, void* v_cache, const int* context_lens,
                         const int* block_tables, int seqs, int heads, int kv_heads, int head_dim, int block_size,
                         int max_blocks, cudaStream_t s) {
  k::paged_attention_forward(out, q, k_cache, v_cache, context_lens, block_tables, seqs, heads, kv_heads, head_dim,
                             block_size, max_blocks, s);
}
void ref_flash_attention(void* out, const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                         const int* context_lens, int seqs, int q_len, int heads, int kv_heads, int head_dim,
                         int max_blocks, cudaStream_t s) {
  k::launch_lucciola_attention(out, q, k_cache, v_cache, block_tables, context_lens, seqs, q_len, heads, kv_heads,
                               head_dim, max_blocks, s);
}
}
"""

SIGNATURES = {
    "ref_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "ref_rope": [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "ref_linear": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "ref_swiglu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ref_add": [c_void_p, c_void_p, c_int, c_void_p],
    "ref_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "ref_argmax": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ref_append_kv": [c_void_p] * 6 + [c_int] * 6 + [c_void_p],
    "ref_paged_attention": [c_void_p] * 6 + [c_int] * 6 + [c_void_p],
    "ref_flash_attention": [c_void_p] * 6 + [c_int] * 6 + [c_void_p],
}


def find_sources() -> Path | None:
    """A folder that holds lucciola's src/kernels and include, or None."""
    for cand in (os.environ.get("LUCCIOLA_REFERENCE_DIR"), STAGED):
        if cand and all((Path(cand) / "src" / "kernels" / f"{k}.cu").is_file() for k in KERNEL_FILES) \
                and (Path(cand) / "include" / "kernels").is_dir():
            return Path(cand)
    return None


def stage(src: str | Path) -> Path:
    """Copy the kernel sources and headers of a lucciola checkout, unchanged, to where find_sources() looks."""
    src = Path(src)
    if STAGED.exists():
        shutil.rmtree(STAGED)
    (STAGED / "src" / "kernels").mkdir(parents=True)
    for k in KERNEL_FILES:
        shutil.copy2(src / "src" / "kernels" / f"{k}.cu", STAGED / "src" / "kernels" / f"{k}.cu")
    shutil.copytree(src / "include", STAGED / "include")
    return STAGED


def build(out_dir: str | Path) -> ctypes.CDLL:
    """Compile lucciola's kernel files as they are, plus the wrappers above, into out_dir and load the library."""
    ref = find_sources()
    if ref is None:
        raise FileNotFoundError("lucciola's kernel sources were not found (set LUCCIOLA_REFERENCE_DIR or stage them)")
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    shim = out_dir / "reference_shim.cu"
    shim.write_text(SHIM)
    lib = out_dir / "liblucciola_reference_kernels.so"
    nvcc = os.environ.get("LUCCIOLA_B200_NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++20", "--expt-relaxed-constexpr",
           "--use_fast_math", "--threads", "0", "-I", str(ref / "include"), "-Xcompiler", "-fPIC", "-shared", "-o", str(lib),
           str(shim)] + [str(ref / "src" / "kernels" / f"{k}.cu") for k in KERNEL_FILES]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on lucciola's kernels:\n{r.stdout}\n{r.stderr}")
    dll = ctypes.CDLL(str(lib))
    for name, sig in SIGNATURES.items():
        fn = getattr(dll, name)
        fn.argtypes, fn.restype = sig, None
    return dll


# ---- timing beside this engine's kernels ------------------------------------------------------------------------
def time_kernels() -> int:
    """Each lucciola kernel and this engine's kernel for the same operation, at the Qwen3-8B layer sizes, for a decode
    step of 8 requests (context 640, the mean of lucciola's 512 -> 768 workload) and a prompt of 2048 tokens: CUDA
    events, 3 warm-up runs, median of 10; a 256 MB buffer is written between runs so that nothing starts from L2."""
    import statistics
    import tempfile

    import torch

    sys.path.insert(0, str(HERE.parent))
    from lucciola_b200 import ops

    dll = build(tempfile.mkdtemp(prefix="lucciola_ref_"))
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    st = torch.cuda.current_stream().cuda_stream
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    H, I, V, nq, nkv, d = 4096, 12288, 151936, 32, 8, 128
    bf = torch.bfloat16

    def timed(fn, runs=10, warm=3):
        times = []
        for i in range(warm + runs):
            flush.fill_(i)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            if i >= warm:
                times.append(a.elapsed_time(b) * 1e3)
        return statistics.median(times)

    def rand(*shape, scale=1.0):
        return (torch.randn(*shape, device=dev) * scale).to(bf)

    rows = []
    for M, what in ((8, "decode, 8 tokens"), (2048, "prompt, 2048 tokens")):
        x = rand(M, H)
        for name, N, K in (("q|k|v", (nq + 2 * nkv) * d, H), ("o", H, nq * d), ("gate|up", 2 * I, H), ("down", H, I)) + \
                ((("lm_head", V, H),) if M == 8 else ()):
            xin, w = rand(M, K), rand(N, K, scale=0.02)
            y = torch.empty(M, N, device=dev, dtype=bf)
            # lucciola runs q, k, v (and gate, up) as separate products; their sum is one product over the stacked rows
            t_ref = timed(lambda: dll.ref_linear(y.data_ptr(), xin.data_ptr(), w.data_ptr(), M, N, K, st), runs=5 if M > 8 else 10)
            t_own = timed(lambda: ops.gemm_tcgen05(y, xin, w, st))
            rows.append((what, f"linear {name} [{N} x {K}]", t_ref, t_own))
        wn = rand(H)
        out = torch.empty_like(x)
        res = torch.randn(M, H, device=dev)
        wn32 = wn.float()
        t_ref = timed(lambda: dll.ref_rmsnorm(out.data_ptr(), x.data_ptr(), wn.data_ptr(), M, H, 1e-6, st))
        t_own = timed(lambda: ops.add_rmsnorm(out, res, x, wn32, 1e-6, st))
        rows.append((what, "rmsnorm (ours: residual add + rmsnorm)", t_ref, t_own))
        g, u, act = rand(M, I), rand(M, I), torch.empty(M, I, device=dev, dtype=bf)
        t_ref = timed(lambda: dll.ref_swiglu(act.data_ptr(), g.data_ptr(), u.data_ptr(), M, I, st))
        t_own = timed(lambda: ops.swiglu(act, g, u, st))
        rows.append((what, "swiglu (ours runs in the gate|up epilogue; stand-alone kernel timed)", t_ref, t_own))
    # attention: decode of 8 requests at 640 keys; a 2048-token prompt
    page, S, ctx = 16, 8, 640
    P = ctx // page
    pool_ref = rand(2, S * P + 1, page, nkv, d)                   # lucciola: [page][slot][kv head][d]
    pool_own = pool_ref.permute(0, 1, 3, 2, 4).contiguous()       # this engine: [page][kv head][slot][d]
    tables = torch.arange(S * P, dtype=torch.int32, device=dev).view(S, P).contiguous()
    lens = torch.full((S,), ctx, dtype=torch.int32, device=dev)
    q, o = rand(S, nq, d), torch.empty(S, nq, d, device=dev, dtype=bf)
    t_ref = timed(lambda: dll.ref_paged_attention(o.data_ptr(), q.data_ptr(), pool_ref[0].data_ptr(), pool_ref[1].data_ptr(),
                                                  lens.data_ptr(), tables.data_ptr(), S, nq, nkv, d, page, P, st))
    pos = torch.full((S,), ctx - 1, dtype=torch.int32, device=dev)
    tiles = torch.tensor([[i, 1, i, 0] for i in range(S)], dtype=torch.int32, device=dev)
    splits = ops.attention_splits(S, nkv, ctx, 4, wide_clusters=ops.attention_wide_clusters(d))
    t_own = timed(lambda: ops.attention_flash(q, o, pool_own[0], pool_own[1], pos, tables, tiles, 4, nq, nkv, d, page, 0,
                                              d ** -0.5, splits, st))
    rows.append(("decode, 8 tokens", "decode attention, 640 keys each", t_ref, t_own))
    T = 2048
    P = T // page
    pool_ref = rand(2, P + 1, page, nkv, d)
    pool_own = pool_ref.permute(0, 1, 3, 2, 4).contiguous()
    tables = torch.arange(P, dtype=torch.int32, device=dev).view(1, P).contiguous()
    lens = torch.tensor([T], dtype=torch.int32, device=dev)
    q, o = rand(T, nq, d), torch.empty(T, nq, d, device=dev, dtype=bf)
    t_ref = timed(lambda: dll.ref_flash_attention(o.data_ptr(), q.data_ptr(), pool_ref[0].data_ptr(), pool_ref[1].data_ptr(),
                                                  tables.data_ptr(), lens.data_ptr(), 1, T, nq, nkv, d, P, st), runs=5)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    per = 2 * (128 // (nq // nkv))
    tiles = torch.tensor([[a, min(per, T - a), 0, 0] for a in range(0, T, per)][::-1], dtype=torch.int32, device=dev)
    t_own = timed(lambda: ops.attention_tcgen05(q, o, pool_own[0], pool_own[1], pos, tables, tiles, nq, nkv, d, page, 0,
                                                d ** -0.5, st))
    rows.append(("prompt, 2048 tokens", "prompt attention, causal", t_ref, t_own))
    print("| workload | operation | lucciola's kernel (us) | this engine's kernel (us) | ratio |")
    print("|---|---|---|---|---|")
    for what, name, a, b in rows:
        print(f"| {what} | {name} | {a:.1f} | {b:.1f} | {a / b:.1f} |")
    assert ops.device_error() == 0
    return 0


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[1] == "stage":
        print(stage(sys.argv[2]))
    elif len(sys.argv) == 2 and sys.argv[1] == "time":
        sys.exit(time_kernels())
    else:
        print(__doc__)
        sys.exit(2)
