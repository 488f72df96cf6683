"""Tensor-level wrappers of the kernel library.

Each function checks what the kernel cannot check for itself (device, type,
contiguity), passes raw pointers and the stream to the C interface, and raises
`KernelError` with the library's message when a call is refused.  There is no
other implementation behind these functions: without the library they raise.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p

import torch

from .csrc import KernelLibraryError, library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dt}")


_SIGNATURES = {
    "lb_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "lb_add_rmsnorm": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "lb_rope_kv": [c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p,
                   c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "lb_attention_plain": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "lb_swiglu": [c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p],
    "lb_gemm_plain": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_longlong,
                      c_longlong, c_void_p],
    "lb_gemm_tcgen05": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p,
                        c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "lb_gemm_tcgen05_addnorm": [c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int, c_void_p],
    "lb_upload": [c_void_p, c_void_p, c_longlong, c_void_p],
    "lb_zero_rows": [c_void_p, c_longlong, c_int, c_void_p, c_int, c_void_p],
    "lb_gemm_tcgen05_heads": [c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p],
    "lb_attention_flash": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                           c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_longlong, c_void_p],
    "lb_attention_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_longlong, c_void_p],
    "lb_sample": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
}

_fn_cache: dict[str, object] = {}


def _fn(name: str):
    f = _fn_cache.get(name)
    if f is None:
        lib = library()
        try:
            f = getattr(lib, name)
        except AttributeError as e:
            raise KernelLibraryError(f"the kernel library lacks {name}") from e
        f.argtypes = _SIGNATURES[name]
        f.restype = c_int
        _fn_cache[name] = f
    return f


def _call(name: str, *args) -> None:
    rc = _fn(name)(*args)
    if rc != 0:
        raise KernelError(library().lb_last_error().decode())


def hash_uniform(key: int, counter: int, i: int) -> float:
    """The sampler's uniform number for (request key, generated index, vocabulary index), on the host."""
    lib = library()
    f = lib.lb_hash_uniform
    f.argtypes = [c_ulonglong, c_uint, c_uint]
    f.restype = c_float
    return float(f(key, counter, i))


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _check(t: torch.Tensor, what: str, dtype: torch.dtype | None = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} must be on the GPU")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, is {t.dtype}")


def current_stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def embedding(out: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, stream: int) -> None:
    """out[t, :] = table[ids[t], :] as float32."""
    _check(out, "embedding output", torch.float32); _check(ids, "token ids", torch.int32); _check(table, "embedding table")
    T, H = out.shape
    _call("lb_embedding", out.data_ptr(), ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype), T, H,
          table.shape[0], stream)


def add_rmsnorm(out: torch.Tensor, residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor,
                eps: float, stream: int, rows: torch.Tensor | None = None) -> None:
    """residual += delta (when rows is None); out = rmsnorm(residual [+ delta]) * weight, on `rows` if given."""
    _check(out, "norm output"); _check(residual, "residual", torch.float32); _check(weight, "norm weight", torch.float32)
    n = out.shape[0]
    H = out.shape[-1]
    if delta is not None:
        _check(delta, "delta")
    if rows is not None:
        _check(rows, "row index", torch.int32)
    _call("lb_add_rmsnorm", out.data_ptr(), dtype_code(out.dtype), residual.data_ptr(), _ptr(delta),
          dtype_code(delta.dtype) if delta is not None else F32, weight.data_ptr(), _ptr(rows), n, H, eps, stream)


def rope_kv(q_in: torch.Tensor, k_in: torch.Tensor, v_in: torch.Tensor, q_out: torch.Tensor,
            positions: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int, eps: float, stream: int,
            q_norm_w: torch.Tensor | None = None, k_norm_w: torch.Tensor | None = None,
            inv_freq: torch.Tensor | None = None, rot_dim: int = 0,
            k_cache: torch.Tensor | None = None, v_cache: torch.Tensor | None = None,
            token_seq: torch.Tensor | None = None, block_table: torch.Tensor | None = None, page_size: int = 0,
            k_out: torch.Tensor | None = None, v_out: torch.Tensor | None = None) -> None:
    """Per-head norm of q and k, rotation, and the write of k and v into pages (or into k_out, v_out).

    q_in, k_in and v_in are 2-d views whose rows may be column ranges of one wider matrix."""
    T = q_in.shape[0]
    dt = q_in.dtype
    for t, w in ((q_in, "q"), (k_in, "k"), (v_in, "v")):
        if not t.is_cuda or t.dtype != dt or t.stride(-1) != 1:
            raise KernelError(f"{w} must be on the GPU, of one type, with unit stride in its last dimension")
    _check(q_out, "q output", dt); _check(positions, "positions", torch.int32)
    max_pages = 0
    if k_cache is not None:
        _check(k_cache, "k pool", dt); _check(v_cache, "v pool", dt)
        _check(token_seq, "token map", torch.int32); _check(block_table, "block table", torch.int32)
        max_pages = block_table.shape[1]
    _call("lb_rope_kv", dtype_code(dt), q_in.data_ptr(), k_in.data_ptr(), v_in.data_ptr(), q_in.stride(0),
          k_in.stride(0), v_in.stride(0), q_out.data_ptr(), _ptr(k_out), _ptr(v_out), _ptr(k_cache), _ptr(v_cache),
          positions.data_ptr(), _ptr(token_seq), _ptr(block_table), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq),
          T, num_q_heads, num_kv_heads, head_dim, rot_dim, page_size, max_pages, eps, stream)


def attention_plain(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    positions: torch.Tensor, token_seq: torch.Tensor, block_table: torch.Tensor,
                    num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                    stream: int) -> None:
    dt = q.dtype
    _check(q, "q"); _check(out, "attention output", dt); _check(k_cache, "k pool", dt); _check(v_cache, "v pool", dt)
    _check(positions, "positions", torch.int32); _check(token_seq, "token map", torch.int32)
    _check(block_table, "block table", torch.int32)
    _call("lb_attention_plain", dtype_code(dt), q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
          positions.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(), q.shape[0], num_q_heads, num_kv_heads,
          head_dim, page_size, block_table.shape[1], window, scale, stream)


def swiglu(out: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, stream: int) -> None:
    """out = silu(gate) * up; gate and up are 2-d views with the same row stride."""
    if gate.stride(0) != up.stride(0) or gate.stride(1) != 1 or up.stride(1) != 1:
        raise KernelError("gate and up need the same row stride and unit column stride")
    _check(out, "swiglu output", gate.dtype)
    T, inter = out.shape
    _call("lb_swiglu", dtype_code(out.dtype), out.data_ptr(), gate.data_ptr(), up.data_ptr(), gate.stride(0), T, inter, stream)


def gemm_plain(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, stream: int) -> None:
    """y[M, N] = x[M, K] . w[N, K]^T on the 32-bit pipes; x and y may be row-strided views."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(y.shape) != (M, N):
        raise KernelError(f"gemm shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if x.stride(1) != 1 or y.stride(1) != 1 or not w.is_contiguous() or not (x.is_cuda and w.is_cuda and y.is_cuda):
        raise KernelError("gemm operands must be on the GPU with unit column stride; w contiguous")
    _call("lb_gemm_plain", y.data_ptr(), dtype_code(y.dtype), x.data_ptr(), dtype_code(x.dtype), w.data_ptr(),
          dtype_code(w.dtype), M, N, K, x.stride(0) if M > 1 else K, y.stride(0) if M > 1 else N, stream)


def sample(tokens: torch.Tensor, logits: torch.Tensor, stream: int, temperature: torch.Tensor | None = None,
           keys: torch.Tensor | None = None, counters: torch.Tensor | None = None) -> None:
    """tokens[r] = greedy or temperature sample of logits[r, :]; see sampling/sampler.py for the key."""
    _check(tokens, "token output", torch.int32); _check(logits, "logits", torch.float32)
    if temperature is not None:
        _check(temperature, "temperature", torch.float32); _check(keys, "keys", torch.int64)
        _check(counters, "counters", torch.int32)
    R, V = logits.shape
    _call("lb_sample", tokens.data_ptr(), logits.data_ptr(), _ptr(temperature), _ptr(keys), _ptr(counters), R, V, stream)


_WORKSPACE_ELEMS = 16 * 1024 * 1024      # float32 partials of split products (64 MB)
_COUNTERS = 4096
_scratch: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}


def _gemm_scratch(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Per device: the workspace for partial sums of split products and the tile counters (zero between launches)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    s = _scratch.get(key)
    if s is None:
        s = (torch.empty(_WORKSPACE_ELEMS, dtype=torch.float32, device=device),
             torch.zeros(_COUNTERS, dtype=torch.int32, device=device))
        _scratch[key] = s
    return s


def gemm_tcgen05_ok(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> bool:
    """The conditions of the tensor-core kernel: bfloat16 operands, K a multiple of 8, 16-byte alignment."""
    K = x.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and y.dtype in (torch.bfloat16, torch.float32)
            and K % 8 == 0 and (x.shape[0] == 1 or x.stride(0) % 8 == 0) and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and w.is_contiguous() and x.stride(1) == 1 and y.stride(1) == 1)


class LbRowScale(ctypes.Structure):
    """Mirror of RowScale in csrc/gemm_tcgen05.cu."""
    _fields_ = [("on", c_int), ("tiles", c_int), ("sumsq", c_void_p), ("inv_width", c_float), ("eps", c_float)]


def _row_scale(sumsq: torch.Tensor | None, width: int, eps: float):
    """The argument for rows that lack their norm's factor: None, or a reference to an LbRowScale."""
    if sumsq is None:
        return None
    _check(sumsq, "partial sums of squares", torch.float32)
    return ctypes.byref(LbRowScale(1, sumsq.shape[1], sumsq.data_ptr(), 1.0 / width, eps))


def gemm_tcgen05(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, stream: int, force_bt: int = 0,
                 force_splits: int = 0, swiglu: bool = False, sumsq: torch.Tensor | None = None, eps: float = 0.0) -> None:
    """y[M, N] = x[M, K] . w[N, K]^T on the tensor cores (tcgen05, accumulators in tensor memory).

    With `swiglu` the rows of w alternate in blocks of 64 between gate rows and up rows of the same 64
    features (see interleave_gate_up), and y[M, N/2] = silu(x . gate^T) * (x . up^T), formed in the epilogue.
    With `sumsq` [M, tiles] the rows of x lack the factor of an RMSNorm over K values: row m of the product is
    multiplied by rsqrt(sum(sumsq[m]) / K + eps), before the activation if there is one (see gemm_tcgen05_addnorm)."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(y.shape) != (M, N // 2 if swiglu else N):
        raise KernelError(f"gemm shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if not gemm_tcgen05_ok(y, x, w):
        raise KernelError("gemm_tcgen05 takes bfloat16 operands with K a multiple of 8, 16-byte aligned, unit column stride")
    ws, counters = _gemm_scratch(x.device)
    _call("lb_gemm_tcgen05", y.data_ptr(), dtype_code(y.dtype), x.data_ptr(), w.data_ptr(), M, N, K,
          x.stride(0) if M > 1 else K, y.stride(0) if M > 1 else y.shape[1], ws.data_ptr(), ws.numel(), counters.data_ptr(),
          counters.numel(), force_bt, force_splits, 1 if swiglu else 0, _row_scale(sumsq, K, eps), stream)


class LbHeadEpilogue(ctypes.Structure):
    """Mirror of HeadEpilogue in csrc/gemm_tcgen05.cu."""
    _fields_ = [("on", c_int), ("num_q_heads", c_int), ("num_kv_heads", c_int), ("page_size", c_int), ("max_pages", c_int),
                ("eps", c_float), ("positions", c_void_p), ("token_seq", c_void_p), ("block_table", c_void_p),
                ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("inv_freq", c_void_p), ("q_out", c_void_p),
                ("k_cache", c_void_p), ("v_cache", c_void_p)]


def gemm_tcgen05_heads_sizes_ok(M: int, N: int, K: int, head_dim: int) -> bool:
    """The sizes the q|k|v product with the head epilogue takes (heads of 128, at most 32 tokens, a split product)."""
    lib = library()
    lib.lb_gemm_tcgen05_heads_ok.argtypes = [c_int, c_int, c_int, c_int]
    lib.lb_gemm_tcgen05_heads_ok.restype = c_int
    return bool(lib.lb_gemm_tcgen05_heads_ok(M, N, K, head_dim))


def gemm_tcgen05_heads_ok(x: torch.Tensor, w: torch.Tensor, head_dim: int, rot_dim: int | None) -> bool:
    """The conditions of the q|k|v product whose epilogue norms, rotates and stores the heads: bfloat16, heads of
    128 rotated whole (or not at all), at most 32 tokens, a product that is split over a cluster."""
    lib = library()
    lib.lb_gemm_tcgen05_heads_ok.argtypes = [c_int, c_int, c_int, c_int]
    lib.lb_gemm_tcgen05_heads_ok.restype = c_int
    M, K = x.shape
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and x.stride(1) == 1
            and (M == 1 or x.stride(0) % 8 == 0) and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and rot_dim in (None, head_dim) and bool(lib.lb_gemm_tcgen05_heads_ok(M, w.shape[0], K, head_dim)))


def gemm_tcgen05_addnorm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """The conditions of the product whose epilogue adds to the residual stream: bfloat16, 16-byte alignment, and sizes
    for which the product is split over a thread-block cluster (few tokens, fewer output tiles than SMs)."""
    lib = library()
    lib.lb_gemm_tcgen05_addnorm_ok.argtypes = [c_int, c_int, c_int]
    lib.lb_gemm_tcgen05_addnorm_ok.restype = c_int
    M, K = x.shape
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and x.stride(1) == 1
            and (M == 1 or x.stride(0) % 8 == 0) and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(lib.lb_gemm_tcgen05_addnorm_ok(M, w.shape[0], K)))


def gemm_tcgen05_addnorm_tiles(M: int, N: int, K: int) -> int:
    """Columns of the partial sums of squares that gemm_tcgen05_addnorm writes for these sizes: blocks of 128 features
    with few tokens, the feature tiles the many-token product chooses otherwise (0: sizes it does not take)."""
    lib = library()
    lib.lb_gemm_tcgen05_addnorm_tiles.argtypes = [c_int, c_int, c_int]
    lib.lb_gemm_tcgen05_addnorm_tiles.restype = c_int
    return int(lib.lb_gemm_tcgen05_addnorm_tiles(M, N, K))


def gemm_tcgen05_addnorm(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, norm_w: torch.Tensor, out: torch.Tensor,
                         sumsq: torch.Tensor, stream: int) -> None:
    """residual += x . w^T; out = (residual * norm_w) rounded to bfloat16, without the factor rsqrt(mean(residual^2) + eps)
    of the RMSNorm; sumsq[m, t] = sum of residual[m]^2 over the t-th block of features (gemm_tcgen05_addnorm_tiles says
    how many blocks these sizes have).  The product that reads
    `out` is given `sumsq` and multiplies its sums by the row's factor (a row's factor commutes with a linear map), so
    the add, the copy and the norm between two products cost no kernel of their own."""
    M, K = x.shape
    N = w.shape[0]
    _check(w, "w", torch.bfloat16); _check(residual, "residual", torch.float32); _check(norm_w, "norm weight", torch.float32)
    _check(out, "normed output", torch.bfloat16); _check(sumsq, "partial sums of squares", torch.float32)
    if tuple(residual.shape) != (M, N) or tuple(out.shape) != (M, N) or sumsq.shape[0] != M or norm_w.shape[0] != N:
        raise KernelError(f"gemm_tcgen05_addnorm shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, residual {tuple(residual.shape)}, sumsq {tuple(sumsq.shape)}")
    _call("lb_gemm_tcgen05_addnorm", x.data_ptr(), w.data_ptr(), M, N, K, x.stride(0) if M > 1 else K, residual.data_ptr(),
          norm_w.data_ptr(), out.data_ptr(), sumsq.data_ptr(), sumsq.shape[1], stream)


def gemm_tcgen05_heads(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
                       block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, num_q_heads: int,
                       num_kv_heads: int, page_size: int, eps: float, stream: int, q_norm_w: torch.Tensor | None = None,
                       k_norm_w: torch.Tensor | None = None, inv_freq: torch.Tensor | None = None,
                       sumsq: torch.Tensor | None = None, row_eps: float = 0.0) -> None:
    """x . w^T for w = [q | k | v] rows with heads of 128, finished per head in the product's epilogue: RMSNorm of
    query and key heads, rotation, queries to q_out [M, nq, 128], keys and values into their cache pages.
    `sumsq`, `row_eps`: the rows of x lack their norm's factor (see gemm_tcgen05)."""
    M, K = x.shape
    _check(x, "x", torch.bfloat16); _check(w, "w", torch.bfloat16); _check(q_out, "q output", torch.bfloat16)
    _check(k_cache, "k pool", torch.bfloat16); _check(v_cache, "v pool", torch.bfloat16)
    _check(positions, "positions", torch.int32); _check(token_seq, "token map", torch.int32)
    _check(block_table, "block table", torch.int32)
    for t, what in ((q_norm_w, "q norm weight"), (k_norm_w, "k norm weight"), (inv_freq, "rotary table")):
        if t is not None:
            _check(t, what, torch.float32)
    he = LbHeadEpilogue(1, num_q_heads, num_kv_heads, page_size, block_table.shape[1], eps, positions.data_ptr(),
                        token_seq.data_ptr(), block_table.data_ptr(), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq),
                        q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr())
    _call("lb_gemm_tcgen05_heads", x.data_ptr(), w.data_ptr(), M, w.shape[0], K, x.stride(0) if M > 1 else K,
          ctypes.byref(he), _row_scale(sumsq, K, row_eps), stream)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[gate rows 0..63 | up rows 0..63 | gate rows 64..127 | up rows 64..127 | ...]: the row order the
    fused SwiGLU epilogue of gemm_tcgen05 expects.  The number of rows must be a multiple of 64."""
    I, K = gate.shape
    if up.shape != gate.shape or I % 64:
        raise KernelError(f"gate and up must have the same shape with a multiple of 64 rows, got {tuple(gate.shape)}, {tuple(up.shape)}")
    return torch.stack([gate.view(I // 64, 64, K), up.view(I // 64, 64, K)], dim=1).reshape(2 * I, K).contiguous()


def zero_rows(state: torch.Tensor, slots: torch.Tensor, stream: int) -> None:
    """state[slots[i]] = 0 for every non-negative entry of slots (int32, on the device)."""
    _check(state, "state"); _check(slots, "slot list", torch.int32)
    row_bytes = state[0].numel() * state.element_size()
    _call("lb_zero_rows", state.data_ptr(), row_bytes, state.shape[0], slots.data_ptr(), slots.shape[0], stream)


def upload(dst_ptr: int, src_ptr: int, nbytes: int, stream: int) -> None:
    """One asynchronous copy from pinned host memory to the device, in the order of `stream`."""
    _call("lb_upload", dst_ptr, src_ptr, nbytes, stream)


def launch_count() -> int:
    """Kernels the library has launched so far in this process."""
    lib = library()
    lib.lb_launch_count.restype = c_ulonglong
    return int(lib.lb_launch_count())


def device_error() -> int:
    """Code that a kernel left when one of its bounded waits gave up (0: none).  Synchronises the device."""
    lib = library()
    lib.lb_device_error.restype = c_int
    lib.lb_attention_tcgen05_device_error.restype = c_int
    lib.lb_attention_flash_device_error.restype = c_int
    return (int(lib.lb_device_error()) or int(lib.lb_attention_tcgen05_device_error())
            or int(lib.lb_attention_flash_device_error()))


def linear(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, stream: int, fast: bool) -> None:
    """y = x . w^T.  `fast` allows the tensor-core kernel where its conditions hold (otherwise, and
    always on the 32-bit path, the product runs on the ordinary pipes)."""
    if fast and gemm_tcgen05_ok(y, x, w):
        gemm_tcgen05(y, x, w, stream)
    else:
        gemm_plain(y, x, w, stream)


_attn_ws: dict[int, torch.Tensor] = {}
_attn_ws_retired: list[torch.Tensor] = []


def _attention_workspace(device: torch.device, elems: int) -> torch.Tensor:
    """Per device: float32 scratch for the partial results of split attention; grows on demand.

    A recorded CUDA graph keeps the address of the workspace it was recorded with, so a workspace that has
    been handed out is never freed: when a larger one is needed the old one is retired, not released (it stays
    valid for the recordings that name it; launches are ordered on one stream, so sharing it is safe).  Sizes at
    least double, which bounds what the retired ones hold to the size of the current one."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _attn_ws.get(key)
    if ws is None or ws.numel() < elems:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the attention workspace cannot grow while a CUDA graph is captured; run the step once before")
        if ws is not None:
            _attn_ws_retired.append(ws)
        ws = torch.empty(max(elems, 1 << 20, 2 * ws.numel() if ws is not None else 0), dtype=torch.float32, device=device)
        _attn_ws[key] = ws
    return ws


def attention_flash_ok(q: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """The conditions of the tensor-core attention kernel."""
    return (q.dtype == torch.bfloat16 and head_dim % 8 == 0 and 8 <= head_dim <= 128
            and num_q_heads % num_kv_heads == 0 and num_q_heads // num_kv_heads <= 64)


def attention_splits(num_tiles: int, num_kv_heads: int, max_span: int, max_rows: int = 64, slots: int = 296,
                     wide_clusters: int = 0) -> int:
    """Into how many key ranges a launch is cut.  `slots` is how many CTAs run at a time (two on each
    of the 148 SMs).  Fewer CTAs than slots: as many ranges as still fit one wave; for tiles of up to
    16 query rows a count below 16 becomes a power of two, because up to 8 ranges of such tiles combine
    inside a thread-block cluster instead of through a workspace and a second kernel.  More CTAs than
    slots: the count (up to 8) that costs least by a model of the last wave and of the CTAs' fixed costs.  A range
    has 256 keys at least.  `wide_clusters`: how many clusters of 16 CTAs the GPU keeps resident (0: none); a launch of
    at most that many tiles x kv heads over up to 24 K keys that would take 16 or more ranges takes 16 in such clusters
    (one request of 8 kv heads at 8 K keys: 12.9 us against 17.5 us with 32 ranges through the workspace)."""
    base = max(num_tiles * num_kv_heads, 1)
    cap = max(1, min(max_span // 256, 64))
    if max_rows > 16 and base >= slots // 2:
        return 1         # portions of prompts fill the SMs by themselves; cutting them only adds partial results
    if base <= slots:
        s = max(1, min(slots // base, cap))
        if max_rows <= 16 and s < 16:
            s = 8 if s >= 8 else 4 if s >= 4 else 2 if s >= 2 else 1
        elif max_rows <= 16 and base <= wide_clusters and max_span <= 24576:
            s = 16
        return s
    # More tiles than slots.  The memory is busy as long as about half the slots are filled, so only a last wave of fewer
    # CTAs than that costs (the more the longer a CTA runs), and every CTA costs its start and its end: measured,
    # about 6 us of a slot per CTA, 0.022 us per key of a CTA's range while a full wave shares the memory.
    best, best_cost = 1, float("inf")
    for s in range(1, min(cap, 8) + 1):
        rest = (base * s) % slots
        tail = 0.6 * (0.022 * max_span / s) * max(0.0, 1.0 - rest / (slots / 2)) if rest else 0.0
        cost = 6.0 * base * s / slots + tail
        if cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


_wide_clusters: dict[int, int] = {}


def attention_wide_clusters(head_dim: int) -> int:
    """How many clusters of 16 CTAs of the decode attention kernel the GPU keeps resident at a time (0: it does not
    schedule clusters of that size)."""
    key = 64 if head_dim <= 64 else 128
    if key not in _wide_clusters:
        lib = library()
        lib.lb_attention_flash_wide_clusters.restype = c_int
        lib.lb_attention_flash_wide_clusters.argtypes = [c_int]
        _wide_clusters[key] = max(0, int(lib.lb_attention_flash_wide_clusters(key)))
    return _wide_clusters[key]


def attention_flash(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    positions: torch.Tensor, block_table: torch.Tensor, tiles: torch.Tensor, max_rows: int,
                    num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                    splits: int, stream: int, force_workspace: bool = False, tma: bool = True) -> None:
    """Tensor-core attention over pages.  tiles: int32 [n, 4] of (first token, tokens, request index, 0).
    `force_workspace` sends the partial results of the splits through the workspace and the combining
    kernel even where a cluster could combine them.  Tiles of at most 16 query rows (decoded tokens) over pages of
    8 to 128 tokens run in the kernel whose keys and values a warp of its own fetches by TMA; `tma=False` keeps them
    in the kernel that fetches with 16-byte copies, which takes every page size."""
    _check(q, "q", torch.bfloat16); _check(out, "attention output", torch.bfloat16)
    _check(k_cache, "k pool", torch.bfloat16); _check(v_cache, "v pool", torch.bfloat16)
    _check(positions, "positions", torch.int32); _check(block_table, "block table", torch.int32)
    _check(tiles, "tiles", torch.int32)
    n = tiles.shape[0]
    ws, ws_elems = None, 0
    by_tma = tma and max_rows <= 16 and page_size in (8, 16, 32, 64, 128)
    in_cluster = max_rows <= 16 and not force_workspace and (2 <= splits <= 8 or (splits <= 16 and by_tma))
    if splits > 1 and not in_cluster:
        ws_elems = n * num_kv_heads * splits * max_rows * (head_dim + 2)
        ws = _attention_workspace(q.device, ws_elems)
        ws_elems = ws.numel()
    _call("lb_attention_flash", q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
          positions.data_ptr(), block_table.data_ptr(), tiles.data_ptr(), n, num_q_heads, num_kv_heads, head_dim,
          page_size, block_table.shape[1], k_cache.shape[0] if tma else 0, window, scale,
          -splits if force_workspace else splits, max_rows, _ptr(ws), ws_elems, stream)


def attention_tcgen05_ok(q: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                         max_pages: int = 0) -> bool:
    """The conditions of the tensor-memory attention kernel: bfloat16, head size 128, at most 128 query heads per
    kv head, pages of 8, 16, 32, 64 or 128 tokens, at most 4096 pages a request."""
    lib = library()
    lib.lb_attention_tcgen05_ok.restype = c_int
    return (q.dtype == torch.bfloat16 and max_pages <= 4096
            and bool(lib.lb_attention_tcgen05_ok(num_q_heads, num_kv_heads, head_dim, page_size)))


def attention_tcgen05_splits(num_tiles: int, num_kv_heads: int, max_span: int, sms: int = 148) -> int:
    """Into how many key ranges the work items of the tensor-memory kernel are cut.  A CTA takes a whole SM, so a launch
    of fewer CTAs than SMs (one portion of a few hundred tokens behind a long context) leaves SMs idle for as long as
    its longest item lasts, and one of a few more CTAs than SMs runs a second round for them.  By a model fitted to
    measurements (8 kv heads, items of 64 tokens): a CTA takes 6 us plus 0.0177 us per key it visits (8 us when it
    leaves partial results), the launch as many rounds of that as its CTAs need on the SMs, and the second kernel
    6 us plus 0.06 us per CTA (266 KB of partial results written and read again).  A cut must promise 5 % at least.  64 CTAs behind 7680 keys: 140 us whole, 87 us in two ranges; 8 CTAs behind 16 K keys:
    240 and 43 us in eight.  A range has four blocks of 64 keys at least.  The count depends on the launch's shape alone
    (tiles, kv heads, the bound of the context), never on where the requests stand, so a recorded step keeps it; it
    takes every item to see `max_span` keys, which overrates whole prompts, whose items see half of that on average,
    but those either fill the SMs many times over or are short."""
    ctas = max(num_tiles * num_kv_heads, 1)
    per_key = 0.0177 * max_span
    best, best_cost = 1, -(-ctas // sms) * (6.0 + per_key)
    for s in range(2, min(8, max_span // 256) + 1):
        cost = -(-ctas * s // sms) * (8.0 + per_key / s) + 6.0 + 0.06 * ctas * s
        if cost < 0.95 * best_cost:
            best, best_cost = s, cost
    return best


def attention_tcgen05(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      positions: torch.Tensor, block_table: torch.Tensor, tiles: torch.Tensor, num_q_heads: int,
                      num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float, stream: int,
                      key_splits: int = 1) -> None:
    """Attention of portions of prompts on tcgen05 (S and O in tensor memory).  tiles: int32 [n, 4] of
    (first token, tokens, request index, 0) with tokens <= 2 * (128 // (nq // nkv)).  With key_splits > 1 the keys of
    every tile are cut into that many ranges, a CTA each, combined by a second kernel."""
    _check(q, "q", torch.bfloat16); _check(out, "attention output", torch.bfloat16)
    _check(k_cache, "k pool", torch.bfloat16); _check(v_cache, "v pool", torch.bfloat16)
    _check(positions, "positions", torch.int32); _check(block_table, "block table", torch.int32)
    _check(tiles, "tiles", torch.int32)
    ws, ws_elems = None, 0
    if key_splits > 1:
        ws = _attention_workspace(q.device, tiles.shape[0] * num_kv_heads * key_splits * 256 * (head_dim + 2))
        ws_elems = ws.numel()
    _call("lb_attention_tcgen05", q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
          positions.data_ptr(), block_table.data_ptr(), tiles.data_ptr(), tiles.shape[0], q.shape[0], num_q_heads,
          num_kv_heads, head_dim, page_size, k_cache.shape[0], block_table.shape[1], window, scale, key_splits,
          _ptr(ws), ws_elems, stream)


def attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, step, group: int,
              num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
              stream: int, plan=None) -> None:
    """Causal attention of this step's queries over the pages of their requests.  With a `plan` (tile lists
    by kind on the device, see parts/attention.py) the tensor-core kernels run where their conditions hold:
    portions of prompts go to the tcgen05 kernel, the rest (decoded tokens, short portions, other head
    sizes) to the mma.sync kernels; everything else, and every step without a plan, goes to the plain kernel."""
    if plan is None or not attention_flash_ok(q, num_q_heads, num_kv_heads, head_dim):
        attention_plain(q, out, k_cache, v_cache, step.positions, step.token_seq, step.block_tables[group],
                        num_q_heads, num_kv_heads, head_dim, page_size, window, scale, stream)
        return
    meta, most_rows = plan.arrays, plan.host["rows"]
    longest = step.span_hint or step.max_context_len                 # a recorded step plans for a bucket of lengths
    span = min(longest, window + step.max_q_len) if window > 0 else longest
    kinds = ["all"]
    if "big" in meta and attention_tcgen05_ok(q, num_q_heads, num_kv_heads, head_dim, page_size,
                                              step.block_tables[group].shape[1]):
        attention_tcgen05(q, out, k_cache, v_cache, step.positions, step.block_tables[group], meta["big"],
                          num_q_heads, num_kv_heads, head_dim, page_size, window, scale, stream,
                          key_splits=attention_tcgen05_splits(meta["big"].shape[0], num_kv_heads, span))
        kinds = ["rest"] if "rest" in meta else []
    for kind in kinds:
        tiles = meta[kind]
        rows = min(most_rows[kind], 64)
        wide = attention_wide_clusters(head_dim) if rows <= 16 and page_size in (8, 16, 32, 64, 128) else 0
        splits = attention_splits(tiles.shape[0], num_kv_heads, span, rows, wide_clusters=wide)
        attention_flash(q, out, k_cache, v_cache, step.positions, step.block_tables[group], tiles, rows,
                        num_q_heads, num_kv_heads, head_dim, page_size, window, scale, splits, stream)
