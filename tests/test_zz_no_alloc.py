"""The matrix product for callers that cannot allocate device memory, called through its exported C
symbol (GPU).  This file is named so that pytest collects it last.

lb_gemm_tcgen05_static_scratch keeps its scratch (partial sums and tile counters of a product whose K
is split) in an array inside the library, for callers that have no allocator to ask: a host that gave
all device memory to its own pool, a loop that must not take cudaMalloc's device-wide synchronisation,
a program in another language.  The test calls it twice in a row, with different inputs, and compares
each result with the ordinary entry point, which gets its scratch from the caller."""
import ctypes
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

PARTIALS, COUNTERS = 2 * 1024 * 1024, 1024        # LB_STATIC_SCRATCH_PARTIALS, LB_STATIC_SCRATCH_COUNTERS


def static_scratch_fn():
    from lucciola_b200.csrc import library
    lib = library()
    fn = lib.lb_gemm_tcgen05_static_scratch
    fn.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p]
    fn.restype = c_int
    return lib, fn


def rel(a, b):
    return ((a.double() - b.double()).abs().max() / b.double().abs().max()).item()


@pytest.mark.parametrize("M,N,K,ydt", [(8, 4096, 4096, torch.bfloat16), (3, 1000, 776, torch.float32), (64, 384, 2048, torch.bfloat16),
                                      (300, 512, 256, torch.bfloat16)])
def test_two_calls_in_a_row_equal_the_ordinary_entry_point(M, N, K, ydt):
    from lucciola_b200 import ops
    lib, fn = static_scratch_fn()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                                 # the second call finds what the first left in the scratch
        g = torch.Generator(device=dev).manual_seed(100 * call + M)
        x = (torch.randn(M, K, device=dev, generator=g) * (1 + call)).bfloat16()
        w = torch.randn(N, K, device=dev, generator=g).bfloat16()
        want = torch.empty(M, N, device=dev, dtype=ydt)
        ops.gemm_tcgen05(want, x, w, stream)
        got = torch.full((M, N), float("nan"), device=dev, dtype=ydt)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(dev)
        free_before = torch.cuda.mem_get_info(dev)[0]       # the driver's own count: it sees a cudaMalloc that torch's does not
        rc = fn(got.data_ptr(), ops.dtype_code(ydt), x.data_ptr(), w.data_ptr(), M, N, K, K, N, stream)
        assert rc == 0, lib.lb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before
        if call == 1:       # the first call on a device may load the kernel's code; from the second on nothing may change
            assert torch.cuda.mem_get_info(dev)[0] >= free_before
        assert ops.device_error() == 0
        tol = 2e-6 if ydt == torch.float32 else 5e-3        # the tolerances of tests/test_kernels_gpu.py
        assert rel(got, x.double() @ w.double().t()) < tol
        assert rel(got, want) < tol


def test_sizes_beyond_the_built_in_scratch_are_refused():
    from lucciola_b200 import ops
    lib, fn = static_scratch_fn()
    dev = torch.device("cuda:0")
    M, N, K = 256, 6144, 4096                             # a split product: splits x 1.57 M partial sums > 2 M
    x = torch.zeros(M, K, device=dev, dtype=torch.bfloat16)
    w = torch.zeros(N, K, device=dev, dtype=torch.bfloat16)
    y = torch.full((M, N), 7.0, device=dev, dtype=torch.bfloat16)
    rc = fn(y.data_ptr(), ops.BF16, x.data_ptr(), w.data_ptr(), M, N, K, K, N, torch.cuda.current_stream().cuda_stream)
    msg = lib.lb_last_error().decode()
    assert rc != 0 and "built-in scratch holds" in msg and str(PARTIALS) in msg
    torch.cuda.synchronize()
    assert (y == 7.0).all()                               # nothing was launched
