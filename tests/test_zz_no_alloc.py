"""``ug_gemm_noalloc``: the GEMM entry point for callers that may not allocate device memory
(runtime plug-in callbacks that only get pre-allocated buffers, processes whose GPU memory is
fully reserved by another allocator, loops that cannot take cudaMalloc's implicit
synchronisation).  All its scratch - descriptors, tables, counters, staging - is one static
device array inside the library.

The test calls the exported C symbol directly through ctypes, twice in a row per case (the
second call reuses the array and must clear the first call's counters), and compares with the
regular entry point (``ops.gemm.gemm``, whose tables and staging are torch allocations) within
the tolerance the other kernel tests use.  It also checks that an oversized problem is rejected
without a launch.  This file sorts last so that a ``-x`` run has finished every other test first.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from universal_gemm_b200.ops import native

    fn = native.lib().ug_gemm_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_uint64, ctypes.c_int64, ctypes.c_uint64, ctypes.c_int64, ctypes.c_uint64, ctypes.c_int64,
                   ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64,
                   ctypes.c_void_p]
    return fn


def _call(fn, a, b, c, mode, status):
    stream = torch.cuda.current_stream(c.device).cuda_stream
    code = 0 if c.dtype == torch.float32 else 1
    return fn(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), c.data_ptr(), c.stride(0), c.shape[0], c.shape[1],
              a.shape[1], code, mode, 0 if status is None else status.data_ptr(), ctypes.c_void_p(stream))


@pytest.mark.parametrize("m,n,k,pad", [(256, 512, 384, 0),      # aligned: tables only
                                       (300, 520, 200, 0),      # aligned pitches, ragged tiles
                                       (200, 333, 264, 3),      # odd pitches: A and B staged in the static array
                                       (130, 1000, 1001, 1)])
@pytest.mark.parametrize("c_dtype", [torch.float32, torch.bfloat16])
def test_noalloc_matches_regular_entry_point(m, n, k, pad, c_dtype):
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.gemm import gemm

    dev = torch.device("cuda", 0)
    fn = _entry()
    torch.manual_seed(m * 7 + n + k)
    a = torch.randn(m, k + pad, device=dev).bfloat16()[:, :k]
    b = (torch.randn(k, n + pad, device=dev) / k ** 0.5).bfloat16()[:, :n]
    c0 = torch.randn(m, n, device=dev).to(c_dtype)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    tol = 2e-3 if c_dtype == torch.float32 else 3e-2

    # call 1: C = A @ B ; call 2 right after it: C += A @ B
    c_new, c_ref = c0.clone(), c0.clone()
    assert _call(fn, a, b, c_new, native.C_STORE, status) == 0
    assert _call(fn, a, b, c_new, native.C_ADD, status) == 0
    gemm(a, b, c_ref, mode=native.C_STORE)
    gemm(a, b, c_ref, mode=native.C_ADD)
    torch.cuda.synchronize()
    assert status.item() == 0
    torch.testing.assert_close(c_new.float(), c_ref.float(), rtol=tol, atol=tol)
    want = 2 * (a.float() @ b.float())
    torch.testing.assert_close(c_new.float(), want, rtol=tol * 2, atol=tol * 2)


def test_noalloc_rejects_what_does_not_fit(capfd):
    from universal_gemm_b200.ops import native

    dev = torch.device("cuda", 0)
    fn = _entry()
    m, n, k = 128, 4099, 1024            # B has an odd pitch -> 1024 x 4160 bf16 staging > the static array
    a = torch.zeros(m, k, device=dev, dtype=torch.bfloat16)
    b = torch.zeros(k, n, device=dev, dtype=torch.bfloat16)
    c = torch.full((m, n), 7.0, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    assert _call(fn, a, b, c, native.C_STORE, status) == -2
    assert "static" in capfd.readouterr().err
    assert _call(fn, a, b, c, 1, status) == -1          # atomic mode is not offered here
    torch.cuda.synchronize()
    assert c.min().item() == 7.0 and status.item() == 0  # nothing ran


def test_noalloc_leaves_free_memory_unchanged_and_can_keep_its_own_status_word():
    """The property the entry point exists for: once the first call on the device has done its set-up, further
    calls change the amount of free device memory by nothing, whether or not operands have to be staged.  The
    calls here also pass no status word (``status_ptr = 0``): the kernel then reports into a word inside the
    static array, and the results must still match the regular entry point."""
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.gemm import gemm

    dev = torch.device("cuda", 0)
    fn = _entry()
    torch.manual_seed(77)
    cases = []
    for m, n, k, pad in ((256, 512, 384, 0), (200, 333, 264, 3)):
        a = torch.randn(m, k + pad, device=dev).bfloat16()[:, :k]
        b = (torch.randn(k, n + pad, device=dev) / k ** 0.5).bfloat16()[:, :n]
        cases.append((a, b, torch.zeros(m, n, device=dev), torch.zeros(m, n, device=dev)))
    for a, b, _, c_ref in cases:                          # the regular entry point allocates tables and staging
        gemm(a, b, c_ref, mode=native.C_STORE)
    assert _call(fn, *cases[0][:3], native.C_STORE, None) == 0      # first call on the device: set-up included
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(dev)[0]
    for _ in range(2):
        for a, b, c_new, _ in cases:
            assert _call(fn, a, b, c_new, native.C_STORE, None) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(dev)[0] == free_before
    for a, b, c_new, c_ref in cases:
        torch.testing.assert_close(c_new, c_ref, rtol=2e-3, atol=2e-3)
