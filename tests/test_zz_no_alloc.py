"""The allocation-free GEMV entry point, called the way a C host would call it.

Some hosts cannot allocate device memory where they need a GEMV: a serving
loop whose memory all belongs to a pool, a plugin inside another process, a
region that must not synchronise.  `smr_gemv_bf16_noalloc` serves them from a
small array compiled into the library.  This test loads the exported C
symbol with ctypes (no Python binding in between), runs it twice in a row and
compares each result with the library's regular op, which allocates its
workspace through `symm_mem`.  It is collected last so that a failure here
cannot hide another test's result.
"""
import ctypes

import pytest
import torch


def _entry():
    from symm_mem_recipes_b200._ext import C

    lib = ctypes.CDLL(C.__file__)
    fn = lib.smr_gemv_bf16_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    return fn


def _status():
    from symm_mem_recipes_b200._ext import C

    lib = ctypes.CDLL(C.__file__)
    fn = lib.smr_gemv_bf16_noalloc_status
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint * 6), ctypes.c_char_p, ctypes.c_int]
    record = (ctypes.c_uint * 6)()
    err = ctypes.create_string_buffer(256)
    rc = fn(torch.cuda.current_stream().cuda_stream, ctypes.byref(record), err, 256)
    return rc, list(record), err.value.decode()


def _call(fn, x, w, out):
    err = ctypes.create_string_buffer(256)
    rc = fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], w.shape[1],
            torch.cuda.current_stream().cuda_stream, err, 256)
    return rc, err.value.decode()


@pytest.mark.gpu
@pytest.mark.parametrize("B,K,N", [(4, 3584, 8192), (16, 1024, 2048)])
def test_noalloc_gemv_matches_the_allocating_op_twice(B, K, N):
    import symm_mem_recipes_b200 as smr

    torch.cuda.set_device(0)
    fn = _entry()
    g = torch.Generator().manual_seed(B + K + N)
    for call in range(2):                      # second call reuses whatever the first left in the scratch
        x = (torch.randn(B, K, generator=g) * 0.5).to(torch.bfloat16).cuda()
        w = (torch.randn(K, N, generator=g) * 0.05).to(torch.bfloat16).cuda()
        out = torch.full((B, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc, msg = _call(fn, x, w, out)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before      # nothing taken from the framework's allocator
        rc, record, msg = _status()                         # the kernel ran to its end: no wait ran out
        assert rc == 0 and record[0] == 0, (rc, record, msg)
        expect = smr.gemv_all_reduce(x, w)                  # world of one: the plain product
        torch.cuda.synchronize()
        ref = x.double() @ w.double()
        tol = ref.abs() * 2.0 ** -7 + 2e-2
        assert bool(((out.double() - ref).abs() <= tol).all()), f"call {call}: differs from fp64"
        assert torch.allclose(out.float(), expect.float(), rtol=2e-2, atol=2e-2), f"call {call}"


@pytest.mark.gpu
def test_noalloc_gemv_refuses_what_does_not_fit():
    torch.cuda.set_device(0)
    fn = _entry()
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(64, 8192 + 8, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(4, 8192 + 8, dtype=torch.bfloat16, device="cuda")
    rc, msg = _call(fn, x, w, out)
    assert rc == 1 and "8192" in msg           # beyond the static scratch: refused, nothing launched
    x17 = torch.zeros(17, 64, dtype=torch.bfloat16, device="cuda")
    w2 = torch.zeros(64, 128, dtype=torch.bfloat16, device="cuda")
    out2 = torch.zeros(17, 128, dtype=torch.bfloat16, device="cuda")
    rc, msg = _call(fn, x17, w2, out2)
    assert rc == 1 and "batch" in msg
    torch.cuda.synchronize()


@pytest.mark.gpu
def test_noalloc_gemv_after_a_call_of_another_shape():
    """Calls of different shapes (different tile counts and K splits) share the one static array:
    alternating them stays correct and the status record stays clear."""
    torch.cuda.set_device(0)
    fn = _entry()
    g = torch.Generator().manual_seed(5)
    for B, K, N in [(2, 512, 8192), (2, 512, 256), (2, 512, 8192), (16, 4096, 1024), (2, 512, 8192)]:
        x = (torch.randn(B, K, generator=g) * 0.5).to(torch.bfloat16).cuda()
        w = (torch.randn(K, N, generator=g) * 0.05).to(torch.bfloat16).cuda()
        out = torch.full((B, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc, msg = _call(fn, x, w, out)
        assert rc == 0, msg
        rc, record, msg = _status()
        assert rc == 0 and record[0] == 0, (rc, record, msg)
        ref = x.double() @ w.double()
        assert bool(((out.double() - ref).abs() <= ref.abs() * 2.0 ** -7 + 2e-2).all()), (B, K, N)
