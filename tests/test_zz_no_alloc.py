"""The allocation-free decode entry point, qmm_quant_matmul_decode_noalloc.

It serves callers that must not allocate while they run (a server that split its device memory up at
start-up, a plugin under a no-allocation-after-init rule), so its split-K scratch is an array inside
the library image instead of a buffer from the caller.  The test drives it through the C ABI and
requires the very same bits as the regular entry point, on two calls in a row (the second call finds
the array as the first one left it), for both weight layouts and output types, and checks that a
problem too large for the built-in array is refused with a clear message.

Collected last on purpose: a failure here cannot hide the other tests from a run that stops at the
first failure.  It passes on its own in a fresh process and after the rest of the suite.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _noalloc(capi, a, w, scale, pt, bias, out_dtype):
    M, K = a.shape
    N = w.shape[1]
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    rc = capi.lib().qmm_quant_matmul_decode_noalloc(
        a.data_ptr(), K, w.data_ptr(), w.stride(0), w.stride(1),
        None if scale is None else scale.data_ptr(), 0 if scale is None else scale.numel(),
        None if pt is None else pt.data_ptr(), None if bias is None else bias.data_ptr(),
        capi.DTYPE_NONE if bias is None else capi.dtype_code(bias.dtype), out.data_ptr(),
        capi.dtype_code(out_dtype), N, M, N, K, torch.cuda.current_stream().cuda_stream)
    capi.check(rc, "qmm_quant_matmul_decode_noalloc")
    return out


@pytest.mark.parametrize("shape", [(1, 8192, 2048), (8, 1040, 1008), (33, 4096, 7168), (128, 2048, 4096)])
def test_same_bits_as_the_regular_entry_point_twice_in_a_row(capi, dev, shape):
    M, K, N = shape
    g = torch.Generator(device=dev).manual_seed(M * 13 + N)
    for call in range(2):
        a = torch.randint(-127, 128, (M, K), generator=g, device=dev, dtype=torch.int8)
        w = torch.randint(-127, 128, (K, N), generator=g, device=dev, dtype=torch.int8)
        scale = torch.empty(N, device=dev).uniform_(1e-3, 1e-2, generator=g)
        pt = torch.empty(M, device=dev).uniform_(1e-2, 5e-2, generator=g)
        bias = (torch.randn(N, generator=g, device=dev) * 0.1).to(torch.bfloat16)
        want = capi.quant_matmul(a, w, scale, pertoken_scale=pt, bias=bias, output_dtype=torch.bfloat16,
                                 algo=capi.ALGO_STREAMK)
        got = _noalloc(capi, a, w, scale, pt, bias, torch.bfloat16)
        assert torch.equal(got, want), f"call {call}: bf16 output differs"  # tolerance: none, bit-identical
        want_i = capi.quant_matmul(a, w, None, output_dtype=torch.int32, algo=capi.ALGO_STREAMK)
        got_i = _noalloc(capi, a, w, None, None, None, torch.int32)
        assert torch.equal(got_i, want_i), f"call {call}: int32 accumulator differs"
        # the transposed view of an [N,K] weight
        wt = w.t().contiguous().t()
        got_t = _noalloc(capi, a, wt, scale, pt, bias, torch.bfloat16)
        assert torch.equal(got_t, want), f"call {call}: K-major weight differs"


def test_sizes_beyond_the_builtin_scratch_are_refused(capi, dev):
    lib = capi.lib()
    M, K, N = 128, 128, 32768  # 256 tiles x 64 KiB of partial sums + counters > 16 MiB
    a = torch.zeros((M, K), dtype=torch.int8, device=dev)
    w = torch.zeros((K, N), dtype=torch.int8, device=dev)
    out = torch.empty((M, N), dtype=torch.int32, device=dev)
    rc = lib.qmm_quant_matmul_decode_noalloc(a.data_ptr(), K, w.data_ptr(), N, 1, None, 0, None, None,
                                             capi.DTYPE_NONE, out.data_ptr(), capi.DTYPE_I32, N, M, N, K,
                                             torch.cuda.current_stream().cuda_stream)
    assert rc == 6 and b"built-in buffer holds 16777216" in lib.qmm_last_error()
    # the largest N that fits at M = 128 is accepted
    N = 32640
    w = torch.ones((K, N), dtype=torch.int8, device=dev)
    a.fill_(1)
    got = _noalloc(capi, a, w, None, None, None, torch.int32)
    assert int(got.min()) == K and int(got.max()) == K
    # prefill-sized M is not this entry point's business
    big = torch.zeros((256, K), dtype=torch.int8, device=dev)
    out2 = torch.empty((256, N), dtype=torch.int32, device=dev)
    rc = lib.qmm_quant_matmul_decode_noalloc(big.data_ptr(), K, w.data_ptr(), N, 1, None, 0, None, None,
                                             capi.DTYPE_NONE, out2.data_ptr(), capi.DTYPE_I32, N, 256, N, K,
                                             torch.cuda.current_stream().cuda_stream)
    assert rc == 2 and b"1 <= M <= 128" in lib.qmm_last_error()


def test_allocates_nothing_and_reports_timeouts_in_its_own_word(capi, dev):
    """The claim in the name: the device's free memory is the same before and after a call (the first call on
    a device looked the array's address up earlier in this file), and the entry point's own status word - the
    one a timed-out wait would mark - reads 0 after correct runs."""
    M, K, N = 16, 2048, 4096
    a = torch.randint(-127, 128, (M, K), device=dev, dtype=torch.int8)
    w = torch.randint(-127, 128, (K, N), device=dev, dtype=torch.int8)
    out = torch.empty((M, N), dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    lib = capi.lib()

    def call():
        rc = lib.qmm_quant_matmul_decode_noalloc(a.data_ptr(), K, w.data_ptr(), N, 1, None, 0, None, None,
                                                 capi.DTYPE_NONE, out.data_ptr(), capi.DTYPE_I32, N, M, N, K, stream)
        capi.check(rc, "qmm_quant_matmul_decode_noalloc")

    call()  # set-up, if this test runs alone
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"device free memory changed by {free_before - free_after} bytes"
    assert torch.equal(out, capi.quant_matmul(a, w, None, output_dtype=torch.int32, algo=capi.ALGO_STREAMK))
    assert lib.qmm_noalloc_status(0) == 0
