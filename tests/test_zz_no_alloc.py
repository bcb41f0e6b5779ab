"""The allocation-free form of the re-quantising int8 Linear, called straight through the C ABI.

``samb_gemm_i8_requant_static`` is for hosts that cannot hand the library any scratch memory (a plug-in without
access to its server's memory pool, a process whose device memory was given out in full at start-up, a real-time
loop that keeps away from the allocator): it takes inputs and outputs only and keeps its one float of scratch per output row
in an array inside the library's device image.  This test checks it against ``samb_gemm_i8_requant`` (same kernels,
caller-supplied scratch) on two calls in a row, since the built-in array keeps whatever the previous call left in
it, and checks that more rows than the array holds are refused.  The file sorts last on purpose: a run that stops
at the first failure has then already been through every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, fn, xq, sx, wq, sw, bias, out, yq, ys, scratch, epi, status):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    M, K = xq.shape
    N = wq.shape[0]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if scratch is None:
        return fn(p(xq), xq.stride(0), p(sx), p(wq), wq.stride(0), p(sw), p(bias), p(out), out.stride(0), p(yq), p(ys),
                  M, N, K, epi, p(status), stream)
    return fn(p(xq), xq.stride(0), p(sx), p(wq), wq.stride(0), p(sw), p(bias), p(out), out.stride(0), p(yq), p(ys),
              p(scratch), M, N, K, epi, p(status), stream)


def test_requant_without_allocation_matches_the_scratch_form_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from segment_anything_fast_b200 import _lib
    lib = _lib.load()
    assert lib.samb_gemm_i8_requant_static_max_rows() == 262144
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(77)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    epi = _lib.EPI_BIAS | _lib.EPI_GELU
    # two products of different sizes, the larger one first: the second call meets the first call's leftovers
    for M, N, K in [(4096 + 37, 512, 1280), (1000, 256, 320)]:
        xq = torch.randint(-127, 128, (M, K), generator=g, device=dev, dtype=torch.int8)
        wq = torch.randint(-127, 128, (N, K), generator=g, device=dev, dtype=torch.int8)
        sx = torch.rand(M, generator=g, device=dev) * 0.02 + 0.001
        sw = torch.rand(N, generator=g, device=dev) * 0.002 + 0.0001
        bias = torch.randn(N, generator=g, device=dev) * 0.1
        ref = [torch.empty(M, N, dtype=torch.bfloat16, device=dev), torch.empty(M, N, dtype=torch.int8, device=dev),
               torch.empty(M, dtype=torch.float32, device=dev)]
        scratch = torch.full((M,), 123.0, dtype=torch.float32, device=dev)         # stale contents must not matter
        rc = _call(lib, lib.samb_gemm_i8_requant, xq, sx, wq, sw, bias, *ref, scratch, epi, status)
        assert rc == 0, _lib.error_string(rc)
        for _ in range(2):
            got = [torch.zeros_like(t) for t in ref]
            rc = _call(lib, lib.samb_gemm_i8_requant_static, xq, sx, wq, sw, bias, *got, None, epi, status)
            assert rc == 0, _lib.error_string(rc)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            # integer outputs and scales are exact in both forms; the bf16 output comes from the same GEMM launch
            for a, b, name in zip(got, ref, ("out", "yq", "y_scale")):
                assert torch.equal(a, b), name
    # more rows than the built-in array holds: refused on the host, nothing launched, nothing read
    one = torch.zeros(16, dtype=torch.int8, device=dev)
    f = torch.zeros(16, dtype=torch.float32, device=dev)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.samb_gemm_i8_requant_static(p(one), 16, p(f), p(one), 16, p(f), p(f), p(one), 8, p(one), p(f),
                                         262144 + 1, 8, 16, epi, p(status), None)
    assert rc == -2 and b"shape" in lib.samb_error_string(rc)
