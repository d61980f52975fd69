"""fdk_gemm_static, the tensor-core contraction that allocates nothing: its output against fdk_gemm's
tensor-core path through the C ABI, on two calls in a row that share the built-in scratch array, and its
refusal of matrices beyond the array's size.  Collected last on purpose: the array outlives every call,
so this file must pass both in a fresh process and after all other tests have used the library."""
import numpy as np
import pytest

import fdeep_b200
from fdeep_b200 import capi
from util import assert_close

pytestmark = pytest.mark.gpu


def run_pair(M, N, K, seed, relu):
    """One shape through the allocating entry point and through the static one; returns both results."""
    import torch
    g = torch.Generator(device="cpu").manual_seed(seed)
    A = torch.randn(M, K, generator=g).cuda()
    W = torch.randn(N, K, generator=g).cuda()
    bias = torch.randn(N, generator=g).cuda()
    want = torch.full((M, N), float("nan"), device="cuda")
    got = torch.full((M, N), float("nan"), device="cuda")
    torch.cuda.synchronize()
    capi.gemm(1, A.data_ptr(), K, W.data_ptr(), K, want.data_ptr(), N, M, N, K, d_bias=bias.data_ptr(), relu=relu)
    capi.gemm_static(A.data_ptr(), K, W.data_ptr(), K, got.data_ptr(), N, M, N, K, d_bias=bias.data_ptr(), relu=relu)
    assert capi.tc_status() == 0
    torch.cuda.synchronize()
    ref = (A.double() @ W.double().T + bias.double())
    if relu:
        ref = torch.relu(ref)
    return got.cpu().numpy(), want.cpu().numpy(), ref.cpu().numpy()


def test_static_scratch_matches_allocating_path_twice(built_library):
    # First call fills a large part of the array; the second, smaller one finds the first call's halves
    # there and must not be disturbed by them.  A third repeats the first shape with other data.
    cases = [(1000, 384, 512, 11, True), (333, 72, 100, 12, False), (1000, 384, 512, 13, True)]
    for M, N, K, seed, relu in cases:
        got, want, ref = run_pair(M, N, K, seed, relu)
        assert np.isfinite(got).all()
        assert_close(got, want, f"static vs allocating {M}x{N}x{K}")
        assert_close(got, ref.astype(np.float32), f"static vs float64 product {M}x{N}x{K}")


def test_static_scratch_leaves_device_memory_alone(built_library):
    """The property that gives the entry point its name: after a first call on the device (which may load kernels and
    looks the array's address up), further calls change the amount of free device memory by nothing."""
    import torch
    M, N, K = 512, 256, 384
    g = torch.Generator(device="cpu").manual_seed(5)
    A, W = torch.randn(M, K, generator=g).cuda(), torch.randn(N, K, generator=g).cuda()
    out = torch.empty(M, N, device="cuda")
    capi.gemm_static(A.data_ptr(), K, W.data_ptr(), K, out.data_ptr(), N, M, N, K)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        capi.gemm_static(A.data_ptr(), K, W.data_ptr(), K, out.data_ptr(), N, M, N, K)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert capi.tc_status() == 0
    assert free_after == free_before


def test_static_scratch_reads_only_k_floats_per_row(built_library):
    """W as a column slice of a larger matrix (ldw > K) whose last row ends exactly at the end of the allocation:
    nothing beyond the K-th float of a row may be touched, and the padding between rows must not leak into the result
    (it holds NaN here).  Both the static and the allocating tensor-core entry point."""
    import torch
    M, N, K, ldw = 200, 96, 64, 80
    g = torch.Generator(device="cpu").manual_seed(6)
    A = torch.randn(M, K, generator=g).cuda()
    buf = torch.full(((N - 1) * ldw + K,), float("nan"), device="cuda")   # ends with the last row's K-th value
    Wd = torch.randn(N, K, generator=g)
    rows = buf.as_strided((N, K), (ldw, 1))
    rows.copy_(Wd.cuda())
    ref = (A.double().cpu() @ Wd.double().T).numpy().astype(np.float32)
    for entry in (capi.gemm_static, lambda *a, **k: capi.gemm(1, *a, **k)):
        out = torch.full((M, N), float("nan"), device="cuda")
        entry(A.data_ptr(), K, buf.data_ptr(), ldw, out.data_ptr(), N, M, N, K)
        assert capi.tc_status() == 0
        torch.cuda.synchronize()
        assert_close(out.cpu().numpy(), ref, "column slice of a larger matrix")
    with pytest.raises(fdeep_b200.FdeepError, match="row strides"):
        capi.gemm_static(A.data_ptr(), K, buf.data_ptr(), K - 4, out.data_ptr(), N, M, N, K)


def test_static_scratch_refuses_oversize(built_library):
    import torch
    limit = capi.gemm_static_max_weight_floats()
    assert limit == 1 << 20
    N, K = 1024, 1024 + 4  # N * ldw just above the limit
    A = torch.zeros(8, K, device="cuda")
    W = torch.zeros(N, K, device="cuda")
    out = torch.zeros(8, N, device="cuda")
    with pytest.raises(fdeep_b200.FdeepError, match="at most"):
        capi.gemm_static(A.data_ptr(), K, W.data_ptr(), K, out.data_ptr(), N, 8, N, K)
    # exactly at the limit is accepted
    K = 1024
    A = torch.ones(8, K, device="cuda")
    W = torch.full((N, K), 0.5, device="cuda")
    capi.gemm_static(A.data_ptr(), K, W.data_ptr(), K, out.data_ptr(), N, 8, N, K)
    assert capi.tc_status() == 0
    torch.cuda.synchronize()
    np.testing.assert_allclose(out.cpu().numpy(), 512.0, rtol=1e-6)
