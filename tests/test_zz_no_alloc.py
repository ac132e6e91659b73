"""GPU: the allocation-free column-sum entry point against the pooled path.

dnn_cuda_colsum_acc_static() serves callers that may not allocate device memory
when they call (all of HBM already owned by their arenas, no tolerance for the
device-wide stall of an allocation, or a no-allocation-after-start-up policy).
It keeps its partial sums in an array compiled into the library.  The check is
against the library's existing way to get the same numbers: the bias gradient
that tensor_add's backward produces through the C-ABI.  The call is made twice
in a row, with different inputs, because all calls share the one static array.
This file is named so that pytest collects it last.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def reference_colsum(gpu, g_np):
    """Bias gradient through the existing entry points: y = a + bias, backward with upstream g."""
    rows, cols = g_np.shape
    a = gpu.tensor(np.zeros((rows, cols), np.float32), gpu.scratch, True)
    bias = gpu.param(np.zeros(cols, np.float32))
    y = gpu.lib.tensor_add(gpu.scratch, a, bias)
    gpu.backward_from(y, g_np)
    return gpu.download_grad(bias)


# the last pair has more than 128 x 256 rows, so the number of row blocks is clamped to the 128 the array holds
@pytest.mark.parametrize("shapes", [[(1000, 768), (37, 130)], [(16384, 2304), (5, 8192)], [(40000, 96), (70001, 33)]])
def test_static_colsum_matches_pooled_path_twice_in_a_row(gpu, shapes):
    rng = np.random.default_rng(5)
    for rows, cols in shapes:                       # two calls back to back on the shared array
        g_np = rng.standard_normal((rows, cols)).astype(np.float32)
        want = reference_colsum(gpu, g_np)
        exact = g_np.astype(np.float64).sum(axis=0)            # and against plain numpy, independent of the library
        assert np.linalg.norm(want - exact) <= 2e-5 * np.linalg.norm(exact)
        g = gpu.tensor(g_np, gpu.scratch)
        out = gpu.tensor(np.zeros(cols, np.float32), gpu.scratch)
        rc = gpu.lib.dnn_cuda_colsum_acc_static(out.contents.data, g.contents.data, rows, cols)
        assert rc == 0, gpu.lib.dnn_cuda_colsum_acc_static_error()
        got = gpu.download(out)
        gpu.reset_step()
        err = np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want.astype(np.float64))
        assert err <= 2e-5, (rows, cols, err)
        assert np.linalg.norm(got - exact) <= 2e-5 * np.linalg.norm(exact), (rows, cols)


def test_static_colsum_accumulates_and_rejects_oversize(gpu):
    rng = np.random.default_rng(6)
    g_np = rng.standard_normal((300, 64)).astype(np.float32)
    start = rng.standard_normal(64).astype(np.float32)
    g, out = gpu.tensor(g_np, gpu.scratch), gpu.tensor(start, gpu.scratch)
    assert gpu.lib.dnn_cuda_colsum_acc_static(out.contents.data, g.contents.data, 300, 64) == 0
    np.testing.assert_allclose(gpu.download(out), start + g_np.astype(np.float64).sum(0), rtol=2e-5, atol=2e-5)
    launches = gpu.lib.dnn_cuda_launch_count()
    assert gpu.lib.dnn_cuda_colsum_acc_static(out.contents.data, g.contents.data, 1, 8193) == -2
    assert b"8192" in gpu.lib.dnn_cuda_colsum_acc_static_error()
    assert gpu.lib.dnn_cuda_launch_count() == launches          # nothing was launched
    gpu.reset_step()
