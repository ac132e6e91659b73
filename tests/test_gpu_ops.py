"""GPU: every op of the hot path, called through the C-ABI of libdnn_b200.so,
against (a) the numpy oracle on the same seeded inputs and (b) the committed
vectors produced by the unmodified reference library."""
import ctypes as C
import os

import numpy as np
import pytest

from cases import CASES, compare
from golden_util import check

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# ops that go through a GEMM or attention kernel.  Bars: 1e-3 relative L2 with TF32 products, 1e-5 with 3xTF32.
TENSOR_CORE_OPS = ("matmul", "conv2d", "attention")


@pytest.fixture(scope="module")
def ops_golden():
    return np.load(os.path.join(GOLDEN, "ops.npz"))


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_fp32_mode_matches_oracle_and_reference(gpu, binding, ops_golden, case):
    gpu.lib.dnn_cuda_set_gemm_mode(binding.GEMM_FP32)
    inp = case.make(np.random.default_rng(1234))
    got = case.run(gpu, inp)
    gpu.reset_step()
    compare(case, got, case.oracle(inp))
    for k, v in got.items():
        key = case.name + "/" + k
        check(key, v, ops_golden[key], ops_golden[key + "#"], max(case.tol, 1e-6), exact=k in case.golden_exact)


@pytest.mark.parametrize("mode,tol", [("tf32", 1e-3), ("3xtf32", 1e-5)])
@pytest.mark.parametrize("case", [c for c in CASES if c.name.startswith(TENSOR_CORE_OPS)], ids=lambda c: c.name)
def test_tensor_core_modes_match_oracle(gpu, binding, case, mode, tol):
    """The tensor-core kernels themselves at small sizes: the precision policy, which by default sends products
    this small to a more exact path, is switched off so that plain TF32 resp. the three-product split is what runs."""
    gpu.lib.dnn_cuda_set_gemm_mode(binding.GEMM_TF32 if mode == "tf32" else binding.GEMM_3XTF32)
    roles, max_flop = C.c_uint(0), C.c_double(0)
    gpu.lib.dnn_cuda_get_tf32_policy(C.byref(roles), C.byref(max_flop))
    simt = gpu.lib.dnn_cuda_get_exact_policy()
    gpu.lib.dnn_cuda_set_tf32_policy(0, 0.0)
    gpu.lib.dnn_cuda_set_exact_policy(0.0)
    try:
        inp = case.make(np.random.default_rng(1234))
        got = case.run(gpu, inp)
        gpu.reset_step()
        compare(case, got, case.oracle(inp), tol=tol)
    finally:
        gpu.lib.dnn_cuda_set_tf32_policy(roles.value, max_flop.value)
        gpu.lib.dnn_cuda_set_exact_policy(simt)
        gpu.lib.dnn_cuda_set_gemm_mode(binding.GEMM_FP32)


X3_SHAPES = [  # (a shape, b shape, trans_b): one per tile configuration of the one-pass 3xTF32 kernel
    ((100, 200), (200, 300), 0),      # at most 128 rows, wide output: single CTAs with 256-column tiles
    ((100, 200), (300, 200), 1),
    ((64, 4096), (4096, 64), 0),      # long K on few tiles: split-K partials and their reduction
    ((520, 1000), (1000, 264), 0),    # CTA pairs, ragged in M, N and K, several k-blocks per stage ring
    ((520, 1000), (264, 1000), 1),
    ((2, 256, 96), (96, 128), 0),     # 128-column tiles
]


@pytest.mark.parametrize("sa,sb,tb", X3_SHAPES, ids=lambda v: str(v))
@pytest.mark.parametrize("form", ["one-accumulator", "two-accumulators"])
def test_3xtf32_products_hold_1e5_on_every_tile_configuration(gpu, binding, sa, sb, tb, form):
    """Forward, dA and dW of a linear layer as 3xTF32 tensor-core products whatever their size (the kernel splits raw
    tiles in shared memory).  one-accumulator: the form the TF32 mode's precision policy selects, here for every role;
    two-accumulators: the exact mode's form, with its size rule switched off."""
    from oracle import dnn_oracle as O
    rng = np.random.default_rng(77)
    n = sb[-2] if tb else sb[-1]
    a = rng.standard_normal(sa).astype(np.float32)
    b = (0.2 * rng.standard_normal(sb)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    g = rng.standard_normal(sa[:-1] + (n,)).astype(np.float32)
    roles, max_flop = C.c_uint(0), C.c_double(0)
    gpu.lib.dnn_cuda_get_tf32_policy(C.byref(roles), C.byref(max_flop))
    simt = gpu.lib.dnn_cuda_get_exact_policy()
    if form == "one-accumulator":
        gpu.lib.dnn_cuda_set_gemm_mode(binding.GEMM_TF32)
        gpu.lib.dnn_cuda_set_tf32_policy(7, 0.0)
    else:
        gpu.lib.dnn_cuda_set_gemm_mode(binding.GEMM_3XTF32)
        gpu.lib.dnn_cuda_set_exact_policy(0.0)
    try:
        ta = gpu.tensor(a, gpu.scratch, True)
        tw, tbias = gpu.param(b), gpu.param(bias)
        y = gpu.lib.tensor_matmul_add(gpu.scratch, ta, tw, tb, tbias)
        gpu.backward_from(y, g)
        got = dict(y=gpu.download(y), da=gpu.download_grad(ta), db=gpu.download_grad(tw), dbias=gpu.download_grad(tbias))
        gpu.reset_step()
    finally:
        gpu.lib.dnn_cuda_set_tf32_policy(roles.value, max_flop.value)
        gpu.lib.dnn_cuda_set_exact_policy(simt)
        gpu.lib.dnn_cuda_set_gemm_mode(binding.GEMM_FP32)
    wy, wda, wdb, wdbias = O.matmul_add(a, b, tb, bias, g)
    for name, want in (("y", wy), ("da", wda), ("db", wdb), ("dbias", wdbias)):
        err = np.linalg.norm(got[name].astype(np.float64) - want) / np.linalg.norm(want)
        assert err <= 1e-5, (name, err)


def test_same_seed_twice_is_bit_identical(gpu, binding):
    """Determinism on one GPU: no atomics anywhere on the path."""
    gpu.lib.dnn_cuda_set_gemm_mode(binding.GEMM_FP32)
    for case in [c for c in CASES if c.name.startswith(("rms_norm[37", "embedding[V50", "attention[B2 H3", "matmul_add[4, 37, 64][64"))]:
        inp = case.make(np.random.default_rng(99))
        a = case.run(gpu, inp); gpu.reset_step()
        b = case.run(gpu, inp); gpu.reset_step()
        for k in a:
            assert np.array_equal(a[k], b[k]), (case.name, k)


class _TwiceBackward:
    """Proxy of the binding whose backward_from() runs the tape node twice, so the second
    run finds gradient buffers that already hold a value and must add to them."""

    def __init__(self, dnn, binding):
        self._dnn, self._binding = dnn, binding

    class _Lib:
        def __init__(self, lib):
            self._lib = lib

        def __getattr__(self, name):
            return getattr(self._lib, name)

        def dnn_backward(self, scratch, loss):
            self._lib.dnn_backward(scratch, loss)
            self._lib.dnn_backward(scratch, loss)

    @property
    def lib(self):
        return self._Lib(self._dnn.lib)

    def __getattr__(self, name):
        return getattr(self._dnn, name)

    def backward_from(self, out, gout):
        import ctypes as C
        fn = C.cast(out.contents.grad_fn, C.POINTER(self._binding.GradFn))
        g = self._dnn.tensor(np.asarray(gout, dtype=np.float32).reshape(self._dnn.shape_of(out)), pool=self._dnn.scratch)
        fn.contents.backward(fn, g)
        fn.contents.backward(fn, g)
        self._dnn.sync()


OVERWRITING = ("merge_heads", "split_heads")     # their backward stores (src/multihead.c:92,177)


@pytest.mark.parametrize("case", [c for c in CASES if not c.name.startswith(("rope_freqs_init", "transpose+", "mean", "adamw", "clip_grad_norm", "lr_schedules"))],
                         ids=lambda c: c.name)
def test_second_backward_accumulates(gpu, binding, case):
    """The first gradient written to a buffer may be a plain store; every later one must add.
    Running each tape node twice has to give exactly twice the oracle's gradients."""
    gpu.lib.dnn_cuda_set_gemm_mode(binding.GEMM_FP32)
    inp = case.make(np.random.default_rng(4321))
    got = case.run(_TwiceBackward(gpu, binding), inp)
    gpu.reset_step()
    want = case.oracle(inp)
    factor = 1.0 if case.name.startswith(OVERWRITING) else 2.0
    want = {k: (v * factor if k.startswith("d") else v) for k, v in want.items()}
    compare(case, got, want)


def test_attention_kernel_variants_behind_switches_match_oracle():
    """The tensor-core attention has two forms that the defaults do not run: the dQ kernel with one CTA per SM, and
    gradients / outputs written by the threads themselves (taken when a view cannot be described to the copy engine).
    Both are selected by environment switches read at the first launch, so the cases run in a child process."""
    import subprocess
    import sys
    env = dict(os.environ, DNN_CUDA_ATTN_DQ="1", DNN_CUDA_ATTN_TMA_OUT="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_gpu_ops.py"), "-q", "-x", "-p", "no:cacheprovider",
                        "-k", "test_tensor_core_modes_match_oracle and attention and tf32 and not 3xtf32"],
                       capture_output=True, text=True, timeout=900, env=env, cwd=root)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert " passed" in r.stdout and "failed" not in r.stdout, r.stdout[-2000:]
