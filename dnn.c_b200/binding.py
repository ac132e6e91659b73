"""ctypes binding of the dnn.c C API.

The same declarations serve two shared libraries, because they export the
same symbols with the same struct layouts:

  * dnn.c_b200/libdnn_b200.so   this repository's CUDA implementation
    (tensor payloads live in device memory, moved with dnn_cuda_upload /
    dnn_cuda_download);
  * a build of the reference library (CPU; payloads are host memory), used
    only by tests and the benchmark's CPU baseline.

`Dnn(path)` loads one of them and gives numpy-level helpers on top of the raw
C calls.  Nothing here computes: every op is a call into the library.
"""
import ctypes as C
import os

import numpy as np

MAX_DIMS = 8


class MemPool(C.Structure):
    _fields_ = [("buffer", C.c_void_p), ("capacity", C.c_size_t), ("offset", C.c_size_t)]


class DnnCtx(C.Structure):
    _fields_ = [("params", C.POINTER(MemPool)), ("scratch", C.POINTER(MemPool)), ("data", C.POINTER(MemPool))]


class Tensor(C.Structure):
    pass


Tensor._fields_ = [
    ("data", C.c_void_p),
    ("grad", C.c_void_p),
    ("shape", C.c_int * MAX_DIMS),
    ("strides", C.c_int * MAX_DIMS),
    ("ndim", C.c_int),
    ("flags", C.c_uint),          # bit 0 requires_grad, bit 1 contiguous
    ("offset", C.c_int),
    ("parent", C.POINTER(Tensor)),
    ("grad_fn", C.c_void_p),
    ("pool", C.POINTER(MemPool)),
]
TensorP = C.POINTER(Tensor)
assert C.sizeof(Tensor) == 120 and C.sizeof(MemPool) == 24


class GradFn(C.Structure):
    pass


GradFn._fields_ = [
    ("backward", C.CFUNCTYPE(None, C.POINTER(GradFn), TensorP)),
    ("pool", C.POINTER(MemPool)),
    ("inputs", C.POINTER(TensorP)),
    ("n_inputs", C.c_int),
    ("saved_tensors", C.POINTER(C.c_void_p)),
    ("n_saved", C.c_int),
]
assert C.sizeof(GradFn) == 48


class AdamW(C.Structure):
    _fields_ = [
        ("params", C.POINTER(TensorP)), ("n_params", C.c_int), ("lr", C.c_float),
        ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float), ("weight_decay", C.c_float),
        ("t", C.c_int), ("m", C.POINTER(TensorP)), ("v", C.POINTER(TensorP)),
    ]


class LrScheduler(C.Structure):
    _fields_ = [
        ("opt", C.POINTER(AdamW)), ("schedule", C.c_int), ("base_lr", C.c_float), ("min_lr", C.c_float),
        ("warmup_iters", C.c_int), ("total_iters", C.c_int), ("step_size", C.c_int), ("gamma", C.c_float),
        ("t", C.c_int),
    ]


assert C.sizeof(AdamW) == 56


class KernelTime(C.Structure):
    _fields_ = [("name", C.c_char * 56), ("launches", C.c_longlong), ("ms", C.c_double), ("work", C.c_double)]


PoolP = C.POINTER(MemPool)
VP = C.c_void_p
I = C.c_int
F = C.c_float
IP = C.POINTER(C.c_int)

# name -> (restype, argtypes); shared by both libraries
API = {
    "dnn_ctx_init": (I, [C.POINTER(DnnCtx), C.c_size_t, C.c_size_t, C.c_size_t]),
    "dnn_ctx_reset_step": (None, [C.POINTER(DnnCtx)]),
    "dnn_ctx_destroy": (None, [C.POINTER(DnnCtx)]),
    "mem_pool_reset": (None, [PoolP]),
    "mem_pool_mark": (C.c_size_t, [PoolP]),
    "mem_pool_release": (None, [PoolP, C.c_size_t]),
    "_mem_pool_alloc": (VP, [PoolP, C.c_size_t, VP]),
    "dnn_seed": (None, [C.c_uint64]),
    "tensor_zeros": (TensorP, [PoolP, I, IP, I]),
    "tensor_zeros_data": (TensorP, [PoolP, I, IP]),
    "tensor_randn": (TensorP, [PoolP, I, IP, I]),
    "tensor_uniform": (TensorP, [PoolP, I, IP, I, F]),
    "tensor_scratch": (TensorP, [PoolP, I, IP, I]),
    "tensor_slice": (TensorP, [PoolP, TensorP, I, I, I]),
    "tensor_transpose": (TensorP, [PoolP, TensorP, I, I]),
    "tensor_reshape": (TensorP, [PoolP, TensorP, I, IP]),
    "tensor_flatten": (TensorP, [PoolP, TensorP]),
    "tensor_contiguous": (TensorP, [PoolP, TensorP]),
    "tensor_numel": (I, [TensorP]),
    "tensor_zero_grad": (None, [TensorP]),
    "dnn_grad_enabled": (I, []),
    "dnn_backward": (None, [PoolP, TensorP]),
    "tensor_add": (TensorP, [PoolP, TensorP, TensorP]),
    "tensor_cat": (TensorP, [PoolP, TensorP, TensorP, I]),
    "tensor_matmul": (TensorP, [PoolP, TensorP, TensorP]),
    "tensor_matmul_add": (TensorP, [PoolP, TensorP, TensorP, I, TensorP]),
    "tensor_relu": (TensorP, [PoolP, TensorP]),
    "tensor_silu": (TensorP, [PoolP, TensorP]),
    "tensor_swiglu": (TensorP, [PoolP, TensorP, TensorP]),
    "tensor_sub": (TensorP, [PoolP, TensorP, TensorP]),
    "tensor_mul": (TensorP, [PoolP, TensorP, TensorP]),
    "tensor_div": (TensorP, [PoolP, TensorP, TensorP]),
    "tensor_neg": (TensorP, [PoolP, TensorP]),
    "tensor_pow": (TensorP, [PoolP, TensorP, F]),
    "tensor_triu": (TensorP, [PoolP, I, I]),
    "tensor_sigmoid": (TensorP, [PoolP, TensorP]),
    "tensor_softmax": (TensorP, [PoolP, TensorP, I]),
    "tensor_causal_softmax": (TensorP, [PoolP, TensorP]),
    "tensor_dropout": (TensorP, [PoolP, TensorP, F]),
    "tensor_sum": (TensorP, [PoolP, TensorP, I]),
    "tensor_mean": (TensorP, [PoolP, TensorP, I]),
    "tensor_cross_entropy": (TensorP, [PoolP, TensorP, TensorP, I]),
    "tensor_cross_entropy_masked": (TensorP, [PoolP, TensorP, TensorP, TensorP, I]),
    "tensor_embedding": (TensorP, [PoolP, TensorP, TensorP]),
    "tensor_avg_pool2d": (TensorP, [PoolP, TensorP, I, I]),
    "tensor_layer_norm": (TensorP, [PoolP, TensorP, TensorP, TensorP, F]),
    "tensor_rms_norm": (TensorP, [PoolP, TensorP, TensorP, F]),
    "tensor_attention_ex": (TensorP, [PoolP, TensorP, TensorP, TensorP, TensorP, I, I, IP]),
    "tensor_attention": (TensorP, [PoolP, TensorP, TensorP, TensorP, TensorP]),
    "tensor_split_heads": (TensorP, [PoolP, TensorP, I]),
    "tensor_merge_heads": (TensorP, [PoolP, TensorP]),
    "tensor_split_qkv_heads": (None, [PoolP, TensorP, I, C.POINTER(TensorP), C.POINTER(TensorP), C.POINTER(TensorP)]),
    "tensor_rope": (TensorP, [PoolP, TensorP, TensorP, TensorP]),
    "tensor_rope_freqs_init": (None, [PoolP, C.POINTER(TensorP), C.POINTER(TensorP), I, I, F]),
    "tensor_conv2d": (TensorP, [PoolP, TensorP, TensorP, TensorP, I, I]),
    "adamw_create": (C.POINTER(AdamW), [PoolP, C.POINTER(TensorP), I, F, F, F, F, F]),
    "adamw_step": (None, [C.POINTER(AdamW)]),
    "adamw_step_with_lr_multipliers": (None, [C.POINTER(AdamW), C.POINTER(C.c_float)]),
    "adamw_zero_grad": (None, [C.POINTER(AdamW)]),
    "grad_norm": (F, [C.POINTER(TensorP), I]),
    "clip_grad_norm": (F, [C.POINTER(TensorP), I, F]),
    "lr_scheduler_create": (C.POINTER(LrScheduler), [PoolP, C.POINTER(AdamW), I, F, I, I, F, I, F]),
    "lr_scheduler_step": (None, [C.POINTER(LrScheduler)]),
    "lr_scheduler_get_lr": (F, [C.POINTER(LrScheduler)]),
    "lr_scheduler_reset": (None, [C.POINTER(LrScheduler)]),
    "module_parameters": (C.POINTER(TensorP), [VP, IP]),
    "module_num_parameters": (C.c_longlong, [VP]),
    "module_find_param": (TensorP, [VP, C.c_char_p]),
    "module_save": (None, [VP, C.c_char_p]),
    "module_load": (None, [VP, C.c_char_p, I]),
    "linear_create": (VP, [PoolP, I, I]),
    "linear_forward": (TensorP, [PoolP, VP, TensorP]),
    "conv2d_create": (VP, [PoolP, I, I, I, I, I]),
    "conv2d_forward": (TensorP, [PoolP, VP, TensorP]),
    "rms_norm_create": (VP, [PoolP, I, F]),
    "layer_norm_create": (VP, [PoolP, I, F]),
    "embedding_create": (VP, [PoolP, I, I]),
    "swiglu_ffn_create": (VP, [PoolP, I, I]),
    "transformer_block_create": (VP, [PoolP, I, I, I, I]),
    "transformer_block_forward": (TensorP, [PoolP, VP, TensorP]),
    "decoder_lm_create": (VP, [PoolP, I, I, I, I, I, I]),
    "decoder_lm_enable_rope": (None, [PoolP, VP, I, F]),
    "decoder_lm_init_weights": (None, [VP]),
    "decoder_lm_forward": (TensorP, [PoolP, VP, TensorP]),
    "decoder_lm_shift_targets": (TensorP, [PoolP, TensorP]),
    "decoder_lm_generate": (C.POINTER(C.c_int), [PoolP, PoolP, VP, TensorP, I, F, I, C.POINTER(C.c_int)]),
    "vision_lm_generate": (C.POINTER(C.c_int), [PoolP, PoolP, VP, TensorP, TensorP, I, F, I, C.POINTER(C.c_int)]),
    "decoder_lm_argmax_token": (I, [C.POINTER(C.c_float), I]),
    "decoder_lm_sample_with_temp": (I, [C.POINTER(C.c_float), I, F]),
    "kv_cache_create": (VP, [PoolP, I, I, I, I]),
    "transformer_block_forward_cached": (TensorP, [PoolP, VP, TensorP, VP]),
    "decoder_lm_train_step": (TensorP, [PoolP, VP, TensorP, TensorP, C.POINTER(AdamW), F, C.POINTER(C.c_float)]),
    "vision_lm_create": (VP, [PoolP, I, I, I, I, I, I, I, I, I, I, I]),
    "vision_lm_enable_rope": (None, [PoolP, VP, I, F]),
    "vision_lm_init_weights": (None, [VP]),
    "vision_lm_loss_padded": (TensorP, [PoolP, VP, TensorP, TensorP, TensorP, TensorP, IP]),
    "vision_lm_train_step_padded": (TensorP, [PoolP, VP, TensorP, TensorP, TensorP, TensorP, IP, C.POINTER(AdamW), F, C.POINTER(C.c_float)]),
    "vision_lm_train_step": (TensorP, [PoolP, VP, TensorP, TensorP, TensorP, C.POINTER(AdamW), F, C.POINTER(C.c_float)]),
}

# only libdnn_b200.so has these
CUDA_API = {
    "dnn_cuda_init": (I, [I]),
    "dnn_cuda_available": (I, []),
    "dnn_cuda_sync": (I, []),
    "dnn_cuda_last_error": (C.c_char_p, []),
    "dnn_cuda_stream": (VP, []),
    "dnn_cuda_upload": (I, [TensorP, VP, C.c_size_t]),
    "dnn_cuda_download": (I, [TensorP, VP, C.c_size_t]),
    "dnn_cuda_download_grad": (I, [TensorP, VP, C.c_size_t]),
    "dnn_cuda_memcpy_h2d": (I, [VP, VP, C.c_size_t]),
    "dnn_cuda_memcpy_d2h": (I, [VP, VP, C.c_size_t]),
    "dnn_cuda_host_alloc": (VP, [C.c_size_t]),
    "dnn_cuda_host_free": (None, [VP]),
    "dnn_cuda_set_gemm_mode": (I, [I]),
    "dnn_cuda_get_gemm_mode": (I, []),
    "dnn_cuda_set_tf32_policy": (I, [C.c_uint, C.c_double]),
    "dnn_cuda_set_exact_policy": (I, [C.c_double]),
    "dnn_cuda_get_exact_policy": (C.c_double, []),
    "dnn_cuda_get_tf32_policy": (I, [C.POINTER(C.c_uint), C.POINTER(C.c_double)]),
    "dnn_cuda_graph_capture_decoder_lm_step": (VP, [PoolP, VP, TensorP, TensorP, C.POINTER(AdamW), F]),
    "dnn_cuda_graph_replay": (I, [VP, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "dnn_cuda_graph_destroy": (None, [VP]),
    "dnn_cuda_optimizer_save": (I, [C.POINTER(AdamW), C.c_char_p]),
    "dnn_cuda_optimizer_load": (I, [C.POINTER(AdamW), C.c_char_p]),
    "dnn_cuda_train_state_save": (I, [C.POINTER(AdamW), C.POINTER(LrScheduler), C.c_char_p]),
    "dnn_cuda_train_state_load": (I, [C.POINTER(AdamW), C.POINTER(LrScheduler), C.c_char_p]),
    "dnn_cuda_set_fused_attention": (None, [I]),
    "dnn_cuda_get_fused_attention": (I, []),
    "dnn_cuda_colsum_acc_static": (I, [VP, VP, C.c_longlong, I]),
    "dnn_cuda_colsum_acc_static_error": (C.c_char_p, []),
    "dnn_cuda_vlm_stager_create": (VP, [I, I, I, I, I, I, I, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "dnn_cuda_vlm_stager_destroy": (None, [VP]),
    "dnn_cuda_vlm_stager_put": (I, [VP, I, I, C.POINTER(C.c_int), I, VP, I, I]),
    "dnn_cuda_vlm_stager_submit": (I, [VP, I, I]),
    "dnn_cuda_vlm_stager_assemble": (I, [VP, I, TensorP, TensorP, TensorP, TensorP, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "dnn_cuda_vlm_stager_error": (C.c_char_p, []),
    "dnn_cuda_launch_count": (C.c_longlong, []),
    "dnn_cuda_timer_start": (I, []),
    "dnn_cuda_timer_stop_ms": (F, []),
    "dnn_cuda_profile_enable": (I, [I]),
    "dnn_cuda_profile_read": (I, [I, C.POINTER(C.c_longlong), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "dnn_cuda_profile_kernels": (I, [C.POINTER(KernelTime), I]),
    "dnn_cuda_pool_device_used": (C.c_size_t, [PoolP]),
    "dnn_cuda_pool_device_peak": (C.c_size_t, [PoolP]),
    "dnn_cuda_dp_unique_id": (I, [VP]),
    "dnn_cuda_dp_init": (I, [I, I, VP]),
    "dnn_cuda_dp_allreduce_grads": (I, [C.POINTER(TensorP), I]),
    "dnn_cuda_dp_world_size": (I, []),
    "dnn_cuda_dp_finalize": (I, []),
    "dnn_cuda_dp_last_error": (C.c_char_p, []),
    "dnn_cuda_dp_backward": (I, [PoolP, TensorP, C.POINTER(TensorP), I]),
    "dnn_cuda_dp_vision_lm_train_step_padded": (TensorP, [PoolP, VP, TensorP, TensorP, TensorP, TensorP, IP, C.POINTER(AdamW), F, C.POINTER(C.c_float)]),
    "dnn_cuda_dp_decoder_lm_train_step": (TensorP, [PoolP, VP, TensorP, TensorP, C.POINTER(AdamW), F, C.POINTER(C.c_float)]),
}

GEMM_FP32, GEMM_TF32, GEMM_3XTF32 = 0, 1, 2
ATTENTION_CAUSAL, ATTENTION_PREFIX_LM = 0, 1

HERE = os.path.dirname(os.path.abspath(__file__))
B200_LIB = os.environ.get("DNN_B200_LIB") or os.path.join(HERE, "libdnn_b200.so")       # another build of the library, for A/B timing


def _ints(seq):
    return (C.c_int * len(seq))(*[int(x) for x in seq])


class Dnn:
    """One loaded library plus a context (params / scratch / data pools)."""

    def __init__(self, path=B200_LIB, params_mb=256, scratch_mb=1024, data_mb=64, device=0):
        if not os.path.exists(path):
            raise FileNotFoundError("%s is missing: build it first (python dnn.c_b200/build.py)" % path)
        self.lib = C.CDLL(path, mode=C.RTLD_LOCAL)
        self.is_cuda = hasattr(self.lib, "dnn_cuda_upload")
        for name, (res, args) in API.items():
            fn = getattr(self.lib, name)
            fn.restype, fn.argtypes = res, args
        if self.is_cuda:
            for name, (res, args) in CUDA_API.items():
                fn = getattr(self.lib, name)
                fn.restype, fn.argtypes = res, args
            rc = self.lib.dnn_cuda_init(device)
            if rc != 0:
                raise RuntimeError("dnn_cuda_init failed: %s" % self.lib.dnn_cuda_last_error().decode())
        self.ctx = DnnCtx()
        rc = self.lib.dnn_ctx_init(C.byref(self.ctx), params_mb << 20, scratch_mb << 20, data_mb << 20)
        if rc != 0:
            raise MemoryError("dnn_ctx_init failed")
        self.params, self.scratch, self.data = self.ctx.params, self.ctx.scratch, self.ctx.data
        self._keep = []

    def close(self):
        if self.ctx is not None:
            self.sync()
            self.lib.dnn_ctx_destroy(C.byref(self.ctx))
            self.ctx = None

    # ---- payload movement -------------------------------------------------
    def sync(self):
        if self.is_cuda:
            self.lib.dnn_cuda_sync()

    def upload(self, t, arr):
        arr = np.ascontiguousarray(arr)
        assert arr.dtype in (np.float32, np.int32), arr.dtype
        n = self.lib.tensor_numel(t)
        assert arr.size == n, (arr.shape, n)
        if self.is_cuda:
            self._keep.append(arr)
            rc = self.lib.dnn_cuda_upload(t, arr.ctypes.data, arr.nbytes)
            assert rc == 0, self.lib.dnn_cuda_last_error()
            self.sync()
            self._keep.pop()
        else:
            C.memmove(t.contents.data + 4 * t.contents.offset, arr.ctypes.data, arr.nbytes)

    def shape_of(self, t):
        return tuple(t.contents.shape[i] for i in range(t.contents.ndim))

    def download(self, t, dtype=np.float32):
        """Contiguous tensor -> numpy array of its shape."""
        out = np.empty(self.shape_of(t), dtype=dtype)
        if self.is_cuda:
            rc = self.lib.dnn_cuda_download(t, out.ctypes.data, out.nbytes)
            assert rc == 0, self.lib.dnn_cuda_last_error()
        else:
            C.memmove(out.ctypes.data, t.contents.data + 4 * t.contents.offset, out.nbytes)
        return out

    def download_grad(self, t):
        """Gradient buffer of a root tensor (None when it was never written)."""
        if not t.contents.grad:
            return None
        out = np.empty(self.shape_of(t), dtype=np.float32)
        if self.is_cuda:
            rc = self.lib.dnn_cuda_download_grad(t, out.ctypes.data, out.nbytes)
            assert rc == 0, self.lib.dnn_cuda_last_error()
        else:
            C.memmove(out.ctypes.data, t.contents.grad, out.nbytes)
        return out

    def read_raw(self, ptr, n, dtype=np.float32):
        out = np.empty(n, dtype=dtype)
        if self.is_cuda:
            self.lib.dnn_cuda_memcpy_d2h(out.ctypes.data, ptr, out.nbytes)
        else:
            C.memmove(out.ctypes.data, ptr, out.nbytes)
        return out

    # ---- tensor construction ---------------------------------------------
    def tensor(self, arr, pool=None, requires_grad=False):
        """New contiguous tensor holding `arr` (float32 or int32)."""
        arr = np.ascontiguousarray(arr)
        pool = pool or self.data
        shape = arr.shape if arr.ndim else (1,)
        t = self.lib.tensor_scratch(pool, len(shape), _ints(shape), 1 if requires_grad else 0)
        self.upload(t, arr.astype(np.int32 if arr.dtype.kind in "iu" else np.float32))
        return t

    def backward_from(self, out, gout):
        """Runs the tape node of `out` with `gout` as the upstream gradient, the
        way dnn_backward() calls it: grad_fn.backward(fn, &contiguous_wrapper)."""
        assert out.contents.grad_fn, "tensor has no tape node"
        fn = C.cast(out.contents.grad_fn, C.POINTER(GradFn))
        g = self.tensor(np.asarray(gout, dtype=np.float32).reshape(self.shape_of(out)), pool=self.scratch)
        fn.contents.backward(fn, g)
        self.sync()

    def param(self, arr):
        return self.tensor(arr, pool=self.params, requires_grad=True)

    def parameters(self, module):
        n = C.c_int(0)
        arr = self.lib.module_parameters(module, C.byref(n))
        return [arr[i] for i in range(n.value)]

    def reset_step(self):
        self.sync()
        self.lib.dnn_ctx_reset_step(C.byref(self.ctx))

    def scalar(self, t):
        return float(self.download(t).reshape(-1)[0])


def ints(seq):
    return _ints(seq)
