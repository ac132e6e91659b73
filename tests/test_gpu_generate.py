"""GPU: KV-cache generation of the decoder LM and the vision LM against the token sequences the unmodified
reference produced for the same seeded weights, prompt and random stream (tests/golden/generate.npz)."""
import os

import numpy as np
import pytest

import models

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "generate.npz")


@pytest.mark.parametrize("mode", ["fp32", "tf32"])
@pytest.mark.parametrize("case", models.GEN_CASES, ids=[c[0] for c in models.GEN_CASES])
def test_generated_tokens_equal_the_reference(binding, case, mode):
    name, over, prompt, max_new, temp, use_cache = case
    want = np.load(GOLDEN)[name].tolist()
    d = binding.Dnn(binding.B200_LIB, params_mb=64, scratch_mb=512, data_mb=64)
    d.lib.dnn_cuda_set_gemm_mode(binding.GEMM_FP32 if mode == "fp32" else binding.GEMM_TF32)
    try:
        cfg = dict(models.lm_config("tiny")); cfg.update(over)
        got = models.run_generate(d, cfg, prompt, max_new, temp, use_cache, seed=77)
    finally:
        d.lib.dnn_cuda_set_gemm_mode(binding.GEMM_TF32)
        d.close()
    if mode == "fp32":
        assert got == want
    else:
        # TF32 logits differ in the third digit: the greedy sequences of these peaked models still agree;
        # a sampled sequence may legitimately leave the reference's path, so only its prompt and length are held
        assert got[:len(prompt)] == want[:len(prompt)] and len(got) == len(want)
        if temp == 0.0:
            assert got == want


def test_cache_and_full_forward_agree(binding):
    """Greedy generation with the KV cache equals greedy generation that re-runs the whole sequence."""
    cfg = dict(models.lm_config("tiny")); cfg.update(V=96, D=128, L=2, H=4, F=256)
    out = []
    for use_cache in (1, 0):
        d = binding.Dnn(binding.B200_LIB, params_mb=64, scratch_mb=512, data_mb=64)
        d.lib.dnn_cuda_set_gemm_mode(binding.GEMM_FP32)
        out.append(models.run_generate(d, cfg, [5, 6, 7, 8], 16, 0.0, use_cache))
        d.lib.dnn_cuda_set_gemm_mode(binding.GEMM_TF32)
        d.close()
    assert out[0] == out[1]


def test_replayed_token_steps_equal_eager_token_steps(binding):
    """From the third new token on, a cached decoding step is one graph launch; with DNN_CUDA_GEN_GRAPH=0 every step
    launches its kernels one by one.  Greedy and sampled sequences have to be the same either way."""
    cfg = dict(models.lm_config("tiny")); cfg.update(V=96, D=128, L=2, H=4, F=256)
    for temp in (0.0, 0.8):
        out = []
        for graph in ("1", "0"):
            os.environ["DNN_CUDA_GEN_GRAPH"] = graph
            try:
                d = binding.Dnn(binding.B200_LIB, params_mb=64, scratch_mb=512, data_mb=64)
                d.lib.dnn_cuda_set_gemm_mode(binding.GEMM_FP32)
                out.append(models.run_generate(d, cfg, [5, 6, 7, 8], 24, temp, 1, seed=5))
                d.lib.dnn_cuda_set_gemm_mode(binding.GEMM_TF32)
                d.close()
            finally:
                os.environ.pop("DNN_CUDA_GEN_GRAPH", None)
        assert out[0] == out[1] and len(out[0]) > 8


@pytest.mark.parametrize("mode", ["fp32", "tf32"])
@pytest.mark.parametrize("case", models.VLM_GEN_CASES, ids=[c[0] for c in models.VLM_GEN_CASES])
def test_vision_lm_generated_tokens_equal_the_reference(binding, case, mode):
    """vision_lm_generate: prefix-LM prefill of image tokens + prompt, then cached decoding.  The cached and
    uncached reference sequences differ (only the uncached path adds the image positions); both are held."""
    name, prompt, max_new, temp, use_cache, patched = case
    want = np.load(GOLDEN)[name].tolist()
    d = binding.Dnn(binding.B200_LIB, params_mb=64, scratch_mb=512, data_mb=64)
    d.lib.dnn_cuda_set_gemm_mode(binding.GEMM_FP32 if mode == "fp32" else binding.GEMM_TF32)
    try:
        got = models.run_vlm_generate(d, prompt, max_new, temp, use_cache, patched, seed=77)
    finally:
        d.lib.dnn_cuda_set_gemm_mode(binding.GEMM_TF32)
        d.close()
    if mode == "fp32":
        assert got == want
    else:
        assert got[:len(prompt)] == want[:len(prompt)] and len(got) <= len(prompt) + max_new
        if temp == 0.0 and name != "vlm-greedy-nocache":
            assert got == want


def test_generate_gives_back_the_device_memory_of_its_caches(binding):
    """decoder_lm_generate marks the data pool, builds its KV caches there and releases the mark
    (src/gpt.c:220-421).  With a fresh data pool the mark is taken BEFORE the pool owns any device memory
    (the output buffer is a host allocation); the release must still return the caches' device memory."""
    import ctypes as C
    cfg = dict(models.lm_config("tiny"))
    d = binding.Dnn(binding.B200_LIB, params_mb=64, scratch_mb=256, data_mb=64)
    lib = d.lib
    lm = lib.decoder_lm_create(d.params, cfg["V"], cfg["D"], cfg["L"], cfg["H"], cfg["D"] // cfg["H"], cfg["F"])
    lib.decoder_lm_enable_rope(d.params, lm, 32, 10000.0)
    models.seeded_weights(d, lm, models.O.lm_param_names(cfg["L"]), 5, std=0.3)
    ids = d.tensor(np.array([[3, 17, 42, 5]], np.int32), d.scratch)          # prompt NOT in the data pool
    assert lib.dnn_cuda_pool_device_used(d.data) == 0
    n = C.c_int(0)
    out = lib.decoder_lm_generate(d.scratch, d.data, lm, ids, 6, 0.0, 1, C.byref(n))
    assert n.value == 10 and out
    d.sync()
    assert lib.dnn_cuda_pool_device_used(d.data) == 0, "the KV caches stayed allocated on the device"
    d.close()
