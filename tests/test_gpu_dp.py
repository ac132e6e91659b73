"""GPU (needs 2 devices, otherwise skipped): two data-parallel ranks, each on its own
GPU with half of the batch, against one rank with the whole batch, for the three
trained models: the decoder LM (dnn_cuda_dp_decoder_lm_train_step), the vision LM
(dnn_cuda_dp_vision_lm_train_step_padded; parameters outside its graph have no
gradient on any rank) and the CNN driven op by op (dnn_cuda_dp_backward).  The averaged
gradients, the gradient norm and the updated parameters must agree with the
single-process step, and both ranks must hold bit-identical parameters (no parameter
broadcast is ever needed)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

WORKER = r"""
import ctypes as C, os, sys, time
import numpy as np
sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
from conftest import load_binding
import models
from oracle import dnn_oracle as O
B = load_binding()
rank, world, out = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
d = B.Dnn(B.B200_LIB, params_mb=256, scratch_mb=1024, data_mb=16, device=rank if world > 1 else 0)
lib = d.lib
lib.dnn_cuda_set_gemm_mode(B.GEMM_FP32)
if world > 1:
    idfile = os.path.join(out, "nccl_id.bin")
    buf = (C.c_ubyte * 128)()
    if rank == 0:
        assert lib.dnn_cuda_dp_unique_id(buf) == 0
        open(idfile + ".tmp", "wb").write(bytes(buf)); os.rename(idfile + ".tmp", idfile)
    else:
        for _ in range(600):
            if os.path.exists(idfile): break
            time.sleep(0.1)
        buf = (C.c_ubyte * 128)(*open(idfile, "rb").read())
    assert lib.dnn_cuda_dp_init(rank, world, buf) == 0
kind = sys.argv[4] if len(sys.argv) > 4 else "lm"
res = dict()
if kind == "lm":
    cfg = dict(models.lm_config("tiny"), B=4)
    ids_all, _ = models.lm_inputs(cfg)
    per = cfg["B"] // world
    ids_np = ids_all[rank * per:(rank + 1) * per]
    lm = lib.decoder_lm_create(d.params, cfg["V"], cfg["D"], cfg["L"], cfg["H"], cfg["D"] // cfg["H"], cfg["F"])
    lib.decoder_lm_enable_rope(d.params, lm, cfg["N"], 10000.0)
    names = O.lm_param_names(cfg["L"])
    params, _ = models.seeded_weights(d, lm, names, 123)
    arr = (B.TensorP * len(params))(*params)
    opt = lib.adamw_create(d.params, arr, len(params), cfg["lr"], cfg["b1"], cfg["b2"], cfg["eps"], cfg["wd"])
    for step in range(2):
        ids = d.tensor(ids_np, d.data)
        tgt = lib.decoder_lm_shift_targets(d.data, ids)
        gn = C.c_float(0)
        loss = lib.dnn_cuda_dp_decoder_lm_train_step(d.scratch, lm, ids, tgt, opt, cfg["clip"], C.byref(gn))
        res["loss%d" % step] = np.float32(d.scalar(loss)); res["gn%d" % step] = np.float32(gn.value)
        if step == 0:
            for n, t in zip(names, params): res["g/" + n] = d.download_grad(t)
        d.reset_step()
elif kind == "vlm":
    # prefix-LM vision LM, padded step.  Text lengths are chosen so that both halves of the batch have the
    # same number of loss positions: every rank normalises by its own mask sum, so only then is the mean
    # of the per-rank gradients the gradient of the whole batch.  img_proj.* never get a gradient.
    V, D, L, H, F, img, patch, Tmax, Bsz = 40, 32, 2, 2, 48, 32, 16, 8, 4
    vlm = lib.vision_lm_create(d.params, V, D, L, H, D // H, F, 3, img, img, patch, 1)
    lib.vision_lm_enable_rope(d.params, vlm, Tmax, 10000.0)
    names = models.vlm_param_names(L)
    params, _ = models.seeded_weights(d, vlm, names, 123)
    arr = (B.TensorP * len(params))(*params)
    opt = lib.adamw_create(d.params, arr, len(params), 6e-4, 0.9, 0.95, 1e-8, 0.1)
    images, _, ids_all, tgt_all, _ = models.vlm_inputs(3, Bsz, img, V, Tmax)
    lens_all = np.array([3, 6, 6, 3], np.int32)
    mask_all = (np.arange(Tmax)[None, :] < (lens_all[:, None] - 1)).astype(np.float32)
    per = Bsz // world
    sl = slice(rank * per, (rank + 1) * per)
    lens = np.ascontiguousarray(lens_all[sl])
    for step in range(2):
        gn = C.c_float(0)
        loss = lib.dnn_cuda_dp_vision_lm_train_step_padded(d.scratch, vlm, d.tensor(images[sl], d.data), d.tensor(ids_all[sl], d.data),
                                                           d.tensor(tgt_all[sl], d.data), d.tensor(mask_all[sl], d.data),
                                                           lens.ctypes.data_as(C.POINTER(C.c_int)), opt, 1.0, C.byref(gn))
        res["loss%d" % step] = np.float32(d.scalar(loss)); res["gn%d" % step] = np.float32(gn.value)
        if step == 0:
            for n, t in zip(names, params):
                g = d.download_grad(t)
                if g is None:
                    assert n.startswith("img_proj"), n
                else:
                    res["g/" + n] = g
        d.reset_step()
else:
    # the MNIST-shaped CNN driven op by op, as the reference's own loop does (examples/mnist/mnist_train.c:99-114),
    # with dnn_cuda_dp_backward in the place of dnn_backward; no clipping
    Bsz = 8
    c1 = lib.conv2d_create(d.params, 1, 32, 3, 1, 1); c2 = lib.conv2d_create(d.params, 32, 64, 3, 1, 1)
    f1 = lib.linear_create(d.params, 3136, 128); f2 = lib.linear_create(d.params, 128, 10)
    params = []
    for m in (c1, c2, f1, f2): params += d.parameters(m)
    names = models.CNN_NAMES
    rng = np.random.default_rng(2)
    for t in params: d.upload(t, ((rng.random(d.shape_of(t)) * 2 - 1) * 0.05).astype(np.float32))
    arr = (B.TensorP * len(params))(*params)
    opt = lib.adamw_create(d.params, arr, len(params), 1e-3, 0.9, 0.999, 1e-8, 0.01)
    x_all = rng.random((Bsz, 784)).astype(np.float32); y_all = rng.integers(0, 10, size=Bsz).astype(np.int32)
    per = Bsz // world
    sl = slice(rank * per, (rank + 1) * per)
    for step in range(2):
        x, y = d.tensor(x_all[sl], d.data), d.tensor(y_all[sl], d.data)
        h = lib.tensor_reshape(d.scratch, x, 4, B.ints([per, 1, 28, 28]))
        h = lib.tensor_avg_pool2d(d.scratch, lib.tensor_relu(d.scratch, lib.conv2d_forward(d.scratch, c1, h)), 2, 2)
        h = lib.tensor_avg_pool2d(d.scratch, lib.tensor_relu(d.scratch, lib.conv2d_forward(d.scratch, c2, h)), 2, 2)
        h = lib.tensor_reshape(d.scratch, h, 2, B.ints([per, 3136]))
        h = lib.tensor_relu(d.scratch, lib.linear_forward(d.scratch, f1, h))
        loss = lib.tensor_cross_entropy(d.scratch, lib.linear_forward(d.scratch, f2, h), y, 1)
        assert lib.dnn_cuda_dp_backward(d.scratch, loss, arr, len(params)) == 0, lib.dnn_cuda_dp_last_error()
        res["loss%d" % step] = np.float32(d.scalar(loss)); res["gn%d" % step] = np.float32(lib.grad_norm(arr, len(params)))
        if step == 0:
            for n, t in zip(names, params): res["g/" + n] = d.download_grad(t)
        lib.adamw_step(opt); lib.adamw_zero_grad(opt)
        d.reset_step()
for n, t in zip(names, params): res["p/" + n] = d.download(t)
np.savez(os.path.join(out, "rank%d_of%d.npz" % (rank, world)), **res)
if world > 1: lib.dnn_cuda_dp_finalize()
d.close()
"""


@pytest.mark.parametrize("kind", ["lm", "vlm", "cnn"])
@pytest.mark.parametrize("overlap", ["0", "1"], ids=["exchange-after-backward", "exchange-during-backward"])
def test_two_ranks_match_one_rank_with_the_whole_batch(tmp_path, overlap, kind):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "dp_worker.py"
    script.write_text(WORKER.format(root=ROOT))
    # small buckets: the exchange of the second step is split into many all-reduces that start during backward
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", DNN_CUDA_BUCKET_BYTES="16384", DNN_CUDA_DP_OVERLAP=overlap)
    single = subprocess.run([sys.executable, str(script), "0", "1", str(tmp_path), kind], env=env, capture_output=True, text=True, timeout=600)
    assert single.returncode == 0, single.stdout + single.stderr
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", str(tmp_path), kind], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    one = np.load(tmp_path / "rank0_of1.npz")
    r0, r1 = np.load(tmp_path / "rank0_of2.npz"), np.load(tmp_path / "rank1_of2.npz")
    # mean of the per-rank mean losses is the full-batch loss
    assert abs(0.5 * (r0["loss0"] + r1["loss0"]) - one["loss0"]) <= 1e-6 * abs(one["loss0"])
    assert abs(r0["gn0"] - one["gn0"]) <= 1e-5 * one["gn0"] and r0["gn0"] == r1["gn0"]
    for k in one.files:
        if k.startswith(("g/", "p/")):
            a, b = r0[k].astype(np.float64), one[k].astype(np.float64)
            # Gradients agree to fp32 rounding (half and whole batches take different kernels and summation
            # orders).  AdamW divides by sqrt(v): where a gradient is mathematically zero (the key part of a
            # QKV bias) the update is normalised rounding noise, so parameters get a wider bound.
            tol = 2e-5 if k.startswith("g/") else 1e-4
            assert np.linalg.norm(a - b) <= tol * np.linalg.norm(b) + 1e-9, k
            assert np.array_equal(r0[k], r1[k]), "ranks diverged on " + k
