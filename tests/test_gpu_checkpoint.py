"""GPU: a run saved with module_save + dnn_cuda_optimizer_save and loaded into a freshly built
model and optimiser continues bit for bit (weights, AdamW moments and step counter restored)."""
import ctypes as C
import os

import numpy as np
import pytest

import models

pytestmark = pytest.mark.gpu


def _build(binding, cfg):
    d = binding.Dnn(binding.B200_LIB, params_mb=256, scratch_mb=2048, data_mb=32)
    d.lib.dnn_cuda_set_gemm_mode(binding.GEMM_TF32)
    lib = d.lib
    lm = lib.decoder_lm_create(d.params, cfg["V"], cfg["D"], cfg["L"], cfg["H"], cfg["D"] // cfg["H"], cfg["F"])
    lib.decoder_lm_enable_rope(d.params, lm, cfg["N"], 10000.0)
    names = models.O.lm_param_names(cfg["L"])
    params, _ = models.seeded_weights(d, lm, names, cfg["seed"] + 100)
    arr = (binding.TensorP * len(params))(*params)
    opt = lib.adamw_create(d.params, arr, len(params), cfg["lr"], cfg["b1"], cfg["b2"], cfg["eps"], cfg["wd"])
    return d, lm, opt, params, names, arr


def _steps(d, lm, opt, cfg, ids_np, n):
    losses = []
    for _ in range(n):
        ids = d.tensor(ids_np, d.data)
        tgt = d.lib.decoder_lm_shift_targets(d.data, ids)
        gn = C.c_float(0)
        loss = d.lib.decoder_lm_train_step(d.scratch, lm, ids, tgt, opt, cfg["clip"], C.byref(gn))
        losses.append(d.scalar(loss))
        d.reset_step()
    return losses


def test_resume_continues_bit_for_bit(binding, tmp_path):
    cfg = dict(models.lm_config("c1"))
    cfg.update(L=2, B=4, N=64)
    ids_np, _ = models.lm_inputs(cfg)
    wfile, ofile = str(tmp_path / "weights.dnnm").encode(), str(tmp_path / "adamw.dnno").encode()

    d, lm, opt, params, names, keep = _build(binding, cfg)
    first = _steps(d, lm, opt, cfg, ids_np, 2)
    d.lib.module_save(C.cast(lm, C.c_void_p), wfile)
    assert d.lib.dnn_cuda_optimizer_save(opt, ofile) == 0
    straight = _steps(d, lm, opt, cfg, ids_np, 2)
    want = {n: d.download(t) for n, t in zip(names, params)}
    t_end = opt.contents.t
    d.close()

    d2, lm2, opt2, params2, names2, keep2 = _build(binding, dict(cfg, seed=cfg["seed"] + 1))    # different initial weights
    d2.lib.module_load(C.cast(lm2, C.c_void_p), wfile, 1)
    assert d2.lib.dnn_cuda_optimizer_load(opt2, ofile) == 0
    assert opt2.contents.t == 2
    resumed = _steps(d2, lm2, opt2, cfg, ids_np, 2)
    assert resumed == straight, (resumed, straight, first)
    assert opt2.contents.t == t_end
    for n, t in zip(names2, params2):
        assert np.array_equal(d2.download(t), want[n]), n
    d2.close()


def test_optimizer_load_rejects_a_mismatched_file(binding, tmp_path):
    cfg = dict(models.lm_config("tiny"))
    d, lm, opt, params, names, keep = _build(binding, cfg)
    ofile = str(tmp_path / "adamw.dnno").encode()
    assert d.lib.dnn_cuda_optimizer_save(opt, ofile) == 0
    d.close()
    d2, lm2, opt2, *_ = _build(binding, dict(cfg, D=64, H=4))
    assert d2.lib.dnn_cuda_optimizer_load(opt2, ofile) == -3
    assert d2.lib.dnn_cuda_optimizer_load(opt2, str(tmp_path / "missing").encode()) == -2
    d2.close()
