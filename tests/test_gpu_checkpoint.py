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


def test_train_state_restores_scheduler_step_and_host_rng(binding, tmp_path):
    """A run with a warm-up/cosine schedule that also draws a dropout mask every step (from the host generator,
    like src/ops_activation.c:1460): saved after two steps with dnn_cuda_train_state_save and loaded into a fresh
    model, optimiser and scheduler, it continues with the same learning rates, losses, masks and parameters."""
    cfg = dict(models.lm_config("c1"))
    cfg.update(L=1, B=2, N=32)
    ids_np, _ = models.lm_inputs(cfg)
    wfile, sfile = str(tmp_path / "weights.dnnm").encode(), str(tmp_path / "state.dnnt").encode()
    probe = np.ones((4, 50), np.float32)

    def steps(d, lm, opt, sched, n):
        out = []
        for _ in range(n):
            ids = d.tensor(ids_np, d.data)
            tgt = d.lib.decoder_lm_shift_targets(d.data, ids)
            gn = C.c_float(0)
            loss = d.lib.decoder_lm_train_step(d.scratch, lm, ids, tgt, opt, cfg["clip"], C.byref(gn))
            mask = d.download(d.lib.tensor_dropout(d.scratch, d.tensor(probe, d.scratch), 0.5))
            d.lib.lr_scheduler_step(sched)
            out.append((d.scalar(loss), float(opt.contents.lr), mask.tobytes()))
            d.reset_step()
        return out

    d, lm, opt, params, names, keep = _build(binding, cfg)
    d.lib.dnn_seed(99)
    sched = d.lib.lr_scheduler_create(d.params, opt, 1, cfg["lr"], 3, 10, -1.0, 0, 0.0)
    steps(d, lm, opt, sched, 2)
    d.lib.module_save(C.cast(lm, C.c_void_p), wfile)
    assert d.lib.dnn_cuda_train_state_save(opt, sched, sfile) == 0
    straight = steps(d, lm, opt, sched, 3)
    want = {n: d.download(t) for n, t in zip(names, params)}
    d.close()

    d2, lm2, opt2, params2, names2, keep2 = _build(binding, dict(cfg, seed=cfg["seed"] + 1))
    d2.lib.dnn_seed(12345)                                    # a different generator state, to be overwritten
    sched2 = d2.lib.lr_scheduler_create(d2.params, opt2, 1, cfg["lr"], 3, 10, -1.0, 0, 0.0)
    d2.lib.module_load(C.cast(lm2, C.c_void_p), wfile, 1)
    assert d2.lib.dnn_cuda_train_state_load(opt2, sched2, sfile) == 0
    assert sched2.contents.t == 2 and opt2.contents.t == 2
    resumed = steps(d2, lm2, opt2, sched2, 3)
    assert resumed == straight
    for n, t in zip(names2, params2):
        assert np.array_equal(d2.download(t), want[n]), n
    # a file without the tail (optimiser only) is refused by the full loader
    ofile = str(tmp_path / "adamw.dnno").encode()
    assert d2.lib.dnn_cuda_optimizer_save(opt2, ofile) == 0
    assert d2.lib.dnn_cuda_train_state_load(opt2, sched2, ofile) == -3
    d2.close()


def test_weight_files_interchange_with_the_reference(binding, tmp_path):
    """module_save / module_load speak the reference's file format (src/module.c:208-339): for the tiny decoder LM
    with seeded weights this library writes, byte for byte, the file the unmodified reference wrote
    (tests/golden/lm_tiny.dnnm), and loads that file into a model with other weights.  Where a build of the
    reference is present, the reference also loads the file written here."""
    from conftest import REF_LIB
    cfg = models.lm_config("tiny")
    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "lm_tiny.dnnm")
    mine = str(tmp_path / "mine.dnnm")
    d, lm, opt, params, names, keep = _build(binding, cfg)
    d.lib.module_save(C.cast(lm, C.c_void_p), mine.encode())
    want = {n: d.download(t) for n, t in zip(names, params)}
    d.close()
    assert open(mine, "rb").read() == open(golden, "rb").read()

    d2, lm2, opt2, params2, names2, keep2 = _build(binding, dict(cfg, seed=cfg["seed"] + 1))
    assert not np.array_equal(d2.download(params2[0]), want[names2[0]])
    d2.lib.module_load(C.cast(lm2, C.c_void_p), golden.encode(), 1)
    for n, t in zip(names2, params2):
        assert np.array_equal(d2.download(t), want[n]), n
    d2.close()

    if os.path.exists(REF_LIB):
        r = binding.Dnn(REF_LIB, params_mb=64, scratch_mb=64, data_mb=16)
        rlm = r.lib.decoder_lm_create(r.params, cfg["V"], cfg["D"], cfg["L"], cfg["H"], cfg["D"] // cfg["H"], cfg["F"])
        r.lib.module_load(C.cast(rlm, C.c_void_p), mine.encode(), 1)
        for n, t in zip(names, r.parameters(rlm)):
            assert np.array_equal(r.download(t), want[n]), n
        r.close()
