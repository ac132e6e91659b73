"""GPU: the training step recorded as one CUDA graph replays to the same bits as eager steps."""
import ctypes as C

import numpy as np
import pytest

import models
from test_gpu_checkpoint import _build

pytestmark = pytest.mark.gpu


def _eager(d, lm, opt, cfg, ids, tgt, lrs):
    out = []
    for lr in lrs:
        opt.contents.lr = lr
        gn = C.c_float(0)
        loss = d.lib.decoder_lm_train_step(d.scratch, lm, ids, tgt, opt, cfg["clip"], C.byref(gn))
        out.append((d.scalar(loss), float(gn.value)))
        d.reset_step()
    return out


@pytest.mark.parametrize("name,over", [("c1", dict(L=2, B=4, N=64)), ("tiny", {}), ("c1", dict(L=1, B=2, N=200, D=128, H=2))],
                         ids=["d32", "d16-exact-attention", "d64-ragged"])
def test_replayed_steps_equal_eager_steps(binding, name, over):
    cfg = dict(models.lm_config(name)); cfg.update(over)
    ids_np, _ = models.lm_inputs(cfg)
    lrs = [cfg["lr"], cfg["lr"] * 0.5, cfg["lr"] * 0.25, cfg["lr"] * 2.0]      # a schedule: the graph must pick up opt->lr

    d, lm, opt, params, names, keep = _build(binding, cfg)
    ids = d.tensor(ids_np, d.data); tgt = d.lib.decoder_lm_shift_targets(d.data, ids)
    want = _eager(d, lm, opt, cfg, ids, tgt, lrs)
    want_params = {n: d.download(t) for n, t in zip(names, params)}
    d.close()

    d, lm, opt, params, names, keep = _build(binding, cfg)
    ids = d.tensor(ids_np, d.data); tgt = d.lib.decoder_lm_shift_targets(d.data, ids)
    got = _eager(d, lm, opt, cfg, ids, tgt, lrs[:1])                              # warm-up step, eager
    g = d.lib.dnn_cuda_graph_capture_decoder_lm_step(d.scratch, lm, ids, tgt, opt, cfg["clip"])
    assert g, "capture failed"
    before = d.lib.dnn_cuda_launch_count()
    for lr in lrs[1:]:
        opt.contents.lr = lr
        loss, gn = C.c_float(0), C.c_float(0)
        assert d.lib.dnn_cuda_graph_replay(g, C.byref(loss), C.byref(gn)) == 0
        got.append((float(loss.value), float(gn.value)))
    assert d.lib.dnn_cuda_launch_count() - before > 3 * 20, "replays must account for the kernels they run"
    assert got == want, (got, want)
    assert opt.contents.t == len(lrs)
    for n, t in zip(names, params):
        assert np.array_equal(d.download(t), want_params[n]), n
    d.lib.dnn_cuda_graph_destroy(g)
    d.close()


def test_new_batches_go_through_the_same_tensors(binding):
    """Replays read whatever the captured input tensors hold at launch time."""
    cfg = dict(models.lm_config("c1")); cfg.update(L=1, B=2, N=32)
    rng = np.random.default_rng(5)
    batches = [rng.integers(0, cfg["V"], size=(cfg["B"], cfg["N"])).astype(np.int32) for _ in range(3)]

    def run(graph):
        d, lm, opt, params, names, keep = _build(binding, cfg)
        ids = d.tensor(batches[0], d.data); tgt = d.lib.decoder_lm_shift_targets(d.data, ids)
        losses = [x[0] for x in _eager(d, lm, opt, cfg, ids, tgt, [cfg["lr"]])]
        g = d.lib.dnn_cuda_graph_capture_decoder_lm_step(d.scratch, lm, ids, tgt, opt, cfg["clip"]) if graph else None
        for b in batches[1:]:
            d.upload(ids, b); d.upload(tgt, np.ascontiguousarray(b[:, 1:]))
            if graph:
                loss = C.c_float(0)
                assert d.lib.dnn_cuda_graph_replay(g, C.byref(loss), None) == 0
                losses.append(float(loss.value))
            else:
                losses += [x[0] for x in _eager(d, lm, opt, cfg, ids, tgt, [cfg["lr"]])]
        p = {n: d.download(t) for n, t in zip(names, params)}
        if graph:
            d.lib.dnn_cuda_graph_destroy(g)
        d.close()
        return losses, p

    l0, p0 = run(False)
    l1, p1 = run(True)
    assert l0 == l1
    for n in p0:
        assert np.array_equal(p0[n], p1[n]), n


def test_replays_queued_without_readback_equal_eager_steps(binding):
    """Twenty replays launched back to back with NULL outputs (nothing makes the host wait), each with its
    own learning rate.  The graph reads learning rate and bias corrections from pinned host memory when
    it EXECUTES, so every replay needs its own copy of them: the parameters must equal twenty eager steps
    bit for bit."""
    cfg = dict(models.lm_config("c1")); cfg.update(L=2, B=4, N=64)
    ids_np, _ = models.lm_inputs(cfg)
    lrs = [cfg["lr"] * (1.0 + 0.37 * (s % 5)) for s in range(21)]

    d, lm, opt, params, names, keep = _build(binding, cfg)
    ids = d.tensor(ids_np, d.data); tgt = d.lib.decoder_lm_shift_targets(d.data, ids)
    _eager(d, lm, opt, cfg, ids, tgt, lrs)
    want = {n: d.download(t) for n, t in zip(names, params)}
    d.close()

    d, lm, opt, params, names, keep = _build(binding, cfg)
    ids = d.tensor(ids_np, d.data); tgt = d.lib.decoder_lm_shift_targets(d.data, ids)
    _eager(d, lm, opt, cfg, ids, tgt, lrs[:1])
    g = d.lib.dnn_cuda_graph_capture_decoder_lm_step(d.scratch, lm, ids, tgt, opt, cfg["clip"])
    assert g, "capture failed"
    for lr in lrs[1:]:
        opt.contents.lr = lr
        assert d.lib.dnn_cuda_graph_replay(g, None, None) == 0
    d.sync()
    assert opt.contents.t == len(lrs)
    for n, t in zip(names, params):
        assert np.array_equal(d.download(t), want[n]), n
    d.lib.dnn_cuda_graph_destroy(g)
    d.close()
