"""Padded vision-LM batch assembly: the numpy oracle against the batches the unmodified reference
loader built (tests/golden/batch.npz), and the device stager (dnn_cuda_vlm_stager_*) against both.
Everything here is integer or separately rounded fp32 work, so every comparison is bit-exact."""
import ctypes as C
import os

import numpy as np
import pytest

import vlm_batch_data as D
from oracle import dnn_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "batch.npz")
BATCHES = ((0, 3), (3, 5))       # the golden file holds 5 samples as a batch of 3 and a short batch of 2
SEED = 1234


def _oracle_batch(part, version, flips):
    inp, tgt, mask, lens = O.vlm_batch_text([t for _, t, _ in part], D.T_MAX)
    if version < 3:
        img = O.vlm_batch_pixels(np.stack([p for _, _, p in part]), flips, D.MEAN, D.STD)
    else:
        img = np.stack([p for _, _, p in part])
    return dict(img=img, input_ids=inp, target_ids=tgt, loss_mask=mask, text_lens=lens,
                label_ids=np.array([l for l, _, _ in part], np.int32))


@pytest.mark.parametrize("version", [1, 2, 3])
def test_oracle_batches_equal_the_reference_loader(version):
    g = np.load(GOLDEN)
    samples = D.make_samples(SEED + version, 5, version)
    for b, (lo, hi) in enumerate(BATCHES):
        want = _oracle_batch(samples[lo:hi], version, [0] * (hi - lo))
        for k, v in want.items():
            ref = g["v%d/b%d/%s" % (version, b, k)]
            assert v.dtype == ref.dtype and v.tobytes() == ref.tobytes(), (version, b, k)


def _stage(binding, d, st, slot, part, flips):
    for i, (label, text, payload) in enumerate(part):
        buf = np.ascontiguousarray(payload)
        rc = d.lib.dnn_cuda_vlm_stager_put(st, slot, i, text.ctypes.data_as(C.POINTER(C.c_int)), len(text),
                                           buf.ctypes.data_as(C.c_void_p), int(flips[i]), label)
        assert rc == 0, d.lib.dnn_cuda_vlm_stager_error()
    assert d.lib.dnn_cuda_vlm_stager_submit(st, slot, len(part)) == 0


def _assemble(binding, d, st, slot, bs, version, t_batch=D.T_MAX, rows=None):
    rows = rows or bs
    ishape = (rows, 2, 768) if version == 3 else (rows, D.C, D.H, D.W)
    img = d.tensor(np.zeros(ishape, np.float32), d.data)
    ids = d.tensor(np.zeros((rows, t_batch), np.int32), d.data)
    tgt = d.tensor(np.zeros((rows, t_batch), np.int32), d.data)
    mask = d.tensor(np.zeros((rows, t_batch), np.float32), d.data)
    lens, labels = (C.c_int * rows)(), (C.c_int * rows)()
    n = d.lib.dnn_cuda_vlm_stager_assemble(st, slot, img, ids, tgt, mask, lens, labels)
    if n < 0:
        return n, None
    return n, dict(img=d.download(img)[:n], input_ids=d.download(ids, np.int32)[:n], target_ids=d.download(tgt, np.int32)[:n],
                   loss_mask=d.download(mask)[:n], text_lens=np.array(lens[:n], np.int32), label_ids=np.array(labels[:n], np.int32))


def _stager(d, version, slots=2, max_bs=4, H=D.H, W=D.W, Cn=D.C):
    mean, std = (C.c_float * 3)(*D.MEAN), (C.c_float * 3)(*D.STD)
    st = d.lib.dnn_cuda_vlm_stager_create(slots, max_bs, D.T_MAX, H, W, Cn, 1 if version == 3 else 0, mean, std)
    assert st
    return st


@pytest.mark.gpu
@pytest.mark.parametrize("version", [1, 2, 3])
def test_device_batches_equal_the_reference_loader(binding, version):
    """Both batches are staged before either is assembled: slot 1 uploads while slot 0 is consumed."""
    g = np.load(GOLDEN)
    samples = D.make_samples(SEED + version, 5, version)
    d = binding.Dnn(binding.B200_LIB, params_mb=16, scratch_mb=64, data_mb=16)
    st = _stager(d, version)
    try:
        for slot, (lo, hi) in enumerate(BATCHES):
            _stage(binding, d, st, slot, samples[lo:hi], [0] * (hi - lo))
        for slot, (lo, hi) in enumerate(BATCHES):
            n, got = _assemble(binding, d, st, slot, hi - lo, version, rows=3)      # the short batch lands in 3-row tensors
            assert n == hi - lo
            for k, v in got.items():
                ref = g["v%d/b%d/%s" % (version, slot, k)]
                assert v.dtype == ref.dtype and v.tobytes() == ref.tobytes(), (version, slot, k)
    finally:
        d.lib.dnn_cuda_vlm_stager_destroy(st)
        d.close()


@pytest.mark.gpu
@pytest.mark.parametrize("geometry", [(16, 32, 3), (8, 20, 3), (5, 7, 3), (6, 10, 1), (4, 8, 4)], ids=str)
def test_device_pixels_with_flips_equal_the_oracle(binding, geometry):
    """Flipped and unflipped samples, widths that take the vector kernel and widths that do not, and a
    slot that is reused three times in a row."""
    H, W, Cn = geometry
    rng = np.random.default_rng(7)
    d = binding.Dnn(binding.B200_LIB, params_mb=16, scratch_mb=64, data_mb=16)
    mean, std = (C.c_float * 4)(0.485, 0.456, 0.406, 0.5), (C.c_float * 4)(0.229, 0.224, 0.225, 0.25)
    st = d.lib.dnn_cuda_vlm_stager_create(1, 4, D.T_MAX, H, W, Cn, 0, mean, std)
    assert st
    try:
        for trip in range(3):
            bs = 4 - trip
            part = [(int(rng.integers(0, 1000)), rng.integers(0, 257, size=int(rng.integers(1, D.T_MAX))).astype(np.int32),
                     rng.integers(0, 256, size=(H, W, Cn)).astype(np.uint8)) for _ in range(bs)]
            flips = rng.integers(0, 2, size=bs)
            _stage(binding, d, st, 0, part, flips)
            img = d.tensor(np.zeros((bs, Cn, H, W), np.float32), d.data)
            ids = d.tensor(np.zeros((bs, D.T_MAX), np.int32), d.data)
            tgt = d.tensor(np.zeros((bs, D.T_MAX), np.int32), d.data)
            mask = d.tensor(np.zeros((bs, D.T_MAX), np.float32), d.data)
            assert d.lib.dnn_cuda_vlm_stager_assemble(st, 0, img, ids, tgt, mask, None, None) == bs
            want = O.vlm_batch_pixels(np.stack([p for _, _, p in part]), flips, list(mean)[:Cn], list(std)[:Cn])
            assert d.download(img).tobytes() == want.tobytes()
            inp, tg, mk, _ = O.vlm_batch_text([t for _, t, _ in part], D.T_MAX)
            assert (d.download(ids, np.int32) == inp).all() and (d.download(tgt, np.int32) == tg).all() and (d.download(mask) == mk).all()
            d.reset_step()
    finally:
        d.lib.dnn_cuda_vlm_stager_destroy(st)
        d.close()


@pytest.mark.gpu
def test_stager_rejects_what_the_reference_rejects(binding):
    """A text longer than the batch width and an image tensor of the wrong geometry return -1
    (src/imagenet_vlm.c:583, 643); nothing is written."""
    d = binding.Dnn(binding.B200_LIB, params_mb=16, scratch_mb=64, data_mb=16)
    st = _stager(d, 1)
    try:
        text = np.arange(D.T_MAX, dtype=np.int32)                 # stored_len + 1 > T_MAX
        px = np.zeros((D.H, D.W, D.C), np.uint8)
        assert d.lib.dnn_cuda_vlm_stager_put(st, 0, 0, text.ctypes.data_as(C.POINTER(C.c_int)), len(text),
                                             px.ctypes.data_as(C.c_void_p), 0, 1) == -1
        samples = D.make_samples(SEED + 1, 3, 1)
        _stage(binding, d, st, 0, samples, [0, 0, 0])
        n, _ = _assemble(binding, d, st, 0, 3, 1, t_batch=D.T_MAX - 1)      # sample 0 needs the full width
        assert n == -1
        n, _ = _assemble(binding, d, st, 0, 3, 3)                            # patch-shaped tensor for a pixel stager
        assert n == -1
        n, got = _assemble(binding, d, st, 0, 3, 1)
        assert n == 3 and got["text_lens"].tolist() == [len(t) + 1 for _, t, _ in samples]
    finally:
        d.lib.dnn_cuda_vlm_stager_destroy(st)
        d.close()
