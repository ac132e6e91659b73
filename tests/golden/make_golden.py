"""Generates tests/golden/*.npz by running the UNMODIFIED reference library.

    make -C oracle REF=<reference checkout> && OMP_NUM_THREADS=1 python tests/golden/make_golden.py [ops] [generate] [models] [batch] [module]

Without arguments all five files are written; with arguments only the named ones.

Needs oracle/_ref/libdnn_ref.so (built from the reference's own sources by
oracle/Makefile), so it runs only where the reference sources are mounted.
The vectors it writes are what pins the numpy oracle and the CUDA kernels to
the reference on machines that do not have it.  Single-threaded on purpose:
the reference's norm backward races under OpenMP (src/norm.c:299-321).
"""
import os
import sys

os.environ["OMP_NUM_THREADS"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import numpy as np  # noqa: E402

from conftest import REF_LIB, load_binding  # noqa: E402
from cases import CASES  # noqa: E402
from golden_util import pack  # noqa: E402
import models  # noqa: E402

SEED = 1234


def store(dst, prefix, arr):
    sample, stats = pack(arr)
    dst[prefix] = sample
    dst[prefix + "#"] = stats


def write_ops(B):
    ops = {}
    ref = B.Dnn(REF_LIB, params_mb=256, scratch_mb=2048, data_mb=64)
    for case in CASES:
        out = case.run(ref, case.make(np.random.default_rng(SEED)))
        ref.reset_step()
        for k, v in out.items():
            store(ops, case.name + "/" + k, v)
    ref.close()
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **ops)


def write_generate(B):
    gen = {}
    for name, over, prompt, max_new, temp, use_cache in models.GEN_CASES:
        d = B.Dnn(REF_LIB, params_mb=64, scratch_mb=512, data_mb=64)
        cfg = dict(models.lm_config("tiny")); cfg.update(over)
        gen[name] = np.array(models.run_generate(d, cfg, prompt, max_new, temp, use_cache, seed=77), np.int32)
        d.close()
        print("generate", name, gen[name].tolist())
    for name, prompt, max_new, temp, use_cache, patched in models.VLM_GEN_CASES:
        d = B.Dnn(REF_LIB, params_mb=64, scratch_mb=512, data_mb=64)
        gen[name] = np.array(models.run_vlm_generate(d, prompt, max_new, temp, use_cache, patched, seed=77), np.int32)
        d.close()
        print("generate", name, gen[name].tolist())
    np.savez_compressed(os.path.join(HERE, "generate.npz"), **gen)


def write_models(B):
    mdl = {}

    def model(tag, fn, **kw):
        d = B.Dnn(REF_LIB, params_mb=512, scratch_mb=4096, data_mb=64)
        out = fn(d, **kw)
        d.close()
        mdl[tag + "/loss"] = np.array(out["loss"], np.float32)
        if "grad_norm" in out:
            mdl[tag + "/grad_norm"] = np.array(out["grad_norm"], np.float32)
        for n, g in out["grads"].items():
            if g is not None:
                store(mdl, tag + "/grad/" + n, g)
        mdl[tag + "/grad_missing"] = np.array([n for n, g in out["grads"].items() if g is None])
        for n, p in out["params"].items():
            store(mdl, tag + "/param/" + n, p)
        for k in ("logits", "shifted"):
            if k in out:
                store(mdl, tag + "/" + k, out[k])

    for name in ("tiny", "odd", "c1"):
        model("lm_" + name, models.run_lm, cfg=models.lm_config(name), steps=3)
    model("cnn", models.run_cnn, batch=8, steps=2)
    model("cnn512", models.run_cnn, batch=512, steps=1)       # BASELINE config 3 at its full batch
    model("vlm", models.run_vlm, steps=2)
    np.savez_compressed(os.path.join(HERE, "models.npz"), **mdl)
    print("lm_c1 loss", mdl["lm_c1/loss"], "grad_norm", mdl["lm_c1/grad_norm"])


def write_batch(B):
    """Padded vision-LM batches built by the reference's own loader (imagenet_vlm_dl_next_batch) from a
    synthetic dataset written in its on-disk format; shuffle off, so no flips."""
    import ctypes as C
    import tempfile
    import vlm_batch_data as D
    out = {}
    ref = B.Dnn(REF_LIB, params_mb=16, scratch_mb=64, data_mb=16)
    lib = ref.lib
    lib.imagenet_vlm_dl_create.restype = C.c_void_p
    lib.imagenet_vlm_dl_create.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_ulong]
    lib.imagenet_vlm_dl_free.argtypes = [C.c_void_p]
    lib.imagenet_vlm_dl_next_batch.restype = C.c_int
    lib.imagenet_vlm_dl_next_batch.argtypes = [C.c_void_p] + [B.TensorP] * 4 + [C.POINTER(C.c_int)] * 2 + [C.c_int]
    with tempfile.TemporaryDirectory() as root:
        for version in (1, 2, 3):
            split = "v%d" % version
            D.write_dataset(root, split, D.make_samples(SEED + version, 5, version), version)
            dl = lib.imagenet_vlm_dl_create(split.encode(), root.encode(), 0, 1)
            assert dl, "the reference rejected the synthetic dataset"
            for batch, bs in enumerate((3, 3)):        # 5 samples: a full batch, then a short one
                ishape = (bs, 2, 768) if version == 3 else (bs, D.C, D.H, D.W)
                img = ref.tensor(np.zeros(ishape, np.float32), ref.data)
                ids = ref.tensor(np.zeros((bs, D.T_MAX), np.int32), ref.data)
                tgt = ref.tensor(np.zeros((bs, D.T_MAX), np.int32), ref.data)
                mask = ref.tensor(np.zeros((bs, D.T_MAX), np.float32), ref.data)
                lens, labels = (C.c_int * bs)(), (C.c_int * bs)()
                n = lib.imagenet_vlm_dl_next_batch(dl, img, ids, tgt, mask, lens, labels, bs)
                assert n == (3, 2)[batch], n
                tag = "%s/b%d/" % (split, batch)
                out[tag + "img"] = ref.download(img)[:n]
                out[tag + "input_ids"] = ref.download(ids, np.int32)[:n]
                out[tag + "target_ids"] = ref.download(tgt, np.int32)[:n]
                out[tag + "loss_mask"] = ref.download(mask)[:n]
                out[tag + "text_lens"] = np.array(lens[:n], np.int32)
                out[tag + "label_ids"] = np.array(labels[:n], np.int32)
                ref.reset_step()
            lib.imagenet_vlm_dl_free(dl)
    ref.close()
    np.savez_compressed(os.path.join(HERE, "batch.npz"), **out)


def write_module_file(B):
    """A weight file written by the reference's own module_save (src/module.c:208-268) for the tiny decoder LM
    with seeded weights: the bytes a drop-in library has to write, and has to be able to load."""
    import ctypes as C
    d = B.Dnn(REF_LIB, params_mb=64, scratch_mb=64, data_mb=16)
    cfg = models.lm_config("tiny")
    lm = d.lib.decoder_lm_create(d.params, cfg["V"], cfg["D"], cfg["L"], cfg["H"], cfg["D"] // cfg["H"], cfg["F"])
    d.lib.decoder_lm_enable_rope(d.params, lm, cfg["N"], 10000.0)
    models.seeded_weights(d, lm, models.O.lm_param_names(cfg["L"]), cfg["seed"] + 100)
    d.lib.module_save(C.cast(lm, C.c_void_p), os.path.join(HERE, "lm_tiny.dnnm").encode())
    d.close()


def main():
    B = load_binding()
    which = sys.argv[1:] or ["ops", "generate", "models", "batch", "module"]
    if "module" in which:
        write_module_file(B)
        print("lm_tiny.dnnm", os.path.getsize(os.path.join(HERE, "lm_tiny.dnnm")) // 1024, "KiB")
    for name, fn in (("ops", write_ops), ("generate", write_generate), ("models", write_models), ("batch", write_batch)):
        if name in which:
            fn(B)
            print(name + ".npz", os.path.getsize(os.path.join(HERE, name + ".npz")) // 1024, "KiB")


if __name__ == "__main__":
    main()
