"""Generates tests/golden/*.npz by running the UNMODIFIED reference library.

    make -C oracle && OMP_NUM_THREADS=1 python tests/golden/make_golden.py

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


def main():
    B = load_binding()
    ops = {}
    ref = B.Dnn(REF_LIB, params_mb=256, scratch_mb=2048, data_mb=64)
    for case in CASES:
        out = case.run(ref, case.make(np.random.default_rng(SEED)))
        ref.reset_step()
        for k, v in out.items():
            store(ops, case.name + "/" + k, v)
    ref.close()
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **ops)

    gen = {}
    for name, over, prompt, max_new, temp, use_cache in models.GEN_CASES:
        d = B.Dnn(REF_LIB, params_mb=64, scratch_mb=512, data_mb=64)
        cfg = dict(models.lm_config("tiny")); cfg.update(over)
        gen[name] = np.array(models.run_generate(d, cfg, prompt, max_new, temp, use_cache, seed=77), np.int32)
        d.close()
        print("generate", name, gen[name].tolist())
    np.savez_compressed(os.path.join(HERE, "generate.npz"), **gen)

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
    model("vlm", models.run_vlm, steps=2)
    np.savez_compressed(os.path.join(HERE, "models.npz"), **mdl)
    for f in ("ops.npz", "models.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KiB")
    print("lm_c1 loss", mdl["lm_c1/loss"], "grad_norm", mdl["lm_c1/grad_norm"])


if __name__ == "__main__":
    main()
