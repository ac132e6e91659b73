"""CPU: pins the numpy oracle to the reference through the committed golden
vectors (tests/golden/*.npz, written by tests/golden/make_golden.py from the
unmodified reference library)."""
import os

import numpy as np
import pytest

from cases import CASES
from golden_util import check
import models
from oracle import dnn_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def ops_golden():
    return np.load(os.path.join(GOLDEN, "ops.npz"))


@pytest.fixture(scope="module")
def model_golden():
    return np.load(os.path.join(GOLDEN, "models.npz"))


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_oracle_matches_reference_vectors(ops_golden, case):
    want = case.oracle(case.make(np.random.default_rng(1234)))
    for k, v in want.items():
        key = case.name + "/" + k
        check(key, v, ops_golden[key], ops_golden[key + "#"], max(case.tol, 1e-6), exact=k in case.exact)


@pytest.mark.parametrize("name", ["tiny", "odd"])
def test_oracle_lm_step_matches_reference(model_golden, name):
    cfg = models.lm_config(name)
    ids, tgt = models.lm_inputs(cfg)
    rng = np.random.default_rng(cfg["seed"] + 100)
    P = {}
    for n in O.lm_param_names(cfg["L"]):
        shape = {"embed.weight": (cfg["V"], cfg["D"]), "lm_head.bias": (cfg["V"],), "norm.weight": (cfg["D"],)}.get(n)
        if shape is None:
            leaf = n.split(".", 2)[2]
            D, F = cfg["D"], cfg["F"]
            shape = {"qkv_proj.weight": (D, 3 * D), "qkv_proj.bias": (3 * D,), "out_proj.weight": (D, D), "out_proj.bias": (D,),
                     "attn_norm.weight": (D,), "ffn_norm.weight": (D,), "ffn.gate_proj.weight": (D, F), "ffn.gate_proj.bias": (F,),
                     "ffn.up_proj.weight": (D, F), "ffn.up_proj.bias": (F,), "ffn.down_proj.weight": (F, D), "ffn.down_proj.bias": (D,)}[leaf]
        if n.endswith("norm.weight"):
            P[n] = np.ones(shape, np.float32)
        elif n.endswith("bias"):
            P[n] = np.zeros(shape, np.float32)
        else:
            P[n] = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    loss, G = O.lm_loss_and_grads(P, ids, tgt, cfg["L"], cfg["H"])
    tag = "lm_" + name
    assert abs(loss - model_golden[tag + "/loss"][0]) <= 2e-6 * abs(loss)
    gn = O.grad_norm(list(G.values()))
    assert abs(gn - model_golden[tag + "/grad_norm"][0]) <= 1e-5 * gn
    scale = O.clip_scale(gn, cfg["clip"])
    for n, g in G.items():
        key = tag + "/grad/" + n
        check(key, g * scale, model_golden[key], model_golden[key + "#"], 2e-5)


def test_oracle_rng_matches_reference_ids(model_golden):
    cfg = models.lm_config("c1")
    ids, tgt = models.lm_inputs(cfg)
    key = "lm_c1/shifted"
    check(key, tgt, model_golden[key], model_golden[key + "#"], 0, exact=True)
