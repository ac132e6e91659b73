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
    P = models.seeded_values(models.lm_param_shapes(cfg["V"], cfg["D"], cfg["L"], cfg["F"]), cfg["seed"] + 100)
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


def test_oracle_vision_lm_step_matches_reference(model_golden):
    """The float64 restatement of vision_lm_train_step_padded (patch convolution with the reference's
    memory layout, learned image positions, prefix-LM attention with per-sample lengths, masked cross
    entropy on the text rows) against the vectors of the unmodified reference (models.run_vlm defaults)."""
    V, D, L, H, F, img, patch, Tmax, Bsz, seed = 40, 32, 2, 2, 48, 32, 16, 8, 3, 3
    P = models.seeded_values(models.vlm_param_shapes(V, D, L, F, 3, patch, (img // patch) ** 2), seed + 100)
    images, lens, ids, tgt, mask = models.vlm_inputs(seed, Bsz, img, V, Tmax)
    loss, G = O.vlm_loss_and_grads(P, images, ids, tgt, mask, lens, L, H, patch)
    assert abs(loss - model_golden["vlm/loss"][0]) <= 2e-6 * abs(loss)
    gn = O.grad_norm([g for g in G.values() if g is not None])
    assert abs(gn - model_golden["vlm/grad_norm"][0]) <= 1e-5 * gn
    scale = O.clip_scale(gn, 1.0)
    missing = set(model_golden["vlm/grad_missing"].tolist())
    assert missing == {n for n, g in G.items() if g is None}
    for n, g in G.items():
        if g is None:
            continue
        key = "vlm/grad/" + n
        check(key, g * scale, model_golden[key], model_golden[key + "#"], 2e-5)


@pytest.mark.parametrize("tag,batch", [("cnn", 8), ("cnn512", 512)])
def test_oracle_cnn_step_matches_reference(model_golden, tag, batch):
    """The float64 restatement of the MNIST-shaped CNN step against the vectors of the unmodified reference, at
    batch 8 and at BASELINE config 3's batch of 512.  The distance at batch 512 (3e-6 .. 5e-6 on the filter
    gradients, which are serial fp32 sums of up to 401 408 cancelling products in the reference) is the
    reference's own rounding noise: the floor below which a comparison with its vectors says nothing."""
    P, x, y = models.cnn_values(batch)
    loss, G, logits, _ = O.cnn_loss_and_grads(P, x, y)
    assert abs(loss - model_golden[tag + "/loss"][0]) <= 2e-6 * abs(loss)
    if tag == "cnn":
        check("cnn/logits", logits, model_golden["cnn/logits"], model_golden["cnn/logits#"], 2e-5)
    for n, g in G.items():
        key = tag + "/grad/" + n
        err = check(key, g, model_golden[key], model_golden[key + "#"], 1e-5)
        print("reference vs float64 oracle, %s %s: %.2e" % (tag, n, err))
