"""Model-level runs through the C API (decoder LM, MNIST-shaped CNN, vision LM).

The same functions drive the CUDA library and the reference library: they
create the model with the library's own constructors, overwrite every
parameter with seeded values (so both sides start from identical weights),
run training steps with the library's *_train_step and return losses,
gradient norms, gradients and updated parameters as numpy arrays.
"""
import ctypes as C

import numpy as np

from conftest import load_binding
from oracle import dnn_oracle as O

B = load_binding()


def seeded_weights(dnn, module, names, seed, std=0.02):
    """N(0, std) for matrices / conv filters / position tables, 0 for biases, 1 for norm gains."""
    rng = np.random.default_rng(seed)
    params = dnn.parameters(module)
    assert len(params) == len(names), (len(params), len(names))
    vals = {}
    for t, name in zip(params, names):
        shape = dnn.shape_of(t)
        if name.endswith("norm.weight"):
            v = np.ones(shape, np.float32)
        elif name.endswith("bias"):
            v = np.zeros(shape, np.float32)
        else:
            v = (rng.standard_normal(shape) * std).astype(np.float32)
        dnn.upload(t, v)
        vals[name] = v
    return params, vals


def lm_param_shapes(V, D, L, F):
    """Shapes of the decoder LM's parameters in module_parameters() order (src/gpt.c:30-59, src/transformer.c:128-140)."""
    leaf = {"qkv_proj.weight": (D, 3 * D), "qkv_proj.bias": (3 * D,), "out_proj.weight": (D, D), "out_proj.bias": (D,),
            "attn_norm.weight": (D,), "ffn_norm.weight": (D,), "ffn.gate_proj.weight": (D, F), "ffn.gate_proj.bias": (F,),
            "ffn.up_proj.weight": (D, F), "ffn.up_proj.bias": (F,), "ffn.down_proj.weight": (F, D), "ffn.down_proj.bias": (D,)}
    top = {"embed.weight": (V, D), "lm_head.bias": (V,), "norm.weight": (D,)}
    return {n: top[n] if n in top else leaf[n.split(".", 2)[2]] for n in O.lm_param_names(L)}


def seeded_values(shapes, seed, std=0.02):
    """The values seeded_weights() uploads, from shapes alone (no library): same generator, same draw order."""
    rng = np.random.default_rng(seed)
    vals = {}
    for name, shape in shapes.items():
        if name.endswith("norm.weight"):
            vals[name] = np.ones(shape, np.float32)
        elif name.endswith("bias"):
            vals[name] = np.zeros(shape, np.float32)
        else:
            vals[name] = (rng.standard_normal(shape) * std).astype(np.float32)
    return vals


def lm_config(name):
    return {
        # BASELINE config 1: tiny decoder LM
        "c1": dict(V=256, D=128, L=4, H=4, F=512, B=16, N=128, lr=3e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, clip=1.0, seed=0),
        # small enough for the float64 numpy oracle and for golden vectors in git
        "tiny": dict(V=64, D=32, L=2, H=2, F=64, B=2, N=16, lr=1e-3, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, clip=1.0, seed=7),
        "odd": dict(V=50, D=48, L=1, H=3, F=40, B=3, N=33, lr=1e-3, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, clip=0.5, seed=8),
    }[name]


def lm_inputs(cfg):
    """Token ids from the reference's own generator (xorshift128+, src/rng.c)."""
    r = O.Rng(cfg["seed"])
    ids = np.array([r.uniform_int(cfg["V"]) for _ in range(cfg["B"] * cfg["N"])], np.int32).reshape(cfg["B"], cfg["N"])
    return ids, np.ascontiguousarray(ids[:, 1:])


def run_lm(dnn, cfg, steps=1, want_grads=True):
    lib = dnn.lib
    lm = lib.decoder_lm_create(dnn.params, cfg["V"], cfg["D"], cfg["L"], cfg["H"], cfg["D"] // cfg["H"], cfg["F"])
    lib.decoder_lm_enable_rope(dnn.params, lm, cfg["N"], 10000.0)
    names = O.lm_param_names(cfg["L"])
    params, w0 = seeded_weights(dnn, lm, names, cfg["seed"] + 100)
    arr = (B.TensorP * len(params))(*params)
    opt = lib.adamw_create(dnn.params, arr, len(params), cfg["lr"], cfg["b1"], cfg["b2"], cfg["eps"], cfg["wd"])
    ids_np, tgt_np = lm_inputs(cfg)
    out = dict(loss=[], grad_norm=[], names=names, w0=w0, ids=ids_np, targets=tgt_np)
    for s in range(steps):
        ids = dnn.tensor(ids_np, dnn.data)
        tgt = lib.decoder_lm_shift_targets(dnn.data, ids)
        if s == 0:
            out["shifted"] = dnn.download(tgt, np.int32)
        gn = C.c_float(0)
        loss = lib.decoder_lm_train_step(dnn.scratch, lm, ids, tgt, opt, cfg["clip"], C.byref(gn))
        out["loss"].append(dnn.scalar(loss))
        out["grad_norm"].append(float(gn.value))
        if s == 0 and want_grads:
            out["grads"] = {n: dnn.download_grad(t) for n, t in zip(names, params)}   # after clipping
        dnn.reset_step()
    out["params"] = {n: dnn.download(t) for n, t in zip(names, params)}
    out["_keep"] = (arr,)
    return out


def run_generate(dnn, cfg, prompt, max_new, temperature, use_cache, seed=0):
    """decoder_lm_generate on a seeded model; returns the token list (prompt + new)."""
    lib = dnn.lib
    lm = lib.decoder_lm_create(dnn.params, cfg["V"], cfg["D"], cfg["L"], cfg["H"], cfg["D"] // cfg["H"], cfg["F"])
    lib.decoder_lm_enable_rope(dnn.params, lm, len(prompt) + max_new, 10000.0)
    names = O.lm_param_names(cfg["L"])
    seeded_weights(dnn, lm, names, cfg["seed"] + 100, std=0.3)       # large weights: peaked logits, argmax far from ties
    lib.dnn_seed(seed)
    ids = dnn.tensor(np.asarray(prompt, np.int32).reshape(1, -1), dnn.data)
    n = C.c_int(0)
    out = lib.decoder_lm_generate(dnn.scratch, dnn.data, lm, ids, max_new, temperature, use_cache, C.byref(n))
    toks = [int(out[i]) for i in range(n.value)]
    dnn.reset_step()
    return toks


GEN_CASES = [   # name, config overrides, prompt, max_new, temperature, use_cache
    ("greedy-cache", dict(V=64, D=32, L=2, H=2, F=64), [3, 17, 42, 5, 9], 12, 0.0, 1),
    ("greedy-nocache", dict(V=64, D=32, L=2, H=2, F=64), [3, 17, 42, 5, 9], 12, 0.0, 0),
    ("sampled-cache", dict(V=64, D=32, L=2, H=2, F=64), [1, 2, 3], 10, 0.8, 1),
    ("greedy-cache-d32", dict(V=96, D=128, L=2, H=4, F=256), [7, 90, 33, 2, 11, 64, 5], 9, 0.0, 1),
]


# ── MNIST-shaped CNN (BASELINE config 3) ──────────────────────────────────
CNN_NAMES = ["conv1.weight", "conv1.bias", "conv2.weight", "conv2.bias", "fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias"]


CNN_SHAPES = {"conv1.weight": (32, 1, 3, 3), "conv1.bias": (32,), "conv2.weight": (64, 32, 3, 3), "conv2.bias": (64,),
              "fc1.weight": (3136, 128), "fc1.bias": (128,), "fc2.weight": (128, 10), "fc2.bias": (10,)}


def cnn_values(batch, seed=2):
    """Seeded weights (Kaiming-uniform filters, uniform +-1/sqrt(in) linear layers, zero conv biases) and the batch:
    images uniform in [0,1), labels uniform in [0,10).  One generator, fixed draw order."""
    rng = np.random.default_rng(seed)
    P = {}
    for n in CNN_NAMES:
        shape = CNN_SHAPES[n]
        fan_in = int(np.prod(shape[1:])) if len(shape) == 4 else shape[0]
        bound = np.sqrt(6.0 / fan_in) if len(shape) == 4 else 1.0 / np.sqrt(3136 if n.startswith("fc1") else 128)
        P[n] = np.zeros(shape, np.float32) if n.startswith("conv") and n.endswith("bias") else \
            ((rng.random(shape) * 2 - 1) * bound).astype(np.float32)
    x_np = rng.random((batch, 784)).astype(np.float32)
    y_np = rng.integers(0, 10, size=batch).astype(np.int32)
    return P, x_np, y_np


def run_cnn(dnn, batch=8, steps=2, seed=2, want_relu=False):
    lib = dnn.lib
    c1 = lib.conv2d_create(dnn.params, 1, 32, 3, 1, 1)
    c2 = lib.conv2d_create(dnn.params, 32, 64, 3, 1, 1)
    f1 = lib.linear_create(dnn.params, 3136, 128)
    f2 = lib.linear_create(dnn.params, 128, 10)
    params = []
    for m in (c1, c2, f1, f2):
        params += dnn.parameters(m)
    P, x_np, y_np = cnn_values(batch, seed)
    for t, n in zip(params, CNN_NAMES):
        assert dnn.shape_of(t) == CNN_SHAPES[n], (n, dnn.shape_of(t))
        dnn.upload(t, P[n])
    arr = (B.TensorP * len(params))(*params)
    opt = lib.adamw_create(dnn.params, arr, len(params), 1e-3, 0.9, 0.999, 1e-8, 0.01)
    out = dict(loss=[], names=CNN_NAMES)
    for s in range(steps):
        x = dnn.tensor(x_np, dnn.data)
        y = dnn.tensor(y_np, dnn.data)
        h = lib.tensor_reshape(dnn.scratch, x, 4, B.ints([batch, 1, 28, 28]))
        r1 = lib.tensor_relu(dnn.scratch, lib.conv2d_forward(dnn.scratch, c1, h))
        r2 = lib.tensor_relu(dnn.scratch, lib.conv2d_forward(dnn.scratch, c2, lib.tensor_avg_pool2d(dnn.scratch, r1, 2, 2)))
        h = lib.tensor_reshape(dnn.scratch, lib.tensor_avg_pool2d(dnn.scratch, r2, 2, 2), 2, B.ints([batch, 3136]))
        r3 = lib.tensor_relu(dnn.scratch, lib.linear_forward(dnn.scratch, f1, h))
        logits = lib.linear_forward(dnn.scratch, f2, r3)
        loss = lib.tensor_cross_entropy(dnn.scratch, logits, y, 1)
        lib.dnn_backward(dnn.scratch, loss)
        out["loss"].append(dnn.scalar(loss))
        if s == 0:
            out["logits"] = dnn.download(logits)
            out["grads"] = {n: dnn.download_grad(t) for n, t in zip(CNN_NAMES, params)}
            if want_relu:                   # which units of the three ReLUs are on (their outputs are positive)
                out["relu_on"] = {"c1": dnn.download(r1) > 0, "c2": dnn.download(r2) > 0, "h1": dnn.download(r3) > 0}
        lib.adamw_step(opt)
        lib.adamw_zero_grad(opt)
        dnn.reset_step()
    out["params"] = {n: dnn.download(t) for n, t in zip(CNN_NAMES, params)}
    out["_keep"] = (arr,)
    return out


# ── prefix-LM vision LM (BASELINE config 4, reduced) ──────────────────────
def vlm_param_names(n_layers):
    return ["patch_embed.weight", "patch_embed.bias", "img_proj.weight", "img_proj.bias"] + \
           ["lm." + n for n in O.lm_param_names(n_layers)] + ["image_pos"]


def vlm_param_shapes(V, D, L, F, C, patch, n_img):
    shapes = {"patch_embed.weight": (D, C, patch, patch), "patch_embed.bias": (D,), "img_proj.weight": (C * patch * patch, D),
              "img_proj.bias": (D,)}
    shapes.update({"lm." + n: s for n, s in lm_param_shapes(V, D, L, F).items()})
    shapes["image_pos"] = (1, n_img, D)
    return shapes


def vlm_inputs(seed, Bsz, img, V, Tmax, min_len=2):
    """Images ~N(0,1), per-sample text lengths, padded ids / targets and the loss mask with the loader's
    convention mask[b,t] = 1 for t < len-1 (src/imagenet_vlm.c:615-631)."""
    rng = np.random.default_rng(seed)
    images = rng.standard_normal((Bsz, 3, img, img)).astype(np.float32)
    lens = rng.integers(min_len, Tmax + 1, size=Bsz).astype(np.int32)
    ids = rng.integers(0, V, size=(Bsz, Tmax)).astype(np.int32)
    tgt = rng.integers(0, V, size=(Bsz, Tmax)).astype(np.int32)
    mask = (np.arange(Tmax)[None, :] < (lens[:, None] - 1)).astype(np.float32)
    return images, lens, ids, tgt, mask


def run_vlm(dnn, steps=2, seed=3, Bsz=3, img=32, patch=16, V=40, D=32, L=2, H=2, F=48, Tmax=8, min_len=2):
    lib = dnn.lib
    vlm = lib.vision_lm_create(dnn.params, V, D, L, H, D // H, F, 3, img, img, patch, 1)
    lib.vision_lm_enable_rope(dnn.params, vlm, Tmax, 10000.0)
    names = vlm_param_names(L)
    params, _ = seeded_weights(dnn, vlm, names, seed + 100)
    arr = (B.TensorP * len(params))(*params)
    opt = lib.adamw_create(dnn.params, arr, len(params), 6e-4, 0.9, 0.95, 1e-8, 0.1)
    images, lens, ids, tgt, mask = vlm_inputs(seed, Bsz, img, V, Tmax, min_len)
    out = dict(loss=[], grad_norm=[], names=names)
    for s in range(steps):
        ti, tt = dnn.tensor(ids, dnn.data), dnn.tensor(tgt, dnn.data)
        tm, tx = dnn.tensor(mask, dnn.data), dnn.tensor(images, dnn.data)
        gn = C.c_float(0)
        loss = lib.vision_lm_train_step_padded(dnn.scratch, vlm, tx, ti, tt, tm, lens.ctypes.data_as(C.POINTER(C.c_int)),
                                               opt, 1.0, C.byref(gn))
        out["loss"].append(dnn.scalar(loss))
        out["grad_norm"].append(float(gn.value))
        if s == 0:
            out["grads"] = {n: dnn.download_grad(t) for n, t in zip(names, params)}
        dnn.reset_step()
    out["params"] = {n: dnn.download(t) for n, t in zip(names, params)}
    out["_keep"] = (arr,)
    return out


def run_vlm_generate(dnn, prompt, max_new, temperature, use_cache, patched=False, seed=0,
                     img=32, patch=16, V=300, D=32, L=2, H=2, F=48):
    """vision_lm_generate on a seeded model; returns the token list (prompt + new).  V > 258 so that the
    end-of-sequence id can be drawn; `patched` feeds the image as [1, patches, patch_dim]."""
    lib = dnn.lib
    vlm = lib.vision_lm_create(dnn.params, V, D, L, H, D // H, F, 3, img, img, patch, 1)
    lib.vision_lm_enable_rope(dnn.params, vlm, len(prompt) + max_new, 10000.0)
    seeded_weights(dnn, vlm, vlm_param_names(L), seed + 100, std=0.3)
    rng = np.random.default_rng(seed + 5)
    n_patch = (img // patch) ** 2
    image = rng.standard_normal((1, n_patch, 3 * patch * patch) if patched else (1, 3, img, img)).astype(np.float32)
    lib.dnn_seed(seed)
    ids = dnn.tensor(np.asarray(prompt, np.int32).reshape(1, -1), dnn.data)
    n = C.c_int(0)
    out = lib.vision_lm_generate(dnn.scratch, dnn.data, vlm, dnn.tensor(image, dnn.data), ids, max_new, temperature,
                                 use_cache, C.byref(n))
    toks = [int(out[i]) for i in range(n.value)]
    dnn.reset_step()
    return toks


VLM_GEN_CASES = [   # name, prompt, max_new, temperature, use_cache, patched
    ("vlm-greedy-cache", [3, 17, 42, 5], 10, 0.0, 1, False),
    ("vlm-greedy-nocache", [3, 17, 42, 5], 10, 0.0, 0, False),
    ("vlm-sampled-cache", [1, 2, 3], 8, 0.7, 1, False),
    ("vlm-greedy-cache-patched", [9, 8, 7, 6, 5], 6, 0.0, 1, True),
]
