"""Op-level forward / backward microbenchmark (BASELINE config 2) through the C-ABI.

    python dnn.c_b200/opbench.py [--op NAME] [--iters 10] [--small]

For every op of the training hot path at the config-2 shapes it reports device
milliseconds (CUDA events on the library's stream) of the forward and of the
backward launch set, the algorithmic work (bytes for bandwidth-bound ops, FLOP
for matmul and attention) and the fraction of the measured peak
(MEASURED_PEAKS.json: HBM copy bandwidth; TF32 peak taken as half of the
sustained bf16 figure, there being no measured TF32 number).  Inputs are seeded
synthetic tensors; an L2-sized buffer is rewritten between timed iterations.
`--small` shrinks the batch dimension (for profiler captures).
One JSON line per op.
"""
import argparse
import ctypes as C
import importlib.util
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def load_binding():
    name = "dnnc_b200_binding"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(HERE, "binding.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["hbm_gbs"], 0.5 * p["bf16_tflops_sustained"], "measured"
    return 6650.0, 700.0, "fallback"


class Bench:
    def __init__(self, B, iters, small, params_mb=8192, scratch_mb=24 * 1024, echo=True, device=0, tf32_peak=None):
        self.B, self.iters, self.small, self.echo, self.rows = B, iters, small, echo, []
        self.d = B.Dnn(B.B200_LIB, params_mb=params_mb, scratch_mb=scratch_mb, data_mb=256, device=device)
        self.lib = self.d.lib
        self.rng = np.random.default_rng(1)
        # 256 MiB rewritten between iterations: twice the 126 MB L2
        self.flush = self.lib.tensor_zeros(self.d.params, 1, B.ints([64 << 20]), 0)
        self.hbm, self.tf32, self.src = peaks()
        if tf32_peak:                                        # a TF32 figure measured in this run replaces the bf16-derived one
            self.tf32, self.src = tf32_peak, "TF32 matmul measured in this run"

    def dev(self, arr, grad=False):
        return self.d.tensor(arr, self.d.params, grad)         # params pool: survives reset_step

    def flush_l2(self):
        """Rewrites the 256 MiB flush tensor on the device (tensor_zero_grad zero-fills
        t->grad, so grad is pointed at the payload for the duration of the call)."""
        t = self.flush.contents
        saved = t.grad
        t.grad = t.data
        self.lib.tensor_zero_grad(self.flush)
        t.grad = saved

    def time(self, fn):
        self.lib.dnn_cuda_sync()
        self.lib.dnn_cuda_timer_start()
        fn()
        return self.lib.dnn_cuda_timer_stop_ms()

    def run(self, name, build, fwd, gout_shape, work_fwd, work_bwd, bound):
        """build() -> inputs (made once); fwd(inputs) -> output tensor with a tape node."""
        inp = build()
        g = self.dev(self.rng.standard_normal(gout_shape, dtype=np.float32)) if gout_shape else None
        tf, tb = [], []
        for it in range(3 + self.iters):
            self.d.reset_step()
            self.flush_l2()
            holder = {}
            ms_f = self.time(lambda: holder.setdefault("y", fwd(inp)))
            y = holder["y"]
            self.flush_l2()
            if g is not None:
                fn = C.cast(y.contents.grad_fn, C.POINTER(self.B.GradFn))
                ms_b = self.time(lambda: fn.contents.backward(fn, g))
            else:
                ms_b = self.time(lambda: self.lib.dnn_backward(self.d.scratch, y))
            for t in inp.get("_zero", []):
                self.lib.tensor_zero_grad(t)
            if it >= 3:
                tf.append(ms_f); tb.append(ms_b)
        ms_f, ms_b = float(np.median(tf)), float(np.median(tb))
        peak, unit, scale = (self.hbm, "GB/s", 1e9) if bound == "hbm" else (self.tf32, "TFLOP/s", 1e12)
        af, ab = work_fwd / (ms_f * 1e-3) / scale, work_bwd / (ms_b * 1e-3) / scale
        row = {"op": name, "bound": bound, "fwd_ms": round(ms_f, 4), "bwd_ms": round(ms_b, 4),
               "fwd_achieved": round(af, 1), "bwd_achieved": round(ab, 1), "unit": unit, "peak": round(peak, 1),
               "fwd_frac": round(af / peak, 3), "bwd_frac": round(ab / peak, 3), "peak_source": self.src,
               "work_fwd": work_fwd, "work_bwd": work_bwd}
        self.emit(row)
        return row

    def emit(self, row):
        self.rows.append(row)
        if self.echo:
            print(json.dumps(row), flush=True)


class Args:
    """What run_ops needs from the command line: small (reduced batch), shapes (matmul_shapes / step_graph variant), iters."""

    def __init__(self, small=False, shapes="", iters=10, rows=0, batch=0):
        self.small, self.shapes, self.iters, self.rows, self.batch = small, shapes, iters, rows, batch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--gemm", default="tf32", choices=["tf32", "3xtf32", "fp32"])
    ap.add_argument("--pools-mb", default="8192,24576", help="params,scratch arena sizes (small arenas keep profiler captures fast)")
    ap.add_argument("--shapes", default="", help="matmul_shapes only: indices of the shapes to run, e.g. 0,1,2,3")
    ap.add_argument("--rows", type=int, default=0, help="rows of the row-wise operators instead of 8192 (65536 makes every tensor larger than L2)")
    ap.add_argument("--batch", type=int, default=0, help="cnn_step / cnn_ops: images per batch instead of 512")
    ap.add_argument("--roles-3x", type=int, default=-1,
                    help="tf32 mode: bit set of the products that run as 3xTF32 (1 forward, 2 activation gradient, 4 weight gradient; 3 = strict)")
    args = ap.parse_args()
    B = load_binding()
    pm, sm = (int(x) for x in args.pools_mb.split(","))
    b = Bench(B, args.iters, args.small, pm, sm)
    b.lib.dnn_cuda_set_gemm_mode({"fp32": 0, "tf32": 1, "3xtf32": 2}[args.gemm])
    if args.roles_3x >= 0:
        b.lib.dnn_cuda_set_tf32_policy(args.roles_3x, 4e9)
    run_ops(b, args.op.split(","), args)
    b.d.close()


def run_ops(b, ops, args):
    """Runs the named workloads on the Bench `b`; every result is appended to b.rows (and printed when b.echo)."""
    B = b.B
    lib, d, rng = b.lib, b.d, b.rng
    R = args.rows if args.rows else (1024 if args.small else 8192)
    Bt = 2 if args.small else 8

    def want(n):
        return "all" in ops or n in ops

    def randn(*shape, scale=1.0):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale))

    if want("rms_norm"):
        b.run("rms_norm", lambda: dict(x=b.dev(randn(R, 768), True), w=b.dev(np.ones(768, np.float32), True)),
              lambda i: lib.tensor_rms_norm(d.scratch, i["x"], i["w"], 1e-5), (R, 768), 8 * R * 768, 16 * R * 768, "hbm")
    if want("layer_norm"):
        b.run("layer_norm", lambda: dict(x=b.dev(randn(R, 768), True), w=b.dev(np.ones(768, np.float32), True),
                                         bb=b.dev(np.zeros(768, np.float32), True)),
              lambda i: lib.tensor_layer_norm(d.scratch, i["x"], i["w"], i["bb"], 1e-5), (R, 768), 8 * R * 768, 16 * R * 768, "hbm")
    if "relu" in ops or "silu" in ops or "add" in ops:            # element-wise passes of the models, at [R, 2048]
        n = R * 2048
        if "relu" in ops:
            b.run("relu", lambda: dict(x=b.dev(randn(R, 2048), True)), lambda i: lib.tensor_relu(d.scratch, i["x"]), (R, 2048), 8 * n, 12 * n, "hbm")
        if "silu" in ops:
            b.run("silu", lambda: dict(x=b.dev(randn(R, 2048), True)), lambda i: lib.tensor_silu(d.scratch, i["x"]), (R, 2048), 8 * n, 12 * n, "hbm")
        if "add" in ops:
            b.run("add", lambda: dict(x=b.dev(randn(R, 2048), True), y=b.dev(randn(R, 2048), True)),
                  lambda i: lib.tensor_add(d.scratch, i["x"], i["y"]), (R, 2048), 12 * n, 12 * n, "hbm")
    if "embedding" in ops:
        V, D = 32000, 768
        b.run("embedding", lambda: dict(t=b.dev(randn(V, D, scale=0.02), True), ids=b.dev(rng.integers(0, V, size=2 * R).astype(np.int32))),
              lambda i: lib.tensor_embedding(d.scratch, i["t"], i["ids"]), (2 * R, D), 8 * 2 * R * D, 8 * 2 * R * D, "hbm")
    if "cnn_ops" in ops:
        # the convolution and pooling operators of BASELINE config 3 one by one: conv 3x3 (32 -> 64) on [N,32,14,14]
        # (im2col, GEMM, permute forward; permute, two GEMMs, col2im backward) and avg_pool 2x2 on [N,32,28,28]
        Nb = args.batch if args.batch else 512
        w = b.dev((rng.random((64, 32, 3, 3), dtype=np.float32) - 0.5) * 0.1, True)
        bias = b.dev(np.zeros(64, np.float32), True)
        n_in, n_out, col = Nb * 32 * 14 * 14, Nb * 64 * 14 * 14, 288 * Nb * 196
        b.run("conv2d_3x3_32to64", lambda: dict(x=b.dev(randn(Nb, 32, 14, 14), True), _zero=[w, bias]),
              lambda i: lib.tensor_conv2d(d.scratch, i["x"], w, bias, 1, 1), (Nb, 64, 14, 14),
              4.0 * (n_in + 2 * col + 2 * n_out), 4.0 * (2 * n_out + 3 * col + n_in), "hbm")
        n_p = Nb * 32 * 28 * 28
        b.run("avg_pool2d_2x2", lambda: dict(x=b.dev(randn(Nb, 32, 28, 28), True)),
              lambda i: lib.tensor_avg_pool2d(d.scratch, i["x"], 2, 2), (Nb, 32, 14, 14), 5.0 * n_p, 5.0 * n_p, "hbm")
    if want("swiglu"):
        n = R * 2048
        b.run("swiglu", lambda: dict(g=b.dev(randn(R, 2048), True), u=b.dev(randn(R, 2048), True)),
              lambda i: lib.tensor_swiglu(d.scratch, i["g"], i["u"]), (R, 2048), 12 * n, 28 * n, "hbm")
    if want("rope"):
        n = Bt * 12 * 1024 * 64
        cos = np.cos(np.outer(np.arange(1024), 10000.0 ** (-np.arange(32) / 32.0))).astype(np.float32)
        sin = np.sin(np.outer(np.arange(1024), 10000.0 ** (-np.arange(32) / 32.0))).astype(np.float32)
        b.run("rope", lambda: dict(x=b.dev(randn(Bt, 12, 1024, 64), True), c=b.dev(cos), s=b.dev(sin)),
              lambda i: lib.tensor_rope(d.scratch, i["x"], i["c"], i["s"]), (Bt, 12, 1024, 64), 8 * n, 12 * n, "hbm")
    if want("cross_entropy_masked"):
        V = 32000
        mask = (rng.random((Bt, 1024)) >= 0.1).astype(np.float32)
        active = float(mask.sum())
        b.run("cross_entropy_masked",
              lambda: dict(x=b.dev(randn(Bt, 1024, V, scale=2.0), True), t=b.dev(rng.integers(0, V, size=(Bt, 1024)).astype(np.int32)),
                           m=b.dev(mask)),
              lambda i: lib.tensor_cross_entropy_masked(d.scratch, i["x"], i["t"], i["m"], 2), None,
              4 * active * V, 12 * active * V, "hbm")
    if want("matmul_add"):
        M, K, N = R, 768, 3072
        b.run("matmul_add", lambda: dict(a=b.dev(randn(M, K), True), w=b.dev(randn(K, N, scale=0.02), True),
                                         bias=b.dev(np.zeros(N, np.float32), True)),
              lambda i: lib.tensor_matmul_add(d.scratch, i["a"], i["w"], 0, i["bias"]), (M, N), 2.0 * M * N * K, 4.0 * M * N * K, "tensor")
    if "matmul_shapes" in ops:
        # the linear layers of the 124M training step (BASELINE config 5): 16384 tokens
        M = 2048 if args.small else 16384
        shapes = ((768, 2304), (768, 768), (768, 2048), (2048, 768), (768, 32000))
        pick = [int(x) for x in args.shapes.split(",")] if args.shapes else range(len(shapes))
        for K, N in [shapes[i] for i in pick]:
            b.run("matmul_add[%dx%dx%d]" % (M, K, N),
                  lambda: dict(a=b.dev(randn(M, K), True), w=b.dev(randn(K, N, scale=0.02), True), bias=b.dev(np.zeros(N, np.float32), True)),
                  lambda i: lib.tensor_matmul_add(d.scratch, i["a"], i["w"], 0, i["bias"]), (M, N), 2.0 * M * N * K, 4.0 * M * N * K, "tensor")
    for name, mode, prefix in (("attention_causal", 0, 0), ("attention_prefix_lm", 1, 196)):
        if not want(name) and not want("attention"):
            continue
        H, T, D = 12, 1024, 64
        lens = None if mode == 0 else rng.integers(200, 1025, size=Bt).astype(np.int32)
        vis = 0
        for bi in range(Bt):
            nb = T if lens is None else int(lens[bi])
            vis += sum(min(nb, (i + 1) if (mode == 0 or i >= prefix) else prefix) for i in range(nb))
        flop = 4.0 * D * vis * H
        lp = None if lens is None else lens.ctypes.data_as(C.POINTER(C.c_int))
        b.run(name, lambda: dict(q=b.dev(randn(Bt, H, T, D), True), k=b.dev(randn(Bt, H, T, D), True), v=b.dev(randn(Bt, H, T, D), True)),
              lambda i, mode=mode, prefix=prefix, lp=lp: lib.tensor_attention_ex(d.scratch, i["q"], i["k"], i["v"], None, mode, prefix, lp),
              (Bt, H, T, D), flop, 2 * flop, "tensor")
    if "step_graph" in ops:
        # BASELINE config 1 (V 256, d 128, 4 blocks, 4 heads, FFN 512, batch 16 x 128): kernels of a
        # few microseconds, so the step is bound by launch overhead; eager steps against replays of
        # the recorded step, wall time per step including the loss read-back
        V, D, L, H, F, Bsz, N = 256, 128, 4, 4, 512, 16, 128
        if args.shapes == "gpt124m":                      # BASELINE config 5 instead: GPU-bound, shows what launch gaps cost
            V, D, L, H, F, Bsz, N = 32000, 768, 12, 12, 2048, 16, 1024
        lm = lib.decoder_lm_create(d.params, V, D, L, H, D // H, F)
        lib.decoder_lm_enable_rope(d.params, lm, N, 10000.0)
        lib.dnn_seed(4); lib.decoder_lm_init_weights(lm)
        params = d.parameters(lm)
        arr = (B.TensorP * len(params))(*params)
        opt = lib.adamw_create(d.params, arr, len(params), 3e-4, 0.9, 0.95, 1e-8, 0.1)
        ids = d.tensor(rng.integers(0, V, size=(Bsz, N)).astype(np.int32), d.params)
        tgt = lib.decoder_lm_shift_targets(d.params, ids)
        gn = C.c_float(0)

        def eager():
            loss = lib.decoder_lm_train_step(d.scratch, lm, ids, tgt, opt, 1.0, C.byref(gn))
            v = d.scalar(loss); d.reset_step(); return v
        for _ in range(5):
            eager()
        before = lib.dnn_cuda_launch_count()
        t0 = time.perf_counter()
        reps = 50 if D < 512 else 10
        for _ in range(reps):
            eager()
        ms_eager = (time.perf_counter() - t0) * 1e3 / reps
        per_step = (lib.dnn_cuda_launch_count() - before) // reps
        g = lib.dnn_cuda_graph_capture_decoder_lm_step(d.scratch, lm, ids, tgt, opt, 1.0)
        loss = C.c_float(0)
        for _ in range(5):
            lib.dnn_cuda_graph_replay(g, C.byref(loss), None)
        t0 = time.perf_counter()
        for _ in range(reps):
            lib.dnn_cuda_graph_replay(g, C.byref(loss), None)
        ms_graph = (time.perf_counter() - t0) * 1e3 / reps
        lib.dnn_cuda_graph_destroy(g)
        b.emit(({"op": "step_graph", "workload": "decoder LM V%d d%d L%d H%d F%d, %dx%d tokens" % (V, D, L, H, F, Bsz, N),
                          "kernels_per_step": int(per_step), "eager_ms_per_step": round(ms_eager, 3), "graph_ms_per_step": round(ms_graph, 3),
                          "eager_tokens_per_s": round(Bsz * N / ms_eager * 1e3), "graph_tokens_per_s": round(Bsz * N / ms_graph * 1e3),
                          "speedup": round(ms_eager / ms_graph, 2)}))
    if "cnn_step" in ops:
        # BASELINE config 3: 512 images 1x28x28, conv 3x3 (1->32) + pool, conv 3x3 (32->64) + pool, 3136->128->10,
        # cross entropy, backward, AdamW; wall time per step with the loss read back
        Bsz = args.batch if args.batch else (64 if args.small else 512)
        lib.dnn_seed(2)
        c1, c2 = lib.conv2d_create(d.params, 1, 32, 3, 1, 1), lib.conv2d_create(d.params, 32, 64, 3, 1, 1)
        f1, f2 = lib.linear_create(d.params, 3136, 128), lib.linear_create(d.params, 128, 10)
        params = []
        for m in (c1, c2, f1, f2):
            params += d.parameters(m)
        arr = (B.TensorP * len(params))(*params)
        opt = lib.adamw_create(d.params, arr, len(params), 1e-3, 0.9, 0.999, 1e-8, 0.01)
        x = d.tensor(rng.random((Bsz, 1, 28, 28), dtype=np.float32), d.params)
        y = d.tensor(rng.integers(0, 10, size=Bsz).astype(np.int32), d.params)

        def cnn_step():
            lib.adamw_zero_grad(opt)
            h = lib.tensor_avg_pool2d(d.scratch, lib.tensor_relu(d.scratch, lib.conv2d_forward(d.scratch, c1, x)), 2, 2)
            h = lib.tensor_avg_pool2d(d.scratch, lib.tensor_relu(d.scratch, lib.conv2d_forward(d.scratch, c2, h)), 2, 2)
            h = lib.tensor_reshape(d.scratch, h, 2, B.ints([Bsz, 3136]))
            h = lib.tensor_relu(d.scratch, lib.linear_forward(d.scratch, f1, h))
            loss = lib.tensor_cross_entropy(d.scratch, lib.linear_forward(d.scratch, f2, h), y, 1)
            lib.dnn_backward(d.scratch, loss)
            lib.adamw_step(opt)
            v = d.scalar(loss)
            d.reset_step()
            return v

        for _ in range(5):
            cnn_step()
        before = lib.dnn_cuda_launch_count()
        t0 = time.perf_counter()
        reps = 50
        for _ in range(reps):
            last = cnn_step()
        ms = (time.perf_counter() - t0) * 1e3 / reps
        b.emit(({"op": "cnn_step", "workload": "BASELINE config 3: %d images 1x28x28, 2 conv + 2 linear" % Bsz, "ms_per_step": round(ms, 3),
                          "images_per_s": round(Bsz / ms * 1e3), "kernels_per_step": int((lib.dnn_cuda_launch_count() - before) // reps),
                          "loss": round(last, 4)}))
    if "vlm_step" in ops:
        # BASELINE config 4: 64 images 3x224x224 (196 image tokens) + up to 32 text tokens, d 512, 8 blocks, 8 heads,
        # FFN 1376, vocabulary 1024; vision_lm_train_step_padded with per-sample text lengths and loss mask
        Bsz, Tm = (8 if args.small else 64), 32
        vlm = lib.vision_lm_create(d.params, 1024, 512, 8, 8, 64, 1376, 3, 224, 224, 16, 1)
        lib.vision_lm_enable_rope(d.params, vlm, Tm, 10000.0)
        lib.dnn_seed(3); lib.vision_lm_init_weights(vlm)
        params = d.parameters(vlm)
        arr = (B.TensorP * len(params))(*params)
        opt = lib.adamw_create(d.params, arr, len(params), 6e-4, 0.9, 0.95, 1e-8, 0.1)
        lens = rng.integers(8, Tm + 1, size=Bsz).astype(np.int32)
        img = d.tensor(rng.standard_normal((Bsz, 3, 224, 224), dtype=np.float32), d.params)
        ids = d.tensor(rng.integers(0, 1024, size=(Bsz, Tm)).astype(np.int32), d.params)
        tgt = d.tensor(rng.integers(0, 1024, size=(Bsz, Tm)).astype(np.int32), d.params)
        mask = d.tensor((np.arange(Tm)[None, :] < (lens[:, None] - 1)).astype(np.float32), d.params)
        lp = lens.ctypes.data_as(C.POINTER(C.c_int))
        gn = C.c_float(0)

        def vlm_step():
            loss = lib.vision_lm_train_step_padded(d.scratch, vlm, img, ids, tgt, mask, lp, opt, 1.0, C.byref(gn))
            v = d.scalar(loss)
            d.reset_step()
            return v

        for _ in range(3):
            vlm_step()
        before = lib.dnn_cuda_launch_count()
        t0 = time.perf_counter()
        reps = 20
        for _ in range(reps):
            last = vlm_step()
        ms = (time.perf_counter() - t0) * 1e3 / reps
        b.emit(({"op": "vlm_step", "workload": "BASELINE config 4: %d images 3x224x224 + texts <= %d, d 512, 8 blocks" % (Bsz, Tm),
                          "ms_per_step": round(ms, 3), "images_per_s": round(Bsz / ms * 1e3),
                          "tokens_per_s": round(Bsz * (196 + Tm) / ms * 1e3),
                          "kernels_per_step": int((lib.dnn_cuda_launch_count() - before) // reps), "loss": round(last, 4)}))
    if "vlm_batch" in ops:
        # Padded vision-LM batch of BASELINE config 4 (64 images 3x224x224, texts up to 32): device assembly alone
        # (uint8 HWC -> normalised NCHW floats, ids / targets / mask rows) and the whole put + upload + assemble
        # pipeline over two slots, beside the upload of the same batch as ready-made floats.
        Bsz, Hh, Ww, Cc, Tm = (8 if args.small else 64), 224, 224, 3, 32
        mean, std = (C.c_float * 3)(0.485, 0.456, 0.406), (C.c_float * 3)(0.229, 0.224, 0.225)
        st = lib.dnn_cuda_vlm_stager_create(2, Bsz, Tm, Hh, Ww, Cc, 0, mean, std)
        px = rng.integers(0, 256, size=(Bsz, Hh, Ww, Cc)).astype(np.uint8)
        texts = [rng.integers(0, 257, size=int(rng.integers(7, Tm))).astype(np.int32) for _ in range(Bsz)]

        def stage(slot):
            for i in range(Bsz):
                lib.dnn_cuda_vlm_stager_put(st, slot, i, texts[i].ctypes.data_as(C.POINTER(C.c_int)), len(texts[i]),
                                            px[i].ctypes.data_as(C.c_void_p), i & 1, i)
            lib.dnn_cuda_vlm_stager_submit(st, slot, Bsz)

        def tensors():
            return (lib.tensor_scratch(d.scratch, 4, B.ints([Bsz, Cc, Hh, Ww]), 0), lib.tensor_zeros_data(d.data, 2, B.ints([Bsz, Tm])),
                    lib.tensor_zeros_data(d.data, 2, B.ints([Bsz, Tm])), lib.tensor_scratch(d.scratch, 2, B.ints([Bsz, Tm]), 0))

        ts = []
        for it in range(3 + args.iters):
            d.reset_step()
            stage(0)
            img, ids, tgt, mask = tensors()
            lib.dnn_cuda_sync()                    # the copy stream is not the compute stream: wait for the upload on the host
            time.sleep(0.01)
            b.flush_l2()
            ms = b.time(lambda: lib.dnn_cuda_vlm_stager_assemble(st, 0, img, ids, tgt, mask, None, None))
            if it >= 3:
                ts.append(ms)
        ms_dev = float(np.median(ts))
        dev_bytes = Bsz * Hh * Ww * Cc * 5 + Bsz * Tm * 16
        reps = 20
        d.reset_step()
        stage(0)
        lib.dnn_cuda_sync()
        t0 = time.perf_counter()
        for r in range(reps):
            stage((r + 1) & 1)                     # fill and upload the next slot while this one is assembled
            img, ids, tgt, mask = tensors()
            lib.dnn_cuda_vlm_stager_assemble(st, r & 1, img, ids, tgt, mask, None, None)
            lib.dnn_cuda_sync()
            d.reset_step()
        ms_e2e = (time.perf_counter() - t0) * 1e3 / reps
        # the reference's hand-over: a finished float batch in host memory, uploaded as it is
        fl = lib.dnn_cuda_host_alloc(Bsz * Cc * Hh * Ww * 4)
        C.memset(fl, 0, Bsz * Cc * Hh * Ww * 4)
        img = lib.tensor_zeros_data(d.data, 4, B.ints([Bsz, Cc, Hh, Ww]))
        for _ in range(3):
            lib.dnn_cuda_upload(img, fl, Bsz * Cc * Hh * Ww * 4)
        lib.dnn_cuda_sync()
        t0 = time.perf_counter()
        for _ in range(reps):
            lib.dnn_cuda_upload(img, fl, Bsz * Cc * Hh * Ww * 4)
            lib.dnn_cuda_sync()
        ms_float = (time.perf_counter() - t0) * 1e3 / reps
        lib.dnn_cuda_host_free(fl)
        lib.dnn_cuda_vlm_stager_destroy(st)
        a = dev_bytes / (ms_dev * 1e-3) / 1e9
        b.emit(({"op": "vlm_batch", "workload": "%d images %dx%dx%d uint8, texts <= %d" % (Bsz, Cc, Hh, Ww, Tm), "bound": "hbm",
                          "assemble_ms": round(ms_dev, 4), "assemble_bytes": dev_bytes, "achieved": round(a, 1), "unit": "GB/s",
                          "peak": b.hbm, "frac": round(a / b.hbm, 3), "peak_source": b.src,
                          "pipeline_ms_per_batch": round(ms_e2e, 3), "pipeline_images_per_s": round(Bsz / ms_e2e * 1e3),
                          "h2d_bytes_per_batch": Bsz * Hh * Ww * Cc + Bsz * (2 + Tm) * 4,
                          "float_upload_ms_per_batch": round(ms_float, 3), "float_h2d_bytes_per_batch": Bsz * Cc * Hh * Ww * 4}))
    if "generate" in ops:
        # KV-cache generation on the 124M-shaped decoder LM: batch 1, prompt of 128 tokens, greedy; the time of the
        # extra new tokens of a longer run over a shorter one is the cost of a token step (prefill and set-up cancel).
        lm = lib.decoder_lm_create(d.params, 32000, 768, 12, 12, 64, 2048)
        lib.decoder_lm_enable_rope(d.params, lm, 1024, 10000.0)
        lib.dnn_seed(1); lib.decoder_lm_init_weights(lm)
        ids = d.tensor((np.arange(1, 129, dtype=np.int32).reshape(1, -1) % 250), d.params)
        n = C.c_int(0)
        res = {}
        for new in (8, 8, 136):
            lib.dnn_cuda_sync(); t0 = time.perf_counter(); k0 = lib.dnn_cuda_launch_count()
            lib.decoder_lm_generate(d.scratch, d.data, lm, ids, new, 0.0, 1, C.byref(n))
            lib.dnn_cuda_sync()
            res[new] = (time.perf_counter() - t0, lib.dnn_cuda_launch_count() - k0, n.value - 128)
            d.reset_step()
        extra = res[136][2] - res[8][2]
        ms_tok = (res[136][0] - res[8][0]) / max(extra, 1) * 1e3
        b.emit({"op": "generate", "workload": "decoder LM V32000 d768 L12, batch 1, prompt 128, greedy, KV cache",
                "ms_per_new_token": round(ms_tok, 3), "tokens_per_s": round(1e3 / ms_tok, 1),
                "kernels_per_token": int((res[136][1] - res[8][1]) // max(extra, 1)), "new_tokens": res[136][2],
                "ms_prefill_and_8_tokens": round(res[8][0] * 1e3, 2)})
    if want("adamw"):
        P = (16 if args.small else 124) * 1000 * 1000
        t = lib.tensor_zeros(d.params, 1, B.ints([P]), 1)
        arr = (B.TensorP * 1)(t)
        opt = lib.adamw_create(d.params, arr, 1, 6e-4, 0.9, 0.95, 1e-8, 0.1)
        t.contents.grad = lib.tensor_zeros(d.params, 1, B.ints([P]), 0).contents.data
        ts = []
        for it in range(3 + args.iters):
            b.flush_l2()
            ms = b.time(lambda: lib.adamw_step(opt))
            if it >= 3:
                ts.append(ms)
        ms = float(np.median(ts))
        a = 28.0 * P / (ms * 1e-3) / 1e9
        b.emit(({"op": "adamw", "bound": "hbm", "ms": round(ms, 4), "achieved": round(a, 1), "unit": "GB/s", "peak": b.hbm,
                          "frac": round(a / b.hbm, 3), "params": P, "peak_source": b.src}))
    return b.rows


if __name__ == "__main__":
    main()
