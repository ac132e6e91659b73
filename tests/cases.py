"""Op-level parity cases for the dnn.c hot path.

Every case has three parts that share seeded inputs:
  make(rng)        -> dict of numpy inputs
  run(dnn, inp)    -> dict of outputs computed THROUGH THE C API of a loaded
                      library (the CUDA build or the reference build)
  oracle(inp)      -> the same dict computed by the numpy restatement

Backward is exercised the way dnn_backward() does it: the tape node of the
op's output is called with a seeded upstream gradient.
"""
import ctypes as C

import numpy as np

from conftest import load_binding
from oracle import dnn_oracle as O

TensorP = load_binding().TensorP


def _r(rng, *shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float32)


class Case:
    def __init__(self, name, make, run, oracle, tol=2e-5, exact=(), golden_exact=()):
        self.name, self.make, self.run, self.oracle, self.tol, self.exact = name, make, run, oracle, tol, exact
        # keys that must equal the REFERENCE's output bit for bit (golden vectors), although
        # the numpy oracle, whose libm differs, only agrees to rounding
        self.golden_exact = tuple(golden_exact) + tuple(exact)

    def __repr__(self):
        return self.name


CASES = []


def case(name, tol=2e-5, exact=(), golden_exact=()):
    def deco(cls):
        CASES.append(Case(name, cls.make, cls.run, cls.oracle, tol, exact, golden_exact))
        return cls
    return deco


def _grads(dnn, *ts):
    return [dnn.download_grad(t) for t in ts]


# ── rms_norm / layer_norm ─────────────────────────────────────────────────
def _norm_cases():
    for rows, d in ((37, 768), (5, 130), (64, 2048), (3, 4100), (1, 7)):
        @case("rms_norm[%dx%d]" % (rows, d))
        class _:
            @staticmethod
            def make(rng, rows=rows, d=d):
                return dict(x=_r(rng, rows, d), w=_r(rng, d) * 0.5 + 1, g=_r(rng, rows, d))

            @staticmethod
            def run(dnn, i):
                x, w = dnn.tensor(i["x"], dnn.scratch, True), dnn.param(i["w"])
                y = dnn.lib.tensor_rms_norm(dnn.scratch, x, w, 1e-5)
                dnn.backward_from(y, i["g"])
                dx, dw = _grads(dnn, x, w)
                return dict(y=dnn.download(y), dx=dx, dw=dw)

            @staticmethod
            def oracle(i):
                y, dx, dw = O.rms_norm(i["x"], i["w"], 1e-5, i["g"])
                return dict(y=y, dx=dx, dw=dw)

        @case("layer_norm[%dx%d]" % (rows, d))
        class _:
            @staticmethod
            def make(rng, rows=rows, d=d):
                return dict(x=_r(rng, rows, d) + 0.3, w=_r(rng, d) * 0.5 + 1, b=_r(rng, d), g=_r(rng, rows, d))

            @staticmethod
            def run(dnn, i):
                x, w, b = dnn.tensor(i["x"], dnn.scratch, True), dnn.param(i["w"]), dnn.param(i["b"])
                y = dnn.lib.tensor_layer_norm(dnn.scratch, x, w, b, 1e-5)
                dnn.backward_from(y, i["g"])
                dx, dw, db = _grads(dnn, x, w, b)
                return dict(y=dnn.download(y), dx=dx, dw=dw, db=db)

            @staticmethod
            def oracle(i):
                y, dx, dw, db = O.layer_norm(i["x"], i["w"], i["b"], 1e-5, i["g"])
                return dict(y=y, dx=dx, dw=dw, db=db)


_norm_cases()


# ── elementwise ───────────────────────────────────────────────────────────
def _unary(name, libfn, ofn, shapes):
    for shape in shapes:
        @case("%s%s" % (name, list(shape)))
        class _:
            @staticmethod
            def make(rng, shape=shape):
                return dict(x=_r(rng, *shape, scale=2.0), g=_r(rng, *shape))

            @staticmethod
            def run(dnn, i):
                x = dnn.tensor(i["x"], dnn.scratch, True)
                y = getattr(dnn.lib, libfn)(dnn.scratch, x)
                dnn.backward_from(y, i["g"])
                return dict(y=dnn.download(y), dx=dnn.download_grad(x))

            @staticmethod
            def oracle(i):
                y, dx = ofn(i["x"], i["g"])
                return dict(y=y, dx=dx)


_unary("relu", "tensor_relu", O.relu, [(4, 32, 7, 7), (1001,)])
_unary("silu", "tensor_silu", O.silu, [(33, 129), (8,)])


def _binary(name, libfn, ofn, pairs):
    for sa, sb in pairs:
        @case("%s%s%s" % (name, list(sa), list(sb)))
        class _:
            @staticmethod
            def make(rng, sa=sa, sb=sb):
                out = np.broadcast_shapes(sa, sb)
                return dict(a=_r(rng, *sa), b=_r(rng, *sb), g=_r(rng, *out))

            @staticmethod
            def run(dnn, i):
                a, b = dnn.tensor(i["a"], dnn.scratch, True), dnn.tensor(i["b"], dnn.scratch, True)
                y = getattr(dnn.lib, libfn)(dnn.scratch, a, b)
                dnn.backward_from(y, i["g"])
                da, db = _grads(dnn, a, b)
                return dict(y=dnn.download(y), da=da, db=db)

            @staticmethod
            def oracle(i):
                y, da, db = ofn(i["a"], i["b"], i["g"])
                return dict(y=y, da=da, db=db)


_binary("add", "tensor_add", O.add, [((6, 50, 64), (6, 50, 64)), ((3, 7, 33), (33,)), ((33,), (3, 7, 33)),
                                      ((4, 19, 24), (1, 19, 24)), ((5, 1, 8), (1, 6, 8))])
_binary("swiglu", "tensor_swiglu", O.swiglu, [((9, 17, 64), (9, 17, 64)), ((3, 5, 31), (3, 5, 31)), ((4, 6, 8), (1, 6, 8))])

# ── the rest of ops.h: sub, mul, div, neg, pow, sigmoid, sum, mean, softmax, causal softmax, dropout, triu ──
_binary("sub", "tensor_sub", O.sub, [((5, 9, 32), (5, 9, 32)), ((3, 7, 33), (33,)), ((4, 1, 8), (1, 6, 8))])
_binary("mul", "tensor_mul", O.mul, [((5, 9, 32), (5, 9, 32)), ((33,), (3, 7, 33)), ((4, 1, 8), (1, 6, 8)), ((6, 5), (1,))])
_unary("neg", "tensor_neg", O.neg, [(7, 33), (5,)])
_unary("sigmoid", "tensor_sigmoid", O.sigmoid, [(9, 65), (12,)])

for sa, sb in (((6, 40), (6, 40)), ((3, 5, 16), (16,)), ((4, 1, 8), (1, 6, 8))):
    @case("div%s%s" % (list(sa), list(sb)))
    class _:
        @staticmethod
        def make(rng, sa=sa, sb=sb):
            out = np.broadcast_shapes(sa, sb)
            b = (1.5 + 0.3 * _r(rng, *sb)) * np.where(_r(rng, *sb) > 0, 1, -1)       # away from zero, both signs
            return dict(a=_r(rng, *sa), b=b.astype(np.float32), g=_r(rng, *out))

        @staticmethod
        def run(dnn, i):
            a, b = dnn.tensor(i["a"], dnn.scratch, True), dnn.tensor(i["b"], dnn.scratch, True)
            y = dnn.lib.tensor_div(dnn.scratch, a, b)
            dnn.backward_from(y, i["g"])
            da, db = _grads(dnn, a, b)
            return dict(y=dnn.download(y), da=da, db=db)

        @staticmethod
        def oracle(i):
            y, da, db = O.div(i["a"], i["b"], i["g"])
            return dict(y=y, da=da, db=db)

for shape, e in (((8, 33), 2.0), ((5, 7), 2.5), ((64,), -1.0)):
    @case("pow%s^%g" % (list(shape), e))
    class _:
        @staticmethod
        def make(rng, shape=shape, e=e):
            return dict(x=(0.5 + np.abs(_r(rng, *shape))).astype(np.float32), g=_r(rng, *shape), e=e)

        @staticmethod
        def run(dnn, i):
            x = dnn.tensor(i["x"], dnn.scratch, True)
            y = dnn.lib.tensor_pow(dnn.scratch, x, i["e"])
            dnn.backward_from(y, i["g"])
            return dict(y=dnn.download(y), dx=dnn.download_grad(x))

        @staticmethod
        def oracle(i):
            y, dx = O.power(i["x"], i["e"], i["g"])
            return dict(y=y, dx=dx)

for opname, libfn, ofn in (("sum", "tensor_sum", O.sum_dim), ("mean", "tensor_mean", O.mean_dim)):
    for shape, dim in (((5, 17, 9), 1), ((5, 17, 9), -1), ((6, 33), 0), ((40,), 0)):
        @case("%s%s dim%d" % (opname, list(shape), dim))
        class _:
            @staticmethod
            def make(rng, shape=shape, dim=dim):
                out = list(shape); out[dim] = 1
                return dict(x=_r(rng, *shape), g=_r(rng, *out), dim=dim)

            @staticmethod
            def run(dnn, i, libfn=libfn, opname=opname):
                x = dnn.tensor(i["x"], dnn.scratch, True)
                y = getattr(dnn.lib, libfn)(dnn.scratch, x, i["dim"])
                dnn.backward_from(y, i["g"])
                if opname == "mean":
                    # mean = mul(sum(x), 1/n): y's node is the mul; hand its gradient on to the sum node
                    fn = C.cast(y.contents.grad_fn, C.POINTER(load_binding().GradFn))
                    s_ = fn.contents.inputs[0]
                    dnn.backward_from(s_, dnn.download_grad(s_))
                return dict(y=dnn.download(y), dx=dnn.download_grad(x))

            @staticmethod
            def oracle(i, ofn=ofn):
                y, dx = ofn(i["x"], i["dim"], i["g"])
                return dict(y=y, dx=dx)

for shape, dim in (((7, 50), 1), ((7, 50), 0), ((3, 9, 20), 1), ((4, 5, 33), -1)):
    @case("softmax%s dim%d" % (list(shape), dim))
    class _:
        @staticmethod
        def make(rng, shape=shape, dim=dim):
            return dict(x=_r(rng, *shape, scale=2.0), g=_r(rng, *shape), dim=dim)

        @staticmethod
        def run(dnn, i):
            x = dnn.tensor(i["x"], dnn.scratch, True)
            y = dnn.lib.tensor_softmax(dnn.scratch, x, i["dim"])
            dnn.backward_from(y, i["g"])
            return dict(y=dnn.download(y), dx=dnn.download_grad(x))

        @staticmethod
        def oracle(i):
            y, dx = O.softmax(i["x"], i["dim"], i["g"])
            return dict(y=y, dx=dx)

for shape in ((13, 13), (2, 3, 40, 40)):
    @case("causal_softmax%s" % (list(shape),))
    class _:
        @staticmethod
        def make(rng, shape=shape):
            return dict(x=_r(rng, *shape, scale=2.0), g=_r(rng, *shape))

        @staticmethod
        def run(dnn, i):
            x = dnn.tensor(i["x"], dnn.scratch, True)
            y = dnn.lib.tensor_causal_softmax(dnn.scratch, x)
            dnn.backward_from(y, i["g"])
            return dict(y=dnn.download(y), dx=dnn.download_grad(x))

        @staticmethod
        def oracle(i):
            y, dx = O.causal_softmax(i["x"], i["g"])
            return dict(y=y, dx=dx)

for shape, p in (((6, 37), 0.25), ((200,), 0.5)):
    @case("dropout%s p%g" % (list(shape), p))
    class _:
        @staticmethod
        def make(rng, shape=shape, p=p):
            return dict(x=_r(rng, *shape), g=_r(rng, *shape), p=p, seed=1234)

        @staticmethod
        def run(dnn, i):
            dnn.lib.dnn_seed(i["seed"])                       # the mask comes from the host generator, element by element
            x = dnn.tensor(i["x"], dnn.scratch, True)
            y = dnn.lib.tensor_dropout(dnn.scratch, x, i["p"])
            dnn.backward_from(y, i["g"])
            return dict(y=dnn.download(y), dx=dnn.download_grad(x))

        @staticmethod
        def oracle(i):
            y, dx = O.dropout(i["x"], i["p"], i["seed"], i["g"])
            return dict(y=y, dx=dx)

for n, diag in ((9, 1), (6, 0), (5, -2)):
    @case("triu[%d] diag%d" % (n, diag), exact=("y",))
    class _:
        @staticmethod
        def make(rng, n=n, diag=diag):
            return dict(n=n, diag=diag)

        @staticmethod
        def run(dnn, i):
            return dict(y=dnn.download(dnn.lib.tensor_triu(dnn.scratch, i["n"], i["diag"])))

        @staticmethod
        def oracle(i):
            return dict(y=O.triu(i["n"], i["diag"]))

for sa, sb, dim in (((3, 19, 16), (3, 5, 16), 1), ((4, 8), (2, 8), 0), ((2, 3, 4), (2, 3, 9), 2)):
    @case("cat%s%s dim%d" % (list(sa), list(sb), dim))
    class _:
        @staticmethod
        def make(rng, sa=sa, sb=sb, dim=dim):
            out = list(sa); out[dim] += sb[dim]
            return dict(a=_r(rng, *sa), b=_r(rng, *sb), g=_r(rng, *out), dim=dim)

        @staticmethod
        def run(dnn, i):
            a, b = dnn.tensor(i["a"], dnn.scratch, True), dnn.tensor(i["b"], dnn.scratch, True)
            y = dnn.lib.tensor_cat(dnn.scratch, a, b, i["dim"])
            dnn.backward_from(y, i["g"])
            da, db = _grads(dnn, a, b)
            return dict(y=dnn.download(y), da=da, db=db)

        @staticmethod
        def oracle(i):
            y, da, db = O.cat(i["a"], i["b"], i["dim"], i["g"])
            return dict(y=y, da=da, db=db)


# ── matmul_add / matmul ───────────────────────────────────────────────────
MM = [  # (a shape, b shape, trans_b)
    ((4, 37, 64), (64, 96), 0),       # activations x broadcast weight: collapses to one GEMM
    ((4, 37, 64), (96, 64), 1),       # tied-head form
    ((70, 33), (33, 10), 0),          # 2-D, pitch not a multiple of 16 bytes
    ((70, 33), (10, 33), 1),
    ((3, 2, 17, 8), (3, 2, 8, 5), 0), # true batched
    ((2, 128, 256), (256, 128), 0),   # tensor-core sized
    ((2, 128, 256), (128, 256), 1),
    ((300, 200), (200, 520), 0),      # several 128x256 tiles with ragged edges in M, N and K
    ((300, 200), (520, 200), 1),
    ((4096, 136), (136, 96), 0),      # long reduction for dW: split-K path
    ((3, 1100, 72), (72, 40), 0),
]
for sa, sb, tb in MM:
    @case("matmul_add%s%s T%d" % (list(sa), list(sb), tb), tol=3e-5)
    class _:
        @staticmethod
        def make(rng, sa=sa, sb=sb, tb=tb):
            n = sb[-2] if tb else sb[-1]
            out = tuple(np.broadcast_shapes(sa[:-2], sb[:-2])) + (sa[-2], n)
            return dict(a=_r(rng, *sa), b=_r(rng, *sb, scale=0.2), bias=_r(rng, n), g=_r(rng, *out), tb=tb)

        @staticmethod
        def run(dnn, i):
            a = dnn.tensor(i["a"], dnn.scratch, True)
            b, bias = dnn.param(i["b"]), dnn.param(i["bias"])
            y = dnn.lib.tensor_matmul_add(dnn.scratch, a, b, i["tb"], bias)
            dnn.backward_from(y, i["g"])
            da, db, dbias = _grads(dnn, a, b, bias)
            return dict(y=dnn.download(y), da=da, db=db, dbias=dbias)

        @staticmethod
        def oracle(i):
            y, da, db, dbias = O.matmul_add(i["a"], i["b"], i["tb"], i["bias"], i["g"])
            return dict(y=y, da=da, db=db, dbias=dbias)

for sa, sb in (((5, 21, 16), (16, 12)), ((40, 24), (24, 40)), ((2, 3, 9, 4), (2, 3, 4, 6))):
    @case("matmul%s%s" % (list(sa), list(sb)), tol=3e-5)
    class _:
        @staticmethod
        def make(rng, sa=sa, sb=sb):
            out = tuple(np.broadcast_shapes(sa[:-2], sb[:-2])) + (sa[-2], sb[-1])
            return dict(a=_r(rng, *sa), b=_r(rng, *sb), g=_r(rng, *out))

        @staticmethod
        def run(dnn, i):
            a, b = dnn.tensor(i["a"], dnn.scratch, True), dnn.tensor(i["b"], dnn.scratch, True)
            y = dnn.lib.tensor_matmul(dnn.scratch, a, b)
            dnn.backward_from(y, i["g"])
            da, db = _grads(dnn, a, b)
            return dict(y=dnn.download(y), da=da, db=db)

        @staticmethod
        def oracle(i):
            y, da, db, _ = O.matmul_add(i["a"], i["b"], 0, None, i["g"])
            return dict(y=y, da=da, db=db)


# ── attention ─────────────────────────────────────────────────────────────
ATT = [  # B, H, N, d, mode, prefix, seq_lens
    (2, 3, 70, 32, 0, 0, None),
    (1, 2, 1, 64, 0, 0, None),
    (2, 2, 129, 64, 0, 0, None),
    (3, 2, 70, 8, 1, 5, (70, 3, 37)),          # N_b < prefix, padded rows
    (2, 2, 65, 64, 1, 64, (65, 40)),
    (2, 1, 128, 128, 1, 1, None),
    (2, 2, 63, 32, 0, 0, (63, 17)),
]
for B, H, N, d, mode, prefix, lens in ATT:
    @case("attention[B%d H%d N%d d%d mode%d P%d lens=%s]" % (B, H, N, d, mode, prefix, lens), tol=3e-5)
    class _:
        @staticmethod
        def make(rng, B=B, H=H, N=N, d=d, mode=mode, prefix=prefix, lens=lens):
            return dict(q=_r(rng, B, H, N, d), k=_r(rng, B, H, N, d), v=_r(rng, B, H, N, d), g=_r(rng, B, H, N, d),
                        mode=mode, prefix=prefix, lens=None if lens is None else np.array(lens, np.int32))

        @staticmethod
        def run(dnn, i):
            q, k, v = (dnn.tensor(i[n], dnn.scratch, True) for n in "qkv")
            lens = None if i["lens"] is None else i["lens"].ctypes.data_as(C.POINTER(C.c_int))
            o = dnn.lib.tensor_attention_ex(dnn.scratch, q, k, v, None, i["mode"], i["prefix"], lens)
            g = i["g"].copy()
            if i["lens"] is not None:                     # rows beyond seq_len carry no gradient
                for b, nb in enumerate(i["lens"]):
                    g[b, :, nb:] = 0
            dnn.backward_from(o, g)
            dq, dk, dv = _grads(dnn, q, k, v)
            return dict(o=dnn.download(o), dq=dq, dk=dk, dv=dv)

        @staticmethod
        def oracle(i):
            o, dq, dk, dv = O.attention(i["q"], i["k"], i["v"], i["mode"], i["prefix"], i["lens"], i["g"])
            return dict(o=o, dq=dq, dk=dk, dv=dv)


# 4-D masks broadcast over heads / batch; the [40,40] one is read at [b][h] by the reference (see O.attention)
for B, H, N, d, mshape in ((2, 3, 40, 16, (40, 40)), (2, 2, 70, 32, (2, 1, 70, 70)), (1, 2, 33, 64, (1, 2, 33, 33)), (2, 2, 20, 8, (1, 1, 1, 20))):
    @case("attention+mask[B%d H%d N%d d%d mask%s]" % (B, H, N, d, list(mshape)), tol=3e-5)
    class _:
        @staticmethod
        def make(rng, B=B, H=H, N=N, d=d, mshape=mshape):
            return dict(q=_r(rng, B, H, N, d), k=_r(rng, B, H, N, d), v=_r(rng, B, H, N, d), g=_r(rng, B, H, N, d),
                        mask=_r(rng, *mshape, scale=1.5))

        @staticmethod
        def run(dnn, i):
            q, k, v = (dnn.tensor(i[n], dnn.scratch, True) for n in "qkv")
            o = dnn.lib.tensor_attention(dnn.scratch, q, k, v, dnn.tensor(i["mask"], dnn.scratch))
            dnn.backward_from(o, i["g"])
            dq, dk, dv = _grads(dnn, q, k, v)
            return dict(o=dnn.download(o), dq=dq, dk=dk, dv=dv)

        @staticmethod
        def oracle(i):
            o, dq, dk, dv = O.attention(i["q"], i["k"], i["v"], 0, 0, None, i["g"], mask=i["mask"])
            return dict(o=o, dq=dq, dk=dk, dv=dv)


# ── rope / head layout / embedding ────────────────────────────────────────
for shape in ((2, 3, 17, 32), (1, 1, 5, 6), (2, 12, 64, 64)):
    @case("rope%s" % list(shape))
    class _:
        @staticmethod
        def make(rng, shape=shape):
            cos, sin = O.rope_tables(shape[-1], shape[-2])
            return dict(x=_r(rng, *shape), g=_r(rng, *shape), cos=cos, sin=sin)

        @staticmethod
        def run(dnn, i):
            x = dnn.tensor(i["x"], dnn.scratch, True)
            fc, fs = dnn.tensor(i["cos"], dnn.params), dnn.tensor(i["sin"], dnn.params)
            y = dnn.lib.tensor_rope(dnn.scratch, x, fc, fs)
            dnn.backward_from(y, i["g"])
            return dict(y=dnn.download(y), dx=dnn.download_grad(x))

        @staticmethod
        def oracle(i):
            y, dx = O.rope(i["x"], i["cos"], i["sin"], i["g"])
            return dict(y=y, dx=dx)


@case("rope_freqs_init", tol=1e-6, golden_exact=("cos", "sin"))
class _:
    @staticmethod
    def make(rng):
        return dict(dim=64, n=100)

    @staticmethod
    def run(dnn, i):
        fc, fs = TensorP(), TensorP()
        dnn.lib.tensor_rope_freqs_init(dnn.params, C.byref(fc), C.byref(fs), i["dim"], i["n"], 0.0)
        return dict(cos=dnn.download(fc), sin=dnn.download(fs))

    @staticmethod
    def oracle(i):
        c, s = O.rope_tables(i["dim"], i["n"])
        return dict(cos=c, sin=s)


for B, N, H, dk in ((2, 19, 3, 8), (1, 7, 2, 5), (2, 64, 12, 64)):
    @case("split_qkv_heads[B%d N%d H%d dk%d]" % (B, N, H, dk), exact=("q", "k", "v"))
    class _:
        @staticmethod
        def make(rng, B=B, N=N, H=H, dk=dk):
            return dict(x=_r(rng, B, N, 3 * H * dk), H=H, gq=_r(rng, B, H, N, dk), gk=_r(rng, B, H, N, dk), gv=_r(rng, B, H, N, dk))

        @staticmethod
        def run(dnn, i):
            x = dnn.tensor(i["x"], dnn.scratch, True)
            q, k, v = TensorP(), TensorP(), TensorP()
            dnn.lib.tensor_split_qkv_heads(dnn.scratch, x, i["H"], C.byref(q), C.byref(k), C.byref(v))
            for t, g in ((q, i["gq"]), (k, i["gk"]), (v, i["gv"])):
                dnn.backward_from(t, g)
            return dict(q=dnn.download(q), k=dnn.download(k), v=dnn.download(v), dx=dnn.download_grad(x))

        @staticmethod
        def oracle(i):
            q, k, v, dx = O.split_qkv_heads(i["x"], i["H"], i["gq"], i["gk"], i["gv"])
            return dict(q=q, k=k, v=v, dx=dx)

    @case("merge_heads[B%d N%d H%d dk%d]" % (B, N, H, dk), exact=("y", "dx"))
    class _:
        @staticmethod
        def make(rng, B=B, N=N, H=H, dk=dk):
            return dict(x=_r(rng, B, H, N, dk), g=_r(rng, B, N, H * dk))

        @staticmethod
        def run(dnn, i):
            x = dnn.tensor(i["x"], dnn.scratch, True)
            y = dnn.lib.tensor_merge_heads(dnn.scratch, x)
            dnn.backward_from(y, i["g"])
            return dict(y=dnn.download(y), dx=dnn.download_grad(x))

        @staticmethod
        def oracle(i):
            y, dx = O.merge_heads(i["x"], i["g"])
            return dict(y=y, dx=dx)

    @case("split_heads[B%d N%d H%d dk%d]" % (B, N, H, dk), exact=("y", "dx"))
    class _:
        @staticmethod
        def make(rng, B=B, N=N, H=H, dk=dk):
            return dict(x=_r(rng, B, N, H * dk), H=H, g=_r(rng, B, H, N, dk))

        @staticmethod
        def run(dnn, i):
            x = dnn.tensor(i["x"], dnn.scratch, True)
            y = dnn.lib.tensor_split_heads(dnn.scratch, x, i["H"])
            dnn.backward_from(y, i["g"])
            return dict(y=dnn.download(y), dx=dnn.download_grad(x))

        @staticmethod
        def oracle(i):
            y, dx = O.split_heads(i["x"], i["H"], i["g"])
            return dict(y=y, dx=dx)


for V, D, n in ((50, 16, 200), (7, 5, 1), (300, 768, 64)):
    @case("embedding[V%d D%d n%d]" % (V, D, n), exact=("y",))
    class _:
        @staticmethod
        def make(rng, V=V, D=D, n=n):
            return dict(table=_r(rng, V, D), ids=rng.integers(0, V, size=n).astype(np.int32), g=_r(rng, n, D))

        @staticmethod
        def run(dnn, i):
            table = dnn.param(i["table"])
            ids = dnn.tensor(i["ids"], dnn.data)
            y = dnn.lib.tensor_embedding(dnn.scratch, table, ids)
            dnn.backward_from(y, i["g"])
            return dict(y=dnn.download(y), dtable=dnn.download_grad(table))

        @staticmethod
        def oracle(i):
            y, dt = O.embedding(i["table"], i["ids"], i["g"])
            return dict(y=y, dtable=dt)


# ── cross entropy ─────────────────────────────────────────────────────────
def _ce_run(dnn, i):
    full = dnn.tensor(i["logits_full"], dnn.scratch, True)
    logits = full
    if i["slice"] is not None:
        dim, start, ln = i["slice"]
        logits = dnn.lib.tensor_slice(dnn.scratch, full, dim, start, ln)
    target = dnn.tensor(i["target"], dnn.data)
    if i["mask"] is None:
        loss = dnn.lib.tensor_cross_entropy(dnn.scratch, logits, target, i["dim"])
    else:
        mask = dnn.tensor(i["mask"], dnn.data)
        loss = dnn.lib.tensor_cross_entropy_masked(dnn.scratch, logits, target, mask, i["dim"])
    dnn.lib.dnn_backward(dnn.scratch, loss)
    dnn.sync()
    return dict(loss=dnn.download(loss), dlogits=dnn.download_grad(full))


def _ce_oracle(i):
    full = i["logits_full"]
    sl = [slice(None)] * full.ndim
    if i["slice"] is not None:
        dim, start, ln = i["slice"]
        sl[dim] = slice(start, start + ln)
    loss, d = O.cross_entropy(full[tuple(sl)], i["target"], i["mask"])
    dfull = np.zeros_like(full)
    dfull[tuple(sl)] = d
    return dict(loss=np.array([loss], np.float32), dlogits=dfull)


CE = [  # full logits shape, slice (dim,start,len) or None, masked
    ((64, 10), None, False),                 # 2-D classification path
    ((4, 33, 257), (1, 0, 32), False),       # GPT path: [B,N,V] sliced to [B,N-1,V]
    ((3, 20, 1024), (1, 12, 8), True),       # VLM path: text rows of [B,I+T,V], masked
    ((2, 9, 40), None, True),
    ((2, 5, 32000), None, False),            # wide rows, float4 path
]
for shape, slc, masked in CE:
    @case("cross_entropy%s slice=%s masked=%d" % (list(shape), slc, masked))
    class _:
        @staticmethod
        def make(rng, shape=shape, slc=slc, masked=masked):
            full = _r(rng, *shape, scale=2.0)
            tshape = list(shape[:-1])
            if slc is not None:
                tshape[slc[0]] = slc[2]
            target = rng.integers(0, shape[-1], size=tshape).astype(np.int32)
            mask = (rng.random(tshape) > 0.3).astype(np.float32) if masked else None
            return dict(logits_full=full, slice=slc, target=target, mask=mask, dim=len(shape) - 1)

        run = staticmethod(_ce_run)
        oracle = staticmethod(_ce_oracle)


# ── conv2d / avg_pool2d ───────────────────────────────────────────────────
CONV = [  # N, C, H, W, out_C, k, stride, pad
    (3, 1, 28, 28, 8, 3, 1, 1),      # reference takes its Winograd path: true NCHW
    (2, 4, 9, 7, 6, 3, 1, 1),
    (2, 3, 32, 32, 16, 16, 16, 0),   # patch embed: (M, out_C) memory in an NCHW-shaped tensor
    (2, 2, 11, 11, 5, 3, 2, 0),
    (1, 2, 8, 8, 4, 5, 1, 2),
]
for N, Cc, H, W, oc, k, s, p in CONV:
    @case("conv2d[N%d C%d %dx%d oc%d k%d s%d p%d]" % (N, Cc, H, W, oc, k, s, p), tol=3e-5)
    class _:
        @staticmethod
        def make(rng, N=N, Cc=Cc, H=H, W=W, oc=oc, k=k, s=s, p=p):
            Ho, Wo = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
            return dict(x=_r(rng, N, Cc, H, W), w=_r(rng, oc, Cc, k, k, scale=0.3), b=_r(rng, oc), g=_r(rng, N, oc, Ho, Wo), s=s, p=p)

        @staticmethod
        def run(dnn, i):
            x = dnn.tensor(i["x"], dnn.scratch, True)
            w, b = dnn.param(i["w"]), dnn.param(i["b"])
            y = dnn.lib.tensor_conv2d(dnn.scratch, x, w, b, i["s"], i["p"])
            dnn.backward_from(y, i["g"])
            dx, dw, db = _grads(dnn, x, w, b)
            return dict(y=dnn.download(y), dx=dx, dw=dw, db=db)

        @staticmethod
        def oracle(i):
            y, dx, dw, db = O.conv2d(i["x"], i["w"], i["b"], i["s"], i["p"], i["g"])
            return dict(y=y, dx=dx, dw=dw, db=db)

for shape, k, s in (((2, 3, 28, 28), 2, 2), ((2, 2, 9, 9), 2, 1), ((1, 2, 11, 10), 3, 2)):
    @case("avg_pool2d%s k%d s%d" % (list(shape), k, s))
    class _:
        @staticmethod
        def make(rng, shape=shape, k=k, s=s):
            Ho, Wo = (shape[2] - k) // s + 1, (shape[3] - k) // s + 1
            return dict(x=_r(rng, *shape), g=_r(rng, shape[0], shape[1], Ho, Wo), k=k, s=s)

        @staticmethod
        def run(dnn, i):
            x = dnn.tensor(i["x"], dnn.scratch, True)
            y = dnn.lib.tensor_avg_pool2d(dnn.scratch, x, i["k"], i["s"])
            dnn.backward_from(y, i["g"])
            return dict(y=dnn.download(y), dx=dnn.download_grad(x))

        @staticmethod
        def oracle(i):
            y, dx = O.avg_pool2d(i["x"], i["k"], i["s"], i["g"])
            return dict(y=y, dx=dx)


# ── optimiser: AdamW, gradient norm / clipping, LR schedules (src/optim.c:104-316) ─────────
def _give_grads(dnn, params, grads):
    """p.grad += g through the public API only: the backward of p * g started from a non-scalar root,
    whose gradient dnn_backward sets to ones (src/autograd.c:106-110).  None leaves grad == NULL."""
    for p, g in zip(params, grads):
        if g is None:
            continue
        y = dnn.lib.tensor_mul(dnn.scratch, p, dnn.tensor(g, dnn.scratch))
        dnn.lib.dnn_backward(dnn.scratch, y)
    dnn.sync()


ADAM_SHAPES = [(33, 17), (1025,), (8,), (5, 7)]          # the last one never receives a gradient
ADAM_HYPER = dict(lr=1e-3, b1=0.9, b2=0.95, eps=1e-8, wd=0.1)

for mults, lrs in ((None, (1e-3, 1e-3, 1e-3)), ((1.0, 0.5, 2.0, 1.0), (1e-3, 7e-4, 2e-4))):
    @case("adamw[3 steps, lr_mults=%s]" % (mults is not None), tol=1e-6, exact=("t",))
    class _:
        @staticmethod
        def make(rng, mults=mults, lrs=lrs):
            i = dict(mults=None if mults is None else np.array(mults, np.float32), lrs=lrs)
            for k, shape in enumerate(ADAM_SHAPES):
                i["p%d" % k] = _r(rng, *shape, scale=0.05)
                i["m%d" % k] = _r(rng, *shape, scale=0.01)
                i["v%d" % k] = (_r(rng, *shape, scale=0.01) ** 2).astype(np.float32)
                for s in range(3):
                    i["g%d_%d" % (k, s)] = None if k == 3 else _r(rng, *shape, scale=0.02 * (s + 1))
            return i

        @staticmethod
        def run(dnn, i):
            B = load_binding()
            n = len(ADAM_SHAPES)
            params = [dnn.param(i["p%d" % k]) for k in range(n)]
            arr = (B.TensorP * n)(*params)
            h = ADAM_HYPER
            opt = dnn.lib.adamw_create(dnn.params, arr, n, h["lr"], h["b1"], h["b2"], h["eps"], h["wd"])
            for k in range(n):
                dnn.upload(opt.contents.m[k], i["m%d" % k])
                dnn.upload(opt.contents.v[k], i["v%d" % k])
            out = {}
            for s in range(3):
                dnn.lib.adamw_zero_grad(opt)
                _give_grads(dnn, params, [i["g%d_%d" % (k, s)] for k in range(n)])
                opt.contents.lr = i["lrs"][s]                       # what lr_scheduler_step does between steps
                if i["mults"] is None:
                    dnn.lib.adamw_step(opt)
                else:
                    dnn.lib.adamw_step_with_lr_multipliers(opt, i["mults"].ctypes.data_as(C.POINTER(C.c_float)))
                dnn.sync()
                if s == 0:
                    out.update({"p%d_step1" % k: dnn.download(params[k]) for k in range(n)})
                dnn.lib.mem_pool_reset(dnn.scratch)
            for k in range(n):
                out["p%d" % k], out["m%d" % k], out["v%d" % k] = dnn.download(params[k]), dnn.download(opt.contents.m[k]), dnn.download(opt.contents.v[k])
            out["t"] = np.array([opt.contents.t], np.int32)
            return out

        @staticmethod
        def oracle(i):
            h = ADAM_HYPER
            out = {}
            for k in range(len(ADAM_SHAPES)):
                p, m, v = i["p%d" % k], i["m%d" % k], i["v%d" % k]
                for s in range(3):
                    g = i["g%d_%d" % (k, s)]
                    if g is not None:
                        lr = np.float32(i["lrs"][s]) * (np.float32(1.0) if i["mults"] is None else i["mults"][k])
                        p, m, v = O.adamw_update(p, g, m, v, s + 1, lr, h["b1"], h["b2"], h["eps"], h["wd"])
                    if s == 0:
                        out["p%d_step1" % k] = p
                out["p%d" % k], out["m%d" % k], out["v%d" % k] = p, m, v
            out["t"] = np.array([3], np.int32)
            return out


for max_norm in (0.5, 1e6, 0.0, -1.0):
    @case("clip_grad_norm[max %g]" % max_norm, tol=1e-6)
    class _:
        @staticmethod
        def make(rng, max_norm=max_norm):
            return dict(max_norm=max_norm, g0=_r(rng, 40, 9), g1=_r(rng, 1030), g2=_r(rng, 3, 3, 3, scale=4.0))

        @staticmethod
        def run(dnn, i):
            B = load_binding()
            params = [dnn.param(np.ones_like(i[k])) for k in ("g0", "g1", "g2")] + [dnn.param(np.ones((4, 4), np.float32))]
            arr = (B.TensorP * 4)(*params)
            _give_grads(dnn, params, [i["g0"], i["g1"], i["g2"], None])
            before = dnn.lib.grad_norm(arr, 4)
            ret = dnn.lib.clip_grad_norm(arr, 4, i["max_norm"])
            after = dnn.lib.grad_norm(arr, 4)
            dnn.sync()
            out = {"g%d" % k: dnn.download_grad(params[k]) for k in range(3)}
            out["norms"] = np.array([before, ret, after], np.float32)
            assert not params[3].contents.grad, "a parameter outside the graph must keep grad == NULL"
            return out

        @staticmethod
        def oracle(i):
            gs = [i["g0"], i["g1"], i["g2"]]
            total = O.grad_norm(gs)
            if i["max_norm"] <= 0:                                   # src/optim.c:207: no-op that returns 0
                return dict(g0=gs[0], g1=gs[1], g2=gs[2], norms=np.array([total, 0.0, total], np.float32))
            scale = O.clip_scale(total, i["max_norm"])
            gs = [(g * scale).astype(np.float32) for g in gs]
            return dict(g0=gs[0], g1=gs[1], g2=gs[2], norms=np.array([total, total, O.grad_norm(gs)], np.float32))


LR_SCHEDULES = [  # schedule id (include/optim.h:113-118), warmup, total, step_size, gamma, min_lr
    (0, 0, 100, 0, 0.0, -1.0), (1, 10, 100, 0, 0.0, -1.0), (2, 5, 50, 0, 0.0, -1.0), (3, 0, 40, 0, 0.0, 1e-5),
    (4, 3, 100, 7, 0.5, -1.0), (5, 0, 30, 0, 0.9, -1.0), (1, 100, 10000, 0, 0.0, -1.0), (1, 8, 8, 0, 0.0, -1.0),
]


@case("lr_schedules", tol=1e-6, golden_exact=tuple("lr%d" % k for k in range(len(LR_SCHEDULES))) + ("get_lr", "after_reset"))
class _:
    @staticmethod
    def make(rng):
        return dict(base=6e-4, steps=130)

    @staticmethod
    def run(dnn, i):
        B = load_binding()
        out, get, reset = {}, [], []
        for k, (sched, warmup, total, step, gamma, min_lr) in enumerate(LR_SCHEDULES):
            opt = B.AdamW()
            s = dnn.lib.lr_scheduler_create(dnn.params, C.byref(opt), sched, i["base"], warmup, total, min_lr, step, gamma)
            lrs = []
            for t in range(i["steps"]):
                lrs.append(opt.lr)
                dnn.lib.lr_scheduler_step(s)
            out["lr%d" % k] = np.array(lrs, np.float32)
            get.append(dnn.lib.lr_scheduler_get_lr(s))
            dnn.lib.lr_scheduler_reset(s)
            reset.append(opt.lr)
        out["get_lr"], out["after_reset"] = np.array(get, np.float32), np.array(reset, np.float32)
        return out

    @staticmethod
    def oracle(i):
        out, get, reset = {}, [], []
        for k, (sched, warmup, total, step, gamma, min_lr) in enumerate(LR_SCHEDULES):
            f = lambda t: O.lr_schedule(sched, i["base"], min_lr, warmup, total, step, gamma, t)
            out["lr%d" % k] = np.array([f(t) for t in range(i["steps"])], np.float32)
            get.append(f(i["steps"]))
            reset.append(f(0))
        out["get_lr"], out["after_reset"] = np.array(get, np.float32), np.array(reset, np.float32)
        return out


# ── views ─────────────────────────────────────────────────────────────────
@case("transpose+contiguous+reshape (VLM image-embed path)", exact=("y", "dx"))
class _:
    @staticmethod
    def make(rng):
        return dict(x=_r(rng, 2, 6, 3, 4), g=_r(rng, 2, 12, 6))

    @staticmethod
    def run(dnn, i):
        x = dnn.tensor(i["x"], dnn.scratch, True)
        t = dnn.lib.tensor_transpose(dnn.scratch, x, 1, 2)
        t = dnn.lib.tensor_transpose(dnn.scratch, t, 2, 3)
        c = dnn.lib.tensor_contiguous(dnn.scratch, t)
        dnn.backward_from(c, i["g"].reshape(2, 3, 4, 6))
        y = dnn.lib.tensor_reshape(dnn.scratch, c, 3, load_binding().ints([2, 12, 6]))
        return dict(y=dnn.download(y), dx=dnn.download_grad(x))

    @staticmethod
    def oracle(i):
        y = np.ascontiguousarray(i["x"].transpose(0, 2, 3, 1)).reshape(2, 12, 6)
        dx = np.ascontiguousarray(i["g"].reshape(2, 3, 4, 6).transpose(0, 3, 1, 2))
        return dict(y=y, dx=dx)


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a - b))


def compare(case, got, want, tol=None, golden=False):
    tol = case.tol if tol is None else tol
    exact = case.golden_exact if golden else case.exact
    assert set(got) == set(want), (sorted(got), sorted(want))
    for k in sorted(want):
        assert got[k] is not None, "%s: %s was never written" % (case.name, k)
        assert got[k].shape == want[k].shape, (case.name, k, got[k].shape, want[k].shape)
        if k in exact:
            assert np.array_equal(got[k], want[k]), "%s: %s not bit-exact" % (case.name, k)
        elif np.linalg.norm(want[k]) < 1e-6 * np.sqrt(want[k].size) and tol >= 1e-3:
            # a gradient that is exactly zero in exact arithmetic (single-key softmax): TF32
            # leaves rounding-sized residue of the O(1) intermediates; bound it absolutely
            e = float(np.linalg.norm(got[k])) / np.sqrt(want[k].size)
            assert e <= tol, "%s: %s should vanish, rms %.3g > %.1g" % (case.name, k, e, tol)
        else:
            e = rel_l2(got[k], want[k])
            assert e <= tol, "%s: %s relative L2 error %.3g > %.1g" % (case.name, k, e, tol)
