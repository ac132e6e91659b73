"""CPU restatement of the dnn.c training hot path — TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA kernels: numpy restatements of the
forward and backward formulas of masc-it/dnn.c, each citing the reference
file:line it follows.  Only tests/, __graft_entry__.smoke() and bench.py's
cpu_baseline leg may import it; the product (dnn.c_b200/) never does.

Arithmetic is done in float64 and returned as float32: the reference computes
in fp32 with a fixed loop order, so this oracle is its exact-arithmetic limit
and both the reference and the kernels must agree with it to rounding.

Parity status: PINNED.  tests/test_oracle_golden.py checks every function here
against tests/golden/*.npz, which tests/golden/make_golden.py produced by
running the unmodified reference (oracle/_ref/libdnn_ref.so, built from the
reference's own sources by oracle/Makefile) on seeded inputs.
"""
import numpy as np

F64 = np.float64


def _f32(x):
    return np.asarray(x, dtype=np.float32)


def _unbroadcast(g, shape):
    """Sum `g` over the dims that were broadcast from `shape` (src/ops_elem.c:83-105)."""
    g = np.asarray(g)
    while g.ndim > len(shape):
        g = g.sum(axis=0)
    for d, s in enumerate(shape):
        if s == 1 and g.shape[d] != 1:
            g = g.sum(axis=d, keepdims=True)
    return g


# ── elementwise (src/ops_elem.c:33-175, src/ops_activation.c:16-333) ──────
def add(a, b, gout):
    y = a.astype(F64) + b.astype(F64)
    g = gout.astype(F64)
    return _f32(y), _f32(_unbroadcast(g, a.shape)), _f32(_unbroadcast(g, b.shape))


# ── the rest of ops.h (src/ops_elem.c:178-680, src/ops_reduce.c:12-153, src/ops_activation.c:70-130,300-800,1410-1500)
def sub(a, b, gout):
    g = gout.astype(F64)
    return _f32(a.astype(F64) - b.astype(F64)), _f32(_unbroadcast(g, a.shape)), _f32(_unbroadcast(-g, b.shape))


def mul(a, b, gout):
    a64, b64, g = a.astype(F64), b.astype(F64), gout.astype(F64)
    return _f32(a64 * b64), _f32(_unbroadcast(g * b64, a.shape)), _f32(_unbroadcast(g * a64, b.shape))


def div(a, b, gout):
    a64, b64, g = a.astype(F64), b.astype(F64), gout.astype(F64)
    return _f32(a64 / b64), _f32(_unbroadcast(g / b64, a.shape)), _f32(_unbroadcast(-g * a64 / (b64 * b64), b.shape))


def neg(x, gout):
    return _f32(-x), _f32(-gout)


def power(x, e, gout):
    x64 = x.astype(F64)
    return _f32(x64 ** e), _f32(e * x64 ** (e - 1.0) * gout.astype(F64))


def sigmoid(x, gout):
    s = 1.0 / (1.0 + np.exp(-x.astype(F64)))
    return _f32(s), _f32(s * (1.0 - s) * gout.astype(F64))


def sum_dim(x, dim, gout):
    """keepdim sum; gout has the output shape (size 1 along dim)."""
    y = x.astype(F64).sum(axis=dim, keepdims=True)
    return _f32(y), _f32(np.broadcast_to(gout.astype(F64), x.shape))


def mean_dim(x, dim, gout):
    y = x.astype(F64).mean(axis=dim, keepdims=True)
    return _f32(y), _f32(np.broadcast_to(gout.astype(F64), x.shape) / x.shape[dim])


def softmax(x, dim, gout):
    x64 = x.astype(F64)
    e = np.exp(x64 - x64.max(axis=dim, keepdims=True))
    y = e / e.sum(axis=dim, keepdims=True)
    g = gout.astype(F64)
    return _f32(y), _f32(y * (g - (y * g).sum(axis=dim, keepdims=True)))


def causal_softmax(x, gout):
    """softmax over the last dim of (..., N, N) with columns j > i of row i masked out (exact zeros)."""
    x64 = x.astype(F64)
    n = x.shape[-1]
    keep = np.tril(np.ones((n, n), bool))
    xm = np.where(keep, x64, -np.inf)
    e = np.exp(xm - xm.max(axis=-1, keepdims=True))
    y = e / e.sum(axis=-1, keepdims=True)
    g = gout.astype(F64)
    return _f32(y), _f32(np.where(keep, y * (g - (y * g).sum(axis=-1, keepdims=True)), 0.0))


def dropout(x, p, seed, gout):
    """keep mask from the reference generator in element order: uniform() >= p (src/ops_activation.c:1460)."""
    r = Rng(seed)
    keep = np.array([1.0 if r.uniform() >= p else 0.0 for _ in range(x.size)], F64).reshape(x.shape)
    scale = 1.0 / (1.0 - p)
    return _f32(keep * x.astype(F64) * scale), _f32(keep * gout.astype(F64) * scale)


def triu(n, diagonal):
    i, j = np.indices((n, n))
    return np.where(j >= i + diagonal, -np.inf, 0.0).astype(np.float32)


def cat(a, b, dim, gout):
    y = np.concatenate([a, b], axis=dim)
    ga, gb = np.split(gout, [a.shape[dim]], axis=dim)
    return _f32(y), _f32(ga), _f32(gb)


def relu(x, gout):
    return _f32(np.maximum(x, 0)), _f32(np.where(x > 0, gout, 0))


def silu(x, gout):
    x64 = x.astype(F64)
    s = 1.0 / (1.0 + np.exp(-x64))
    return _f32(x64 * s), _f32(gout * s * (1.0 + x64 - x64 * s))


def swiglu(gate, up, gout):
    g, u, go = gate.astype(F64), up.astype(F64), gout.astype(F64)
    s = 1.0 / (1.0 + np.exp(-g))
    y = g * s * u
    dg = go * (s * (1.0 + g - g * s)) * u
    du = go * (g * s)
    return _f32(y), _f32(_unbroadcast(dg, gate.shape)), _f32(_unbroadcast(du, up.shape))


# ── norms (src/norm.c:281-495 rms, :13-277 layer) ─────────────────────────
def rms_norm(x, w, eps, gout):
    x64, g = x.astype(F64), gout.astype(F64)
    d = x.shape[-1]
    rs = 1.0 / np.sqrt((x64 * x64).mean(-1, keepdims=True) + eps)
    wv = np.ones(d) if w is None else w.astype(F64)
    y = x64 * rs * wv
    dw = (g * x64 * rs).reshape(-1, d).sum(0)
    dy = g * wv
    S = (dy * x64).sum(-1, keepdims=True)
    dx = rs * dy - rs * (rs * rs / d * S) * x64
    return _f32(y), _f32(dx), _f32(dw)


def layer_norm(x, w, b, eps, gout):
    x64, g = x.astype(F64), gout.astype(F64)
    d = x.shape[-1]
    mu = x64.mean(-1, keepdims=True)
    var = ((x64 - mu) ** 2).mean(-1, keepdims=True)
    rs = 1.0 / np.sqrt(var + eps)
    wv = np.ones(d) if w is None else w.astype(F64)
    bv = np.zeros(d) if b is None else b.astype(F64)
    xmu = x64 - mu
    y = xmu * rs * wv + bv
    dw = (g * xmu * rs).reshape(-1, d).sum(0)
    db = g.reshape(-1, d).sum(0)
    dy = g * wv
    mdy = dy.mean(-1, keepdims=True)
    mdx = (dy * xmu).mean(-1, keepdims=True)
    dx = rs * (dy - mdy - xmu * mdx * rs * rs)
    return _f32(y), _f32(dx), _f32(dw), _f32(db)


# ── matmul (src/ops_matrix.c:48-1206) ─────────────────────────────────────
def matmul_add(a, b, trans_b, bias, gout):
    """y = a @ b (+T) + bias with numpy batch broadcasting; grads keep operand layouts."""
    a64, b64, g = a.astype(F64), b.astype(F64), gout.astype(F64)
    bop = np.swapaxes(b64, -1, -2) if trans_b else b64
    y = a64 @ bop
    if bias is not None:
        y = y + bias.astype(F64)
    da = _unbroadcast(g @ np.swapaxes(bop, -1, -2), a.shape)
    dbop = np.swapaxes(a64, -1, -2) @ g
    db = np.swapaxes(dbop, -1, -2) if trans_b else dbop
    db = _unbroadcast(db, b.shape)
    dbias = None if bias is None else g.reshape(-1, g.shape[-1]).sum(0)
    return _f32(y), _f32(da), _f32(db), (None if dbias is None else _f32(dbias))


# ── attention (src/attention.c:39-64 visibility, :259-380 fwd, :387-540 bwd) ─
def visible_len(mode, i, prefix_len, n_b):
    v = i + 1 if (mode == 0 or i >= prefix_len) else prefix_len
    return min(v, n_b)


def attention(q, k, v, mode, prefix_len, seq_lens, gout, mask=None):
    """mask: additive, added to the scaled scores of the visible columns (src/attention.c:314-325); it gets no
    gradient.  The reference looks it up with _bcast_off(mask, mask->ndim, {b,h,i,j}) (src/broadcast.h:26-44), i.e.
    dimension k of the mask is indexed by the k-th of (b, h, i, j): a 4-D mask broadcasts as documented, a mask of
    fewer dimensions is read by the LEADING coordinates ([N,N] is read at [b][h]).  Kept as it is."""
    B, H, N, d = q.shape
    mfull = None
    if mask is not None:
        m = np.asarray(mask, F64)
        ext = (B, H, N, N)
        idx = np.ix_(*[np.zeros(ext[k], int) if m.shape[k] == 1 else np.arange(ext[k]) for k in range(m.ndim)])
        sub = m[idx]                                          # shape ext[:ndim]
        mfull = np.broadcast_to(sub.reshape(sub.shape + (1,) * (4 - m.ndim)), ext)
    scale = 1.0 / np.sqrt(np.float32(d)).astype(F64)
    o = np.zeros(q.shape, F64)
    dq, dk, dv = (np.zeros(q.shape, F64) for _ in range(3))
    for b in range(B):
        nb = N if seq_lens is None else int(seq_lens[b])
        vis = np.array([visible_len(mode, i, prefix_len, nb) for i in range(nb)])
        allow = np.arange(nb)[None, :] < vis[:, None]              # [nb, nb]
        for h in range(H):
            Q, K, V = (t[b, h, :nb].astype(F64) for t in (q, k, v))
            S = scale * (Q @ K.T)
            if mfull is not None:
                S = S + mfull[b, h, :nb, :nb]
            S = np.where(allow, S, -np.inf)
            P = np.exp(S - S.max(-1, keepdims=True))
            P = np.where(allow, P, 0.0)
            P /= P.sum(-1, keepdims=True)
            o[b, h, :nb] = P @ V
            G = gout[b, h, :nb].astype(F64)
            dv[b, h, :nb] = P.T @ G
            dP = G @ V.T
            dS = P * (dP - (P * dP).sum(-1, keepdims=True)) * scale
            dq[b, h, :nb] = dS @ K
            dk[b, h, :nb] = dS.T @ Q
    return _f32(o), _f32(dq), _f32(dk), _f32(dv)


# ── rope (src/rope.c:60-171) ──────────────────────────────────────────────
def rope_tables(dim, max_seq, base=10000.0):
    """float32 libm arithmetic as in src/rope.c:163-169."""
    k = np.arange(dim // 2, dtype=np.float32)
    theta = np.power(np.float32(base), (np.float32(-2.0) * k / np.float32(dim)).astype(np.float32)).astype(np.float32)
    ang = (np.arange(max_seq, dtype=np.float32)[:, None] * theta[None, :]).astype(np.float32)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def rope(x, cos, sin, gout):
    x64, g = x.astype(F64), gout.astype(F64)
    c, s = cos.astype(F64), sin.astype(F64)
    xe, xo = x64[..., 0::2], x64[..., 1::2]
    y = np.empty_like(x64)
    y[..., 0::2] = xe * c - xo * s
    y[..., 1::2] = xe * s + xo * c
    ge, go = g[..., 0::2], g[..., 1::2]
    dx = np.empty_like(x64)
    dx[..., 0::2] = ge * c + go * s
    dx[..., 1::2] = -ge * s + go * c
    return _f32(y), _f32(dx)


# ── head layout (src/multihead.c) ─────────────────────────────────────────
def split_qkv_heads(qkv, H, gq, gk, gv):
    B, N, D = qkv.shape
    dk = D // (3 * H)
    x = qkv.reshape(B, N, 3, H, dk)
    q, k, v = (np.ascontiguousarray(x[:, :, i].transpose(0, 2, 1, 3)) for i in range(3))
    g = np.stack([t.transpose(0, 2, 1, 3) for t in (gq, gk, gv)], axis=2).reshape(B, N, D)
    return q, k, v, _f32(g)


def merge_heads(x, gout):
    B, H, N, dk = x.shape
    y = np.ascontiguousarray(x.transpose(0, 2, 1, 3)).reshape(B, N, H * dk)
    dx = np.ascontiguousarray(gout.reshape(B, N, H, dk).transpose(0, 2, 1, 3))
    return y, dx


def split_heads(x, H, gout):
    B, N, D = x.shape
    dk = D // H
    y = np.ascontiguousarray(x.reshape(B, N, H, dk).transpose(0, 2, 1, 3))
    dx = np.ascontiguousarray(gout.transpose(0, 2, 1, 3)).reshape(B, N, D)
    return y, dx


# ── embedding (src/embedding.c:18-110) ────────────────────────────────────
def embedding(table, ids, gout):
    y = table[ids]
    dt = np.zeros(table.shape, F64)
    np.add.at(dt, ids, gout.astype(F64))
    return _f32(y), _f32(dt)


# ── cross entropy (src/ops_activation.c:852-1145, masked :1154-1410) ──────
def cross_entropy(logits, target, mask=None, gout=1.0):
    """Class dim is the last one.  Returns (loss, dlogits)."""
    x = logits.astype(F64)
    C = x.shape[-1]
    x2 = x.reshape(-1, C)
    t = np.asarray(target).reshape(-1)
    mx = x2.max(-1, keepdims=True)
    se = np.exp(x2 - mx).sum(-1, keepdims=True)
    lse = (mx + np.log(se))[:, 0]
    nll = lse - x2[np.arange(len(t)), t]
    sm = np.exp(x2 - mx) / se
    onehot = np.zeros_like(sm)
    onehot[np.arange(len(t)), t] = 1.0
    if mask is None:
        inv = 1.0 / len(t)
        loss = nll.sum() * inv
        d = (sm - onehot) * (gout * inv)
    else:
        m = np.broadcast_to(np.asarray(mask, F64), np.asarray(target).shape).reshape(-1)
        inv = 1.0 / max(m.sum(), 1.0)
        loss = (nll * m).sum() * inv
        d = (sm - onehot) * (gout * inv) * m[:, None]
    return np.float32(loss), _f32(d.reshape(logits.shape))


# ── conv / pool (src/conv.c, src/ops_pool.c) ──────────────────────────────
def _im2col(x, kH, kW, stride, pad):
    N, C, H, W = x.shape
    Ho, Wo = (H + 2 * pad - kH) // stride + 1, (W + 2 * pad - kW) // stride + 1
    xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad)))
    col = np.empty((N, Ho, Wo, C, kH, kW), x.dtype)
    for kh in range(kH):
        for kw in range(kW):
            col[:, :, :, :, kh, kw] = xp[:, :, kh:kh + stride * Ho:stride, kw:kw + stride * Wo:stride].transpose(0, 2, 3, 1)
    return col.reshape(N * Ho * Wo, C * kH * kW), Ho, Wo


def conv2d(x, w, bias, stride, pad, gout):
    """Returns (y, dx, dw, dbias) as flat MEMORY images shaped [N, out_C, Ho, Wo] / operand shapes.

    3x3/s1/p1 is true NCHW (the reference's Winograd path, src/conv.c:719-800).
    Every other geometry stores the GEMM result (M, out_C) in the NCHW-declared
    buffer, reads the upstream gradient the same way (src/conv.c:437-506,847-863)
    but sums the bias gradient with NCHW indexing (:418-435)."""
    N, C, H, W = x.shape
    oc, _, kH, kW = w.shape
    col, Ho, Wo = _im2col(x.astype(F64), kH, kW, stride, pad)        # (M, K)
    wm = w.reshape(oc, -1).astype(F64)
    nchw = (kH == 3 and kW == 3 and stride == 1 and pad == 1)
    y_mc = col @ wm.T + (0 if bias is None else bias.astype(F64))
    g = gout.astype(F64)
    dbias = None if bias is None else g.reshape(N, oc, Ho * Wo).sum((0, 2))
    if nchw:
        y = y_mc.reshape(N, Ho, Wo, oc).transpose(0, 3, 1, 2)
        g_mc = g.transpose(0, 2, 3, 1).reshape(-1, oc)
    else:
        y = y_mc.reshape(N, oc, Ho, Wo)                              # memory image, not a transpose
        g_mc = g.reshape(-1, oc)
    dw = (g_mc.T @ col).reshape(w.shape)
    dcol = (g_mc @ wm).reshape(N, Ho, Wo, C, kH, kW)
    dxp = np.zeros((N, C, H + 2 * pad, W + 2 * pad), F64)
    for kh in range(kH):
        for kw in range(kW):
            dxp[:, :, kh:kh + stride * Ho:stride, kw:kw + stride * Wo:stride] += dcol[:, :, :, :, kh, kw].transpose(0, 3, 1, 2)
    dx = dxp[:, :, pad:pad + H, pad:pad + W]
    return _f32(y), _f32(dx), _f32(dw), (None if dbias is None else _f32(dbias))


def avg_pool2d(x, k, stride, gout):
    N, C, H, W = x.shape
    if stride <= 0:
        stride = k
    Ho, Wo = (H - k) // stride + 1, (W - k) // stride + 1
    y = np.zeros((N, C, Ho, Wo), F64)
    dx = np.zeros(x.shape, F64)
    g = gout.astype(F64) / (k * k)
    for di in range(k):
        for dj in range(k):
            y += x[:, :, di:di + stride * Ho:stride, dj:dj + stride * Wo:stride]
            dx[:, :, di:di + stride * Ho:stride, dj:dj + stride * Wo:stride] += g
    return _f32(y / (k * k)), _f32(dx)


# ── optimiser (src/optim.c:104-316) ───────────────────────────────────────
def grad_norm(grads):
    return np.float32(np.sqrt(np.float32(sum(float((g.astype(F64) ** 2).sum()) for g in grads if g is not None))))


def clip_scale(total_norm, max_norm):
    return np.float32(max_norm) / np.float32(total_norm) if total_norm > max_norm else np.float32(1.0)


def adamw_update(p, g, m, v, t, lr, b1, b2, eps, wd):
    """One AdamW step in fp32, operation order of src/optim.c:270-310.  t is the step count AFTER increment."""
    f = np.float32
    p, g, m, v = (a.astype(np.float32) for a in (p, g, m, v))
    bc1 = f(1.0) - f(np.power(f(b1), f(t)))
    bc2s = np.sqrt(f(1.0) - f(np.power(f(b2), f(t)))).astype(np.float32)
    m = f(b1) * m + (f(1.0) - f(b1)) * g
    v = f(b2) * v + (f(1.0) - f(b2)) * g * g
    denom = np.sqrt(v) / bc2s + f(eps)
    p = p * (f(1.0) - f(lr) * f(wd))
    p = p - (f(lr) / bc1) * m / denom
    return p, m, v


def lr_schedule(schedule, base, min_lr, warmup, total, step_size, gamma, t):
    f = np.float32
    if min_lr < 0:
        min_lr = f(base) / f(10.0)                       # src/optim.c:165, float division
    if warmup > 0 and t < warmup:
        return f(f(base) * f(t + 1) / f(warmup))
    post = max(t - warmup, 0)
    if schedule in (1, 3):
        decay = total - warmup
        if decay <= 0:
            return f(base)
        c = f(0.5) * (f(1.0) + np.cos(f(np.pi) * f(post) / f(decay), dtype=np.float32))
        return f(f(min_lr) + (f(base) - f(min_lr)) * c)
    if schedule == 4:
        return f(base) if step_size <= 0 else f(f(base) * np.power(f(gamma), f(post // step_size)))
    if schedule == 5:
        return f(base) if post == 0 else f(f(base) * np.power(f(gamma), f(post)))
    return f(base)


# ── xorshift128+ / SplitMix64 (src/rng.c:6-66) ────────────────────────────
_M64 = (1 << 64) - 1


class Rng:
    def __init__(self, seed):
        def mix(z):
            z = (z + 0x9E3779B97F4A7C15) & _M64
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
            return z ^ (z >> 31)
        self.s0 = mix(seed)
        self.s1 = mix(self.s0)

    def next(self):
        s1, s0 = self.s0, self.s1
        self.s0 = s0
        s1 ^= (s1 << 23) & _M64
        self.s1 = s1 ^ s0 ^ (s1 >> 18) ^ (s0 >> 5)
        return (self.s1 + s0) & _M64

    def uniform(self):
        return np.float32(np.float32(self.next() >> 11) * np.float32(2.0 ** -53))

    def uniform_int(self, n):
        if n <= 1:
            return 0
        mask = n
        for sh in (1, 2, 4, 8, 16):
            mask |= mask >> sh
        while True:
            v = (self.next() >> 32) & mask
            if v < n:
                return int(v)


# ── decoder LM training step (src/transformer.c:151-201, src/gpt.c:66-216) ─
def lm_param_names(n_layers):
    names = ["embed.weight"]
    for i in range(n_layers):
        p = "blocks.%d." % i
        names += [p + s for s in ("qkv_proj.weight", "qkv_proj.bias", "out_proj.weight", "out_proj.bias",
                                  "attn_norm.weight", "ffn_norm.weight", "ffn.gate_proj.weight", "ffn.gate_proj.bias",
                                  "ffn.up_proj.weight", "ffn.up_proj.bias", "ffn.down_proj.weight", "ffn.down_proj.bias")]
    return names + ["norm.weight", "lm_head.bias"]


def lm_loss_and_grads(P, ids, targets, n_layers, n_heads, rope_base=10000.0, eps=1e-5,
                      mode=0, prefix_len=0, seq_lens=None, embeds=None, loss_slice=None, loss_mask=None):
    """Forward + backward of the decoder LM in float64.  P maps the names of
    lm_param_names() to arrays.  Returns (loss, {name: grad}).
    embeds: run from given input embeddings [B,S,D] instead of gathering ids
    (decoder_lm_forward_embeds_ex, src/gpt.c:95-122); their gradient is returned under "__embeds__"
    and the embedding table only gets the tied-head part.  loss_slice=(start, n): the loss reads
    logits[:, start:start+n] (src/vlm.c:262-268); loss_mask: cross_entropy_masked."""
    P = {k: v.astype(F64) for k, v in P.items()}
    E = P["embed.weight"]
    D = E.shape[1]
    if embeds is not None:
        x = np.asarray(embeds, F64)
        B, N = x.shape[:2]
    else:
        B, N = ids.shape
        x = E[ids]                                         # [B,N,D]
    dk = D // n_heads
    cos, sin = rope_tables(dk, N, rope_base)
    cos, sin = cos.astype(F64), sin.astype(F64)
    tape = []

    def rms_f(x, w):
        rs = 1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
        return x * rs * w, rs

    def rms_b(x, w, rs, g):
        dw = (g * x * rs).reshape(-1, D).sum(0)
        dy = g * w
        S = (dy * x).sum(-1, keepdims=True)
        return rs * dy - rs * (rs * rs / D * S) * x, dw

    def rot(t, inverse=False):
        s = -sin if inverse else sin
        out = np.empty_like(t)
        te, to = t[..., 0::2], t[..., 1::2]
        out[..., 0::2] = te * cos - to * s
        out[..., 1::2] = te * s + to * cos
        return out

    def heads(t):
        return t.reshape(B, N, n_heads, dk).transpose(0, 2, 1, 3)

    def unheads(t):
        return t.transpose(0, 2, 1, 3).reshape(B, N, D)

    allow = []
    for b in range(B):
        nb = N if seq_lens is None else int(seq_lens[b])
        a = np.zeros((N, N), bool)
        for i in range(nb):
            a[i, :visible_len(mode, i, prefix_len, nb)] = True
        allow.append(a)
    allow = np.stack(allow)[:, None]                       # [B,1,N,N]
    live = allow.any(-1, keepdims=True)
    scale = 1.0 / np.sqrt(np.float32(dk)).astype(F64)

    for i in range(n_layers):
        p = "blocks.%d." % i
        x0 = x
        h1, rs1 = rms_f(x0, P[p + "attn_norm.weight"])
        qkv = h1 @ P[p + "qkv_proj.weight"] + P[p + "qkv_proj.bias"]
        q, k, v = (heads(qkv[..., j * D:(j + 1) * D]) for j in range(3))
        q, k = rot(q), rot(k)
        S = np.where(allow, scale * (q @ k.transpose(0, 1, 3, 2)), -np.inf)
        S = np.where(live, S, 0.0)
        Pm = np.exp(S - S.max(-1, keepdims=True))
        Pm = np.where(allow, Pm, 0.0)
        den = Pm.sum(-1, keepdims=True)
        Pm = np.where(live, Pm / np.where(den == 0, 1.0, den), 0.0)
        att = Pm @ v
        merged = unheads(att)
        x1 = x0 + merged @ P[p + "out_proj.weight"] + P[p + "out_proj.bias"]
        h2, rs2 = rms_f(x1, P[p + "ffn_norm.weight"])
        gate = h2 @ P[p + "ffn.gate_proj.weight"] + P[p + "ffn.gate_proj.bias"]
        up = h2 @ P[p + "ffn.up_proj.weight"] + P[p + "ffn.up_proj.bias"]
        sg = 1.0 / (1.0 + np.exp(-gate))
        hid = gate * sg * up
        x = x1 + hid @ P[p + "ffn.down_proj.weight"] + P[p + "ffn.down_proj.bias"]
        tape.append((x0, h1, rs1, q, k, v, Pm, merged, x1, h2, rs2, gate, up, sg, hid))
    hf, rsf = rms_f(x, P["norm.weight"])
    logits = hf @ E.T + P["lm_head.bias"]                  # [B,N,V]
    if loss_slice is not None:
        s0, sn = loss_slice
        loss, dl = cross_entropy(logits[:, s0:s0 + sn], targets, loss_mask)
        dlogits = np.zeros(logits.shape, F64)
        dlogits[:, s0:s0 + sn] = dl
    elif targets.shape[1] == N - 1:                        # next-token loss on logits[:, :-1]
        loss, dl = cross_entropy(logits[:, :N - 1], targets)
        dlogits = np.zeros(logits.shape, F64)
        dlogits[:, :N - 1] = dl
    else:
        loss, dl = cross_entropy(logits, targets)
        dlogits = dl.astype(F64)

    G = {}
    G["lm_head.bias"] = dlogits.reshape(-1, E.shape[0]).sum(0)
    G["embed.weight"] = dlogits.reshape(-1, E.shape[0]).T @ hf.reshape(-1, D)
    dx, G["norm.weight"] = rms_b(x, P["norm.weight"], rsf, dlogits @ E)
    for i in reversed(range(n_layers)):
        p = "blocks.%d." % i
        x0, h1, rs1, q, k, v, Pm, merged, x1, h2, rs2, gate, up, sg, hid = tape[i]
        G[p + "ffn.down_proj.bias"] = dx.reshape(-1, D).sum(0)
        G[p + "ffn.down_proj.weight"] = hid.reshape(-1, hid.shape[-1]).T @ dx.reshape(-1, D)
        dhid = dx @ P[p + "ffn.down_proj.weight"].T
        dgate = dhid * (sg * (1.0 + gate - gate * sg)) * up
        dup = dhid * (gate * sg)
        F_ = gate.shape[-1]
        G[p + "ffn.gate_proj.bias"] = dgate.reshape(-1, F_).sum(0)
        G[p + "ffn.up_proj.bias"] = dup.reshape(-1, F_).sum(0)
        G[p + "ffn.gate_proj.weight"] = h2.reshape(-1, D).T @ dgate.reshape(-1, F_)
        G[p + "ffn.up_proj.weight"] = h2.reshape(-1, D).T @ dup.reshape(-1, F_)
        dh2 = dgate @ P[p + "ffn.gate_proj.weight"].T + dup @ P[p + "ffn.up_proj.weight"].T
        d1, G[p + "ffn_norm.weight"] = rms_b(x1, P[p + "ffn_norm.weight"], rs2, dh2)
        dx1 = dx + d1
        G[p + "out_proj.bias"] = dx1.reshape(-1, D).sum(0)
        G[p + "out_proj.weight"] = merged.reshape(-1, D).T @ dx1.reshape(-1, D)
        datt = heads(dx1 @ P[p + "out_proj.weight"].T)
        dv = Pm.transpose(0, 1, 3, 2) @ datt
        dP = datt @ v.transpose(0, 1, 3, 2)
        dS = Pm * (dP - (Pm * dP).sum(-1, keepdims=True)) * scale
        dq = rot(dS @ k, inverse=True)
        dk_ = rot(dS.transpose(0, 1, 3, 2) @ q, inverse=True)
        dqkv = np.concatenate([unheads(dq), unheads(dk_), unheads(dv)], axis=-1)
        G[p + "qkv_proj.bias"] = dqkv.reshape(-1, 3 * D).sum(0)
        G[p + "qkv_proj.weight"] = h1.reshape(-1, D).T @ dqkv.reshape(-1, 3 * D)
        d0, G[p + "attn_norm.weight"] = rms_b(x0, P[p + "attn_norm.weight"], rs1, dqkv @ P[p + "qkv_proj.weight"].T)
        dx = dx1 + d0
    if embeds is not None:
        G["__embeds__"] = dx
        return np.float32(loss), {k: (v if k == "__embeds__" else _f32(v)) for k, v in G.items()}
    dE = np.zeros(E.shape, F64)
    np.add.at(dE, ids.reshape(-1), dx.reshape(-1, D))
    G["embed.weight"] = G["embed.weight"] + dE
    return np.float32(loss), {k: _f32(v) for k, v in G.items()}


# ── prefix-LM vision LM, padded training step (src/vlm.c:150-381) ─────────
def vlm_param_names(n_layers):
    return ["patch_embed.weight", "patch_embed.bias", "img_proj.weight", "img_proj.bias"] + \
           ["lm." + n for n in lm_param_names(n_layers)] + ["image_pos"]


def vlm_loss_and_grads(P, images, input_ids, target_ids, loss_mask, text_lens, n_layers, n_heads, patch):
    """vision_lm_loss_padded + backward in float64 (src/vlm.c:303-346).  Image tokens come from the
    patch convolution, whose im2col path leaves (M, out_C) data in an NCHW-shaped tensor that the model
    then transposes as if it were NCHW (src/conv.c:847-863, src/vlm.c:176-185); conv2d() above keeps
    that memory layout.  img_proj.* are outside the graph for [B,C,H,W] images: no gradient (None)."""
    B, T = input_ids.shape
    w = P["patch_embed.weight"]
    Dm = w.shape[0]
    ph, pw = images.shape[2] // patch, images.shape[3] // patch
    I = ph * pw
    zero_g = np.zeros((B, Dm, ph, pw), np.float32)
    y, _, _, _ = conv2d(images, w, P["patch_embed.bias"], patch, 0, zero_g)
    img = np.ascontiguousarray(y.astype(F64).transpose(0, 2, 3, 1)).reshape(B, I, Dm)
    img = img + P["image_pos"].astype(F64)
    lmP = {k[3:]: v for k, v in P.items() if k.startswith("lm.")}
    txt = lmP["embed.weight"].astype(F64)[input_ids]
    embeds = np.concatenate([img, txt], axis=1)
    lens = np.array([I + min(int(n), T) for n in text_lens], np.int32)
    loss, G = lm_loss_and_grads(lmP, None, target_ids, n_layers, n_heads, mode=1, prefix_len=I, seq_lens=lens,
                                embeds=embeds, loss_slice=(I, T), loss_mask=loss_mask)
    de = G.pop("__embeds__")
    out = {"lm." + k: v for k, v in G.items()}
    dE = np.zeros(lmP["embed.weight"].shape, F64)
    np.add.at(dE, input_ids.reshape(-1), de[:, I:].reshape(-1, Dm))
    out["lm.embed.weight"] = _f32(out["lm.embed.weight"].astype(F64) + dE)
    dimg = de[:, :I]
    out["image_pos"] = _f32(dimg.sum(0, keepdims=True))
    g_nchw = np.ascontiguousarray(dimg.reshape(B, ph, pw, Dm).transpose(0, 3, 1, 2))
    _, _, dw, db = conv2d(images, w, P["patch_embed.bias"], patch, 0, _f32(g_nchw))
    # the convolution's own gradients are rounded to float32 on the way in (g_nchw); negligible at 1e-7
    out["patch_embed.weight"], out["patch_embed.bias"] = dw, db
    out["img_proj.weight"] = out["img_proj.bias"] = None
    return loss, out


# ── MNIST-shaped CNN step (examples/mnist/mnist_cnn_pool_model.c, mnist_train.c:99-114) ──
CNN_PARAM_NAMES = ["conv1.weight", "conv1.bias", "conv2.weight", "conv2.bias", "fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias"]


def cnn_loss_and_grads(P, x, labels, relu_on=None):
    """conv3x3(1->32) relu avgpool2 conv3x3(32->64) relu avgpool2 linear(3136->128) relu linear(128->10),
    cross entropy; composed from the operator restatements above (float64 inside every operator, float32
    between operators, as the library stores its activations).  x: [B, 784] or [B,1,28,28].
    relu_on: optional {"c1" | "c2" | "h1": bool array} -- which units of a ReLU are on, used in place of
    (pre-activation > 0) in forward and backward.  A ReLU is discontinuous in its derivative at zero, so two
    correct fp32 implementations may decide a unit whose pre-activation is zero to within rounding differently;
    a checker passes the decisions of the implementation under test for exactly those units.
    Returns (loss, grads, logits, pre) with pre = the three pre-activation arrays."""
    n = x.shape[0]
    x = x.reshape(n, 1, 28, 28).astype(np.float32)

    def on(name, pre):
        return (pre > 0) if relu_on is None or name not in relu_on else np.asarray(relu_on[name], bool).reshape(pre.shape)

    def fwd_conv(inp, w, b):
        oc = w.shape[0]
        return conv2d(inp, w, b, 1, 1, np.zeros((inp.shape[0], oc, inp.shape[2], inp.shape[3]), np.float32))[0]
    c1 = fwd_conv(x, P["conv1.weight"], P["conv1.bias"])
    m1 = on("c1", c1)
    r1 = np.where(m1, c1, np.float32(0))
    p1 = avg_pool2d(r1, 2, 2, np.zeros((n, 32, 14, 14), np.float32))[0]
    c2 = fwd_conv(p1, P["conv2.weight"], P["conv2.bias"])
    m2 = on("c2", c2)
    r2 = np.where(m2, c2, np.float32(0))
    p2 = avg_pool2d(r2, 2, 2, np.zeros((n, 64, 7, 7), np.float32))[0]
    flat = p2.reshape(n, 3136)
    h1 = matmul_add(flat, P["fc1.weight"], 0, P["fc1.bias"], np.zeros((n, 128), np.float32))[0]
    m3 = on("h1", h1)
    a1 = np.where(m3, h1, np.float32(0))
    logits = matmul_add(a1, P["fc2.weight"], 0, P["fc2.bias"], np.zeros((n, 10), np.float32))[0]
    loss, dlogits = cross_entropy(logits, labels)
    G = {}
    _, da1, G["fc2.weight"], G["fc2.bias"] = matmul_add(a1, P["fc2.weight"], 0, P["fc2.bias"], dlogits)
    dh1 = np.where(m3, da1, np.float32(0))
    _, dflat, G["fc1.weight"], G["fc1.bias"] = matmul_add(flat, P["fc1.weight"], 0, P["fc1.bias"], dh1)
    dr2 = avg_pool2d(r2, 2, 2, dflat.reshape(n, 64, 7, 7))[1]
    dc2 = np.where(m2, dr2, np.float32(0))
    _, dp1, G["conv2.weight"], G["conv2.bias"] = conv2d(p1, P["conv2.weight"], P["conv2.bias"], 1, 1, dc2)
    dr1 = avg_pool2d(r1, 2, 2, dp1)[1]
    dc1 = np.where(m1, dr1, np.float32(0))
    _, _, G["conv1.weight"], G["conv1.bias"] = conv2d(x, P["conv1.weight"], P["conv1.bias"], 1, 1, dc1)
    return np.float32(loss), G, logits, {"c1": c1, "c2": c2, "h1": h1}


# ── padded vision-LM batch assembly (src/imagenet_vlm.c:31-46, 598-647) ───
BOS_ID, EOS_ID, PAD_ID = 257, 258, 259          # include/tokenizer.h:23-25


def vlm_batch_text(texts, t_max):
    """Rows of a padded batch from stored token lists (no BOS; src/imagenet_vlm.c:612-629):
    input = BOS + text + PAD..., target = text + PAD..., mask = 1 on the first len(text) slots,
    text_lens = len(text) + 1.  Integer work: bit-exact."""
    n = len(texts)
    inp = np.full((n, t_max), PAD_ID, np.int32)
    tgt = np.full((n, t_max), PAD_ID, np.int32)
    mask = np.zeros((n, t_max), np.float32)
    lens = np.zeros(n, np.int32)
    for b, t in enumerate(texts):
        t = np.asarray(t, np.int32)
        assert len(t) + 1 <= t_max
        inp[b, 0] = BOS_ID
        inp[b, 1:1 + len(t)] = t
        tgt[b, :len(t)] = t
        mask[b, :len(t)] = 1.0
        lens[b] = len(t) + 1
    return inp, tgt, mask, lens


def vlm_batch_pixels(pixels_hwc, flips, mean, std):
    """uint8 [B,H,W,C] -> normalised float32 [B,C,H,W], optional horizontal flip per sample
    (convert_pixels, src/imagenet_vlm.c:31-46).  Each operation is rounded to fp32 on its own, as the
    reference's scalar code does, so the result is bit-exact."""
    px = np.asarray(pixels_hwc, np.uint8)
    out = np.empty((px.shape[0], px.shape[3], px.shape[1], px.shape[2]), np.float32)
    inv255 = np.float32(1.0) / np.float32(255.0)
    mean, std = np.asarray(mean, np.float32), np.asarray(std, np.float32)
    for b in range(px.shape[0]):
        src = px[b, :, ::-1, :] if flips[b] else px[b]
        val = src.astype(np.float32) * inv255
        out[b] = np.transpose(((val - mean) / std).astype(np.float32), (2, 0, 1))
    return out
