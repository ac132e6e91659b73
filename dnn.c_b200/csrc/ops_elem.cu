// Element-wise ops and their gradients: add (with broadcasting), cat, relu,
// silu, swiglu.  All are HBM-bound: contiguous operands move as float4 and one
// thread handles 4 elements per grid-stride step.
// replaces src/ops_elem.c:18-175,660-945 and src/ops_activation.c:14-333.
#include "common.cuh"
#include "device_utils.cuh"
#include <vector>
#include <cstdio>

namespace dnnb {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// Generic element-wise launcher: OP::apply on float4 lanes when every pointer is
// 16-byte aligned and n % 4 == 0, scalar otherwise.
template <typename F>
__global__ void ew_kernel(int64_t n, F f) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) f(i);
}
template <typename F>
static void ew_launch(const char *name, int64_t n, F f) {
    if (n <= 0) return;
    ew_kernel<<<grid_for(n, 256), 256, 0, stream()>>>(n, f);
    LAUNCHED(name);
}

// ---- add -------------------------------------------------------------------
struct AddV4 {
    float4 *o; const float4 *a, *b;
    __device__ void operator()(int64_t i) const {
        float4 x = a[i], y = b[i];
        o[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    }
};
struct Add1 {
    float *o; const float *a, *b;
    __device__ void operator()(int64_t i) const { o[i] = a[i] + b[i]; }
};
struct AddBias {   // o[i] = a[i] + b[i % C]
    float *o; const float *a, *b; int C;
    __device__ void operator()(int64_t i) const { o[i] = a[i] + b[i % C]; }
};
__device__ __forceinline__ int64_t voff(const View &v, int64_t flat) {
    int64_t off = v.offset;
#pragma unroll
    for (int d = DNN_MAX_DIMS - 1; d >= 0; d--)
        if (d < v.ndim) { int c = (int)(flat % v.shape[d]); flat /= v.shape[d]; off += (int64_t)c * v.strides[d]; }
    return off;
}
struct AddBcast {
    float *o; const float *a, *b; View va, vb;
    __device__ void operator()(int64_t i) const { o[i] = a[voff(va, i)] + b[voff(vb, i)]; }
};

// Gradient of a broadcast operand: every element of the operand sums the
// upstream gradient over the dims it was broadcast along, in index order, so
// the result is deterministic (the reference scatters serially,
// src/ops_elem.c:83-105).
struct BcastReduce {
    float *dst; const float *g; View dv; int out_ndim; int out_shape[DNN_MAX_DIMS]; int acc;
    int64_t n_dst;     // logical elements of the operand
    int t_ndim; int t_shape[DNN_MAX_DIMS]; int t_strides[DNN_MAX_DIMS]; int t_offset;
    __device__ void operator()(int64_t e) const {
        // coordinates of operand element e (in the operand's own shape)
        int tc[DNN_MAX_DIMS]; int64_t r = e; int64_t toff = t_offset;
        for (int d = t_ndim - 1; d >= 0; d--) { tc[d] = (int)(r % t_shape[d]); r /= t_shape[d]; toff += (int64_t)tc[d] * t_strides[d]; }
        int lead = out_ndim - t_ndim;
        // iterate over the broadcast extent
        int64_t bext = 1;
        for (int d = 0; d < out_ndim; d++) { int td = d - lead; if (td < 0 || (t_shape[td] == 1 && out_shape[d] != 1)) bext *= out_shape[d]; }
        float s = 0.f;
        for (int64_t bi = 0; bi < bext; bi++) {
            int64_t rem = bi, flat = 0, mul = 1;
            // build the flat output index, last dim fastest
            for (int d = out_ndim - 1; d >= 0; d--) {
                int td = d - lead; int c;
                if (td < 0 || (t_shape[td] == 1 && out_shape[d] != 1)) { c = (int)(rem % out_shape[d]); rem /= out_shape[d]; }
                else c = tc[td];
                flat += (int64_t)c * mul; mul *= out_shape[d];
            }
            s += g[flat];
        }
        dst[toff] = acc ? dst[toff] + s : s;
    }
};

static bool same_contig(const tensor *a, const tensor *b) {
    if (a->ndim != b->ndim || !a->contiguous || !b->contiguous) return false;
    for (int i = 0; i < a->ndim; i++) if (a->shape[i] != b->shape[i]) return false;
    return true;
}
static bool grad_contig(const tensor *t, const tensor *g) {
    if (t->ndim != g->ndim || !t->contiguous) return false;
    for (int i = 0; i < t->ndim; i++) if (t->shape[i] != g->shape[i]) return false;
    return true;
}
static bool lastdim_bias(const tensor *bias, const tensor *out) {
    return bias->ndim == 1 && out->ndim >= 2 && bias->shape[0] == out->shape[out->ndim - 1];
}

static void bcast_reduce_into(tensor *t, float *tg, const tensor *g, bool acc = true) {
    BcastReduce f;
    f.acc = acc ? 1 : 0;
    f.dst = tg; f.g = (const float *)g->data + g->offset; f.out_ndim = g->ndim;
    for (int d = 0; d < DNN_MAX_DIMS; d++) {
        f.out_shape[d] = d < g->ndim ? g->shape[d] : 1;
        f.t_shape[d] = d < t->ndim ? t->shape[d] : 1;
        f.t_strides[d] = d < t->ndim ? t->strides[d] : 0;
    }
    f.t_ndim = t->ndim; f.t_offset = t->offset; f.n_dst = numel_of(t);
    ew_launch("add_bcast_grad_kernel", f.n_dst, f);
}

static void add_backward(grad_fn *fn, tensor *g) {
    tensor *a = fn->inputs[0], *b = fn->inputs[1];
    int64_t n = numel_of(g);
    const float *gd = (const float *)g->data + g->offset;
    tensor *ops[2] = {a, b};
    for (tensor *t : ops) {
        if (!wants_grad(t)) continue;
        bool acc = true;
        float *tg = grad_full(t, &acc);        // each branch writes every element of t
        if (grad_contig(t, g)) { if (acc) k_axpy_acc(tg + t->offset, gd, n); else k_copy(tg + t->offset, gd, n); }
        else if (lastdim_bias(t, g)) k_colsum_acc(tg + t->offset, gd, n / t->shape[0], t->shape[0], acc);
        else bcast_reduce_into(t, tg, g, acc);
    }
}

// ---- cat --------------------------------------------------------------------
static void cat_backward(grad_fn *fn, tensor *g) {
    tensor *a = fn->inputs[0], *b = fn->inputs[1];
    int dim = *(int *)fn->saved_tensors[0];
    const float *gd = (const float *)g->data;
    // Each operand receives its slab of the upstream gradient; expressed as a
    // strided view of the upstream gradient gathered into / added onto the
    // operand's gradient (which follows the operand's own strides).
    tensor *ops[2] = {a, b};
    int start = 0;
    for (int k = 0; k < 2; k++) {
        tensor *t = ops[k];
        if (wants_grad(t)) {
            float *tg = _grad_ensure(t);
            // destination view: the operand's strides (the contiguous fast path
            // of the reference ignores the operand's offset, src/ops_elem.c:690-720)
            View dv = view_of(t);
            if (t->contiguous) dv.offset = 0;
            // source: slab [start, start + t->shape[dim]) of g along dim
            View sv = view_of(g);
            sv.shape[dim] = t->shape[dim];
            sv.offset = g->offset + start * g->strides[dim];
            int64_t n = numel_of(t);
            // dst[dv(i)] += src[sv(i)] : go through a packed temporary only when needed
            if (t->contiguous && dim == 0) {
                k_axpy_acc(tg + dv.offset, gd + sv.offset, n);
            } else {
                float *tmp = dev_alloc_t<float>(fn->pool, (size_t)n);
                k_gather(tmp, gd, sv, n);
                if (t->contiguous) k_axpy_acc(tg + dv.offset, tmp, n);
                else k_scatter(tg, dv, tmp, n, true);
            }
        }
        start += t->shape[dim];
    }
}

// ---- relu / silu / swiglu -----------------------------------------------------
struct ReluF  { float *o; const float *x; __device__ void operator()(int64_t i) const { float v = x[i]; o[i] = v > 0.f ? v : 0.f; } };
struct ReluF4 { float4 *o; const float4 *x; __device__ void operator()(int64_t i) const {
    float4 v = x[i]; o[i] = make_float4(v.x > 0.f ? v.x : 0.f, v.y > 0.f ? v.y : 0.f, v.z > 0.f ? v.z : 0.f, v.w > 0.f ? v.w : 0.f); } };
struct ReluB  { float *dx; const float *x, *g; int acc; __device__ void operator()(int64_t i) const {
    float d = acc ? dx[i] : 0.f; if (x[i] > 0.f) d += g[i]; dx[i] = d; } };
struct ReluB4 { float4 *dx; const float4 *x, *g; int acc; __device__ void operator()(int64_t i) const {
    float4 v = x[i], gg = g[i], d = acc ? dx[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    if (v.x > 0.f) d.x += gg.x; if (v.y > 0.f) d.y += gg.y; if (v.z > 0.f) d.z += gg.z; if (v.w > 0.f) d.w += gg.w; dx[i] = d; } };

struct SiluF { float *o; const float *x; __device__ void operator()(int64_t i) const { float v = x[i]; o[i] = v / (1.0f + expf(-v)); } };
struct SiluB { float *dx; const float *x, *g; int acc; __device__ void operator()(int64_t i) const {
    float v = x[i], s = sigmoidf_(v), r = s * (1.0f + v - v * s) * g[i]; dx[i] = acc ? dx[i] + r : r; } };
// the same with 128-bit accesses (same expressions per element, so the same bits)
__device__ __forceinline__ float silu1(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float silu_b1(float v, float g) { float s = sigmoidf_(v); return s * (1.0f + v - v * s) * g; }
struct SiluF4 { float4 *o; const float4 *x; __device__ void operator()(int64_t i) const {
    float4 v = x[i]; o[i] = make_float4(silu1(v.x), silu1(v.y), silu1(v.z), silu1(v.w)); } };
struct SiluB4 { float4 *dx; const float4 *x, *g; int acc; __device__ void operator()(int64_t i) const {
    float4 v = x[i], gg = g[i], d = acc ? dx[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 r = make_float4(silu_b1(v.x, gg.x), silu_b1(v.y, gg.y), silu_b1(v.z, gg.z), silu_b1(v.w, gg.w));
    dx[i] = acc ? make_float4(d.x + r.x, d.y + r.y, d.z + r.z, d.w + r.w) : r; } };

__device__ __forceinline__ float swiglu1(float g, float u) { return (g / (1.0f + expf(-g))) * u; }
struct SwigluF  { float *o; const float *g, *u; __device__ void operator()(int64_t i) const { o[i] = swiglu1(g[i], u[i]); } };
struct SwigluF4 { float4 *o; const float4 *g, *u; __device__ void operator()(int64_t i) const {
    float4 a = g[i], b = u[i]; o[i] = make_float4(swiglu1(a.x, b.x), swiglu1(a.y, b.y), swiglu1(a.z, b.z), swiglu1(a.w, b.w)); } };
__device__ __forceinline__ void swiglu_b1(float gate, float up, float go, float &dg, float &du) {
    float s = sigmoidf_(gate);
    dg += go * (s * (1.0f + gate - gate * s)) * up;
    du += go * (gate * s);
}
struct SwigluB  { float *dg, *du; const float *g, *u, *go; int acc_g, acc_u; __device__ void operator()(int64_t i) const {
    float a = 0.f, b = 0.f; swiglu_b1(g[i], u[i], go[i], a, b);
    if (dg) dg[i] = acc_g ? dg[i] + a : a; if (du) du[i] = acc_u ? du[i] + b : b; } };
struct SwigluB4 { float4 *dg, *du; const float4 *g, *u, *go; int acc_g, acc_u; __device__ void operator()(int64_t i) const {
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 a = g[i], b = u[i], o = go[i], x = acc_g ? dg[i] : z, y = acc_u ? du[i] : z;
    swiglu_b1(a.x, b.x, o.x, x.x, y.x); swiglu_b1(a.y, b.y, o.y, x.y, y.y);
    swiglu_b1(a.z, b.z, o.z, x.z, y.z); swiglu_b1(a.w, b.w, o.w, x.w, y.w);
    dg[i] = x; du[i] = y; } };
struct SwigluBcast { float *o; const float *g, *u; View vg, vu;
    __device__ void operator()(int64_t i) const { o[i] = swiglu1(g[voff(vg, i)], u[voff(vu, i)]); } };

// SwiGLU backward for packed [rows, C] operands with fresh gradient buffers: a CTA owns 128 columns
// and a slab of rows, stores d(gate) and d(up) and keeps their running column sums, which end up
// in part_g / part_u [slab][C].  The consumers of the two gradients are linear layers whose bias
// gradients are exactly these sums, so the separate pass over each buffer disappears.
__global__ void __launch_bounds__(256)
swiglu_bwd_colsum_kernel(const float *__restrict__ gate, const float *__restrict__ up, const float *__restrict__ go,
                         float *__restrict__ dgate, float *__restrict__ dup, float *__restrict__ part_g, float *__restrict__ part_u,
                         int64_t rows, int C, int rows_per) {
    __shared__ float4 tile[2][8][33];
    const int c = (blockIdx.x * 32 + threadIdx.x) * 4;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per;
    int64_t r1 = r0 + rows_per; if (r1 > rows) r1 = rows;
    float4 sg = make_float4(0.f, 0.f, 0.f, 0.f), su = sg;
    if (c < C) {
#pragma unroll 2
        for (int64_t r = r0 + threadIdx.y; r < r1; r += 8) {
            const int64_t i = r * C + c;
            const float4 a = *reinterpret_cast<const float4 *>(gate + i), b = *reinterpret_cast<const float4 *>(up + i),
                         o = *reinterpret_cast<const float4 *>(go + i);
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f), y = x;
            swiglu_b1(a.x, b.x, o.x, x.x, y.x); swiglu_b1(a.y, b.y, o.y, x.y, y.y);
            swiglu_b1(a.z, b.z, o.z, x.z, y.z); swiglu_b1(a.w, b.w, o.w, x.w, y.w);
            *reinterpret_cast<float4 *>(dgate + i) = x;
            *reinterpret_cast<float4 *>(dup + i) = y;
            sg.x += x.x; sg.y += x.y; sg.z += x.z; sg.w += x.w;
            su.x += y.x; su.y += y.y; su.z += y.z; su.w += y.w;
        }
    }
    tile[0][threadIdx.y][threadIdx.x] = sg;
    tile[1][threadIdx.y][threadIdx.x] = su;
    __syncthreads();
    if (threadIdx.y < 2 && c < C) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; j++) { float4 v = tile[threadIdx.y][j][threadIdx.x]; t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w; }
        *reinterpret_cast<float4 *>((threadIdx.y ? part_u : part_g) + (int64_t)blockIdx.y * C + c) = t;
    }
}

static bool v4ok(int64_t n, std::initializer_list<const void *> ps) {
    if (n % 4) return false;
    for (auto p : ps) if (p && !aligned16(p)) return false;
    return true;
}

static void relu_backward(grad_fn *fn, tensor *g) {
    tensor *a = fn->inputs[0];
    if (!wants_grad(a)) return;
    int64_t n = numel_of(a);
    bool acc = true;
    float *ag = grad_full(a, &acc);
    const float *gd = (const float *)g->data;
    if (a->contiguous) {
        float *dx = ag + a->offset; const float *x = (const float *)a->data + a->offset;
        prof_work((acc ? 16.0 : 12.0) * n);                     // read x, g (and dx when accumulating), write dx
        if (v4ok(n, {dx, x, gd})) ew_launch("relu_bwd_kernel", n / 4, ReluB4{(float4 *)dx, (const float4 *)x, (const float4 *)gd, acc});
        else ew_launch("relu_bwd_kernel", n, ReluB{dx, x, gd, acc});
    } else {
        float *xt = dev_alloc_t<float>(fn->pool, (size_t)n), *dt = dev_alloc_t<float>(fn->pool, (size_t)n);
        k_gather(xt, (const float *)a->data, view_of(a), n);
        ew_launch("relu_bwd_kernel", n, ReluB{dt, xt, gd, 0});
        k_scatter(ag, view_of(a), dt, n, true);
    }
}

static void silu_backward(grad_fn *fn, tensor *g) {
    tensor *a = fn->inputs[0];
    if (!wants_grad(a)) return;
    int64_t n = numel_of(a);
    bool acc = true;
    float *ag = grad_full(a, &acc);
    const float *gd = (const float *)g->data;
    if (a->contiguous) {
        prof_work((acc ? 16.0 : 12.0) * n);
        float *dx = ag + a->offset;
        const float *x = (const float *)a->data + a->offset;
        if (v4ok(n, {dx, x, gd})) ew_launch("silu_bwd_kernel", n / 4, SiluB4{(float4 *)dx, (const float4 *)x, (const float4 *)gd, acc});
        else ew_launch("silu_bwd_kernel", n, SiluB{dx, x, gd, acc});
    } else {
        float *xt = dev_alloc_t<float>(fn->pool, (size_t)n), *dt = dev_alloc_t<float>(fn->pool, (size_t)n);
        k_gather(xt, (const float *)a->data, view_of(a), n);
        ew_launch("silu_bwd_kernel", n, SiluB{dt, xt, gd, 0});
        k_scatter(ag, view_of(a), dt, n, true);
    }
}

static void swiglu_backward(grad_fn *fn, tensor *go) {
    tensor *gate = fn->inputs[0], *up = fn->inputs[1];
    int64_t n = numel_of(go);
    const float *god = (const float *)go->data + go->offset;
    bool ng = wants_grad(gate), nu = wants_grad(up);
    bool acc_g = true, acc_u = true;
    float *ag = ng ? grad_full(gate, &acc_g) : nullptr, *bg = nu ? grad_full(up, &acc_u) : nullptr;
    if (gate == up) acc_u = true;            // same buffer: the second write must add
    if (grad_contig(gate, go) && grad_contig(up, go)) {
        float *dg = ag ? ag + gate->offset : nullptr, *du = bg ? bg + up->offset : nullptr;
        const float *g = (const float *)gate->data + gate->offset, *u = (const float *)up->data + up->offset;
        const int C = go->shape[go->ndim - 1];
        const int64_t rows = C > 0 ? n / C : 0;
        // both buffers fresh and whole: the tiled kernel that also leaves the column sums of d(gate) and d(up)
        if (dg && du && dg != du && !acc_g && !acc_u && gate->offset == 0 && up->offset == 0 && C % 4 == 0 && C >= 128 && rows >= 256 &&
            v4ok(n, {dg, du, g, u, god})) {
            // one wave: 8 CTAs of 256 threads per SM, column groups x row slabs
            const int col_groups = (C / 4 + 31) / 32;
            int nslabs = kNumSMs * 8 / col_groups;
            if (nslabs < 1) nslabs = 1;
            if ((int64_t)nslabs * 32 > rows) nslabs = (int)(rows / 32);
            int per = (int)((rows + nslabs - 1) / nslabs);
            nslabs = (int)((rows + per - 1) / per);
            float *pg = dev_alloc_t<float>(fn->pool, (size_t)nslabs * C), *pu = dev_alloc_t<float>(fn->pool, (size_t)nslabs * C);
            dim3 grid((C / 4 + 31) / 32, nslabs), block(32, 8);
            swiglu_bwd_colsum_kernel<<<grid, block, 0, stream()>>>(g, u, god, dg, du, pg, pu, rows, C, per);
            prof_work(20.0 * rows * C);                          // read gate, up, d(out); write d(gate), d(up)
            LAUNCHED("swiglu_bwd_kernel");
            float *sums_g = colsum_cache_reserve(C);
            colsum_cache_publish(dg, rows, C);
            float *sums_u = colsum_cache_reserve(C);
            colsum_cache_publish(du, rows, C);
            k_colsum_finish2(sums_g, pg, sums_u, pu, nslabs, C);
            return;
        }
        if (dg && du && dg != du && v4ok(n, {dg, du, g, u, god}))
            ew_launch("swiglu_bwd_kernel", n / 4, SwigluB4{(float4 *)dg, (float4 *)du, (const float4 *)g, (const float4 *)u, (const float4 *)god, acc_g, acc_u});
        else
            ew_launch("swiglu_bwd_kernel", n, SwigluB{dg, du, g, u, god, acc_g, acc_u});
        return;
    }
    // Broadcast operands: expand to the output shape, differentiate there, then
    // reduce each operand's gradient over its broadcast dims.
    float *ge = dev_alloc_t<float>(fn->pool, (size_t)n), *ue = dev_alloc_t<float>(fn->pool, (size_t)n);
    float *dge = dev_alloc_t<float>(fn->pool, (size_t)n, true), *due = dev_alloc_t<float>(fn->pool, (size_t)n, true);
    k_gather(ge, (const float *)gate->data, bcast_view(gate, go->ndim, go->shape), n);
    k_gather(ue, (const float *)up->data, bcast_view(up, go->ndim, go->shape), n);
    ew_launch("swiglu_bwd_kernel", n, SwigluB{dge, due, ge, ue, god, 1, 1});
    tensor tmp = *go;
    if (ag) { tmp.data = dge; tmp.offset = 0; bcast_reduce_into(gate, ag, &tmp, acc_g); }
    if (bg) { tmp.data = due; tmp.offset = 0; bcast_reduce_into(up, bg, &tmp, acc_u); }
}


// ══════════ the rest of the element-wise / reduction surface of ops.h ══════════
// sub, mul, div (broadcasting), neg, pow, sigmoid, sum, mean, softmax, causal_softmax, dropout,
// triu.  None of them is on the training path of the models; they are simple, correct, HBM-bound
// kernels that keep the reference's semantics (src/ops_elem.c:178-680, src/ops_reduce.c,
// src/ops_activation.c:70-130,300-800,1410-1500).

enum { BIN_SUB = 0, BIN_MUL = 1, BIN_DIV = 2 };
struct BinF {
    float *o; const float *a, *b; View va, vb; int op;
    __device__ void operator()(int64_t i) const {
        float x = a[voff(va, i)], y = b[voff(vb, i)];
        o[i] = op == BIN_SUB ? x - y : op == BIN_MUL ? x * y : x / y;
    }
};
// per-element operand gradients in the OUTPUT shape (reduced over broadcast dims afterwards)
struct BinB {
    float *da, *db; const float *a, *b, *g; View va, vb; int op;
    __device__ void operator()(int64_t i) const {
        float x = a[voff(va, i)], y = b[voff(vb, i)], gg = g[i];
        if (op == BIN_SUB) { if (da) da[i] = gg; if (db) db[i] = -gg; }
        else if (op == BIN_MUL) { if (da) da[i] = y * gg; if (db) db[i] = x * gg; }
        else { if (da) da[i] = (1.0f / y) * gg; if (db) db[i] = (-x / (y * y)) * gg; }
    }
};

template <int OP>
static void binary_backward(grad_fn *fn, tensor *go) {
    tensor *a = fn->inputs[0], *b = fn->inputs[1];
    if ((OP == BIN_SUB || OP == BIN_DIV) && a == b) {          // d(a-a) = d(a/a) = 0 (src/ops_elem.c:183-188,395-399)
        if (a->requires_grad && !a->grad_fn) _grad_ensure(a);
        return;
    }
    int64_t n = numel_of(go);
    const float *gd = (const float *)go->data + go->offset;
    bool na = wants_grad(a), nb = wants_grad(b);
    if (!na && !nb) return;
    float *dae = na ? dev_alloc_t<float>(fn->pool, (size_t)n) : nullptr, *dbe = nb ? dev_alloc_t<float>(fn->pool, (size_t)n) : nullptr;
    ew_launch("binary_bwd_kernel", n, BinB{dae, dbe, (const float *)a->data, (const float *)b->data, gd,
                                           bcast_view(a, go->ndim, go->shape), bcast_view(b, go->ndim, go->shape), OP});
    tensor tmp = *go;
    tmp.offset = 0;
    tensor *ops[2] = {a, b}; float *parts[2] = {dae, dbe};
    for (int k = 0; k < 2; k++) {
        if (!parts[k]) continue;
        tensor *t = ops[k];
        float *tg = _grad_ensure(t);
        tmp.data = parts[k];
        if (grad_contig(t, go)) k_axpy_acc(tg + t->offset, parts[k], n);
        else bcast_reduce_into(t, tg, &tmp, true);
    }
}

template <int OP>
static tensor *binary_forward(struct mem_pool *scratch, const tensor *a, const tensor *b, const char *name) {
    require_device_payloads(name, {a, b});
    DNN_CHECK(a && b, "binary op: NULL operand");
    int shape[DNN_MAX_DIMS];
    int nd = bcast_shape(a->ndim, a->shape, b->ndim, b->shape, shape);
    if (nd <= 0) { fprintf(stderr, "%s: incompatible shapes\n", name); abort(); }
    tensor *out = tensor_scratch(scratch, nd, shape, 0);
    ew_launch("binary_fwd_kernel", numel_of(out), BinF{(float *)out->data, (const float *)a->data, (const float *)b->data,
                                                       bcast_view(a, nd, shape), bcast_view(b, nd, shape), OP});
    if (dnn_grad_enabled() && (a->requires_grad || b->requires_grad)) {
        grad_fn *fn = attach(scratch, out, binary_backward<OP>, 2, 0);
        fn->inputs[0] = (tensor *)a; fn->inputs[1] = (tensor *)b;
    }
    return out;
}

// ---- unary: neg, pow, sigmoid ----
enum { UN_NEG = 0, UN_POW = 1, UN_SIGMOID = 2 };
struct UnF { float *o; const float *x; View vx; int op; float e;
    __device__ void operator()(int64_t i) const {
        float v = x[voff(vx, i)];
        o[i] = op == UN_NEG ? -v : op == UN_POW ? powf(v, e) : 1.0f / (1.0f + expf(-v));
    } };
// dx[view(i)] += f'(.) * g[i]; `y` is the saved output for sigmoid
struct UnB { float *dx; const float *x, *y, *g; View vx; int op; float e;
    __device__ void operator()(int64_t i) const {
        int64_t o = voff(vx, i);
        float d;
        if (op == UN_NEG) d = -g[i];
        else if (op == UN_POW) d = e * powf(x[o], e - 1.0f) * g[i];
        else { float sg = y[i]; d = sg * (1.0f - sg) * g[i]; }
        dx[o] += d;
    } };
struct UnSaved { int op; float e; tensor *out; };
static void unary_backward(grad_fn *fn, tensor *go) {
    tensor *a = fn->inputs[0];
    if (!wants_grad(a)) return;
    UnSaved *sv = (UnSaved *)fn->saved_tensors[0];
    float *ag = _grad_ensure(a);
    // a view whose elements alias (broadcast strides) would race on +=; views of this library never do
    ew_launch("unary_bwd_kernel", numel_of(a), UnB{ag, (const float *)a->data, sv->out ? (const float *)sv->out->data : nullptr,
                                                   (const float *)go->data + go->offset, view_of(a), sv->op, sv->e});
}
static tensor *unary_forward(struct mem_pool *scratch, const tensor *t, int op, float e) {
    require_device_payloads("unary op", {t});
    DNN_CHECK(t, "unary op: NULL input");
    tensor *out = tensor_scratch(scratch, t->ndim, t->shape, 0);
    ew_launch("unary_fwd_kernel", numel_of(t), UnF{(float *)out->data, (const float *)t->data, view_of(t), op, e});
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, out, unary_backward, 1, 1);
        fn->inputs[0] = (tensor *)t;
        UnSaved *sv = host_alloc_t<UnSaved>(scratch);
        sv->op = op; sv->e = e; sv->out = op == UN_SIGMOID ? out : nullptr;
        fn->saved_tensors[0] = (tensor *)sv;
    }
    return out;
}

// ---- sum over one dim (keepdim) ----
// input viewed as [outer, D, inner] (through the view for non-contiguous inputs); one thread per output
struct SumF { float *o; const float *x; View vx; int D; int64_t inner;
    __device__ void operator()(int64_t i) const {
        int64_t oi = i / inner, in = i - oi * inner;
        float s = 0.f;
        for (int k = 0; k < D; k++) s += x[voff(vx, (oi * D + k) * inner + in)];
        o[i] = s;
    } };
struct SumB { float *dx; const float *g; View vx; int D; int64_t inner;
    __device__ void operator()(int64_t i) const {          // i over the INPUT elements
        int64_t oi = i / (D * inner), in = i % inner;
        dx[voff(vx, i)] += g[oi * inner + in];
    } };
static void sum_backward(grad_fn *fn, tensor *go) {
    tensor *t = fn->inputs[0];
    if (!wants_grad(t)) return;
    int dim = *(int *)fn->saved_tensors[0];
    int64_t inner = 1;
    for (int d = dim + 1; d < t->ndim; d++) inner *= t->shape[d];
    float *tg = _grad_ensure(t);
    ew_launch("sum_bwd_kernel", numel_of(t), SumB{tg, (const float *)go->data + go->offset, view_of(t), t->shape[dim], inner});
}

// ---- softmax over one dim / causal softmax over the last dim ----
// one warp per slice; a slice is D elements `inner` apart in the packed [outer, D, inner] input
__global__ void softmax_fwd_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t slices, int D, int64_t inner, int causal_n) {
    int lane = threadIdx.x & 31;
    int64_t s = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (s >= slices) return;
    int64_t oi = s / inner, in = s - oi * inner;
    const float *xs = x + oi * D * inner + in;
    float *ys = y + oi * D * inner + in;
    int len = causal_n ? (int)(s % causal_n) + 1 : D;          // causal: row i sees columns 0..i
    float m = -INFINITY;
    for (int k = lane; k < len; k += 32) m = fmaxf(m, xs[k * inner]);
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
    for (int k = lane; k < len; k += 32) sum += expf(xs[k * inner] - m);
    sum = warp_sum(sum);
    for (int k = lane; k < D; k += 32) ys[k * inner] = k < len ? expf(xs[k * inner] - m) / sum : 0.f;
}
// dx = y * (g - sum(y*g)) over the slice
__global__ void softmax_bwd_kernel(const float *__restrict__ y, const float *__restrict__ g, float *__restrict__ d,
                                   int64_t slices, int D, int64_t inner, int causal_n) {
    int lane = threadIdx.x & 31;
    int64_t s = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (s >= slices) return;
    int64_t oi = s / inner, in = s - oi * inner, base = oi * D * inner + in;
    int len = causal_n ? (int)(s % causal_n) + 1 : D;
    float dot = 0.f;
    for (int k = lane; k < len; k += 32) dot += y[base + k * inner] * g[base + k * inner];
    dot = warp_sum(dot);
    for (int k = lane; k < D; k += 32) d[base + k * inner] = k < len ? y[base + k * inner] * (g[base + k * inner] - dot) : 0.f;
}
struct SoftSaved { tensor *out; int dim; int causal_n; };
static void softmax_backward(grad_fn *fn, tensor *go) {
    tensor *a = fn->inputs[0];
    if (!wants_grad(a)) return;
    SoftSaved *sv = (SoftSaved *)fn->saved_tensors[0];
    int64_t n = numel_of(a), inner = 1;
    for (int d = sv->dim + 1; d < a->ndim; d++) inner *= a->shape[d];
    int D = a->shape[sv->dim];
    int64_t slices = n / D;
    float *d = dev_alloc_t<float>(fn->pool, (size_t)n);
    softmax_bwd_kernel<<<(unsigned)((slices + 7) / 8), 256, 0, stream()>>>((const float *)sv->out->data, (const float *)go->data + go->offset, d,
                                                                          slices, D, inner, sv->causal_n);
    LAUNCHED("softmax_bwd_kernel");
    float *ag = _grad_ensure(a);
    if (a->contiguous) k_axpy_acc(ag + a->offset, d, n);
    else k_scatter(ag, view_of(a), d, n, true);
}
static tensor *softmax_forward(struct mem_pool *scratch, const tensor *t, int dim, int causal_n) {
    tensor *out = tensor_scratch(scratch, t->ndim, t->shape, 0);
    int64_t n = numel_of(t), inner = 1;
    for (int d = dim + 1; d < t->ndim; d++) inner *= t->shape[d];
    int D = t->shape[dim];
    int64_t slices = D > 0 ? n / D : 0;
    const float *x = (const float *)t->data + t->offset;
    if (!t->contiguous) {
        float *tmp = dev_alloc_t<float>(scratch, (size_t)n);
        k_gather(tmp, (const float *)t->data, view_of(t), n);
        x = tmp;
    }
    if (slices > 0) {
        softmax_fwd_kernel<<<(unsigned)((slices + 7) / 8), 256, 0, stream()>>>(x, (float *)out->data, slices, D, inner, causal_n);
        LAUNCHED("softmax_fwd_kernel");
    }
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, out, softmax_backward, 1, 1);
        fn->inputs[0] = (tensor *)t;
        SoftSaved *sv = host_alloc_t<SoftSaved>(scratch);
        sv->out = out; sv->dim = dim; sv->causal_n = causal_n;
        fn->saved_tensors[0] = (tensor *)sv;
    }
    return out;
}

// ---- dropout: the keep mask comes from the host generator in element order, as in the reference ----
struct DropF { float *o; const float *x, *mask; View vx; float scale;
    __device__ void operator()(int64_t i) const { o[i] = mask[i] * x[voff(vx, i)] * scale; } };
struct DropB { float *dx; const float *g, *mask; View vx; float scale;
    __device__ void operator()(int64_t i) const { dx[voff(vx, i)] += g[i] * mask[i] * scale; } };
struct DropSaved { const float *mask; float scale; };
static void dropout_backward(grad_fn *fn, tensor *go) {
    tensor *a = fn->inputs[0];
    if (!a->requires_grad) return;
    DropSaved *sv = (DropSaved *)fn->saved_tensors[0];
    float *ag = _grad_ensure(a);
    ew_launch("dropout_bwd_kernel", numel_of(a), DropB{ag, (const float *)go->data + go->offset, sv->mask, view_of(a), sv->scale});
}

struct TriuF { float *o; int N, diag;
    __device__ void operator()(int64_t i) const { int r = (int)(i / N), c = (int)(i - (int64_t)r * N); o[i] = c >= r + diag ? -INFINITY : 0.0f; } };

}  // namespace dnnb

using namespace dnnb;

extern "C" {

tensor *tensor_add(struct mem_pool *scratch, const tensor *a, const tensor *b) {
    require_device_payloads("tensor_add", {a, b});
    DNN_CHECK(a && b, "tensor_add: NULL operand");
    int shape[DNN_MAX_DIMS];
    int nd = bcast_shape(a->ndim, a->shape, b->ndim, b->shape, shape);
    DNN_CHECK(nd > 0, "tensor_add: incompatible shapes");
    tensor *out = tensor_scratch(scratch, nd, shape, 0);
    int64_t n = numel_of(out);
    float *od = (float *)out->data;
    const float *af = (const float *)a->data + a->offset, *bf = (const float *)b->data + b->offset;
    if (same_contig(a, b)) {
        prof_work(12.0 * n);
        if (v4ok(n, {od, af, bf})) ew_launch("add_kernel", n / 4, AddV4{(float4 *)od, (const float4 *)af, (const float4 *)bf});
        else ew_launch("add_kernel", n, Add1{od, af, bf});
    } else if (a->contiguous && lastdim_bias(b, out) && numel_of(a) == n) {
        ew_launch("add_bias_kernel", n, AddBias{od, af, bf, b->shape[0]});
    } else if (lastdim_bias(a, out) && b->contiguous && numel_of(b) == n) {
        ew_launch("add_bias_kernel", n, AddBias{od, bf, af, a->shape[0]});
    } else {
        ew_launch("add_bcast_kernel", n, AddBcast{od, (const float *)a->data, (const float *)b->data,
                                                   bcast_view(a, nd, shape), bcast_view(b, nd, shape)});
    }
    if (dnn_grad_enabled() && (a->requires_grad || b->requires_grad)) {
        grad_fn *fn = attach(scratch, out, add_backward, 2, 0);
        fn->inputs[0] = (tensor *)a; fn->inputs[1] = (tensor *)b;
    }
    return out;
}

tensor *tensor_cat(struct mem_pool *scratch, const tensor *a, const tensor *b, int dim) {
    require_device_payloads("tensor_cat", {a, b});
    DNN_CHECK(a && b && a->ndim == b->ndim, "tensor_cat: ndim must match");
    int nd = a->ndim;
    if (dim < 0) dim += nd;
    DNN_CHECK(dim >= 0 && dim < nd, "tensor_cat: dim out of range");
    int shape[DNN_MAX_DIMS];
    for (int d = 0; d < nd; d++) {
        if (d != dim) DNN_CHECK(a->shape[d] == b->shape[d], "tensor_cat: shape mismatch");
        shape[d] = a->shape[d];
    }
    shape[dim] = a->shape[dim] + b->shape[dim];
    tensor *out = tensor_scratch(scratch, nd, shape, 0);
    const tensor *ops[2] = {a, b};
    int start = 0;
    for (int k = 0; k < 2; k++) {
        const tensor *t = ops[k];
        int64_t n = numel_of(t);
        View dv = view_of(out);
        dv.shape[dim] = t->shape[dim];
        dv.offset = start * out->strides[dim];
        if (t->contiguous) {
            k_scatter((float *)out->data, dv, (const float *)t->data + t->offset, n, false);
        } else {
            float *tmp = dev_alloc_t<float>(scratch, (size_t)n);
            k_gather(tmp, (const float *)t->data, view_of(t), n);
            k_scatter((float *)out->data, dv, tmp, n, false);
        }
        start += t->shape[dim];
    }
    if (dnn_grad_enabled() && (a->requires_grad || b->requires_grad)) {
        grad_fn *fn = attach(scratch, out, cat_backward, 2, 1);
        fn->inputs[0] = (tensor *)a; fn->inputs[1] = (tensor *)b;
        int *sd = host_alloc_t<int>(scratch); *sd = dim;
        fn->saved_tensors[0] = (tensor *)sd;
    }
    return out;
}

tensor *tensor_relu(struct mem_pool *scratch, const tensor *t) {
    require_device_payloads("tensor_relu", {t});
    DNN_CHECK(t, "tensor_relu: NULL input");
    tensor *out = tensor_scratch(scratch, t->ndim, t->shape, 0);
    int64_t n = numel_of(t);
    const float *x = (const float *)t->data + t->offset;
    if (!t->contiguous) {
        float *tmp = dev_alloc_t<float>(scratch, (size_t)n);
        k_gather(tmp, (const float *)t->data, view_of(t), n);
        x = tmp;
    }
    float *od = (float *)out->data;
    prof_work(8.0 * n);
    if (v4ok(n, {od, x})) ew_launch("relu_fwd_kernel", n / 4, ReluF4{(float4 *)od, (const float4 *)x});
    else ew_launch("relu_fwd_kernel", n, ReluF{od, x});
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, out, relu_backward, 1, 0);
        fn->inputs[0] = (tensor *)t;
    }
    return out;
}

tensor *tensor_silu(struct mem_pool *scratch, const tensor *t) {
    require_device_payloads("tensor_silu", {t});
    DNN_CHECK(t, "tensor_silu: NULL input");
    tensor *out = tensor_scratch(scratch, t->ndim, t->shape, 0);
    int64_t n = numel_of(t);
    const float *x = (const float *)t->data + t->offset;
    if (!t->contiguous) {
        float *tmp = dev_alloc_t<float>(scratch, (size_t)n);
        k_gather(tmp, (const float *)t->data, view_of(t), n);
        x = tmp;
    }
    prof_work(8.0 * n);
    if (v4ok(n, {(float *)out->data, x})) ew_launch("silu_fwd_kernel", n / 4, SiluF4{(float4 *)out->data, (const float4 *)x});
    else ew_launch("silu_fwd_kernel", n, SiluF{(float *)out->data, x});
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, out, silu_backward, 1, 0);
        fn->inputs[0] = (tensor *)t;
    }
    return out;
}

tensor *tensor_swiglu(struct mem_pool *scratch, const tensor *gate, const tensor *up) {
    require_device_payloads("tensor_swiglu", {gate, up});
    DNN_CHECK(gate && up, "tensor_swiglu: NULL operand");
    int shape[DNN_MAX_DIMS];
    int nd = bcast_shape(gate->ndim, gate->shape, up->ndim, up->shape, shape);
    DNN_CHECK(nd > 0, "tensor_swiglu: incompatible shapes");
    tensor *out = tensor_scratch(scratch, nd, shape, 0);
    int64_t n = numel_of(out);
    float *od = (float *)out->data;
    if (same_contig(gate, up)) {
        const float *g = (const float *)gate->data + gate->offset, *u = (const float *)up->data + up->offset;
        prof_work(12.0 * n);
        if (v4ok(n, {od, g, u})) ew_launch("swiglu_fwd_kernel", n / 4, SwigluF4{(float4 *)od, (const float4 *)g, (const float4 *)u});
        else ew_launch("swiglu_fwd_kernel", n, SwigluF{od, g, u});
    } else {
        ew_launch("swiglu_fwd_kernel", n, SwigluBcast{od, (const float *)gate->data, (const float *)up->data,
                                                      bcast_view(gate, nd, shape), bcast_view(up, nd, shape)});
    }
    if (dnn_grad_enabled() && (gate->requires_grad || up->requires_grad)) {
        grad_fn *fn = attach(scratch, out, swiglu_backward, 2, 0);
        fn->inputs[0] = (tensor *)gate; fn->inputs[1] = (tensor *)up;
    }
    return out;
}

tensor *tensor_sub(struct mem_pool *scratch, const tensor *a, const tensor *b) { return binary_forward<BIN_SUB>(scratch, a, b, "tensor_sub"); }
tensor *tensor_mul(struct mem_pool *scratch, const tensor *a, const tensor *b) { return binary_forward<BIN_MUL>(scratch, a, b, "tensor_mul"); }
tensor *tensor_div(struct mem_pool *scratch, const tensor *a, const tensor *b) { return binary_forward<BIN_DIV>(scratch, a, b, "tensor_div"); }
tensor *tensor_neg(struct mem_pool *scratch, const tensor *t) { return unary_forward(scratch, t, UN_NEG, 0.f); }
tensor *tensor_pow(struct mem_pool *scratch, const tensor *t, float exp) { return unary_forward(scratch, t, UN_POW, exp); }
tensor *tensor_sigmoid(struct mem_pool *scratch, const tensor *t) { return unary_forward(scratch, t, UN_SIGMOID, 0.f); }

tensor *tensor_sum(struct mem_pool *scratch, const tensor *t, int dim) {
    require_device_payloads("tensor_sum", {t});
    DNN_CHECK(t, "tensor_sum: NULL input");
    int nd = t->ndim;
    if (dim < 0) dim += nd;
    DNN_CHECK(dim >= 0 && dim < nd, "tensor_sum: dim out of range");
    int shape[DNN_MAX_DIMS];
    for (int d = 0; d < nd; d++) shape[d] = t->shape[d];
    shape[dim] = 1;                                           // keepdim
    tensor *out = tensor_scratch(scratch, nd, shape, 0);
    int64_t inner = 1;
    for (int d = dim + 1; d < nd; d++) inner *= t->shape[d];
    ew_launch("sum_fwd_kernel", numel_of(out), SumF{(float *)out->data, (const float *)t->data, view_of(t), t->shape[dim], inner});
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, out, sum_backward, 1, 1);
        fn->inputs[0] = (tensor *)t;
        int *sd = host_alloc_t<int>(scratch); *sd = dim;
        fn->saved_tensors[0] = (tensor *)sd;
    }
    return out;
}

// mean = sum * (1/n) through tensor_mul with a one-element tensor, like the reference (src/ops_reduce.c:138-153)
tensor *tensor_mean(struct mem_pool *scratch, const tensor *t, int dim) {
    require_device_payloads("tensor_mean", {t});
    DNN_CHECK(t, "tensor_mean: NULL input");
    int d = dim < 0 ? dim + t->ndim : dim;
    DNN_CHECK(d >= 0 && d < t->ndim, "tensor_mean: dim out of range");
    tensor *s = tensor_sum(scratch, t, dim);
    int one = 1;
    tensor *scale = tensor_scratch(scratch, 1, &one, 0);
    k_fill((float *)scale->data, 1, 1.0f / (float)t->shape[d]);
    return tensor_mul(scratch, s, scale);
}

tensor *tensor_softmax(struct mem_pool *scratch, const tensor *t, int dim) {
    require_device_payloads("tensor_softmax", {t});
    DNN_CHECK(t, "tensor_softmax: NULL input");
    if (dim < 0) dim += t->ndim;
    DNN_CHECK(dim >= 0 && dim < t->ndim, "tensor_softmax: dim out of range");
    return softmax_forward(scratch, t, dim, 0);
}

tensor *tensor_causal_softmax(struct mem_pool *scratch, const tensor *t) {
    require_device_payloads("tensor_causal_softmax", {t});
    DNN_CHECK(t && t->ndim >= 2, "tensor_causal_softmax: need at least 2 dims");
    DNN_CHECK(t->shape[t->ndim - 2] == t->shape[t->ndim - 1], "tensor_causal_softmax: last two dims must be equal");
    return softmax_forward(scratch, t, t->ndim - 1, t->shape[t->ndim - 1]);
}

tensor *tensor_dropout(struct mem_pool *scratch, const tensor *t, float p) {
    require_device_payloads("tensor_dropout", {t});
    DNN_CHECK(t, "tensor_dropout: NULL input");
    DNN_CHECK(p >= 0.0f && p < 1.0f, "tensor_dropout: p must be in [0, 1)");
    if (!dnn_grad_enabled()) return (tensor *)t;              // evaluation: identity (src/ops_activation.c:1449)
    int64_t n = numel_of(t);
    float scale = 1.0f / (1.0f - p);
    tensor *out = tensor_scratch(scratch, t->ndim, t->shape, 0);
    // same draws, same order as the reference's serial loop (src/ops_activation.c:1460-1463)
    std::vector<float> keep((size_t)n);
    for (int64_t i = 0; i < n; i++) keep[(size_t)i] = dnn_rng_uniform(dnn_get_rng()) >= p ? 1.0f : 0.0f;
    float *mask = dev_alloc_t<float>(scratch, (size_t)n);
    if (n > 0) {
        CUDA_OK(cudaMemcpyAsync(mask, keep.data(), (size_t)n * 4, cudaMemcpyHostToDevice, stream()));
        CUDA_OK(cudaStreamSynchronize(stream()));             // `keep` is pageable and about to go away
    }
    ew_launch("dropout_fwd_kernel", n, DropF{(float *)out->data, (const float *)t->data, mask, view_of(t), scale});
    if (t->requires_grad) {
        grad_fn *fn = attach(scratch, out, dropout_backward, 1, 1);
        fn->inputs[0] = (tensor *)t;
        DropSaved *sv = host_alloc_t<DropSaved>(scratch);
        sv->mask = mask; sv->scale = scale;
        fn->saved_tensors[0] = (tensor *)sv;
    }
    return out;
}

tensor *tensor_triu(struct mem_pool *scratch, int N, int diagonal) {
    DNN_CHECK(N > 0, "tensor_triu: N must be positive");
    int shape[2] = {N, N};
    tensor *out = tensor_scratch(scratch, 2, shape, 0);
    ew_launch("triu_kernel", (int64_t)N * N, TriuF{(float *)out->data, N, diagonal});
    return out;
}

}  // extern "C"
