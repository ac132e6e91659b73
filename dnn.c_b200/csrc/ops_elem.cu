// Element-wise ops and their gradients: add (with broadcasting), cat, relu,
// silu, swiglu.  All are HBM-bound: contiguous operands move as float4 and one
// thread handles 4 elements per grid-stride step.
// replaces src/ops_elem.c:18-175,660-945 and src/ops_activation.c:14-333.
#include "common.cuh"
#include "device_utils.cuh"

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
        ew_launch("silu_bwd_kernel", n, SiluB{ag + a->offset, (const float *)a->data + a->offset, gd, acc});
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

}  // namespace dnnb

using namespace dnnb;

extern "C" {

tensor *tensor_add(struct mem_pool *scratch, const tensor *a, const tensor *b) {
    DNN_CHECK(a && b, "tensor_add: NULL operand");
    int shape[DNN_MAX_DIMS];
    int nd = bcast_shape(a->ndim, a->shape, b->ndim, b->shape, shape);
    DNN_CHECK(nd > 0, "tensor_add: incompatible shapes");
    tensor *out = tensor_scratch(scratch, nd, shape, 0);
    int64_t n = numel_of(out);
    float *od = (float *)out->data;
    const float *af = (const float *)a->data + a->offset, *bf = (const float *)b->data + b->offset;
    if (same_contig(a, b)) {
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
    if (v4ok(n, {od, x})) ew_launch("relu_fwd_kernel", n / 4, ReluF4{(float4 *)od, (const float4 *)x});
    else ew_launch("relu_fwd_kernel", n, ReluF{od, x});
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, out, relu_backward, 1, 0);
        fn->inputs[0] = (tensor *)t;
    }
    return out;
}

tensor *tensor_silu(struct mem_pool *scratch, const tensor *t) {
    DNN_CHECK(t, "tensor_silu: NULL input");
    tensor *out = tensor_scratch(scratch, t->ndim, t->shape, 0);
    int64_t n = numel_of(t);
    const float *x = (const float *)t->data + t->offset;
    if (!t->contiguous) {
        float *tmp = dev_alloc_t<float>(scratch, (size_t)n);
        k_gather(tmp, (const float *)t->data, view_of(t), n);
        x = tmp;
    }
    ew_launch("silu_fwd_kernel", n, SiluF{(float *)out->data, x});
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, out, silu_backward, 1, 0);
        fn->inputs[0] = (tensor *)t;
    }
    return out;
}

tensor *tensor_swiglu(struct mem_pool *scratch, const tensor *gate, const tensor *up) {
    DNN_CHECK(gate && up, "tensor_swiglu: NULL operand");
    int shape[DNN_MAX_DIMS];
    int nd = bcast_shape(gate->ndim, gate->shape, up->ndim, up->shape, shape);
    DNN_CHECK(nd > 0, "tensor_swiglu: incompatible shapes");
    tensor *out = tensor_scratch(scratch, nd, shape, 0);
    int64_t n = numel_of(out);
    float *od = (float *)out->data;
    if (same_contig(gate, up)) {
        const float *g = (const float *)gate->data + gate->offset, *u = (const float *)up->data + up->offset;
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

}  // extern "C"
