// Tensor structs, constructors and views.
// replaces src/tensor.c of the reference: same host-side struct logic, but the
// payload of every tensor is a device allocation and every element-touching
// loop is a kernel launch.
#include "common.cuh"
#include <vector>

using namespace dnnb;

namespace dnnb {

static void packed_strides(int ndim, const int *shape, int *strides) {
    int s = 1;
    for (int i = ndim - 1; i >= 0; i--) { strides[i] = s; s *= shape[i]; }
}
static bool is_packed(const int *shape, const int *strides, int ndim) {
    int s = 1;
    for (int d = ndim - 1; d >= 0; d--) { if (strides[d] != s) return false; s *= shape[d]; }
    return true;
}
static int64_t count(const int *shape, int ndim) {
    int64_t n = 1;
    for (int i = 0; i < ndim; i++) n *= shape[i];
    return n;
}

static tensor *make_tensor(struct mem_pool *pool, int ndim, const int *shape, int requires_grad, bool zero) {
    DNN_CHECK(pool, "tensor: pool is NULL");
    DNN_CHECK(ndim >= 0 && ndim <= DNN_MAX_DIMS, "tensor: ndim out of range");
    tensor *t = host_alloc_t<tensor>(pool);
    t->ndim = ndim;
    memcpy(t->shape, shape, ndim * sizeof(int));
    packed_strides(ndim, shape, t->strides);
    int64_t n = count(shape, ndim);
    DNN_CHECK(n <= INT32_MAX, "tensor: more than 2^31-1 elements");
    t->data = dev_alloc(pool, (size_t)n * sizeof(float), zero);
    t->pool = pool;
    t->requires_grad = requires_grad ? 1 : 0;
    t->contiguous = 1;
    return t;
}

int bcast_shape(int na, const int *sa, int nb, const int *sb, int *out) {
    int n = na > nb ? na : nb;
    for (int i = 0; i < n; i++) {
        int da = i - (n - na), db = i - (n - nb);
        int a = da >= 0 ? sa[da] : 1, b = db >= 0 ? sb[db] : 1;
        if (a != b && a != 1 && b != 1) return 0;
        out[i] = a > b ? a : b;
    }
    return n;
}

View bcast_view(const tensor *t, int out_ndim, const int *out_shape) {
    View v; v.ndim = out_ndim; v.offset = t->offset;
    int lead = out_ndim - t->ndim;
    // A contiguous tensor is indexed by its packed strides, as the reference's
    // contiguous fast path does; otherwise by its stored strides.
    int ps[DNN_MAX_DIMS];
    packed_strides(t->ndim, t->shape, ps);
    for (int d = 0; d < DNN_MAX_DIMS; d++) {
        v.shape[d] = d < out_ndim ? out_shape[d] : 1;
        int td = d - lead;
        if (d >= out_ndim || td < 0 || t->shape[td] == 1) v.strides[d] = 0;
        else v.strides[d] = t->contiguous ? ps[td] : t->strides[td];
    }
    return v;
}

grad_fn *attach(struct mem_pool *scratch, tensor *out, void (*bw)(grad_fn *, tensor *), int n_inputs, int n_saved) {
    grad_fn *fn = _grad_fn_create(scratch);
    fn->backward = bw;
    fn->n_inputs = n_inputs;
    fn->inputs = n_inputs ? host_alloc_t<tensor *>(scratch, n_inputs) : nullptr;
    fn->n_saved = n_saved;
    fn->saved_tensors = n_saved ? host_alloc_t<tensor *>(scratch, n_saved) : nullptr;
    out->requires_grad = 1;
    out->grad_fn = fn;
    return fn;
}

// ---- view backwards (src/tensor.c:40-64, 166-272) -------------------------
static View with_shape_of(const tensor *g, const tensor *parent) {
    View v; v.ndim = g->ndim; v.offset = parent->offset;
    for (int d = 0; d < DNN_MAX_DIMS; d++) {
        v.shape[d] = d < g->ndim ? g->shape[d] : 1;
        v.strides[d] = (d < g->ndim && d < parent->ndim) ? parent->strides[d] : 0;
    }
    return v;
}

static void copy_strided_backward(grad_fn *fn, tensor *g) {
    tensor *parent = fn->inputs[0];
    if (!wants_grad(parent)) return;
    float *pg = _grad_ensure(parent);
    k_scatter(pg, with_shape_of(g, parent), (const float *)g->data + g->offset, numel_of(g), true);
}

static void slice_backward(grad_fn *fn, tensor *g) {
    tensor *parent = fn->inputs[0];
    if (!wants_grad(parent)) return;
    float *pg = _grad_ensure(parent);
    int dim = *(int *)fn->saved_tensors[0], start = *(int *)fn->saved_tensors[1];
    View v = with_shape_of(g, parent);
    v.offset += start * parent->strides[dim];
    k_scatter(pg, v, (const float *)g->data + g->offset, numel_of(g), true);
}

static void transpose_backward(grad_fn *fn, tensor *g) {
    tensor *parent = fn->inputs[0];
    if (!wants_grad(parent)) return;
    float *pg = _grad_ensure(parent);
    int d1 = *(int *)fn->saved_tensors[0], d2 = *(int *)fn->saved_tensors[1];
    View v = with_shape_of(g, parent);
    int s1 = parent->strides[d1], s2 = parent->strides[d2];
    v.strides[d1] = s2; v.strides[d2] = s1;
    k_scatter(pg, v, (const float *)g->data + g->offset, numel_of(g), true);
}

static void reshape_backward(grad_fn *fn, tensor *g) {
    tensor *parent = fn->inputs[0];
    if (!wants_grad(parent)) return;
    float *pg = _grad_ensure(parent);
    if (g->contiguous && parent->contiguous)
        k_axpy_acc(pg + parent->offset, (const float *)g->data + g->offset, numel_of(g));
    else
        k_scatter(pg, with_shape_of(g, parent), (const float *)g->data + g->offset, numel_of(g), true);
}

static tensor *copy_strided(struct mem_pool *scratch, const tensor *t) {
    tensor *out = tensor_scratch(scratch, t->ndim, t->shape, t->requires_grad);
    k_gather((float *)out->data, (const float *)t->data, view_of(t), numel_of(t));
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, out, copy_strided_backward, 1, 0);
        fn->inputs[0] = (tensor *)t;
    }
    return out;
}

static int *save_int(struct mem_pool *pool, int v) { int *p = host_alloc_t<int>(pool); *p = v; return p; }

}  // namespace dnnb

extern "C" {

tensor *tensor_scratch(struct mem_pool *pool, int ndim, const int *shape, int requires_grad) {
    return make_tensor(pool, ndim, shape, requires_grad, false);
}
tensor *tensor_zeros(struct mem_pool *pool, int ndim, const int *shape, int requires_grad) {
    return make_tensor(pool, ndim, shape, requires_grad, true);
}
tensor *tensor_zeros_data(struct mem_pool *pool, int ndim, const int *shape) {
    return make_tensor(pool, ndim, shape, 0, true);
}

// Host RNG draws in the reference's order (src/tensor.c:142-162), then one upload.
tensor *tensor_randn(struct mem_pool *pool, int ndim, const int *shape, int requires_grad) {
    tensor *t = make_tensor(pool, ndim, shape, requires_grad, false);
    int64_t n = numel_of(t);
    std::vector<float> h((size_t)n);
    for (int64_t i = 0; i < n; i++) h[i] = dnn_rng_normal(dnn_get_rng());
    dnn_cuda_upload(t, h.data(), (size_t)n * 4);
    return t;
}
tensor *tensor_uniform(struct mem_pool *pool, int ndim, const int *shape, int requires_grad, float bound) {
    tensor *t = make_tensor(pool, ndim, shape, requires_grad, false);
    int64_t n = numel_of(t);
    std::vector<float> h((size_t)n);
    for (int64_t i = 0; i < n; i++) h[i] = (2.0f * dnn_rng_uniform(dnn_get_rng()) - 1.0f) * bound;
    dnn_cuda_upload(t, h.data(), (size_t)n * 4);
    return t;
}

// ── views (src/tensor.c:274-399) ─────────────────────────────────────────
tensor *tensor_slice(struct mem_pool *scratch, tensor *t, int dim, int start, int len) {
    DNN_CHECK(dim < t->ndim && start >= 0 && start + len <= t->shape[dim], "tensor_slice: range");
    tensor *v = (tensor *)_mem_pool_alloc(scratch, sizeof(tensor), t);
    v->shape[dim] = len;
    v->offset = t->offset + start * t->strides[dim];
    v->parent = t; v->grad_fn = nullptr; v->grad = nullptr; v->pool = nullptr;
    v->contiguous = is_packed(v->shape, v->strides, v->ndim);
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, v, slice_backward, 1, 2);
        fn->inputs[0] = t;
        fn->saved_tensors[0] = (tensor *)save_int(scratch, dim);
        fn->saved_tensors[1] = (tensor *)save_int(scratch, start);
    }
    return v;
}

tensor *tensor_transpose(struct mem_pool *scratch, tensor *t, int d1, int d2) {
    DNN_CHECK(d1 < t->ndim && d2 < t->ndim, "tensor_transpose: dim");
    tensor *v = (tensor *)_mem_pool_alloc(scratch, sizeof(tensor), t);
    v->shape[d1] = t->shape[d2]; v->shape[d2] = t->shape[d1];
    v->strides[d1] = t->strides[d2]; v->strides[d2] = t->strides[d1];
    v->parent = t; v->grad_fn = nullptr; v->grad = nullptr; v->pool = nullptr;
    v->contiguous = is_packed(v->shape, v->strides, v->ndim);
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, v, transpose_backward, 1, 2);
        fn->inputs[0] = t;
        fn->saved_tensors[0] = (tensor *)save_int(scratch, d1);
        fn->saved_tensors[1] = (tensor *)save_int(scratch, d2);
    }
    return v;
}

tensor *tensor_reshape(struct mem_pool *scratch, tensor *t, int ndim, const int *shape) {
    DNN_CHECK(ndim <= DNN_MAX_DIMS, "tensor_reshape: ndim exceeds DNN_MAX_DIMS");
    int resolved[DNN_MAX_DIMS];
    int inferred = -1;
    int64_t product = 1;
    for (int i = 0; i < ndim; i++) {
        if (shape[i] == -1) { DNN_CHECK(inferred == -1, "tensor_reshape: only one -1 allowed"); inferred = i; }
        else { DNN_CHECK(shape[i] > 0, "tensor_reshape: dims must be positive or -1"); product *= shape[i]; }
        resolved[i] = shape[i];
    }
    int64_t total = numel_of(t);
    if (inferred >= 0) {
        DNN_CHECK(total % product == 0, "tensor_reshape: -1 dim must divide evenly");
        resolved[inferred] = (int)(total / product);
    } else {
        DNN_CHECK(product == total, "tensor_reshape: shape must match numel");
    }
    if (!t->contiguous) return tensor_reshape(scratch, copy_strided(scratch, t), ndim, resolved);

    tensor *v = (tensor *)_mem_pool_alloc(scratch, sizeof(tensor), t);
    v->ndim = ndim;
    memcpy(v->shape, resolved, ndim * sizeof(int));
    packed_strides(ndim, resolved, v->strides);
    v->offset = t->offset;
    v->parent = t; v->contiguous = 1; v->grad_fn = nullptr; v->grad = nullptr; v->pool = nullptr;
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, v, reshape_backward, 1, 0);
        fn->inputs[0] = t;
    }
    return v;
}

tensor *tensor_contiguous(struct mem_pool *scratch, tensor *t) {
    require_device_payloads("tensor_contiguous", {t});
    return t->contiguous ? t : copy_strided(scratch, t);
}
tensor *tensor_flatten(struct mem_pool *scratch, tensor *t) {
    int m1 = -1;
    return tensor_reshape(scratch, t, 1, &m1);
}

// ── accessors (src/tensor.c:403-474) ─────────────────────────────────────
float *tensor_data_ptr(tensor *t) {
    DNN_CHECK(t->contiguous, "tensor_data_ptr: tensor must be contiguous");
    return (float *)t->data + t->offset;
}
int tensor_numel(const tensor *t) { return (int)numel_of(t); }
int tensor_ndim(const tensor *t) { return t->ndim; }
int tensor_shape(const tensor *t, int dim) { return t->shape[dim]; }
int tensor_is_leaf(const tensor *t) { return t->requires_grad && t->grad_fn == nullptr; }
int tensor_is_contiguous(const tensor *t) { return t->contiguous; }
int tensor_requires_grad(const tensor *t) { return t->requires_grad; }
void tensor_set_requires_grad(tensor *t, int req) { t->requires_grad = req ? 1 : 0; }
float *tensor_grad(const tensor *t) { grad_settle((tensor *)t); return t->grad; }
tensor *tensor_root(tensor *t) { while (t->parent) t = t->parent; return t; }

void tensor_retain_grad(tensor *t) {
    if (t->grad) return;
    tensor *base = tensor_root(t);
    t->grad = (float *)dev_alloc(base->pool, (size_t)numel_of(t) * 4, true);
}
void tensor_zero_grad(tensor *t) {
    if (t->grad) { k_fill(t->grad, numel_of(t), 0.0f); t->grad_fresh = 0; }
}

void tensor_print(const tensor *t) {
    printf("tensor(shape=[");
    for (int i = 0; i < t->ndim; i++) printf("%s%d", i ? "," : "", t->shape[i]);
    printf("], strides=[");
    for (int i = 0; i < t->ndim; i++) printf("%s%d", i ? "," : "", t->strides[i]);
    int64_t n = numel_of(t);
    int show = n < 16 ? (int)n : 16;
    float h[16];
    dnn_cuda_memcpy_d2h(h, (const float *)t->data + t->offset, (size_t)show * 4);
    printf("], data=[");
    for (int i = 0; i < show; i++) printf("%s%.4f", i ? "," : "", h[i]);
    if (n > 16) printf(",...");
    printf("])\n");
}

}  // extern "C"
