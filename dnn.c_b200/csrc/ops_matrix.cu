// matmul / matmul_add and their gradients: host-side shape logic.
// replaces src/ops_matrix.c:48-1206 of the reference.
//
// The reference runs one sgemm per batch element (src/ops_matrix.c:1109-1183)
// and, in backward, adds each batch element's weight gradient into the same
// buffer (:858-861).  Here the common "activations [B,N,K] times a broadcast
// weight" case collapses into ONE GEMM with M = B*N rows (forward, dA) or a
// reduction dimension of B*N (dW).  Other batch patterns run as one batched
// launch when every operand's batch offsets are affine, or batch by batch.
#include "common.cuh"
#include <vector>

namespace dnnb {

struct Operand {            // a 2-D slice family: element (r,c) of batch bi
    const tensor *t;
    int64_t rs, cs;         // strides of the last two dims
    std::vector<int64_t> off;   // element offset of each batch slice
    bool affine; int64_t bstride;
};

static int64_t batch_offset(const tensor *t, int batch_ndim, const int *coord) {
    int tb = t->ndim - 2;
    int lead = batch_ndim - tb;
    int64_t off = t->offset;
    for (int d = 0; d < tb; d++) {
        int c = coord[lead + d];
        if (t->shape[d] == 1) c = 0;
        off += (int64_t)c * t->strides[d];
    }
    return off;
}

static Operand make_operand(const tensor *t, int batch_ndim, const int *batch_shape, int batch) {
    Operand o; o.t = t;
    o.rs = t->strides[t->ndim - 2]; o.cs = t->strides[t->ndim - 1];
    o.off.resize(batch);
    int coord[DNN_MAX_DIMS] = {0};
    for (int bi = 0; bi < batch; bi++) {
        int r = bi;
        for (int d = batch_ndim - 1; d >= 0; d--) { coord[d] = r % batch_shape[d]; r /= batch_shape[d]; }
        o.off[bi] = batch_offset(t, batch_ndim, coord);
    }
    o.bstride = batch > 1 ? o.off[1] - o.off[0] : 0;
    o.affine = true;
    for (int bi = 1; bi < batch; bi++) if (o.off[bi] - o.off[bi - 1] != o.bstride) { o.affine = false; break; }
    return o;
}

// C(bi) (=|+=) X(bi) * Y(bi) [+ bias], where each of X, Y, C is given by
// base pointer, per-batch offsets and (row, col) strides.  `c_shared` means all
// batches add into the same C (a broadcast operand's gradient).
struct Side { const float *p; const Operand *o; int64_t rs, cs; };

static void run_batched(Side X, Side Y, float *Cp, const Operand *co, int64_t c_rs, int64_t c_cs,
                        int M, int N, int K, int batch, const float *bias, bool accumulate) {
    GemmArgs g;
    g.M = M; g.N = N; g.K = K; g.bias = bias; g.accumulate = accumulate;
    g.a_rs = X.rs; g.a_cs = X.cs; g.b_rs = Y.rs; g.b_cs = Y.cs; g.c_rs = c_rs; g.c_cs = c_cs;
    bool c_shared = batch > 1 && co->affine && co->bstride == 0;
    if (batch == 1 || (X.o->affine && Y.o->affine && co->affine && !c_shared)) {
        g.A = X.p + X.o->off[0]; g.B = Y.p + Y.o->off[0]; g.C = Cp + co->off[0];
        g.a_bs = X.o->bstride; g.b_bs = Y.o->bstride; g.c_bs = co->bstride; g.batch = batch;
        gemm(g);
        return;
    }
    // batch by batch, in order (stream order makes the shared-C accumulation safe)
    g.batch = 1; g.a_bs = g.b_bs = g.c_bs = 0;
    for (int bi = 0; bi < batch; bi++) {
        g.A = X.p + X.o->off[bi]; g.B = Y.p + Y.o->off[bi]; g.C = Cp + co->off[bi];
        g.accumulate = accumulate || (c_shared && bi > 0);
        gemm(g);
    }
}

struct MM {
    int M, N, K, batch, batch_ndim;
    int batch_shape[DNN_MAX_DIMS];
    Operand a, b;
    Operand c;          // packed output / upstream gradient [batch..., M, N]
    bool collapse;      // weight broadcast and rows of `a` continue across batches
};

static MM plan(const tensor *a, const tensor *b, int trans_b) {
    MM p;
    int na = a->ndim, nb = b->ndim;
    p.K = a->shape[na - 1]; p.M = a->shape[na - 2];
    p.N = trans_b ? b->shape[nb - 2] : b->shape[nb - 1];
    p.batch_ndim = bcast_shape(na - 2, a->shape, nb - 2, b->shape, p.batch_shape);
    p.batch = 1;
    for (int i = 0; i < p.batch_ndim; i++) p.batch *= p.batch_shape[i];
    p.a = make_operand(a, p.batch_ndim, p.batch_shape, p.batch);
    p.b = make_operand(b, p.batch_ndim, p.batch_shape, p.batch);
    p.c.t = nullptr; p.c.rs = p.N; p.c.cs = 1;
    p.c.off.resize(p.batch);
    for (int bi = 0; bi < p.batch; bi++) p.c.off[bi] = (int64_t)bi * p.M * p.N;
    p.c.affine = true; p.c.bstride = (int64_t)p.M * p.N;
    p.collapse = p.batch > 1 && p.b.affine && p.b.bstride == 0 && p.a.affine &&
                 p.a.bstride == (int64_t)p.M * p.a.rs;
    return p;
}

static void mm_forward(const MM &p, const tensor *a, const tensor *b, int trans_b, const float *bias, float *out) {
    const float *ad = (const float *)a->data, *bd = (const float *)b->data;
    // B as a (K x N) operand: element (k,n) at k*b_rs' + n*b_cs'
    int64_t bk = trans_b ? p.b.cs : p.b.rs, bn = trans_b ? p.b.rs : p.b.cs;
    gemm_set_role(GEMM_ROLE_FORWARD);
    if (p.collapse) {
        GemmArgs g;
        g.A = ad + p.a.off[0]; g.a_rs = p.a.rs; g.a_cs = p.a.cs; g.a_bs = 0;
        g.B = bd + p.b.off[0]; g.b_rs = bk; g.b_cs = bn; g.b_bs = 0;
        g.C = out; g.c_rs = p.N; g.c_cs = 1; g.c_bs = 0;
        g.bias = bias; g.M = p.M * p.batch; g.N = p.N; g.K = p.K; g.batch = 1; g.accumulate = false;
        gemm(g);
        return;
    }
    run_batched(Side{ad, &p.a, p.a.rs, p.a.cs}, Side{bd, &p.b, bk, bn}, out, &p.c, p.N, 1,
                p.M, p.N, p.K, p.batch, bias, false);
}

// dA(bi) += G(bi) * op(B(bi))^T ;  dB(bi) += A(bi)^T * G(bi)  (laid out like B)
static void mm_backward(const MM &p, tensor *a, tensor *b, int trans_b, const float *gd) {
    const float *ad = (const float *)a->data, *bd = (const float *)b->data;
    int64_t bk = trans_b ? p.b.cs : p.b.rs, bn = trans_b ? p.b.rs : p.b.cs;
    bool need_a = wants_grad(a), need_b = wants_grad(b);
    bool self = (a == b);
    // dA and dW each write the whole of their operand's gradient, so a fresh buffer is
    // stored into rather than added to (grad_full); a broadcast operand is summed over
    // batches and run_batched turns that into store-then-add on its own.
    bool acc_a = true, acc_b = true;
    float *ag = need_a ? grad_full(a, &acc_a) : nullptr;
    float *bg = (need_b && !self) ? grad_full(b, &acc_b) : nullptr;

    if (need_a) {
        gemm_set_role(GEMM_ROLE_DA);
        // dA[m,k] += sum_n G[m,n] * Bop[k,n]   ->  X = G (M x N), Y = Bop^T (N x K)
        if (p.collapse) {
            GemmArgs g;
            g.A = gd; g.a_rs = p.N; g.a_cs = 1; g.a_bs = 0;
            g.B = bd + p.b.off[0]; g.b_rs = bn; g.b_cs = bk; g.b_bs = 0;
            g.C = ag + p.a.off[0]; g.c_rs = p.a.rs; g.c_cs = p.a.cs; g.c_bs = 0;
            g.bias = nullptr; g.M = p.M * p.batch; g.N = p.K; g.K = p.N; g.batch = 1; g.accumulate = acc_a;
            gemm(g);
        } else {
            run_batched(Side{gd, &p.c, p.N, 1}, Side{bd, &p.b, bn, bk}, ag, &p.a, p.a.rs, p.a.cs,
                        p.M, p.K, p.N, p.batch, nullptr, acc_a);
        }
    }
    if ((need_b && !self) || (self && need_a)) {
        float *dst = self ? ag : bg;
        bool acc = self ? true : acc_b;
        gemm_set_role(GEMM_ROLE_DW);
        // dBop[k,n] += sum_m A[m,k] * G[m,n]  ->  X = A^T (K x M), Y = G (M x N); C strides follow B's layout
        if (p.collapse) {
            GemmArgs g;
            g.A = ad + p.a.off[0]; g.a_rs = p.a.cs; g.a_cs = p.a.rs; g.a_bs = 0;
            g.B = gd; g.b_rs = p.N; g.b_cs = 1; g.b_bs = 0;
            g.C = dst + p.b.off[0]; g.c_rs = bk; g.c_cs = bn; g.c_bs = 0;
            g.bias = nullptr; g.M = p.K; g.N = p.N; g.K = p.M * p.batch; g.batch = 1; g.accumulate = acc;
            gemm(g);
        } else {
            run_batched(Side{ad, &p.a, p.a.cs, p.a.rs}, Side{gd, &p.c, p.N, 1}, dst, &p.b, bk, bn,
                        p.K, p.N, p.M, p.batch, nullptr, acc);
        }
    }
    gemm_set_role(GEMM_ROLE_FORWARD);
}

static void matmul_backward(grad_fn *fn, tensor *go) {
    tensor *a = fn->inputs[0], *b = fn->inputs[1];
    MM p = plan(a, b, 0);
    mm_backward(p, a, b, 0, (const float *)go->data);
}

static void matmul_add_backward(grad_fn *fn, tensor *go) {
    tensor *a = fn->inputs[0], *b = fn->inputs[1], *bias = fn->inputs[2];
    int trans_b = *(int *)fn->saved_tensors[0];
    MM p = plan(a, b, trans_b);
    mm_backward(p, a, b, trans_b, (const float *)go->data);
    if (wants_grad(bias)) {
        bool acc = true;
        float *bg = grad_full(bias, &acc);
        int nbias = bias->shape[0];
        k_colsum_acc(bg + bias->offset, (const float *)go->data, numel_of(go) / nbias, nbias, acc);
    }
}

// inputs: a, b, bias, x (the residual).  d(out)/dx = identity; the rest is matmul_add's backward.
static void matmul_add_residual_backward(grad_fn *fn, tensor *go) {
    tensor *x = fn->inputs[3];
    if (wants_grad(x) && !grad_defer_copy(x, (const float *)go->data)) {     // usually deferred: the norm backward that writes dx next adds go
        bool acc = true;
        float *xg = grad_full(x, &acc);
        int64_t n = numel_of(go);
        if (acc) k_axpy_acc(xg + x->offset, (const float *)go->data, n);
        else k_copy(xg + x->offset, (const float *)go->data, n);
    }
    matmul_add_backward(fn, go);
}

static tensor *mm_out(struct mem_pool *scratch, const MM &p) {
    int shape[DNN_MAX_DIMS];
    for (int i = 0; i < p.batch_ndim; i++) shape[i] = p.batch_shape[i];
    shape[p.batch_ndim] = p.M; shape[p.batch_ndim + 1] = p.N;
    return tensor_scratch(scratch, p.batch_ndim + 2, shape, 0);
}

tensor *matmul_add_residual(struct mem_pool *scratch, const tensor *a, const tensor *b, int trans_b, const tensor *bias, const tensor *x) {
    // the fused form needs x to have exactly the output's shape, packed
    // (TF32 mode: the tensor-core kernel's epilogue; at most four rows, any mode: the sliced kernel's reduction)
    bool fits = x && x->contiguous && a->ndim >= 2 && b->ndim == 2 && bias && bias->ndim == 1;
    if (fits) {
        int64_t rows = numel_of(a) / a->shape[a->ndim - 1];
        int ncols = trans_b ? b->shape[0] : b->shape[1];
        fits = (gemm_mode() == DNN_CUDA_GEMM_TF32 || rows <= 4) && x->ndim == a->ndim && numel_of(x) == rows * ncols && x->shape[x->ndim - 1] == ncols && ncols % 4 == 0;
        for (int d = 0; fits && d < a->ndim - 1; d++) fits = x->shape[d] == a->shape[d];
    }
    if (!fits) return tensor_add(scratch, x, tensor_matmul_add(scratch, a, b, trans_b, bias));
    MM p = plan(a, b, trans_b);
    DNN_CHECK(bias->shape[0] == p.N, "matmul_add_residual: bias size != out cols");
    tensor *out = mm_out(scratch, p);
    const float *xd = (const float *)x->data + x->offset;
    gemm_residual_request(xd, p.N);
    mm_forward(p, a, b, trans_b, (const float *)bias->data + bias->offset, (float *)out->data);
    if (!gemm_residual_take()) k_axpy_acc((float *)out->data, xd, numel_of(out));        // the GEMM took another route
    if (dnn_grad_enabled() && (a->requires_grad || b->requires_grad || bias->requires_grad || x->requires_grad)) {
        grad_fn *fn = attach(scratch, out, matmul_add_residual_backward, 4, 1);
        fn->inputs[0] = (tensor *)a; fn->inputs[1] = (tensor *)b; fn->inputs[2] = (tensor *)bias; fn->inputs[3] = (tensor *)x;
        int *st = host_alloc_t<int>(scratch); *st = trans_b;
        fn->saved_tensors[0] = (tensor *)st;
    }
    return out;
}

}  // namespace dnnb

using namespace dnnb;

extern "C" {

tensor *tensor_matmul(struct mem_pool *scratch, const tensor *a, const tensor *b) {
    require_device_payloads("tensor_matmul", {a, b});
    DNN_CHECK(a && b, "tensor_matmul: NULL operand");
    DNN_CHECK(a->ndim >= 2 && b->ndim >= 2, "tensor_matmul: need at least 2D");
    DNN_CHECK(a->shape[a->ndim - 1] == b->shape[b->ndim - 2], "tensor_matmul: inner dim mismatch");
    MM p = plan(a, b, 0);
    DNN_CHECK(p.batch_ndim > 0 || (a->ndim == 2 && b->ndim == 2), "tensor_matmul: incompatible batch dims");
    tensor *out = mm_out(scratch, p);
    mm_forward(p, a, b, 0, nullptr, (float *)out->data);
    if (dnn_grad_enabled() && (a->requires_grad || b->requires_grad)) {
        grad_fn *fn = attach(scratch, out, matmul_backward, 2, 0);
        fn->inputs[0] = (tensor *)a; fn->inputs[1] = (tensor *)b;
    }
    return out;
}

tensor *tensor_matmul_add(struct mem_pool *scratch, const tensor *a, const tensor *b, int trans_b, const tensor *bias) {
    require_device_payloads("tensor_matmul_add", {a, b, bias});
    DNN_CHECK(a && b && bias, "tensor_matmul_add: NULL operand");
    DNN_CHECK(a->ndim >= 2 && b->ndim >= 2, "tensor_matmul_add: need at least 2D");
    DNN_CHECK(bias->ndim == 1, "tensor_matmul_add: bias must be 1-D");
    int nb = b->ndim;
    int b_inner = trans_b ? b->shape[nb - 1] : b->shape[nb - 2];
    DNN_CHECK(a->shape[a->ndim - 1] == b_inner, "tensor_matmul_add: inner dim mismatch");
    MM p = plan(a, b, trans_b);
    DNN_CHECK(bias->shape[0] == p.N, "tensor_matmul_add: bias size != out cols");
    tensor *out = mm_out(scratch, p);
    mm_forward(p, a, b, trans_b, (const float *)bias->data + bias->offset, (float *)out->data);
    if (dnn_grad_enabled() && (a->requires_grad || b->requires_grad || bias->requires_grad)) {
        grad_fn *fn = attach(scratch, out, matmul_add_backward, 3, 1);
        fn->inputs[0] = (tensor *)a; fn->inputs[1] = (tensor *)b; fn->inputs[2] = (tensor *)bias;
        int *st = host_alloc_t<int>(scratch); *st = trans_b;
        fn->saved_tensors[0] = (tensor *)st;
    }
    return out;
}

}  // extern "C"
