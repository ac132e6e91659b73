// Autograd tape walk.  replaces src/autograd.c of the reference.
//
// The host algorithm is the reference's: depth-first topological order from
// the loss (views pull their base tensors into the order), the loss gradient
// is set to ones, then nodes run in reverse order and a node whose output
// never received a gradient is skipped.  What changes is that every gradient
// buffer is device memory, zero-filled with a stream-ordered memset, and each
// node's `backward` launches kernels instead of looping.
#include "common.cuh"
#include <vector>
#include <unordered_set>

using namespace dnnb;

static thread_local int g_grad_enabled = 1;

extern "C" {

int dnn_grad_enabled(void) { return g_grad_enabled; }
dnn_grad_ctx dnn_no_grad_enter(void) {
    dnn_grad_ctx c; c._prev = g_grad_enabled;
    g_grad_enabled = 0;
    return c;
}
void dnn_no_grad_exit(dnn_grad_ctx ctx) { g_grad_enabled = ctx._prev; }

grad_fn *_grad_fn_create(struct mem_pool *pool) {
    grad_fn *fn = host_alloc_t<grad_fn>(pool);
    fn->pool = pool;
    return fn;
}

// src/autograd.c:37-51 — gradients live with the root of a view chain, in the
// root's pool, and start at zero.
float *_grad_ensure(tensor *t) {
    tensor *base = t;
    while (base->parent) base = base->parent;
    if (!base->pool) {
        fprintf(stderr, "_grad_ensure: tensor %p has NULL pool (ndim=%d)\n", (void *)base, base->ndim);
        abort();
    }
    if (!base->grad)
        base->grad = (float *)dev_alloc(base->pool, (size_t)numel_of(base) * sizeof(float), true);
    return base->grad;
}

}  // extern "C"

namespace {

struct Topo {
    std::vector<tensor *> order;
    std::unordered_set<tensor *> seen;
    void visit(tensor *t) {
        if (!t->grad_fn) return;
        if (!seen.insert(t).second) return;
        grad_fn *fn = t->grad_fn;
        for (int i = 0; i < fn->n_inputs; i++) visit(fn->inputs[i]);
        for (int i = 0; i < fn->n_inputs; i++) {
            tensor *p = fn->inputs[i];
            while (p->parent) { p = p->parent; visit(p); }
        }
        order.push_back(t);
    }
};

}  // namespace

extern "C" void dnn_backward(struct mem_pool *scratch, tensor *loss) {
    (void)scratch;
    DNN_CHECK(loss, "dnn_backward: loss is NULL");
    Topo topo;
    topo.visit(loss);

    int64_t n = numel_of(loss);
    if (!loss->grad) {
        DNN_CHECK(loss->pool, "dnn_backward: root tensor has no pool");
        loss->grad = (float *)dev_alloc(loss->pool, (size_t)n * sizeof(float), false);
    }
    k_fill(loss->grad, n, 1.0f);

    for (size_t i = topo.order.size(); i-- > 0;) {
        tensor *t = topo.order[i];
        grad_fn *fn = t->grad_fn;
        if (!fn || !t->grad) continue;
        tensor gv;
        memset(&gv, 0, sizeof gv);
        gv.data = (void *)t->grad;
        gv.ndim = t->ndim;
        int s = 1;
        for (int d = t->ndim - 1; d >= 0; d--) { gv.shape[d] = t->shape[d]; gv.strides[d] = s; s *= t->shape[d]; }
        gv.contiguous = 1;
        fn->backward(fn, &gv);
    }
}
