// Autograd tape walk.  replaces src/autograd.c of the reference.
//
// The host algorithm is the reference's: depth-first topological order from
// the loss (views pull their base tensors into the order), the loss gradient
// is set to ones, then nodes run in reverse order and a node whose output
// never received a gradient is skipped.  What changes is that every gradient
// buffer is device memory, zero-filled with a stream-ordered memset, and each
// node's `backward` launches kernels instead of looping.
#include "common.cuh"
#include "device_utils.cuh"
#include <vector>
#include <unordered_set>
#include <unordered_map>

using namespace dnnb;

static thread_local int g_grad_enabled = 1;

namespace dnnb {
// Gradients whose first contribution is a plain copy that has not been carried out yet
// (grad_defer_copy).  A handful at most: a residual stream defers one per add.
struct DeferredCopy { tensor *base; const float *src; };
static std::vector<DeferredCopy> g_deferred;

// The fresh bit shares a 32-bit unit with the reference's two public flags, so a caller that fills a tensor
// struct in by hand may leave it set by accident.  It only means something on a gradient buffer this
// library allocated: anything else (no buffer, or a buffer outside the pool arenas) is not fresh.
static inline void trust_fresh_bit(tensor *base) {
    if (base->grad_fresh && !(base->grad && dev_ptr_in_arena(base->grad))) base->grad_fresh = 0;
}

static void settle_deferred(tensor *base) {
    trust_fresh_bit(base);
    if (g_deferred.empty()) return;
    for (size_t i = 0; i < g_deferred.size(); i++)
        if (g_deferred[i].base == base) {
            const float *src = g_deferred[i].src;
            g_deferred.erase(g_deferred.begin() + (long)i);
            k_copy(base->grad, src, numel_of(base));
            return;
        }
}
static void settle_all_deferred() {
    while (!g_deferred.empty()) settle_deferred(g_deferred.back().base);
}
// Pools call this before they hand memory out again: a pending copy runs while its source still
// exists (stream order keeps it ahead of whatever reuses the memory).
void grad_settle_all_deferred() { settle_all_deferred(); }
}  // namespace dnnb

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
    dnnb::settle_deferred(base);
    if (!base->pool) {
        fprintf(stderr, "_grad_ensure: tensor %p has NULL pool (ndim=%d)\n", (void *)base, base->ndim);
        abort();
    }
    if (!base->grad) {
        base->grad = (float *)dev_alloc(base->pool, (size_t)numel_of(base) * sizeof(float), true);
        base->grad_fresh = 0;
    } else if (base->grad_fresh) {
        k_fill(base->grad, numel_of(base), 0.0f);
        base->grad_fresh = 0;
    }
    dnnb::colsum_cache_forget(base->grad);        // the caller is about to write this buffer
    return base->grad;
}

}  // extern "C"

namespace dnnb {

float *grad_full(tensor *t, bool *accumulate) {
    tensor *base = t;
    while (base->parent) base = base->parent;
    settle_deferred(base);
    // the caller writes every element of t; that is every element of the root's buffer only
    // if t spans it (the root itself, or a contiguous reshape of all of it)
    bool spans = t->contiguous && t->offset == 0 && numel_of(t) == numel_of(base);
    if (!spans) { *accumulate = true; return _grad_ensure(t); }
    if (!base->grad) {
        DNN_CHECK(base->pool, "gradient requested for a tensor without a pool");
        base->grad = (float *)dev_alloc(base->pool, (size_t)numel_of(base) * sizeof(float), false);
        base->grad_fresh = 0;
        *accumulate = false;
    } else if (base->grad_fresh) {
        base->grad_fresh = 0;
        *accumulate = false;
    } else {
        *accumulate = true;
    }
    colsum_cache_forget(base->grad);
    return base->grad;
}

// Zeroes, in each of `blocks` runs of `pitch` floats, the elements outside [lo, hi).
__global__ void zero_outside_kernel(float *__restrict__ p, int64_t pitch, int64_t blocks, int64_t lo, int64_t hi) {
    int64_t gap = pitch - (hi - lo);
    int64_t total = blocks * gap;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t b = i / gap, r = i % gap;
        p[b * pitch + (r < lo ? r : r - lo + hi)] = 0.0f;
    }
}

float *grad_rows(tensor *t, bool *accumulate) {
    tensor *base = t;
    while (base->parent) base = base->parent;
    settle_deferred(base);
    bool fresh = !base->grad || base->grad_fresh;
    int nd = t->ndim;
    if (!fresh || nd < 1 || t == base) return grad_full(t, accumulate);
    int64_t inner = 1;
    bool packed = true;
    for (int d = nd - 1; d >= 1; d--) { if (t->strides[d] != inner) packed = false; inner *= t->shape[d]; }
    int64_t total = numel_of(base);
    int64_t pitch = t->shape[0] > 1 ? (int64_t)t->strides[0] : total;
    int64_t lo = t->offset;
    bool slab = packed && inner > 0 && pitch >= inner && (int64_t)t->shape[0] * pitch == total && lo >= 0 && lo + inner <= pitch;
    if (!slab) { *accumulate = true; return _grad_ensure(t); }
    if (!base->grad) {
        DNN_CHECK(base->pool, "gradient requested for a tensor without a pool");
        base->grad = (float *)dev_alloc(base->pool, (size_t)total * sizeof(float), false);
    }
    base->grad_fresh = 0;
    colsum_cache_forget(base->grad);
    if (pitch > inner) {
        int64_t gaps = (int64_t)t->shape[0] * (pitch - inner);
        zero_outside_kernel<<<grid_for(gaps, 256), 256, 0, stream()>>>(base->grad, pitch, t->shape[0], lo, lo + inner);
        LAUNCHED("zero_outside_kernel");
    }
    *accumulate = false;
    return base->grad;
}

bool grad_defer_copy(tensor *t, const float *src) {
    tensor *base = t;
    while (base->parent) base = base->parent;
    const bool spans = t->contiguous && t->offset == 0 && numel_of(t) == numel_of(base);
    trust_fresh_bit(base);
    if (!spans || !base->pool || (base->grad && !base->grad_fresh)) return false;
    if (!base->grad) base->grad = (float *)dev_alloc(base->pool, (size_t)numel_of(base) * sizeof(float), false);
    base->grad_fresh = 0;                      // it has content now, even if the content is still a promise
    colsum_cache_forget(base->grad);
    g_deferred.push_back(DeferredCopy{base, src});
    return true;
}

float *grad_full_based(tensor *t, bool *accumulate, const float **basep) {
    *basep = nullptr;
    if (!g_deferred.empty()) {
        tensor *base = t;
        while (base->parent) base = base->parent;
        const bool spans = t->contiguous && t->offset == 0 && numel_of(t) == numel_of(base);
        for (size_t i = 0; spans && i < g_deferred.size(); i++)
            if (g_deferred[i].base == base) {
                *basep = g_deferred[i].src;
                g_deferred.erase(g_deferred.begin() + (long)i);
                *accumulate = false;
                colsum_cache_forget(base->grad);
                return base->grad;
            }
    }
    return grad_full(t, accumulate);
}

void grad_settle(tensor *t) {
    tensor *base = t;
    while (base->parent) base = base->parent;
    settle_deferred(base);
    if (t->grad && t->grad_fresh) { k_fill(t->grad, numel_of(t), 0.0f); t->grad_fresh = 0; }
}

}  // namespace dnnb

namespace dnnb {
// Told, during dnn_backward, when the gradient of a leaf (a root tensor without a tape node that
// requires grad) has received its last contribution.  Used to start the data-parallel exchange of
// a gradient bucket while backward is still running.
static void (*g_leaf_ready)(tensor *leaf) = nullptr;
void set_leaf_ready_observer(void (*fn)(tensor *leaf)) { g_leaf_ready = fn; }
}  // namespace dnnb

namespace {

inline tensor *root_of(tensor *t) { while (t->parent) t = t->parent; return t; }

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
    require_device_payloads("dnn_backward", {loss});
    Topo topo;
    topo.visit(loss);
    colsum_cache_forget(nullptr);                // cached column sums never outlive one backward pass

    int64_t n = numel_of(loss);
    if (!loss->grad) {
        DNN_CHECK(loss->pool, "dnn_backward: root tensor has no pool");
        loss->grad = (float *)dev_alloc(loss->pool, (size_t)n * sizeof(float), false);
    }
    k_fill(loss->grad, n, 1.0f);
    loss->grad_fresh = 0;

    // number of tape nodes that still owe each leaf a contribution
    std::unordered_map<tensor *, int> owed;
    if (g_leaf_ready)
        for (tensor *t : topo.order) {
            grad_fn *fn = t->grad_fn;
            for (int i = 0; i < fn->n_inputs; i++) {
                tensor *r = root_of(fn->inputs[i]);
                if (!r->grad_fn && r->requires_grad) owed[r]++;
            }
        }

    for (size_t i = topo.order.size(); i-- > 0;) {
        tensor *t = topo.order[i];
        grad_fn *fn = t->grad_fn;
        if (!fn) continue;
        settle_deferred(root_of(t));         // a copy nobody folded into a later write happens now
        if (t->grad) {                       // a node whose output never received a gradient is skipped
            tensor gv;
            memset(&gv, 0, sizeof gv);
            gv.data = (void *)t->grad;
            gv.ndim = t->ndim;
            int s = 1;
            for (int d = t->ndim - 1; d >= 0; d--) { gv.shape[d] = t->shape[d]; gv.strides[d] = s; s *= t->shape[d]; }
            gv.contiguous = 1;
            fn->backward(fn, &gv);
        }
        if (g_leaf_ready)                    // run or skipped, this node owes its leaves nothing more
            for (int k = 0; k < fn->n_inputs; k++) {
                tensor *r = root_of(fn->inputs[k]);
                auto it = owed.find(r);
                if (it != owed.end() && --it->second == 0) g_leaf_ready(r);
            }
    }
    settle_all_deferred();
    colsum_cache_forget(nullptr);
}
