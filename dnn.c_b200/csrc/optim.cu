// AdamW, gradient norm / clipping, zero_grad and the LR schedules.
// replaces src/optim.c:67-316 of the reference.
//
// The reference loops over parameter tensors with OpenMP, which is badly
// balanced (one 24.6 M-element embedding next to 768-element gains).  Here all
// tensors of one call are described by a small table and ONE launch covers
// them: a CTA owns a fixed-size chunk of one tensor.  AdamW is HBM-bound at
// 28 bytes per parameter (read p, g, m, v; write p, m, v).
#include "common.cuh"
#include <cstdio>
#include <cstring>
#include "device_utils.cuh"
#include <vector>
#include <algorithm>

namespace dnnb {

constexpr int kChunk = 8192;       // elements per CTA (256 threads x 8 float4)

struct TensorRef { float *p, *g, *m, *v; int64_t n; float lr; int first_chunk; };

__device__ __forceinline__ int find_tensor(const TensorRef *tab, int nt, int chunk) {
    int lo = 0, hi = nt - 1;
    while (lo < hi) { int mid = (lo + hi + 1) >> 1; if (tab[mid].first_chunk <= chunk) lo = mid; else hi = mid - 1; }
    return lo;
}

struct AdamHyper { float b1, b2, eps, wd, bc1, bc2_sqrt; };

__device__ __forceinline__ void adam1(float &p, float &m, float &v, float g, float lr, float step, const AdamHyper &h) {
    m = h.b1 * m + (1.0f - h.b1) * g;
    v = h.b2 * v + (1.0f - h.b2) * g * g;
    float denom = sqrtf(v) / h.bc2_sqrt + h.eps;
    p *= 1.0f - lr * h.wd;
    p -= step * m / denom;
}

__global__ void __launch_bounds__(256) adamw_kernel(const TensorRef *__restrict__ tab, int nt, AdamHyper h) {
    int t = find_tensor(tab, nt, blockIdx.x);
    TensorRef r = tab[t];
    int64_t start = (int64_t)(blockIdx.x - r.first_chunk) * kChunk;
    int64_t end = start + kChunk < r.n ? start + kChunk : r.n;
    float step = r.lr / h.bc1;
    bool vec = ((((uintptr_t)r.p | (uintptr_t)r.g | (uintptr_t)r.m | (uintptr_t)r.v) & 15) == 0);
    if (vec) {
        int64_t e4 = start + ((end - start) & ~(int64_t)3);
        for (int64_t i = start + threadIdx.x * 4; i < e4; i += 1024) {
            float4 p = *(float4 *)(r.p + i), g = *(const float4 *)(r.g + i), m = *(float4 *)(r.m + i), v = *(float4 *)(r.v + i);
            adam1(p.x, m.x, v.x, g.x, r.lr, step, h); adam1(p.y, m.y, v.y, g.y, r.lr, step, h);
            adam1(p.z, m.z, v.z, g.z, r.lr, step, h); adam1(p.w, m.w, v.w, g.w, r.lr, step, h);
            *(float4 *)(r.p + i) = p; *(float4 *)(r.m + i) = m; *(float4 *)(r.v + i) = v;
        }
        start = e4;
    }
    for (int64_t i = start + threadIdx.x; i < end; i += 256) adam1(r.p[i], r.m[i], r.v[i], r.g[i], r.lr, step, h);
}

// sum of squares per chunk in double (the reference accumulates in double, src/optim.c:194-204)
__global__ void __launch_bounds__(256) sumsq_kernel(const TensorRef *__restrict__ tab, int nt, double *__restrict__ partial) {
    __shared__ double sh[8];
    int t = find_tensor(tab, nt, blockIdx.x);
    TensorRef r = tab[t];
    int64_t start = (int64_t)(blockIdx.x - r.first_chunk) * kChunk;
    int64_t end = start + kChunk < r.n ? start + kChunk : r.n;
    double s = 0.0;
    for (int64_t i = start + threadIdx.x; i < end; i += 256) { double g = (double)r.g[i]; s += g * g; }
    s = warp_sum_d(s);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) { double tt = 0.0; for (int w = 0; w < 8; w++) tt += sh[w]; partial[blockIdx.x] = tt; }
}
__global__ void sumsq_final_kernel(const double *__restrict__ partial, int n, float *__restrict__ out_norm, double *__restrict__ out_sq) {
    __shared__ double sh[32];
    double s = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
    s = warp_sum_d(s);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tt = 0.0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) tt += sh[w];
        out_sq[0] = tt;
        out_norm[0] = sqrtf((float)tt);
    }
}
__global__ void __launch_bounds__(256) scale_kernel(const TensorRef *__restrict__ tab, int nt, float scale) {
    int t = find_tensor(tab, nt, blockIdx.x);
    TensorRef r = tab[t];
    int64_t start = (int64_t)(blockIdx.x - r.first_chunk) * kChunk;
    int64_t end = start + kChunk < r.n ? start + kChunk : r.n;
    for (int64_t i = start + threadIdx.x; i < end; i += 256) r.g[i] *= scale;
}

// Device-resident staging for the tables and reduction partials; grown on demand.
struct OptScratch { TensorRef *tab = nullptr; size_t tab_cap = 0; double *partial = nullptr; size_t part_cap = 0;
                    float *norm = nullptr; double *sq = nullptr; };
static OptScratch g_os;

// ── variants for a captured step ─────────────────────────────────────────
// A CUDA graph bakes kernel arguments in, so what changes from step to step (learning rate,
// bias corrections) is read from a small device struct that the graph refreshes from pinned
// host memory, and the clipping decision is taken on the device from the norm just computed.
struct StepState { float lr, bc1, bc2_sqrt, max_norm; };

__global__ void __launch_bounds__(256) scale_dev_kernel(const TensorRef *__restrict__ tab, int nt, const float *__restrict__ norm,
                                                        const StepState *__restrict__ st) {
    const float total = norm[0], max_norm = st->max_norm;
    if (!(max_norm > 0.0f) || !(total > max_norm)) return;          // same rule as clip_grad_norm: no scaling at or below the bound
    const float scale = max_norm / total;
    int t = find_tensor(tab, nt, blockIdx.x);
    TensorRef r = tab[t];
    int64_t start = (int64_t)(blockIdx.x - r.first_chunk) * kChunk;
    int64_t end = start + kChunk < r.n ? start + kChunk : r.n;
    for (int64_t i = start + threadIdx.x; i < end; i += 256) r.g[i] *= scale;
}
// TensorRef.lr holds the per-tensor multiplier here; the step's learning rate comes from the state
__global__ void __launch_bounds__(256) adamw_dev_kernel(const TensorRef *__restrict__ tab, int nt, AdamHyper h0,
                                                        const StepState *__restrict__ st) {
    AdamHyper h = h0;
    h.bc1 = st->bc1; h.bc2_sqrt = st->bc2_sqrt;
    int t = find_tensor(tab, nt, blockIdx.x);
    TensorRef r = tab[t];
    r.lr = st->lr * r.lr;
    int64_t start = (int64_t)(blockIdx.x - r.first_chunk) * kChunk;
    int64_t end = start + kChunk < r.n ? start + kChunk : r.n;
    float step = r.lr / h.bc1;
    bool vec = ((((uintptr_t)r.p | (uintptr_t)r.g | (uintptr_t)r.m | (uintptr_t)r.v) & 15) == 0);
    if (vec) {
        int64_t e4 = start + ((end - start) & ~(int64_t)3);
        for (int64_t i = start + threadIdx.x * 4; i < e4; i += 1024) {
            float4 p = *(float4 *)(r.p + i), g = *(const float4 *)(r.g + i), m = *(float4 *)(r.m + i), v = *(float4 *)(r.v + i);
            adam1(p.x, m.x, v.x, g.x, r.lr, step, h); adam1(p.y, m.y, v.y, g.y, r.lr, step, h);
            adam1(p.z, m.z, v.z, g.z, r.lr, step, h); adam1(p.w, m.w, v.w, g.w, r.lr, step, h);
            *(float4 *)(r.p + i) = p; *(float4 *)(r.m + i) = m; *(float4 *)(r.v + i) = v;
        }
        start = e4;
    }
    for (int64_t i = start + threadIdx.x; i < end; i += 256) adam1(r.p[i], r.m[i], r.v[i], r.g[i], r.lr, step, h);
}

static int upload_table(std::vector<TensorRef> &tab) {
    int chunks = 0;
    for (auto &r : tab) { r.first_chunk = chunks; chunks += (int)((r.n + kChunk - 1) / kChunk); }
    if (tab.size() > g_os.tab_cap) {
        CUDA_OK(cudaStreamSynchronize(stream()));
        if (g_os.tab) CUDA_OK(cudaFree(g_os.tab));
        g_os.tab_cap = tab.size() * 2 + 64;
        CUDA_OK(cudaMalloc((void **)&g_os.tab, g_os.tab_cap * sizeof(TensorRef)));
    }
    if ((size_t)chunks > g_os.part_cap) {
        CUDA_OK(cudaStreamSynchronize(stream()));
        if (g_os.partial) CUDA_OK(cudaFree(g_os.partial));
        g_os.part_cap = (size_t)chunks * 2 + 1024;
        CUDA_OK(cudaMalloc((void **)&g_os.partial, g_os.part_cap * sizeof(double)));
    }
    if (!g_os.norm) { CUDA_OK(cudaMalloc((void **)&g_os.norm, sizeof(float))); CUDA_OK(cudaMalloc((void **)&g_os.sq, sizeof(double))); }
    CUDA_OK(cudaMemcpyAsync(g_os.tab, tab.data(), tab.size() * sizeof(TensorRef), cudaMemcpyHostToDevice, stream()));
    return chunks;
}

static std::vector<TensorRef> grad_table(tensor **params, int n_params) {
    std::vector<TensorRef> tab;
    for (int i = 0; i < n_params; i++) {
        float *g = params[i]->grad;
        if (!g) continue;
        grad_settle(params[i]);
        TensorRef r; r.p = nullptr; r.g = g; r.m = r.v = nullptr; r.n = numel_of(params[i]); r.lr = 0.f; r.first_chunk = 0;
        if (r.n > 0) tab.push_back(r);
    }
    return tab;
}

// Sum of squared gradients -> device scalars; returns false when no grads exist.
static bool grad_sumsq_device(tensor **params, int n_params, std::vector<TensorRef> &tab, int &chunks) {
    tab = grad_table(params, n_params);
    if (tab.empty()) return false;
    chunks = upload_table(tab);
    sumsq_kernel<<<chunks, 256, 0, stream()>>>(g_os.tab, (int)tab.size(), g_os.partial);
    { double b = 0; for (auto &r : tab) b += 4.0 * (double)r.n; prof_work(b); }
    LAUNCHED("grad_sumsq_kernel");
    sumsq_final_kernel<<<1, 1024, 0, stream()>>>(g_os.partial, chunks, g_os.norm, g_os.sq);
    LAUNCHED("grad_sumsq_final_kernel");
    return true;
}

static float lr_at(const lr_scheduler *s, int t) {
    // src/optim.c:104-150
    float base = s->base_lr;
    if (s->warmup_iters > 0 && t < s->warmup_iters) return base * (float)(t + 1) / (float)s->warmup_iters;
    int post = t - s->warmup_iters;
    if (post < 0) post = 0;
    switch (s->schedule) {
    case LR_SCHEDULE_COSINE:
    case LR_SCHEDULE_LINEAR_WARMUP_COSINE: {
        int decay = s->total_iters - s->warmup_iters;
        if (decay <= 0) return base;
        float c = 0.5f * (1.0f + cosf((float)M_PI * post / decay));
        return s->min_lr + (base - s->min_lr) * c;
    }
    case LR_SCHEDULE_STEP:
        if (s->step_size <= 0) return base;
        return base * powf(s->gamma, (float)(post / s->step_size));
    case LR_SCHEDULE_EXPONENTIAL:
        if (post == 0) return base;
        return base * powf(s->gamma, (float)post);
    default:
        return base;
    }
}

}  // namespace dnnb

using namespace dnnb;

extern "C" {

adamw_opt *adamw_create(struct mem_pool *params_pool, tensor **params, int n_params, float lr,
                        float beta1, float beta2, float eps, float weight_decay) {
    adamw_opt *opt = host_alloc_t<adamw_opt>(params_pool);
    opt->params = params; opt->n_params = n_params; opt->lr = lr;
    opt->beta1 = beta1; opt->beta2 = beta2; opt->eps = eps; opt->weight_decay = weight_decay; opt->t = 0;
    opt->m = host_alloc_t<tensor *>(params_pool, n_params);
    opt->v = host_alloc_t<tensor *>(params_pool, n_params);
    for (int i = 0; i < n_params; i++) {
        opt->m[i] = tensor_zeros(params_pool, params[i]->ndim, params[i]->shape, 0);
        opt->v[i] = tensor_zeros(params_pool, params[i]->ndim, params[i]->shape, 0);
    }
    return opt;
}
void adamw_free(adamw_opt *opt) { (void)opt; }

// ── optimiser state files ────────────────────────────────────────────────
// The reference saves weights only (module_save, src/module.c:208-268), so a run cannot be
// resumed.  This file holds what is missing: magic "DNNO", u32 version = 1, u32 n_params,
// i32 t, f32 lr, beta1, beta2, eps, weight_decay, then per parameter u32 numel, float m[numel],
// float v[numel], in the optimiser's parameter order.  Together with module_save it restores a
// run bit for bit (the kernels are deterministic).
int dnn_cuda_optimizer_save(const adamw_opt *opt, const char *path) {
    if (!opt || !path) return -1;
    FILE *f = fopen(path, "wb");
    if (!f) return -2;
    uint32_t version = 1, n = (uint32_t)opt->n_params;
    int32_t t = opt->t;
    float hyper[5] = {opt->lr, opt->beta1, opt->beta2, opt->eps, opt->weight_decay};
    bool ok = fwrite("DNNO", 1, 4, f) == 4 && fwrite(&version, 4, 1, f) == 1 && fwrite(&n, 4, 1, f) == 1 &&
              fwrite(&t, 4, 1, f) == 1 && fwrite(hyper, 4, 5, f) == 5;
    std::vector<float> host;
    for (int i = 0; ok && i < opt->n_params; i++) {
        uint32_t numel = (uint32_t)numel_of(opt->params[i]);
        host.resize(numel);
        ok = fwrite(&numel, 4, 1, f) == 1;
        for (tensor *s : {opt->m[i], opt->v[i]}) {
            ok = ok && dnn_cuda_download(s, host.data(), (size_t)numel * 4) == 0 && fwrite(host.data(), 4, numel, f) == numel;
        }
    }
    ok = (fclose(f) == 0) && ok;
    return ok ? 0 : -3;
}

// Loads into an optimiser created for the same parameters (count and sizes are checked).
// Hyper-parameters come from the file as well, t included.
int dnn_cuda_optimizer_load(adamw_opt *opt, const char *path) {
    if (!opt || !path) return -1;
    FILE *f = fopen(path, "rb");
    if (!f) return -2;
    char magic[4]; uint32_t version = 0, n = 0; int32_t t = 0; float hyper[5];
    bool ok = fread(magic, 1, 4, f) == 4 && memcmp(magic, "DNNO", 4) == 0 && fread(&version, 4, 1, f) == 1 && version == 1 &&
              fread(&n, 4, 1, f) == 1 && (int)n == opt->n_params && fread(&t, 4, 1, f) == 1 && fread(hyper, 4, 5, f) == 5;
    std::vector<float> host;
    for (int i = 0; ok && i < opt->n_params; i++) {
        uint32_t numel = 0;
        ok = fread(&numel, 4, 1, f) == 1 && (int64_t)numel == numel_of(opt->params[i]);
        if (!ok) break;
        host.resize(numel);
        for (tensor *s : {opt->m[i], opt->v[i]})
            ok = ok && fread(host.data(), 4, numel, f) == numel && dnn_cuda_upload(s, host.data(), (size_t)numel * 4) == 0;
    }
    fclose(f);
    if (!ok) return -3;
    opt->t = t; opt->lr = hyper[0]; opt->beta1 = hyper[1]; opt->beta2 = hyper[2]; opt->eps = hyper[3]; opt->weight_decay = hyper[4];
    return 0;
}

// Whole resume state: the optimiser file above followed by a tail with what else a run carries between
// steps -- the scheduler's step count (it keeps its own, src/optim.c:104-189) and the state of the calling
// thread's default host generator (dropout masks and weight initialisation draw from it,
// src/ops_activation.c:1460, src/rng.c:70).  Tail: magic "DNNT", u32 has_scheduler, i32 scheduler_t,
// u64 rng_s0, u64 rng_s1.
int dnn_cuda_train_state_save(const adamw_opt *opt, const lr_scheduler *sched, const char *path) {
    int rc = dnn_cuda_optimizer_save(opt, path);
    if (rc != 0) return rc;
    FILE *f = fopen(path, "ab");
    if (!f) return -2;
    uint32_t has = sched ? 1u : 0u;
    int32_t st = sched ? sched->t : 0;
    const dnn_rng *r = dnn_get_rng();
    uint64_t s[2] = {r->s[0], r->s[1]};
    bool ok = fwrite("DNNT", 1, 4, f) == 4 && fwrite(&has, 4, 1, f) == 1 && fwrite(&st, 4, 1, f) == 1 && fwrite(s, 8, 2, f) == 2;
    ok = (fclose(f) == 0) && ok;
    return ok ? 0 : -3;
}
// Restores the optimiser, then the tail: sched->t and the learning rate that follows from it (when both the
// file and the caller have a scheduler) and the default host generator.
int dnn_cuda_train_state_load(adamw_opt *opt, lr_scheduler *sched, const char *path) {
    int rc = dnn_cuda_optimizer_load(opt, path);
    if (rc != 0) return rc;
    FILE *f = fopen(path, "rb");
    if (!f) return -2;
    char magic[4]; uint32_t has = 0; int32_t st = 0; uint64_t s[2] = {0, 0};
    bool ok = fseek(f, -28L, SEEK_END) == 0 && fread(magic, 1, 4, f) == 4 && memcmp(magic, "DNNT", 4) == 0 &&
              fread(&has, 4, 1, f) == 1 && fread(&st, 4, 1, f) == 1 && fread(s, 8, 2, f) == 2;
    fclose(f);
    if (!ok) return -3;
    if (sched && has) { sched->t = st; sched->opt->lr = lr_at(sched, st); }
    dnn_rng *r = dnn_get_rng();
    r->s[0] = s[0]; r->s[1] = s[1];
    return 0;
}

// The reference memsets every parameter gradient here (src/optim.c:93-100).  The buffers are
// only marked fresh: the first backward contribution of the step (a dW GEMM that covers the
// whole tensor) stores instead of adding, and whatever is still fresh when gradients are
// read (grad norm, clipping, AdamW, all-reduce, download) is zero-filled then.
void adamw_zero_grad(adamw_opt *opt) {
    for (int i = 0; i < opt->n_params; i++)
        if (opt->params[i]->grad) opt->params[i]->grad_fresh = 1;
}

float grad_norm(tensor **params, int n_params) {
    std::vector<TensorRef> tab; int chunks = 0;
    if (!grad_sumsq_device(params, n_params, tab, chunks)) return 0.0f;
    float h = 0.f;
    dnn_cuda_memcpy_d2h(&h, g_os.norm, sizeof h);
    return h;
}

float clip_grad_norm(tensor **params, int n_params, float max_norm) {
    if (max_norm <= 0.0f) return 0.0f;
    std::vector<TensorRef> tab; int chunks = 0;
    if (!grad_sumsq_device(params, n_params, tab, chunks)) return 0.0f;
    float total = 0.f;
    dnn_cuda_memcpy_d2h(&total, g_os.norm, sizeof total);     // the API returns the norm: one sync per step
    if (total > max_norm) {
        float scale = max_norm / total;
        scale_kernel<<<chunks, 256, 0, stream()>>>(g_os.tab, (int)tab.size(), scale);
        { double b = 0; for (auto &r : tab) b += 8.0 * (double)r.n; prof_work(b); }
        LAUNCHED("grad_scale_kernel");
    }
    return total;
}

void adamw_step_with_lr_multipliers(adamw_opt *opt, const float *lr_mults) {
    opt->t++;
    AdamHyper h;
    h.b1 = opt->beta1; h.b2 = opt->beta2; h.eps = opt->eps; h.wd = opt->weight_decay;
    h.bc1 = 1.0f - powf(h.b1, (float)opt->t);
    h.bc2_sqrt = sqrtf(1.0f - powf(h.b2, (float)opt->t));
    std::vector<TensorRef> tab;
    for (int i = 0; i < opt->n_params; i++) {
        tensor *p = opt->params[i];
        if (!p->grad) continue;                    // not in the backward graph (src/optim.c:287)
        grad_settle(p);
        TensorRef r;
        r.p = tensor_data_ptr(p); r.g = p->grad; r.m = tensor_data_ptr(opt->m[i]); r.v = tensor_data_ptr(opt->v[i]);
        r.n = numel_of(p); r.lr = opt->lr * (lr_mults ? lr_mults[i] : 1.0f); r.first_chunk = 0;
        if (r.n > 0) tab.push_back(r);
    }
    if (tab.empty()) return;
    int chunks = upload_table(tab);
    double bytes = 0;
    for (auto &r : tab) bytes += 28.0 * (double)r.n;        // read p,g,m,v; write p,m,v
    prof_begin(1);
    adamw_kernel<<<chunks, 256, 0, stream()>>>(g_os.tab, (int)tab.size(), h);
    prof_work(bytes);
    LAUNCHED("adamw_kernel");
    prof_end(1, bytes);
}
void adamw_step(adamw_opt *opt) { adamw_step_with_lr_multipliers(opt, nullptr); }

}  // extern "C"

namespace dnnb {

// Optimiser tail of a captured step: its own tables and reduction buffers (the eager path's are
// re-uploaded on every call, which a graph cannot replay), a device StepState and its pinned
// host copy.
// The graph's copy node reads pinned host memory when the graph EXECUTES, not when it is
// launched, so replays queued back to back without a readback must not share one host struct:
// the state lives in a ring of kStateSlots pinned structs, each replay points the copy node at
// the next slot (cudaGraphExecMemcpyNodeSetParams1D) and a slot is rewritten only after the
// replay that last read it has finished (one event per slot).
constexpr int kStateSlots = 8;
struct OptGraph {
    TensorRef *tab = nullptr; int nt = 0, chunks = 0;
    double *partial = nullptr, *sq = nullptr; float *norm = nullptr;
    StepState *state_dev = nullptr, *state_host = nullptr;       // state_host: kStateSlots structs
    cudaEvent_t slot_done[kStateSlots] = {};
    bool slot_used[kStateSlots] = {};
    int next_slot = 0;
    float max_norm = 0.0f;
    AdamHyper h;
};

// Outside capture.  Every parameter must already own a gradient buffer (one eager step has run).
OptGraph *opt_graph_prepare(adamw_opt *opt, float grad_clip) {
    OptGraph *og = new OptGraph();
    std::vector<TensorRef> tab;
    int chunks = 0;
    for (int i = 0; i < opt->n_params; i++) {
        tensor *p = opt->params[i];
        if (!p->grad) continue;
        TensorRef r;
        r.p = tensor_data_ptr(p); r.g = p->grad; r.m = tensor_data_ptr(opt->m[i]); r.v = tensor_data_ptr(opt->v[i]);
        r.n = numel_of(p); r.lr = 1.0f; r.first_chunk = chunks;
        if (r.n <= 0) continue;
        chunks += (int)((r.n + kChunk - 1) / kChunk);
        tab.push_back(r);
    }
    DNN_CHECK(!tab.empty(), "step graph: no parameter has a gradient yet; run one eager step first");
    og->nt = (int)tab.size(); og->chunks = chunks;
    CUDA_OK(cudaMalloc((void **)&og->tab, tab.size() * sizeof(TensorRef)));
    CUDA_OK(cudaMemcpy(og->tab, tab.data(), tab.size() * sizeof(TensorRef), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMalloc((void **)&og->partial, (size_t)chunks * sizeof(double)));
    CUDA_OK(cudaMalloc((void **)&og->sq, sizeof(double)));
    CUDA_OK(cudaMalloc((void **)&og->norm, sizeof(float)));
    CUDA_OK(cudaMalloc((void **)&og->state_dev, sizeof(StepState)));
    CUDA_OK(cudaMallocHost((void **)&og->state_host, kStateSlots * sizeof(StepState)));
    memset(og->state_host, 0, kStateSlots * sizeof(StepState));
    for (int i = 0; i < kStateSlots; i++) CUDA_OK(cudaEventCreateWithFlags(&og->slot_done[i], cudaEventDisableTiming));
    og->h.b1 = opt->beta1; og->h.b2 = opt->beta2; og->h.eps = opt->eps; og->h.wd = opt->weight_decay; og->h.bc1 = og->h.bc2_sqrt = 1.0f;
    og->max_norm = grad_clip;
    return og;
}
// Inside capture, after backward: norm, clip, AdamW.
void opt_graph_launch(OptGraph *og, adamw_opt *opt) {
    for (int i = 0; i < opt->n_params; i++) if (opt->params[i]->grad) grad_settle(opt->params[i]);
    CUDA_OK(cudaMemcpyAsync(og->state_dev, og->state_host, sizeof(StepState), cudaMemcpyHostToDevice, stream()));
    sumsq_kernel<<<og->chunks, 256, 0, stream()>>>(og->tab, og->nt, og->partial);
    LAUNCHED("grad_sumsq_kernel");
    sumsq_final_kernel<<<1, 1024, 0, stream()>>>(og->partial, og->chunks, og->norm, og->sq);
    LAUNCHED("grad_sumsq_final_kernel");
    scale_dev_kernel<<<og->chunks, 256, 0, stream()>>>(og->tab, og->nt, og->norm, og->state_dev);
    LAUNCHED("grad_scale_kernel");
    adamw_dev_kernel<<<og->chunks, 256, 0, stream()>>>(og->tab, og->nt, og->h, og->state_dev);
    LAUNCHED("adamw_kernel");
}
// Before every replay: the step counter moves on the host, the graph reads the derived numbers.
// Returns the pinned struct this replay's copy node must read (see kStateSlots).
const void *opt_graph_advance(OptGraph *og, adamw_opt *opt) {
    opt->t++;
    const int slot = og->next_slot;
    og->next_slot = (slot + 1) % kStateSlots;
    if (og->slot_used[slot]) CUDA_OK(cudaEventSynchronize(og->slot_done[slot]));   // the replay kStateSlots ago
    StepState *st = og->state_host + slot;
    st->lr = opt->lr;
    st->bc1 = 1.0f - powf(opt->beta1, (float)opt->t);
    st->bc2_sqrt = sqrtf(1.0f - powf(opt->beta2, (float)opt->t));
    st->max_norm = og->max_norm;
    return st;
}
// After the replay has been launched: marks when the slot handed out by the last advance is free again.
void opt_graph_launched(OptGraph *og) {
    const int slot = (og->next_slot + kStateSlots - 1) % kStateSlots;
    CUDA_OK(cudaEventRecord(og->slot_done[slot], stream()));
    og->slot_used[slot] = true;
}
const void *opt_graph_state_dev(const OptGraph *og) { return og->state_dev; }
size_t opt_graph_state_bytes() { return sizeof(StepState); }
const float *opt_graph_norm(const OptGraph *og) { return og->norm; }
void opt_graph_destroy(OptGraph *og) {
    if (!og) return;
    cudaFree(og->tab); cudaFree(og->partial); cudaFree(og->sq); cudaFree(og->norm); cudaFree(og->state_dev); cudaFreeHost(og->state_host);
    for (int i = 0; i < kStateSlots; i++) if (og->slot_done[i]) cudaEventDestroy(og->slot_done[i]);
    delete og;
}

}  // namespace dnnb

extern "C" {

lr_scheduler *lr_scheduler_create(struct mem_pool *params_pool, adamw_opt *opt, int schedule, float base_lr,
                                  int warmup_iters, int total_iters, float min_lr, int step_size, float gamma) {
    lr_scheduler *s = host_alloc_t<lr_scheduler>(params_pool);
    s->opt = opt; s->schedule = schedule; s->base_lr = base_lr; s->warmup_iters = warmup_iters;
    s->total_iters = total_iters; s->step_size = step_size; s->gamma = gamma; s->t = 0;
    s->min_lr = (min_lr < 0.0f) ? base_lr / 10.0f : min_lr;
    opt->lr = lr_at(s, 0);
    return s;
}
void  lr_scheduler_step(lr_scheduler *s) { s->t++; s->opt->lr = lr_at(s, s->t); }
float lr_scheduler_get_lr(const lr_scheduler *s) { return lr_at(s, s->t); }
void  lr_scheduler_reset(lr_scheduler *s) { s->t = 0; s->opt->lr = lr_at(s, 0); }
void  lr_scheduler_destroy(lr_scheduler *s) { (void)s; }

}  // extern "C"
