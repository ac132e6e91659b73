// Device runtime: the compute stream, the device arenas that shadow each
// mem_pool, payload transfer and error reporting.
//
// Pools: replaces src/pool.c:8-57 and src/context.c:5-35 of the reference.
// A mem_pool keeps its three public fields; `buffer` is a host mapping that
// holds structs and saved scalars, and a device arena of the same capacity is
// created on first payload allocation and found again through `buffer`.
#include "common.cuh"
#include <sys/mman.h>
#include <unordered_map>
#include <vector>
#include <mutex>
#include <string>

namespace dnnb {

struct Arena {
    char  *base = nullptr;
    size_t cap = 0, off = 0, peak = 0;
    size_t born_at = 0;                             // host offset of the pool when the arena was created (device offset 0)
    std::vector<std::pair<size_t, size_t>> marks;   // (host offset, device offset)
};

struct Runtime {
    bool         ready = false;
    int          device = 0;
    cudaStream_t compute = nullptr;
    int          gemm_mode = DNN_CUDA_GEMM_TF32;
    long long    launches = 0;
    std::string  last_error;
    std::unordered_map<const void *, Arena> arenas;   // keyed by mem_pool.buffer
};
static Runtime g_rt;
static std::mutex g_mu;

static void set_error(const std::string &s) { g_rt.last_error = s; }

void cuda_fail(cudaError_t e, const char *what, const char *file, int line) {
    char buf[512];
    snprintf(buf, sizeof buf, "CUDA error %d (%s) at %s:%d: %s", (int)e, cudaGetErrorString(e), file, line, what);
    set_error(buf);
    fprintf(stderr, "dnn_b200: %s\n", buf);
    abort();
}

static int init_device(int device, bool may_abort) {
    if (g_rt.ready) return 0;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        set_error(std::string("no usable CUDA device: ") + cudaGetErrorString(e));
        (void)cudaGetLastError();
        if (may_abort) {
            fprintf(stderr, "dnn_b200: %s. This library runs on the GPU only; there is no CPU fallback.\n",
                    g_rt.last_error.c_str());
            abort();
        }
        return -1;
    }
    if (device < 0 || device >= n) { set_error("device index out of range"); if (may_abort) abort(); return -2; }
    CUDA_OK(cudaSetDevice(device));
    CUDA_OK(cudaStreamCreateWithFlags(&g_rt.compute, cudaStreamNonBlocking));
    g_rt.device = device;
    const char *mode = getenv("DNN_CUDA_GEMM");
    if (mode) {
        if (!strcmp(mode, "fp32")) g_rt.gemm_mode = DNN_CUDA_GEMM_FP32;
        else if (!strcmp(mode, "tf32")) g_rt.gemm_mode = DNN_CUDA_GEMM_TF32;
        else if (!strcmp(mode, "3xtf32")) g_rt.gemm_mode = DNN_CUDA_GEMM_3XTF32;
    }
    g_rt.ready = true;
    return 0;
}

cudaStream_t stream() {
    if (!g_rt.ready) init_device(0, true);
    return g_rt.compute;
}

// Per-launch timeline (dnn_cuda_profile_enable(2)): one event after every launch on the compute stream.
// Launches are serialised on that stream and the host runs ahead of the device, so the time between two
// consecutive events is the duration of the later kernel.
struct LaunchRec { const char *name; cudaEvent_t after; double work; };
static bool g_timeline_on = false;
static std::vector<LaunchRec> g_timeline;
static cudaEvent_t g_timeline_start = nullptr;
static double g_next_work = 0.0;
static cudaEvent_t get_event();
void prof_work(double work) { g_next_work = work; }

void launched(const char *name) {
    g_rt.launches++;
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        char buf[256];
        snprintf(buf, sizeof buf, "launch of %s", name);
        cuda_fail(e, buf, __FILE__, __LINE__);
    }
    if (g_timeline_on) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(g_rt.compute, &cs) == cudaSuccess && cs == cudaStreamCaptureStatusNone) {
            cudaEvent_t ev = get_event();
            CUDA_OK(cudaEventRecord(ev, g_rt.compute));
            g_timeline.push_back(LaunchRec{name, ev, g_next_work});
        }
    }
    g_next_work = 0.0;
}

// kernels that ran (or, negative, were only recorded) without passing through launched()
void add_launches(long long n) { g_rt.launches += n; }

int gemm_mode() { return g_rt.gemm_mode; }

// ---- profiling ------------------------------------------------------------------
struct ProfRec { cudaEvent_t a, b; double work; };
struct ProfClass { std::vector<ProfRec> recs; cudaEvent_t pending = nullptr; };
static bool g_prof_on = false;
static ProfClass g_prof[2];
static std::vector<cudaEvent_t> g_event_pool;
static cudaEvent_t g_timer_a = nullptr, g_timer_b = nullptr;

static cudaEvent_t get_event() {
    if (!g_event_pool.empty()) { cudaEvent_t e = g_event_pool.back(); g_event_pool.pop_back(); return e; }
    cudaEvent_t e; CUDA_OK(cudaEventCreate(&e)); return e;
}
void prof_begin(int c) {
    if (!g_prof_on) return;
    g_prof[c].pending = get_event();
    CUDA_OK(cudaEventRecord(g_prof[c].pending, stream()));
}
void prof_end(int c, double work) {
    if (!g_prof_on || !g_prof[c].pending) return;
    cudaEvent_t b = get_event();
    CUDA_OK(cudaEventRecord(b, stream()));
    g_prof[c].recs.push_back(ProfRec{g_prof[c].pending, b, work});
    g_prof[c].pending = nullptr;
}

static Arena *arena_of(const mem_pool *pool, bool create) {
    DNN_CHECK(pool && pool->buffer, "pool is NULL or destroyed");
    auto it = g_rt.arenas.find(pool->buffer);
    if (it != g_rt.arenas.end()) return &it->second;
    if (!create) return nullptr;
    stream();   // make sure the device is initialised (aborts without one)
    Arena a;
    a.cap = pool->capacity;
    a.born_at = pool->offset;
    cudaError_t e = cudaMalloc((void **)&a.base, a.cap ? a.cap : 256);
    if (e != cudaSuccess) {
        fprintf(stderr, "dnn_b200: cannot reserve %zu bytes of device memory for a pool\n", a.cap);
        cuda_fail(e, "cudaMalloc(pool arena)", __FILE__, __LINE__);
    }
    return &(g_rt.arenas[pool->buffer] = a);
}

bool dev_ptr_in_arena(const void *p) {
    const char *c = (const char *)p;
    for (auto &kv : g_rt.arenas)
        if (c >= kv.second.base && c < kv.second.base + kv.second.cap) return true;
    return false;
}

void require_device_payloads(const char *op, std::initializer_list<const tensor *> ts) {
    for (const tensor *t : ts) {
        if (!t || !t->data || dev_ptr_in_arena(t->data)) continue;
        cudaPointerAttributes at;
        cudaError_t e = cudaPointerGetAttributes(&at, t->data);
        if (e == cudaSuccess && (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged)) continue;
        cudaGetLastError();
        fprintf(stderr, "dnn_b200: %s: a tensor's payload (data = %p, pool = %p) is host memory.  This library computes on the GPU: "
                        "create tensors with tensor_scratch / tensor_zeros* in a dnn.c pool and fill them with dnn_cuda_upload "
                        "(read results with dnn_cuda_download); hand-built tensor structs around malloc'd buffers are not accepted.\n",
                op, t->data, (void *)t->pool);
        abort();
    }
}

void *dev_alloc(struct mem_pool *pool, size_t bytes, bool zero) {
    Arena *a = arena_of(pool, true);
    size_t need = (bytes + 255) & ~(size_t)255;
    if (need == 0) need = 256;
    if (a->off + need > a->cap) {
        fprintf(stderr, "dnn_b200: pool out of device memory (capacity %zu, used %zu, wanted %zu)\n",
                a->cap, a->off, need);
        abort();
    }
    void *p = a->base + a->off;
    a->off += need;
    if (a->off > a->peak) a->peak = a->off;
    if (zero) CUDA_OK(cudaMemsetAsync(p, 0, bytes, stream()));
    return p;
}

void *dev_put(struct mem_pool *pool, const void *host, size_t bytes) {
    void *d = dev_alloc(pool, bytes, false);
    // pageable source: the runtime stages it before returning, so `host` may die
    CUDA_OK(cudaMemcpyAsync(d, host, bytes, cudaMemcpyHostToDevice, stream()));
    return d;
}

}  // namespace dnnb

using namespace dnnb;

extern "C" {

// ── pools ───────────────────────────────────────────────────────────────
mem_pool mem_pool_create(size_t capacity) {
    mem_pool p;
    // Host side: address space only; pages are committed when touched.
    void *m = mmap(nullptr, capacity ? capacity : 4096, PROT_READ | PROT_WRITE,
                   MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    DNN_CHECK(m != MAP_FAILED, "mem_pool_create: cannot map host buffer");
    p.buffer = (char *)m;
    p.capacity = capacity;
    p.offset = 0;
    return p;
}

void mem_pool_destroy(mem_pool *pool) {
    if (!pool || !pool->buffer) return;
    grad_settle_all_deferred();
    auto it = g_rt.arenas.find(pool->buffer);
    if (it != g_rt.arenas.end()) {
        cudaStreamSynchronize(g_rt.compute);
        cudaFree(it->second.base);
        g_rt.arenas.erase(it);
    }
    munmap(pool->buffer, pool->capacity ? pool->capacity : 4096);
    pool->buffer = nullptr;
    pool->capacity = 0;
    pool->offset = 0;
}

void mem_pool_reset(mem_pool *pool) {
    grad_settle_all_deferred();
    pool->offset = 0;
    Arena *a = arena_of(pool, false);
    if (a) { a->off = 0; a->born_at = 0; a->marks.clear(); }
}

size_t mem_pool_mark(mem_pool *pool) {
    Arena *a = arena_of(pool, false);
    if (a) a->marks.emplace_back(pool->offset, a->off);
    return pool->offset;
}

void mem_pool_release(mem_pool *pool, size_t mark) {
    grad_settle_all_deferred();
    pool->offset = mark;
    Arena *a = arena_of(pool, false);
    if (!a) return;
    while (!a->marks.empty() && a->marks.back().first > mark) a->marks.pop_back();
    if (!a->marks.empty() && a->marks.back().first == mark) {
        a->off = a->marks.back().second;
        a->marks.pop_back();
    } else if (mark <= a->born_at) {
        // a mark taken before the pool had a device arena (nothing was on the device yet): everything goes
        a->off = 0;
    }
}

static inline size_t host_round(size_t b) { return (b + 15) & ~(size_t)15; }

void *_mem_pool_alloc(struct mem_pool *pool, size_t bytes, const void *src) {
    size_t need = host_round(bytes);
    DNN_CHECK(pool->offset + need <= pool->capacity, "_mem_pool_alloc: out of memory");
    void *p = pool->buffer + pool->offset;
    if (src) memcpy(p, src, bytes); else memset(p, 0, bytes);
    pool->offset += need;
    return p;
}

void *_mem_pool_alloc_nz(struct mem_pool *pool, size_t bytes) {
    size_t need = host_round(bytes);
    DNN_CHECK(pool->offset + need <= pool->capacity, "_mem_pool_alloc_nz: out of memory");
    void *p = pool->buffer + pool->offset;
    pool->offset += need;
    return p;
}

int dnn_ctx_init(dnn_ctx *ctx, size_t params_sz, size_t scratch_sz, size_t data_sz) {
    mem_pool *p = (mem_pool *)malloc(sizeof(mem_pool));
    mem_pool *s = (mem_pool *)malloc(sizeof(mem_pool));
    mem_pool *d = (mem_pool *)malloc(sizeof(mem_pool));
    if (!p || !s || !d) { free(p); free(s); free(d); return -1; }
    *p = mem_pool_create(params_sz);
    *s = mem_pool_create(scratch_sz);
    *d = mem_pool_create(data_sz);
    ctx->params = p; ctx->scratch = s; ctx->data = d;
    return 0;
}

void dnn_ctx_reset_step(dnn_ctx *ctx) {
    mem_pool_reset(ctx->scratch);
    mem_pool_reset(ctx->data);
}

void dnn_ctx_destroy(dnn_ctx *ctx) {
    mem_pool **ps[3] = {&ctx->params, &ctx->scratch, &ctx->data};
    for (auto pp : ps) if (*pp) { mem_pool_destroy(*pp); free(*pp); *pp = nullptr; }
}

// ── dnn_cuda_* ──────────────────────────────────────────────────────────
int dnn_cuda_init(int device) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_rt.ready) return g_rt.device == device ? 0 : -3;
    return init_device(device, false);
}

int dnn_cuda_available(void) {
    if (g_rt.ready) return 1;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    return n > 0;
}

int dnn_cuda_sync(void) {
    cudaError_t e = cudaStreamSynchronize(stream());
    if (e != cudaSuccess) { set_error(cudaGetErrorString(e)); return -1; }
    int ge = gemm_tc_error();
    int ae = attn_tc_error();
    int ne = norm_error();
    if (ge || ae || ne) {
        char buf[200];
        snprintf(buf, sizeof buf, "a bounded barrier wait gave up (gemm code 0x%x, attention code 0x%x, norm backward %d)", ge, ae, ne);
        set_error(buf);
        return -5;
    }
    return 0;
}

const char *dnn_cuda_last_error(void) { return g_rt.last_error.c_str(); }
void *dnn_cuda_stream(void) { return (void *)stream(); }

static int xfer(void *dst, const void *src, size_t bytes, cudaMemcpyKind kind, bool wait) {
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, kind, stream());
    if (e == cudaSuccess && wait) e = cudaStreamSynchronize(stream());
    if (e != cudaSuccess) { set_error(std::string("copy failed: ") + cudaGetErrorString(e)); return -1; }
    return 0;
}

int dnn_cuda_upload(tensor *t, const void *host_src, size_t bytes) {
    if (!t || !t->data || !t->contiguous) { set_error("upload: tensor must be contiguous with a payload"); return -2; }
    if (bytes > (size_t)numel_of(t) * 4) { set_error("upload: more bytes than the tensor holds"); return -3; }
    return xfer((float *)t->data + t->offset, host_src, bytes, cudaMemcpyHostToDevice, false);
}

int dnn_cuda_download(const tensor *t, void *host_dst, size_t bytes) {
    if (!t || !t->data || !t->contiguous) { set_error("download: tensor must be contiguous with a payload"); return -2; }
    if (bytes > (size_t)numel_of(t) * 4) { set_error("download: more bytes than the tensor holds"); return -3; }
    return xfer(host_dst, (const float *)t->data + t->offset, bytes, cudaMemcpyDeviceToHost, true);
}

int dnn_cuda_download_grad(const tensor *t, void *host_dst, size_t bytes) {
    if (!t || !t->grad) { set_error("download_grad: tensor has no grad"); return -2; }
    grad_settle((tensor *)t);
    if (bytes > (size_t)numel_of(t) * 4) { set_error("download_grad: more bytes than the tensor holds"); return -3; }
    return xfer(host_dst, t->grad, bytes, cudaMemcpyDeviceToHost, true);
}

int dnn_cuda_memcpy_h2d(void *dev_dst, const void *host_src, size_t bytes) {
    return xfer(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, false);
}
int dnn_cuda_memcpy_d2h(void *host_dst, const void *dev_src, size_t bytes) {
    return xfer(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, true);
}

void *dnn_cuda_host_alloc(size_t bytes) {
    stream();
    void *p = nullptr;
    if (cudaMallocHost(&p, bytes) != cudaSuccess) { set_error("cudaMallocHost failed"); return nullptr; }
    return p;
}
void dnn_cuda_host_free(void *p) { if (p) cudaFreeHost(p); }

int dnn_cuda_timer_start(void) {
    if (!g_timer_a) { CUDA_OK(cudaEventCreate(&g_timer_a)); CUDA_OK(cudaEventCreate(&g_timer_b)); }
    CUDA_OK(cudaEventRecord(g_timer_a, stream()));
    return 0;
}
float dnn_cuda_timer_stop_ms(void) {
    if (!g_timer_a) return -1.0f;
    CUDA_OK(cudaEventRecord(g_timer_b, stream()));
    CUDA_OK(cudaEventSynchronize(g_timer_b));
    float ms = 0.f;
    CUDA_OK(cudaEventElapsedTime(&ms, g_timer_a, g_timer_b));
    return ms;
}
int dnn_cuda_profile_enable(int on) {
    CUDA_OK(cudaStreamSynchronize(stream()));
    for (auto &c : g_prof) { for (auto &r : c.recs) { g_event_pool.push_back(r.a); g_event_pool.push_back(r.b); } c.recs.clear(); c.pending = nullptr; }
    for (auto &r : g_timeline) g_event_pool.push_back(r.after);
    g_timeline.clear();
    g_prof_on = on == 1;
    g_timeline_on = on == 2;
    if (g_timeline_on) {
        if (!g_timeline_start) CUDA_OK(cudaEventCreate(&g_timeline_start));
        CUDA_OK(cudaEventRecord(g_timeline_start, stream()));
    }
    return 0;
}
// Sums the timeline by kernel name.  Returns the number of distinct names; fills up to `cap` rows.
int dnn_cuda_profile_kernels(dnn_cuda_kernel_time *rows, int cap) {
    CUDA_OK(cudaStreamSynchronize(stream()));
    std::vector<dnn_cuda_kernel_time> acc;
    cudaEvent_t prev = g_timeline_start;
    for (auto &r : g_timeline) {
        float ms = 0.f;
        CUDA_OK(cudaEventElapsedTime(&ms, prev, r.after));
        prev = r.after;
        size_t i = 0;
        for (; i < acc.size(); i++) if (!strcmp(acc[i].name, r.name)) break;
        if (i == acc.size()) {
            dnn_cuda_kernel_time t;
            memset(&t, 0, sizeof t);
            snprintf(t.name, sizeof t.name, "%s", r.name);
            acc.push_back(t);
        }
        acc[i].launches++; acc[i].ms += ms; acc[i].work += r.work;
    }
    for (int i = 0; i < (int)acc.size() && i < cap; i++) rows[i] = acc[i];
    return (int)acc.size();
}
int dnn_cuda_profile_read(int kernel_class, long long *launches, double *ms, double *work) {
    if (kernel_class < 0 || kernel_class > 1) return -1;
    CUDA_OK(cudaStreamSynchronize(stream()));
    double tms = 0, tw = 0;
    for (auto &r : g_prof[kernel_class].recs) { float e = 0; CUDA_OK(cudaEventElapsedTime(&e, r.a, r.b)); tms += e; tw += r.work; }
    if (launches) *launches = (long long)g_prof[kernel_class].recs.size();
    if (ms) *ms = tms;
    if (work) *work = tw;
    return 0;
}

int dnn_cuda_set_tf32_policy(unsigned roles_3x, double max_flop_3x) {
    gemm_reread_env();
    if (roles_3x > 7u || !(max_flop_3x >= 0.0)) { set_error("tf32 policy: roles is a 3-bit mask, max_flop must be >= 0"); return -1; }
    gemm_set_policy(roles_3x, max_flop_3x);
    return 0;
}
int dnn_cuda_set_exact_policy(double simt_max_flop) {
    if (!(simt_max_flop >= 0.0)) { set_error("exact policy: simt_max_flop must be >= 0"); return -1; }
    gemm_set_exact_policy(simt_max_flop);
    return 0;
}
double dnn_cuda_get_exact_policy(void) { return gemm_get_exact_policy(); }
int dnn_cuda_get_tf32_policy(unsigned *roles_3x, double *max_flop_3x) {
    if (!roles_3x || !max_flop_3x) return -1;
    gemm_get_policy(roles_3x, max_flop_3x);
    return 0;
}

int dnn_cuda_set_gemm_mode(int mode) {
    if (mode < 0 || mode > 2) { set_error("unknown gemm mode"); return -1; }
    g_rt.gemm_mode = mode;
    return 0;
}
int dnn_cuda_get_gemm_mode(void) { return g_rt.gemm_mode; }
long long dnn_cuda_launch_count(void) { return g_rt.launches; }

size_t dnn_cuda_pool_device_used(const mem_pool *pool) {
    Arena *a = arena_of(pool, false);
    return a ? a->off : 0;
}
size_t dnn_cuda_pool_device_peak(const mem_pool *pool) {
    Arena *a = arena_of(pool, false);
    return a ? a->peak : 0;
}

}  // extern "C"
