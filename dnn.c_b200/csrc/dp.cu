// Data-parallel gradient exchange over NCCL (one process per GPU).
//
// The reference is single-process; this is the one exchange step data
// parallelism needs: after backward every rank holds the gradient of its own
// micro-batch, and the ranks average them in place.  Parameter gradients are
// bump-allocated back to back in the params arena (in the order backward first
// touches them), so neighbouring gradients are merged into address ranges and
// each range of up to DNN_CUDA_BUCKET_MB (default 64 MiB) is one ncclAllReduce.
// NCCL is opened with dlopen so that single-GPU use has no NCCL dependency.
#include "common.cuh"
#include <nccl.h>
#include <dlfcn.h>
#include <vector>
#include <utility>
#include <algorithm>
#include <string>

namespace dnnb {

struct NcclApi {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};
static NcclApi g_nccl;
static ncclComm_t g_comm = nullptr;
static int g_world = 1;
static std::string g_dp_error;

static bool load_nccl() {
    if (g_nccl.lib) return true;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) { g_nccl.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (g_nccl.lib) break; }
    if (!g_nccl.lib) { g_dp_error = std::string("cannot load libnccl: ") + dlerror(); return false; }
#define SYM(field, name) *(void **)(&g_nccl.field) = dlsym(g_nccl.lib, name); \
    if (!g_nccl.field) { g_dp_error = std::string("libnccl lacks ") + name; return false; }
    SYM(GetUniqueId, "ncclGetUniqueId") SYM(CommInitRank, "ncclCommInitRank") SYM(AllReduce, "ncclAllReduce")
    SYM(GroupStart, "ncclGroupStart") SYM(GroupEnd, "ncclGroupEnd") SYM(CommDestroy, "ncclCommDestroy")
    SYM(CommAbort, "ncclCommAbort") SYM(CommGetAsyncError, "ncclCommGetAsyncError") SYM(GetErrorString, "ncclGetErrorString")
#undef SYM
    return true;
}

static int nccl_fail(ncclResult_t r, const char *what) {
    g_dp_error = std::string(what) + ": " + (g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "nccl error");
    fprintf(stderr, "dnn_b200: %s\n", g_dp_error.c_str());
    return -1;
}

// Merges gradient buffers that sit back to back (up to the allocator's
// 256-byte padding) into spans and cuts the spans into buckets.
struct Span { char *p; size_t bytes; };
std::vector<Span> plan_buckets(std::vector<Span> grads, size_t bucket_bytes) {
    std::sort(grads.begin(), grads.end(), [](const Span &a, const Span &b) { return a.p < b.p; });
    std::vector<Span> merged;
    for (const Span &g : grads) {
        if (!merged.empty()) {
            Span &m = merged.back();
            char *end = m.p + m.bytes;
            char *pad_end = (char *)(((uintptr_t)end + 255) & ~(uintptr_t)255);
            if (g.p >= end && g.p <= pad_end) { m.bytes = (size_t)(g.p + g.bytes - m.p); continue; }
        }
        merged.push_back(g);
    }
    std::vector<Span> out;
    for (const Span &m : merged)
        for (size_t off = 0; off < m.bytes; off += bucket_bytes)
            out.push_back(Span{m.p + off, std::min(bucket_bytes, m.bytes - off)});
    return out;
}

// Every rank must issue the same collectives: same number of buckets, same sizes, same order.  A rank
// whose model differs (a parameter without a gradient, another allocation order) would leave the others
// waiting inside NCCL with no diagnosis.  So whenever a rank's bucket plan changes (first step, and the
// step after the gradient buffers were allocated) the ranks compare a fingerprint of the plan -- bucket
// count and a hash of the sizes -- with one tiny all-reduce (max of h and of ~h: both equal the local
// values on every rank only if all ranks hold the same h) and return an error instead of entering the
// exchange when they differ.
static uint64_t g_plan_seen = 0;
static unsigned long long *g_plan_dev = nullptr;
static uint64_t plan_fingerprint(const std::vector<Span> &buckets) {
    uint64_t h = 0xcbf29ce484222325ull ^ (uint64_t)buckets.size();
    for (const Span &b : buckets) { h ^= (uint64_t)b.bytes; h *= 0x100000001b3ull; }
    return h ? h : 1;
}
static int plan_agree(const std::vector<Span> &buckets, cudaStream_t s) {
    const uint64_t h = plan_fingerprint(buckets);
    if (h == g_plan_seen) return 0;
    if (!g_plan_dev) CUDA_OK(cudaMalloc((void **)&g_plan_dev, 2 * sizeof(unsigned long long)));
    unsigned long long host[2] = {h, ~h}, got[2] = {0, 0};
    CUDA_OK(cudaMemcpyAsync(g_plan_dev, host, sizeof host, cudaMemcpyHostToDevice, s));
    ncclResult_t r = g_nccl.AllReduce(g_plan_dev, g_plan_dev, 2, ncclUint64, ncclMax, g_comm, s);
    if (r != ncclSuccess) return nccl_fail(r, "ncclAllReduce (plan fingerprint)");
    CUDA_OK(cudaMemcpyAsync(got, g_plan_dev, sizeof got, cudaMemcpyDeviceToHost, s));
    CUDA_OK(cudaStreamSynchronize(s));
    if (got[0] != host[0] || got[1] != host[1]) {
        g_dp_error = "data-parallel ranks disagree on the gradient buckets (a different set of parameters has gradients, or they "
                     "were allocated in another order); no gradient was exchanged";
        fprintf(stderr, "dnn_b200: %s\n", g_dp_error.c_str());
        return -5;
    }
    g_plan_seen = h;
    return 0;
}

// ── exchange overlapped with backward ────────────────────────────────────
// Gradient buffers keep their addresses from the second step on, so the buckets are planned up
// front.  dnn_backward reports every parameter whose gradient is final; when all parameters
// that touch a bucket are final, the bucket's all-reduce is queued on a second stream behind an
// event recorded on the compute stream.  Buckets complete in the order backward finishes them,
// which is the same on every rank (same model, same tape), so the ranks issue their collectives
// in the same order.  The compute stream waits for the exchange before the gradient norm.
struct Overlap {
    bool active = false;
    cudaStream_t comm = nullptr;
    cudaEvent_t done = nullptr;
    std::vector<cudaEvent_t> ready;
    std::vector<Span> buckets;
    std::vector<int> remaining;                                // parameters not yet final, per bucket
    std::vector<char> launched;
    std::vector<std::pair<tensor *, std::vector<int>>> owners; // parameter -> buckets it touches
    std::vector<tensor *> all_params;
    int rc = 0;
};
static Overlap g_ov;

static size_t bucket_bytes() {
    size_t b = (size_t)64 << 20;
    if (const char *e = getenv("DNN_CUDA_BUCKET_MB")) { long v = atol(e); if (v > 0) b = (size_t)v << 20; }
    if (const char *e = getenv("DNN_CUDA_BUCKET_BYTES")) { long v = atol(e); if (v >= 1024) b = (size_t)v & ~(size_t)255; }
    return b;
}
static void launch_bucket(int b) {
    if (g_ov.launched[b]) return;
    g_ov.launched[b] = 1;
    if ((int)g_ov.ready.size() <= b) g_ov.ready.resize(b + 1, nullptr);
    if (!g_ov.ready[b]) CUDA_OK(cudaEventCreateWithFlags(&g_ov.ready[b], cudaEventDisableTiming));
    CUDA_OK(cudaEventRecord(g_ov.ready[b], stream()));
    CUDA_OK(cudaStreamWaitEvent(g_ov.comm, g_ov.ready[b], 0));
    const Span &s = g_ov.buckets[b];
    ncclResult_t r = g_nccl.AllReduce(s.p, s.p, s.bytes / 4, ncclFloat32, ncclAvg, g_comm, g_ov.comm);
    if (r != ncclSuccess) g_ov.rc = nccl_fail(r, "ncclAllReduce (overlapped)");
}
static void on_leaf_ready(tensor *leaf) {
    if (!g_ov.active) return;
    for (auto &o : g_ov.owners) {
        if (o.first != leaf) continue;
        grad_settle(leaf);                                   // a gradient nobody wrote this step is zeros
        for (int b : o.second)
            if (--g_ov.remaining[b] == 0) launch_bucket(b);
        return;
    }
}
bool dp_overlap_begin(tensor **params, int n_params) {
    g_ov.active = false;
    if (g_world == 1 || !g_comm) return false;
    // Off unless DNN_CUDA_DP_OVERLAP=1: on NVLink the exchange of the 124M model takes about 1.2 ms
    // of a 37 ms step, and run beside backward its kernels take SMs away from the persistent GEMMs,
    // which costs as much as it hides (measured on 2 GPUs: 37.7 ms overlapped, 37.4 ms in sequence).
    const char *ov = getenv("DNN_CUDA_DP_OVERLAP");
    if (!ov || ov[0] != '1') return false;
    // Parameters that own a gradient buffer take part.  On the first step none does (the buffers are allocated
    // during backward): the exchange then runs after backward.  A parameter outside the graph (img_proj.* of the
    // vision LM fed with images) never gets one and is skipped here as it is by AdamW; one that gets its first
    // buffer during THIS backward is exchanged after backward (dp_overlap_finish).
    std::vector<Span> grads;
    for (int i = 0; i < n_params; i++)
        if (params[i]->grad) grads.push_back(Span{(char *)params[i]->grad, (size_t)numel_of(params[i]) * 4});
    if (grads.empty()) return false;
    g_ov.all_params.assign(params, params + n_params);
    if (!g_ov.comm) {
        CUDA_OK(cudaStreamCreateWithFlags(&g_ov.comm, cudaStreamNonBlocking));
        CUDA_OK(cudaEventCreateWithFlags(&g_ov.done, cudaEventDisableTiming));
    }
    g_ov.buckets = plan_buckets(grads, bucket_bytes());
    if (plan_agree(g_ov.buckets, stream()) != 0) return false;       // the serial path reports the disagreement
    const int nb = (int)g_ov.buckets.size();
    g_ov.remaining.assign(nb, 0);
    g_ov.launched.assign(nb, 0);
    g_ov.owners.clear();
    g_ov.rc = 0;
    for (int i = 0; i < n_params; i++) {
        if (!params[i]->grad) continue;
        char *lo = (char *)params[i]->grad, *hi = lo + (size_t)numel_of(params[i]) * 4;
        std::vector<int> touch;
        for (int b = 0; b < nb; b++) {
            const Span &s = g_ov.buckets[b];
            if (lo < s.p + s.bytes && hi > s.p) { touch.push_back(b); g_ov.remaining[b]++; }
        }
        g_ov.owners.emplace_back(params[i], touch);
    }
    g_ov.active = true;
    set_leaf_ready_observer(on_leaf_ready);
    return true;
}
int dp_overlap_finish() {
    set_leaf_ready_observer(nullptr);
    if (!g_ov.active) return 0;
    g_ov.active = false;
    // parameters outside the tape never report: settle them and send what is left
    for (auto &o : g_ov.owners) grad_settle(o.first);
    for (int b = 0; b < (int)g_ov.buckets.size(); b++) launch_bucket(b);
    CUDA_OK(cudaEventRecord(g_ov.done, g_ov.comm));
    CUDA_OK(cudaStreamWaitEvent(stream(), g_ov.done, 0));
    if (g_ov.rc) return g_ov.rc;
    // gradients that were allocated during this backward were not in the plan: exchange them now
    std::vector<tensor *> late;
    for (tensor *t : g_ov.all_params) {
        if (!t->grad) continue;
        bool planned = false;
        for (auto &o : g_ov.owners) if (o.first == t) { planned = true; break; }
        if (!planned) late.push_back(t);
    }
    if (!late.empty()) { int rc = dnn_cuda_dp_allreduce_grads(late.data(), (int)late.size()); if (rc) return rc; }
    ncclResult_t async = ncclSuccess;
    ncclResult_t r = g_nccl.CommGetAsyncError(g_comm, &async);
    if (r != ncclSuccess || async != ncclSuccess) return nccl_fail(r != ncclSuccess ? r : async, "ncclCommGetAsyncError");
    return 0;
}

}  // namespace dnnb

using namespace dnnb;

extern "C" {

int dnn_cuda_dp_unique_id(void *out_128_bytes) {
    if (!load_nccl()) return -1;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    ncclUniqueId id;
    ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
    memcpy(out_128_bytes, &id, 128);
    return 0;
}

int dnn_cuda_dp_init(int rank, int world_size, const void *id_128_bytes) {
    if (world_size < 1 || rank < 0 || rank >= world_size) { g_dp_error = "dp_init: bad rank/world"; return -2; }
    if (g_comm) { g_dp_error = "dp_init: already initialised"; return -3; }
    g_world = world_size;
    if (world_size == 1) return 0;
    if (!load_nccl()) { g_world = 1; return -1; }
    stream();       // binds the device chosen by dnn_cuda_init()
    ncclUniqueId id;
    memcpy(&id, id_128_bytes, 128);
    ncclResult_t r = g_nccl.CommInitRank(&g_comm, world_size, id, rank);
    if (r != ncclSuccess) { g_comm = nullptr; g_world = 1; return nccl_fail(r, "ncclCommInitRank"); }
    g_plan_seen = 0;
    return 0;
}

int dnn_cuda_dp_world_size(void) { return g_world; }

// Host-only view of the bucket planner (no device work): given n buffers (address, bytes),
// writes up to `cap` buckets and returns how many there are.
int dnn_cuda_dp_plan_buckets(const size_t *addrs, const size_t *bytes, int n, size_t bucket_bytes,
                             size_t *out_addrs, size_t *out_bytes, int cap) {
    if (n < 0 || bucket_bytes == 0) return -1;
    std::vector<Span> grads;
    for (int i = 0; i < n; i++) grads.push_back(Span{(char *)addrs[i], bytes[i]});
    std::vector<Span> b = plan_buckets(grads, bucket_bytes);
    for (int i = 0; i < (int)b.size() && i < cap; i++) { out_addrs[i] = (size_t)b[i].p; out_bytes[i] = b[i].bytes; }
    return (int)b.size();
}

int dnn_cuda_dp_allreduce_grads(tensor **params, int n_params) {
    if (g_world == 1) return 0;
    if (!g_comm) { g_dp_error = "dp_allreduce: communicator not initialised"; return -2; }
    std::vector<Span> grads;
    for (int i = 0; i < n_params; i++)
        if (params[i]->grad) grad_settle(params[i]);
    for (int i = 0; i < n_params; i++)
        if (params[i]->grad) grads.push_back(Span{(char *)params[i]->grad, (size_t)numel_of(params[i]) * 4});
    if (grads.empty()) return 0;
    std::vector<Span> buckets = plan_buckets(grads, bucket_bytes());
    if (int rc = plan_agree(buckets, stream())) return rc;
    ncclResult_t r = g_nccl.GroupStart();
    if (r != ncclSuccess) return nccl_fail(r, "ncclGroupStart");
    for (const Span &b : buckets) {
        // padding floats between merged gradients are averaged too; they are never read
        r = g_nccl.AllReduce(b.p, b.p, b.bytes / 4, ncclFloat32, ncclAvg, g_comm, stream());
        if (r != ncclSuccess) { g_nccl.GroupEnd(); return nccl_fail(r, "ncclAllReduce"); }
    }
    r = g_nccl.GroupEnd();
    if (r != ncclSuccess) return nccl_fail(r, "ncclGroupEnd");
    ncclResult_t async = ncclSuccess;
    r = g_nccl.CommGetAsyncError(g_comm, &async);
    if (r != ncclSuccess || async != ncclSuccess) return nccl_fail(r != ncclSuccess ? r : async, "ncclCommGetAsyncError");
    return 0;
}

const char *dnn_cuda_dp_last_error(void) { return g_dp_error.c_str(); }

// dnn_backward followed by the exchange; from the second step on (gradient buffers allocated) and with the
// overlap on, buckets are sent while backward still runs.
int dnn_cuda_dp_backward(struct mem_pool *scratch, tensor *loss, tensor **params, int n_params) {
    const bool dp = g_world > 1;
    const bool overlapped = dp && dp_overlap_begin(params, n_params);
    dnn_backward(scratch, loss);
    if (!dp) return 0;
    return overlapped ? dp_overlap_finish() : dnn_cuda_dp_allreduce_grads(params, n_params);
}

int dnn_cuda_dp_finalize(void) {
    if (g_comm) {
        cudaStreamSynchronize(stream());
        g_nccl.CommDestroy(g_comm);
        g_comm = nullptr;
    }
    if (g_plan_dev) { cudaFree(g_plan_dev); g_plan_dev = nullptr; }
    g_plan_seen = 0;
    g_world = 1;
    return 0;
}

}  // extern "C"
