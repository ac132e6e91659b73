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
    if (!load_nccl()) return -1;
    stream();       // binds the device chosen by dnn_cuda_init()
    ncclUniqueId id;
    memcpy(&id, id_128_bytes, 128);
    ncclResult_t r = g_nccl.CommInitRank(&g_comm, world_size, id, rank);
    if (r != ncclSuccess) { g_comm = nullptr; return nccl_fail(r, "ncclCommInitRank"); }
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
    size_t mb = 64;
    if (const char *e = getenv("DNN_CUDA_BUCKET_MB")) { long v = atol(e); if (v > 0) mb = (size_t)v; }
    std::vector<Span> buckets = plan_buckets(grads, mb << 20);
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

int dnn_cuda_dp_finalize(void) {
    if (g_comm) {
        cudaStreamSynchronize(stream());
        g_nccl.CommDestroy(g_comm);
        g_comm = nullptr;
    }
    g_world = 1;
    return 0;
}

}  // extern "C"
