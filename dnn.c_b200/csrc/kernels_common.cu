// Small bandwidth-bound utility kernels used by several ops: fill, copy,
// accumulate, strided gather / scatter and column sums.
#include "common.cuh"
#include "device_utils.cuh"

namespace dnnb {

// ---- fill / copy / accumulate (128-bit when the pointers allow it) -------
__global__ void fill_kernel(float *__restrict__ p, int64_t n, float v) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) p[i] = v;
}

__global__ void acc_kernel_v4(float4 *__restrict__ dst, const float4 *__restrict__ src, int64_t n4) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n4; i += stride) {
        float4 d = dst[i], s = src[i];
        d.x += s.x; d.y += s.y; d.z += s.z; d.w += s.w;
        dst[i] = d;
    }
}
__global__ void acc_kernel(float *__restrict__ dst, const float *__restrict__ src, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] += src[i];
}

void k_fill(float *p, int64_t n, float v) {
    if (n <= 0) return;
    if (v == 0.0f) { CUDA_OK(cudaMemsetAsync(p, 0, (size_t)n * 4, stream())); return; }
    fill_kernel<<<grid_for(n, 256), 256, 0, stream()>>>(p, n, v);
    LAUNCHED("fill_kernel");
}

void k_axpy_acc(float *dst, const float *src, int64_t n) {
    if (n <= 0) return;
    if (aligned16(dst) && aligned16(src) && n % 4 == 0) {
        acc_kernel_v4<<<grid_for(n / 4, 256), 256, 0, stream()>>>((float4 *)dst, (const float4 *)src, n / 4);
        LAUNCHED("acc_kernel_v4");
    } else {
        acc_kernel<<<grid_for(n, 256), 256, 0, stream()>>>(dst, src, n);
        LAUNCHED("acc_kernel");
    }
}

void k_copy(float *dst, const float *src, int64_t n) {
    if (n <= 0) return;
    CUDA_OK(cudaMemcpyAsync(dst, src, (size_t)n * 4, cudaMemcpyDeviceToDevice, stream()));
}

// ---- strided gather / scatter ---------------------------------------------
__device__ __forceinline__ int64_t view_offset(const View &v, int64_t flat) {
    int64_t off = v.offset;
#pragma unroll
    for (int d = DNN_MAX_DIMS - 1; d >= 0; d--) {
        if (d < v.ndim) {
            int c = (int)(flat % v.shape[d]);
            flat /= v.shape[d];
            off += (int64_t)c * v.strides[d];
        }
    }
    return off;
}

__global__ void gather_kernel(float *__restrict__ dst, const float *__restrict__ src, View sv, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = src[view_offset(sv, i)];
}

// Each destination address is written by exactly one i when the view has no
// zero strides over extents > 1; callers guarantee that.
__global__ void scatter_kernel(float *__restrict__ dst, View dv, const float *__restrict__ src, int64_t n, int acc) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        int64_t o = view_offset(dv, i);
        dst[o] = acc ? dst[o] + src[i] : src[i];
    }
}

void k_gather(float *dst, const float *src, const View &sv, int64_t n) {
    if (n <= 0) return;
    gather_kernel<<<grid_for(n, 256), 256, 0, stream()>>>(dst, src, sv, n);
    LAUNCHED("gather_kernel");
}

void k_scatter(float *dst, const View &dv, const float *src, int64_t n, bool accumulate) {
    if (n <= 0) return;
    scatter_kernel<<<grid_for(n, 256), 256, 0, stream()>>>(dst, dv, src, n, accumulate ? 1 : 0);
    LAUNCHED("scatter_kernel");
}

// ---- column sums: out[c] += sum_r g[r*C + c] ------------------------------
// Stage 1: CTA (cx, ry) sums rows [ry*rows_per, ...) of 32 columns into
// partial[ry][c]; stage 2 adds the partials in row-block order, so the result
// does not depend on scheduling.
__global__ void colsum_partial_kernel(const float *__restrict__ g, float *__restrict__ partial,
                                      int64_t rows, int C, int rows_per) {
    __shared__ float tile[32][33];
    int c = blockIdx.x * 32 + threadIdx.x;
    int64_t r0 = (int64_t)blockIdx.y * rows_per;
    int64_t r1 = r0 + rows_per; if (r1 > rows) r1 = rows;
    float s = 0.f;
    if (c < C)
        for (int64_t r = r0 + threadIdx.y; r < r1; r += blockDim.y) s += g[r * C + c];
    tile[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float t = 0.f;
#pragma unroll
        for (int j = 0; j < 32; j++) t += tile[j][threadIdx.x];
        partial[(int64_t)blockIdx.y * C + c] = t;
    }
}
// float4 variant: CTA = 32 x 8 threads covering 128 columns, 16-byte loads.
// Arrival counters of the fused column sum, one per group of 128 columns.  The last CTA of a
// group to finish resets its counter, so the array is all zero between launches.
constexpr int kColsumGroups = 2048;
__device__ unsigned int g_colsum_arrivals[kColsumGroups];

// out != nullptr: the CTA that finishes last in its column group adds the partials of all row
// slabs in slab order (fixed order: the result does not depend on which CTA is last) and
// writes `out`, which saves the second launch.
__global__ void colsum_partial_v4_kernel(const float *__restrict__ g, float *__restrict__ partial,
                                         int64_t rows, int C, int rows_per, float *__restrict__ out, int acc) {
    __shared__ float4 tile[8][33];
    __shared__ int is_last;
    int c = (blockIdx.x * 32 + threadIdx.x) * 4;
    int64_t r0 = (int64_t)blockIdx.y * rows_per;
    int64_t r1 = r0 + rows_per; if (r1 > rows) r1 = rows;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < C)
        for (int64_t r = r0 + threadIdx.y; r < r1; r += 8) {
            float4 v = *reinterpret_cast<const float4 *>(g + r * C + c);
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
    tile[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; j++) { float4 v = tile[j][threadIdx.x]; t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w; }
        *reinterpret_cast<float4 *>(partial + (int64_t)blockIdx.y * C + c) = t;
    }
    if (out == nullptr) return;
    __threadfence();                         // this CTA's partials are visible before its arrival
    __syncthreads();
    if (threadIdx.x == 0 && threadIdx.y == 0) {
        unsigned prev = atomicAdd(&g_colsum_arrivals[blockIdx.x], 1u);
        is_last = (prev == gridDim.y - 1);
        if (is_last) g_colsum_arrivals[blockIdx.x] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // 256 threads over the 128 columns of this group: threadIdx.y picks one of 8 slab lanes
    // (p = y, y+8, ...), lane sums are combined in lane order
    float4 s2 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < C)
        for (int p = threadIdx.y; p < (int)gridDim.y; p += 8) {
            float4 v = __ldcg(reinterpret_cast<const float4 *>(partial + (int64_t)p * C + c));      // L2: written by other CTAs
            s2.x += v.x; s2.y += v.y; s2.z += v.z; s2.w += v.w;
        }
    tile[threadIdx.y][threadIdx.x] = s2;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; j++) { float4 v = tile[j][threadIdx.x]; t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w; }
        float4 *o4 = reinterpret_cast<float4 *>(out + c);
        if (acc) { float4 o = *o4; t.x += o.x; t.y += o.y; t.z += o.z; t.w += o.w; }
        *o4 = t;
    }
}
__global__ void colsum_final_kernel(float *__restrict__ out, const float *__restrict__ partial, int nparts, int C, int acc) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float s = 0.f;
    for (int p = 0; p < nparts; p++) s += partial[(int64_t)p * C + c];
    out[c] = acc ? out[c] + s : s;
}

// ── column sums a producer has already computed ──────────────────────────────
// A backward kernel that writes a whole gradient buffer can sum its columns on the way (the
// bias gradient of the layer that consumes the buffer needs exactly that) and leave the sums
// here.  k_colsum_acc uses them when it is asked for the same buffer, rows and width, which saves
// a pass over the buffer.  The entry dies with any later write to the buffer (the gradient
// helpers call colsum_cache_forget) and at both ends of dnn_backward.
// A few entries, used round-robin: one backward kernel may leave sums for two buffers (SwiGLU
// backward writes d(gate) and d(up), each consumed by its own linear layer).
struct ColsumEntry { const float *src = nullptr; int64_t rows = 0; int C = 0; float *sums = nullptr; size_t cap = 0; bool valid = false; };
constexpr int kColsumEntries = 4;
static ColsumEntry g_cc[kColsumEntries];
static int g_cc_last = 0;
float *colsum_cache_reserve(int C) {
    g_cc_last = (g_cc_last + 1) % kColsumEntries;
    ColsumEntry &e = g_cc[g_cc_last];
    if ((size_t)C > e.cap) {
        CUDA_OK(cudaStreamSynchronize(stream()));
        if (e.sums) CUDA_OK(cudaFree(e.sums));
        e.cap = (size_t)C * 2;
        CUDA_OK(cudaMalloc((void **)&e.sums, e.cap * sizeof(float)));
    }
    e.valid = false;
    return e.sums;
}
// Describes what the sums handed out by the latest colsum_cache_reserve() belong to.
void colsum_cache_publish(const float *src, int64_t rows, int C) {
    ColsumEntry &e = g_cc[g_cc_last];
    e.src = src; e.rows = rows; e.C = C; e.valid = true;
}
void colsum_cache_forget(const void *buffer) {
    for (auto &e : g_cc) if (buffer == nullptr || buffer == (const void *)e.src) e.valid = false;
}
static const ColsumEntry *colsum_cache_find(const float *g, int64_t rows, int C) {
    for (auto &e : g_cc) if (e.valid && e.src == g && e.rows == rows && e.C == C) return &e;
    return nullptr;
}

__global__ void colsum_apply_kernel(float *__restrict__ out, const float *__restrict__ sums, int C, int acc) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < C) out[c] = acc ? out[c] + sums[c] : sums[c];
}

// Partials [nparts, C] -> sums[C] for one or two producers' outputs in one launch (blockIdx.y picks
// the job).  CTA = 32 columns x 32 slab lanes: lane y adds slabs y, y+32, ... and the 32 lane sums
// are added in lane order, so the result does not depend on scheduling.
struct FinishJobs { float *sums[2]; const float *part[2]; };
__global__ void colsum_finish_kernel(FinishJobs jobs, int nparts, int C) {
    __shared__ float tile[32][33];
    float *__restrict__ sums = jobs.sums[blockIdx.y];
    const float *__restrict__ part = jobs.part[blockIdx.y];
    const int c = blockIdx.x * 32 + threadIdx.x;
    float s = 0.f;
    if (c < C)
        for (int p = threadIdx.y; p < nparts; p += 32) s += part[(int64_t)p * C + c];
    tile[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float t = 0.f;
#pragma unroll
        for (int y = 0; y < 32; y++) t += tile[y][threadIdx.x];
        sums[c] = t;
    }
}
void k_colsum_finish2(float *sums0, const float *part0, float *sums1, const float *part1, int nparts, int C) {
    FinishJobs jobs;
    jobs.sums[0] = sums0; jobs.part[0] = part0; jobs.sums[1] = sums1; jobs.part[1] = part1;
    colsum_finish_kernel<<<dim3((C + 31) / 32, sums1 ? 2 : 1), dim3(32, 32), 0, stream()>>>(jobs, nparts, C);
    LAUNCHED("colsum_finish_kernel");
}
void k_colsum_finish(float *sums, const float *partial, int nparts, int C) { k_colsum_finish2(sums, partial, nullptr, nullptr, nparts, C); }

// Scratch for the partials lives in a small cache owned by this file, grown
// on demand (never shrinks; one per process).
static float *g_colsum_scratch = nullptr;
static size_t g_colsum_cap = 0;

void k_colsum_acc(float *out, const float *g, int64_t rows, int C, bool accumulate) {
    if (rows <= 0 || C <= 0) return;
    if (const ColsumEntry *e = colsum_cache_find(g, rows, C)) {                      // the producer of g left its column sums
        colsum_apply_kernel<<<(C + 255) / 256, 256, 0, stream()>>>(out, e->sums, C, accumulate ? 1 : 0);
        LAUNCHED("colsum_apply_kernel");
        return;
    }
    int nparts = (int)((rows + 255) / 256);
    if (nparts > 512) nparts = 512;
    int rows_per = (int)((rows + nparts - 1) / nparts);
    nparts = (int)((rows + rows_per - 1) / rows_per);
    size_t need = (size_t)nparts * C * sizeof(float);
    if (need > g_colsum_cap) {
        CUDA_OK(cudaStreamSynchronize(stream()));
        if (g_colsum_scratch) CUDA_OK(cudaFree(g_colsum_scratch));
        g_colsum_cap = need * 2;
        CUDA_OK(cudaMalloc((void **)&g_colsum_scratch, g_colsum_cap));
    }
    if (C % 4 == 0 && aligned16(g)) {
        dim3 grid((C / 4 + 31) / 32, nparts), block(32, 8);
        bool fused = (int)grid.x <= kColsumGroups && aligned16(out);
        colsum_partial_v4_kernel<<<grid, block, 0, stream()>>>(g, g_colsum_scratch, rows, C, rows_per, fused ? out : nullptr,
                                                               accumulate ? 1 : 0);
        prof_work(4.0 * rows * C);
        LAUNCHED("colsum_partial_v4_kernel");
        if (fused) return;
    } else {
        dim3 grid((C + 31) / 32, nparts), block(32, 32);
        colsum_partial_kernel<<<grid, block, 0, stream()>>>(g, g_colsum_scratch, rows, C, rows_per);
        LAUNCHED("colsum_partial_kernel");
    }
    colsum_final_kernel<<<(C + 127) / 128, 128, 0, stream()>>>(out, g_colsum_scratch, nparts, C, accumulate ? 1 : 0);
    LAUNCHED("colsum_final_kernel");
}

}  // namespace dnnb
