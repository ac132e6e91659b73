// RMSNorm and LayerNorm, forward and backward.
// replaces src/norm.c:13-495 of the reference.
//
// All four kernels are HBM-bound.  One warp owns one row at a time and walks
// rows grid-stride; lanes read the row as float4 (128-bit, coalesced) and
// reduce with warp shuffles.  In backward each lane also carries the partial
// weight/bias gradients of the columns it owns across all the rows its warp
// visits, writes them once to a [warps, d] partial buffer, and a second small
// kernel adds the partials in a fixed order, so the result is deterministic
// (the reference's own loop is racy under OpenMP, src/norm.c:299-321).
#include "common.cuh"
#include "device_utils.cuh"

namespace dnnb {

constexpr int kWarpsPerCta = 8;

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ void st4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }

// ---- forward ---------------------------------------------------------------
// LN=false: rstd = 1/sqrt(mean(x^2)+eps), y = x*rstd*w
// LN=true : mean, rstd = 1/sqrt(var+eps), y = (x-mean)*rstd*w + b
template <bool LN, bool VEC>
__global__ void norm_fwd_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b,
                                float *__restrict__ y, float *__restrict__ mean_out, float *__restrict__ rstd_out,
                                int64_t rows, int d, float eps) {
    int lane = threadIdx.x & 31;
    int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    int64_t nwarps = (int64_t)gridDim.x * kWarpsPerCta;
    float inv_d = 1.0f / (float)d;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const float *xr = x + r * d;
        float *yr = y + r * d;
        float s = 0.f, mu = 0.f;
        if (LN) {
            if (VEC) for (int j = lane * 4; j < d; j += 128) { float4 v = ld4(xr + j); s += v.x + v.y + v.z + v.w; }
            else     for (int j = lane; j < d; j += 32) s += xr[j];
            mu = warp_sum(s) * inv_d;
            s = 0.f;
            if (VEC) for (int j = lane * 4; j < d; j += 128) { float4 v = ld4(xr + j);
                float a = v.x - mu, bb = v.y - mu, c = v.z - mu, e = v.w - mu; s += a * a + bb * bb + c * c + e * e; }
            else     for (int j = lane; j < d; j += 32) { float a = xr[j] - mu; s += a * a; }
        } else {
            if (VEC) for (int j = lane * 4; j < d; j += 128) { float4 v = ld4(xr + j); s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
            else     for (int j = lane; j < d; j += 32) { float a = xr[j]; s += a * a; }
        }
        s = warp_sum(s);
        float rs = 1.0f / sqrtf(s * inv_d + eps);
        if (lane == 0) { rstd_out[r] = rs; if (LN) mean_out[r] = mu; }
        if (VEC) {
            for (int j = lane * 4; j < d; j += 128) {
                float4 v = ld4(xr + j);
                float4 ww = w ? ld4(w + j) : make_float4(1.f, 1.f, 1.f, 1.f);
                float4 bb = (LN && b) ? ld4(b + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                float4 o;
                o.x = (v.x - mu) * rs * ww.x + bb.x; o.y = (v.y - mu) * rs * ww.y + bb.y;
                o.z = (v.z - mu) * rs * ww.z + bb.z; o.w = (v.w - mu) * rs * ww.w + bb.w;
                st4(yr + j, o);
            }
        } else {
            for (int j = lane; j < d; j += 32)
                yr[j] = (xr[j] - mu) * rs * (w ? w[j] : 1.f) + ((LN && b) ? b[j] : 0.f);
        }
    }
}

// The same with the row held in registers (T 128-bit slots per lane, d <= 128 T, d a multiple of 4): one read of x with all
// of a lane's loads in flight at once instead of two passes; the sums run over the same elements in the same order.
template <bool LN, int T>
__global__ void norm_fwd_reg_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b,
                                    float *__restrict__ y, float *__restrict__ mean_out, float *__restrict__ rstd_out,
                                    int64_t rows, int d, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5), nwarps = (int64_t)gridDim.x * kWarpsPerCta;
    const float inv_d = 1.0f / (float)d;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const float *xr = x + r * d;
        float *yr = y + r * d;
        float4 v[T];
#pragma unroll
        for (int t = 0; t < T; t++) { const int j = (lane + 32 * t) * 4; v[t] = j < d ? ld4(xr + j) : make_float4(0.f, 0.f, 0.f, 0.f); }
        float s = 0.f, mu = 0.f;
        if (LN) {
#pragma unroll
            for (int t = 0; t < T; t++) if ((lane + 32 * t) * 4 < d) s += v[t].x + v[t].y + v[t].z + v[t].w;
            mu = warp_sum(s) * inv_d;
            s = 0.f;
#pragma unroll
            for (int t = 0; t < T; t++) if ((lane + 32 * t) * 4 < d) {
                float a = v[t].x - mu, bb = v[t].y - mu, c = v[t].z - mu, e = v[t].w - mu; s += a * a + bb * bb + c * c + e * e; }
        } else {
#pragma unroll
            for (int t = 0; t < T; t++) if ((lane + 32 * t) * 4 < d) s += v[t].x * v[t].x + v[t].y * v[t].y + v[t].z * v[t].z + v[t].w * v[t].w;
        }
        s = warp_sum(s);
        const float rs = 1.0f / sqrtf(s * inv_d + eps);
        if (lane == 0) { rstd_out[r] = rs; if (LN) mean_out[r] = mu; }
#pragma unroll
        for (int t = 0; t < T; t++) {
            const int j = (lane + 32 * t) * 4;
            if (j >= d) continue;
            float4 ww = w ? ld4(w + j) : make_float4(1.f, 1.f, 1.f, 1.f);
            float4 bb = (LN && b) ? ld4(b + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 o;
            o.x = (v[t].x - mu) * rs * ww.x + bb.x; o.y = (v[t].y - mu) * rs * ww.y + bb.y;
            o.z = (v[t].z - mu) * rs * ww.z + bb.z; o.w = (v[t].w - mu) * rs * ww.w + bb.w;
            st4(yr + j, o);
        }
    }
}

// A handful of rows (a decoding step: one token per sequence): one CTA per row instead of one warp, so that a row of
// 768 floats is two loads per thread and not two dozen in a row.  d a multiple of 4, 16-byte aligned pointers.
template <bool LN>
__global__ void __launch_bounds__(256)
norm_fwd_row_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b,
                    float *__restrict__ y, float *__restrict__ mean_out, float *__restrict__ rstd_out, int d, float eps) {
    __shared__ float red[32];
    const int64_t r = blockIdx.x;
    const float *xr = x + r * d;
    float *yr = y + r * d;
    const float inv_d = 1.0f / (float)d;
    float s = 0.f, mu = 0.f;
    if (LN) {
        for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) { float4 v = ld4(xr + j); s += v.x + v.y + v.z + v.w; }
        mu = block_sum(s, red) * inv_d;
        s = 0.f;
        for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) { float4 v = ld4(xr + j);
            float a = v.x - mu, bb = v.y - mu, c = v.z - mu, e = v.w - mu; s += a * a + bb * bb + c * c + e * e; }
    } else {
        for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) { float4 v = ld4(xr + j); s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
    }
    s = block_sum(s, red);
    const float rs = 1.0f / sqrtf(s * inv_d + eps);
    if (threadIdx.x == 0) { rstd_out[r] = rs; if (LN) mean_out[r] = mu; }
    for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
        float4 v = ld4(xr + j);
        float4 ww = w ? ld4(w + j) : make_float4(1.f, 1.f, 1.f, 1.f);
        float4 bb = (LN && b) ? ld4(b + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 o;
        o.x = (v.x - mu) * rs * ww.x + bb.x; o.y = (v.y - mu) * rs * ww.y + bb.y;
        o.z = (v.z - mu) * rs * ww.z + bb.z; o.w = (v.w - mu) * rs * ww.w + bb.w;
        st4(yr + j, o);
    }
}

// ---- backward --------------------------------------------------------------
// T = float4 slots per lane (d <= 128*T).  Per row:
//   dy = g*w
//   RMS: S = sum(dy*x); dx += rs*dy - rs*(rs^2/d*S)*x;                dw_j += g*x*rs
//   LN : xmu=x-mu; a=mean(dy); c=mean(dy*xmu); dx += rs*(dy-a-xmu*c*rs^2); dw_j += g*xmu*rs; db_j += g
template <bool LN, int T>
__global__ void norm_bwd_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ g,
                                const float *__restrict__ mean, const float *__restrict__ rstd,
                                float *dx, float *__restrict__ dw_part, float *__restrict__ db_part,
                                int64_t rows, int d, const float *addend) {
    int lane = threadIdx.x & 31;
    int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    int64_t nwarps = (int64_t)gridDim.x * kWarpsPerCta;
    float inv_d = 1.0f / (float)d;
    float4 aw[T], ab[LN ? T : 1];
#pragma unroll
    for (int t = 0; t < T; t++) { aw[t] = make_float4(0.f, 0.f, 0.f, 0.f); if (LN) ab[t] = aw[t]; }

    for (int64_t r = warp; r < rows; r += nwarps) {
        const float *xr = x + r * d, *gr = g + r * d;
        float rs = rstd[r], mu = LN ? mean[r] : 0.f;
        float4 xv[T], dyv[T];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int t = 0; t < T; t++) {
            int j = (lane + 32 * t) * 4;
            if (j < d) {
                float4 v = ld4(xr + j), gg = ld4(gr + j);
                float4 ww = w ? ld4(w + j) : make_float4(1.f, 1.f, 1.f, 1.f);
                v.x -= mu; v.y -= mu; v.z -= mu; v.w -= mu;
                float4 dy = make_float4(gg.x * ww.x, gg.y * ww.y, gg.z * ww.z, gg.w * ww.w);
                xv[t] = v; dyv[t] = dy;
                s1 += dy.x * v.x + dy.y * v.y + dy.z * v.z + dy.w * v.w;
                if (LN) s2 += dy.x + dy.y + dy.z + dy.w;
                if (dw_part) {
                    aw[t].x += gg.x * v.x * rs; aw[t].y += gg.y * v.y * rs;
                    aw[t].z += gg.z * v.z * rs; aw[t].w += gg.w * v.w * rs;
                }
                if (LN && db_part) { ab[t].x += gg.x; ab[t].y += gg.y; ab[t].z += gg.z; ab[t].w += gg.w; }
            }
        }
        s1 = warp_sum(s1);
        if (LN) s2 = warp_sum(s2);
        if (dx) {
            float *dxr = dx + r * d;
            float k1 = rs * rs * inv_d * s1;       // RMS: S_scaled ; LN: mean(dy*xmu)*rs^2
            float mdy = LN ? s2 * inv_d : 0.f;
#pragma unroll
            for (int t = 0; t < T; t++) {
                int j = (lane + 32 * t) * 4;
                if (j < d) {
                    float4 o = addend ? ld4(addend + r * d + j) : make_float4(0.f, 0.f, 0.f, 0.f), v = xv[t], dy = dyv[t];
                    o.x += rs * (dy.x - mdy) - rs * k1 * v.x; o.y += rs * (dy.y - mdy) - rs * k1 * v.y;
                    o.z += rs * (dy.z - mdy) - rs * k1 * v.z; o.w += rs * (dy.w - mdy) - rs * k1 * v.w;
                    st4(dxr + j, o);
                }
            }
        }
    }
    // every warp writes its partial (zeros when it saw no row)
#pragma unroll
    for (int t = 0; t < T; t++) {
        int j = (lane + 32 * t) * 4;
        if (j < d) {
            if (dw_part) st4(dw_part + warp * d + j, aw[t]);
            if (LN && db_part) st4(db_part + warp * d + j, ab[t]);
        }
    }
}

// Same computation with the rows staged through shared memory by the copy engine: every warp
// owns two row buffers (x row and g row each) and two mbarriers; while it works on one row, a
// bulk copy (cp.async.bulk, 1-D) of its next row is in flight.  The loads cost no registers and
// never stop, which the register version cannot do: it has nothing in flight while it reduces
// and stores.  Used when two buffers per warp fit (d <= 768 with 8 warps and 2 CTAs per SM).
__device__ __forceinline__ void bulk_load_1d(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src), "r"(bytes),
                   "r"((uint32_t)__cvta_generic_to_shared(bar)) : "memory");
}
__device__ __forceinline__ void bar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(count));
}
__device__ __forceinline__ void bar_expect(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(bytes) : "memory");
}
// bounded: a copy that never lands must not hang the GPU; the caller flags the error
__device__ __forceinline__ bool bar_wait(uint64_t *bar, uint32_t parity) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(bar);
    for (uint32_t it = 0; it < (1u << 24); it++) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ int g_norm_error = 0;

template <bool LN, int T>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 2)
norm_bwd_staged_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ g,
                       const float *__restrict__ mean, const float *__restrict__ rstd,
                       float *dx, float *__restrict__ dw_part, float *__restrict__ db_part,
                       int64_t rows, int d, const float *addend) {
    extern __shared__ __align__(128) uint8_t norm_smem[];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + wid;
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerCta;
    const uint32_t row_bytes = (uint32_t)d * 4;
    // per warp: [2 buffers][x row | g row], then the CTA's barriers
    float *buf = reinterpret_cast<float *>(norm_smem) + (size_t)wid * 4 * d;
    uint64_t *bars = reinterpret_cast<uint64_t *>(norm_smem + (size_t)kWarpsPerCta * 4 * row_bytes) + wid * 2;
    if (lane == 0) { bar_init(&bars[0], 1); bar_init(&bars[1], 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    __syncwarp();
    const float inv_d = 1.0f / (float)d;
    float4 aw[T], ab[LN ? T : 1], wr[T];          // wr: this lane's weights, the same for every row
#pragma unroll
    for (int t = 0; t < T; t++) {
        aw[t] = make_float4(0.f, 0.f, 0.f, 0.f); if (LN) ab[t] = aw[t];
        int j = (lane + 32 * t) * 4;
        wr[t] = (w && j < d) ? ld4(w + j) : make_float4(1.f, 1.f, 1.f, 1.f);
    }
    auto fetch = [&](int64_t r, int b) {
        if (lane == 0) {
            bar_expect(&bars[b], 2 * row_bytes);
            bulk_load_1d(buf + (size_t)b * 2 * d, x + r * d, row_bytes, &bars[b]);
            bulk_load_1d(buf + (size_t)b * 2 * d + d, g + r * d, row_bytes, &bars[b]);
        }
    };
    if (warp < rows) fetch(warp, 0);
    int it = 0;
    for (int64_t r = warp; r < rows; r += nwarps, it++) {
        const int b = it & 1;
        if (r + nwarps < rows) fetch(r + nwarps, b ^ 1);       // the other buffer was consumed in the previous trip
        const float rs = rstd[r], mu = LN ? mean[r] : 0.f;
        int ok = 1;
        if (lane == 0) ok = bar_wait(&bars[b], (uint32_t)(it >> 1) & 1u);       // one poller per warp
        if (!__shfl_sync(0xffffffffu, ok, 0)) { if (lane == 0) atomicCAS(&g_norm_error, 0, 1); break; }
        const float *xs = buf + (size_t)b * 2 * d, *gs = xs + d;
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int t = 0; t < T; t++) {
            int j = (lane + 32 * t) * 4;
            if (j < d) {
                float4 v = ld4(xs + j), gg = ld4(gs + j);
                const float4 ww = wr[t];
                v.x -= mu; v.y -= mu; v.z -= mu; v.w -= mu;
                s1 += gg.x * ww.x * v.x + gg.y * ww.y * v.y + gg.z * ww.z * v.z + gg.w * ww.w * v.w;
                if (LN) s2 += gg.x * ww.x + gg.y * ww.y + gg.z * ww.z + gg.w * ww.w;
                if (dw_part) {
                    aw[t].x += gg.x * v.x * rs; aw[t].y += gg.y * v.y * rs;
                    aw[t].z += gg.z * v.z * rs; aw[t].w += gg.w * v.w * rs;
                }
                if (LN && db_part) { ab[t].x += gg.x; ab[t].y += gg.y; ab[t].z += gg.z; ab[t].w += gg.w; }
            }
        }
        s1 = warp_sum(s1);
        if (LN) s2 = warp_sum(s2);
        if (dx) {
            float *dxr = dx + r * d;
            const float k1 = rs * rs * inv_d * s1, mdy = LN ? s2 * inv_d : 0.f;
#pragma unroll
            for (int t = 0; t < T; t++) {
                int j = (lane + 32 * t) * 4;
                if (j < d) {
                    float4 v = ld4(xs + j), gg = ld4(gs + j);
                    const float4 ww = wr[t];
                    float4 o = addend ? ld4(addend + r * d + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                    v.x -= mu; v.y -= mu; v.z -= mu; v.w -= mu;
                    o.x += rs * (gg.x * ww.x - mdy) - rs * k1 * v.x; o.y += rs * (gg.y * ww.y - mdy) - rs * k1 * v.y;
                    o.z += rs * (gg.z * ww.z - mdy) - rs * k1 * v.z; o.w += rs * (gg.w * ww.w - mdy) - rs * k1 * v.w;
                    st4(dxr + j, o);
                }
            }
        }
        __syncwarp();          // every lane is done with this buffer before lane 0 refills it two trips on
    }
    // The CTA's eight partial sums are added in shared memory (the row buffers are free now; every copy
    // a warp asked for has been waited for), so one row of partials per CTA leaves the kernel.
    __syncthreads();
    float *red = reinterpret_cast<float *>(norm_smem);             // [8 warps][2][d]
#pragma unroll
    for (int t = 0; t < T; t++) {
        int j = (lane + 32 * t) * 4;
        if (j < d) {
            if (dw_part) st4(red + (size_t)(wid * 2) * d + j, aw[t]);
            if (LN && db_part) st4(red + (size_t)(wid * 2 + 1) * d + j, ab[t]);
        }
    }
    __syncthreads();
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        if (dw_part) {
            float s = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < kWarpsPerCta; w8++) s += red[(size_t)(w8 * 2) * d + j];
            dw_part[(int64_t)blockIdx.x * d + j] = s;
        }
        if (LN && db_part) {
            float s = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < kWarpsPerCta; w8++) s += red[(size_t)(w8 * 2 + 1) * d + j];
            db_part[(int64_t)blockIdx.x * d + j] = s;
        }
    }
}

// Scalar fallback for d not a multiple of 4, unaligned rows or d > 2048:
// one CTA per row for dx, column sums done by separate kernels.
template <bool LN>
__global__ void norm_bwd_dx_scalar_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ g,
                                          const float *__restrict__ mean, const float *__restrict__ rstd,
                                          float *dx, int d, const float *addend) {
    __shared__ float sh[32];
    int64_t r = blockIdx.x;
    const float *xr = x + r * d, *gr = g + r * d;
    float rs = rstd[r], mu = LN ? mean[r] : 0.f, inv_d = 1.0f / (float)d;
    float s1 = 0.f, s2 = 0.f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float dy = gr[j] * (w ? w[j] : 1.f), v = xr[j] - mu;
        s1 += dy * v; s2 += dy;
    }
    s1 = block_sum(s1, sh);
    s2 = LN ? block_sum(s2, sh) : 0.f;
    float k1 = rs * rs * inv_d * s1, mdy = LN ? s2 * inv_d : 0.f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float dy = gr[j] * (w ? w[j] : 1.f), v = xr[j] - mu;
        float val = rs * (dy - mdy) - rs * k1 * v;
        dx[r * d + j] = addend ? addend[r * d + j] + val : val;
    }
}
// t[r,j] = g*(x-mu)*rs, to be column-summed
template <bool LN>
__global__ void norm_dw_terms_kernel(const float *__restrict__ x, const float *__restrict__ g, const float *__restrict__ mean,
                                     const float *__restrict__ rstd, float *__restrict__ t, int64_t rows, int d) {
    int64_t n = rows * d;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / d;
        t[i] = g[i] * (x[i] - (LN ? mean[r] : 0.f)) * rstd[r];
    }
}

// out[j] += sum_p part[p*d + j].  CTA = 32 columns x 32 row-lanes; lane y sums
// p = y, y+32, ... and the 32 lane sums are added in lane order (fixed order).
__global__ void norm_part_reduce_kernel(float *__restrict__ out, const float *__restrict__ part, int nparts, int d, int acc) {
    __shared__ float tile[32][33];
    int j = blockIdx.x * 32 + threadIdx.x;
    float s = 0.f;
    if (j < d)
        for (int p = threadIdx.y; p < nparts; p += 32) s += part[(int64_t)p * d + j];
    tile[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && j < d) {
        float t = 0.f;
#pragma unroll
        for (int y = 0; y < 32; y++) t += tile[y][threadIdx.x];
        out[j] = acc ? out[j] + t : t;
    }
}

int norm_error() {
    int e = 0;
    cudaMemcpyFromSymbol(&e, g_norm_error, sizeof e);
    return e;
}

template <bool LN>
static void norm_forward(const float *x, const float *w, const float *b, float *y, float *mean, float *rstd,
                         int64_t rows, int d, float eps) {
    if (rows <= 0) return;
    bool vec = d % 4 == 0 && aligned16(x) && aligned16(y) && (!w || aligned16(w)) && (!b || aligned16(b));
    int grid = (int)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
    int cap = kNumSMs * 8;
    if (grid > cap) grid = cap;
    const int T = (d + 127) / 128;
    if (vec && rows <= 8 && d >= 256) norm_fwd_row_kernel<LN><<<(unsigned)rows, 256, 0, stream()>>>(x, w, b, y, mean, rstd, d, eps);
    else if (vec && T <= 2) norm_fwd_reg_kernel<LN, 2><<<grid, kWarpsPerCta * 32, 0, stream()>>>(x, w, b, y, mean, rstd, rows, d, eps);
    else if (vec && T <= 4) norm_fwd_reg_kernel<LN, 4><<<grid, kWarpsPerCta * 32, 0, stream()>>>(x, w, b, y, mean, rstd, rows, d, eps);
    else if (vec && T <= 6) norm_fwd_reg_kernel<LN, 6><<<grid, kWarpsPerCta * 32, 0, stream()>>>(x, w, b, y, mean, rstd, rows, d, eps);
    else if (vec && T <= 8) norm_fwd_reg_kernel<LN, 8><<<grid, kWarpsPerCta * 32, 0, stream()>>>(x, w, b, y, mean, rstd, rows, d, eps);
    else if (vec) norm_fwd_kernel<LN, true><<<grid, kWarpsPerCta * 32, 0, stream()>>>(x, w, b, y, mean, rstd, rows, d, eps);
    else     norm_fwd_kernel<LN, false><<<grid, kWarpsPerCta * 32, 0, stream()>>>(x, w, b, y, mean, rstd, rows, d, eps);
    prof_work(8.0 * rows * d);                                   // read x, write y
    LAUNCHED(LN ? "layernorm_fwd_kernel" : "rmsnorm_fwd_kernel");
}

// rows staged through shared memory when two CTAs of 8 warps with two row pairs each fit on an SM
static size_t staged_smem(int d) { return (size_t)kWarpsPerCta * 4 * d * sizeof(float) + kWarpsPerCta * 2 * sizeof(uint64_t); }
static bool staged_ok(int d) { return d % 4 == 0 && (d + 127) / 128 <= 6 && staged_smem(d) <= 100 * 1024; }

template <bool LN, int T>
static void launch_bwd(const float *x, const float *w, const float *g, const float *mean, const float *rstd,
                       float *dx, float *dwp, float *dbp, int64_t rows, int d, int grid, const float *addend) {
    const size_t smem = staged_smem(d);
    if (staged_ok(d)) {
        static bool once = false;
        if (!once) {
            CUDA_OK(cudaFuncSetAttribute(norm_bwd_staged_kernel<LN, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
            CUDA_OK(cudaFuncSetAttribute(norm_bwd_staged_kernel<LN, T>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
            once = true;
        }
        norm_bwd_staged_kernel<LN, T><<<grid, kWarpsPerCta * 32, smem, stream()>>>(x, w, g, mean, rstd, dx, dwp, dbp, rows, d, addend);
        prof_work((addend ? 16.0 : 12.0) * rows * d);            // read x, g (and the residual gradient), write dx
        LAUNCHED(LN ? "layernorm_bwd_kernel" : "rmsnorm_bwd_kernel");
        return;
    }
    norm_bwd_kernel<LN, T><<<grid, kWarpsPerCta * 32, 0, stream()>>>(x, w, g, mean, rstd, dx, dwp, dbp, rows, d, addend);
    prof_work((addend ? 16.0 : 12.0) * rows * d);
    LAUNCHED(LN ? "layernorm_bwd_kernel" : "rmsnorm_bwd_kernel");
}

template <bool LN>
static void norm_backward(struct mem_pool *pool, const float *x, const float *w, const float *g, const float *mean,
                          const float *rstd, float *dx, float *dw, float *db, int64_t rows, int d,
                          const float *addend, bool acc_dw, bool acc_db) {
    if (rows <= 0) return;
    bool vec = d % 4 == 0 && d <= 2048 && aligned16(x) && aligned16(g) && (!w || aligned16(w)) && (!dx || aligned16(dx)) && (!addend || aligned16(addend));
    if (vec) {
        int grid = (int)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
        int cap = kNumSMs * 2;
        if (grid > cap) grid = cap;
        int nparts = staged_ok(d) ? grid : grid * kWarpsPerCta;      // the staged kernel adds its warps' partials itself
        float *dwp = dw ? dev_alloc_t<float>(pool, (size_t)nparts * d) : nullptr;
        float *dbp = (LN && db) ? dev_alloc_t<float>(pool, (size_t)nparts * d) : nullptr;
        int T = (d + 127) / 128;
        if (T <= 1)      launch_bwd<LN, 1>(x, w, g, mean, rstd, dx, dwp, dbp, rows, d, grid, addend);
        else if (T <= 2) launch_bwd<LN, 2>(x, w, g, mean, rstd, dx, dwp, dbp, rows, d, grid, addend);
        else if (T <= 4) launch_bwd<LN, 4>(x, w, g, mean, rstd, dx, dwp, dbp, rows, d, grid, addend);
        else if (T <= 6) launch_bwd<LN, 6>(x, w, g, mean, rstd, dx, dwp, dbp, rows, d, grid, addend);
        else if (T <= 8) launch_bwd<LN, 8>(x, w, g, mean, rstd, dx, dwp, dbp, rows, d, grid, addend);
        else             launch_bwd<LN, 16>(x, w, g, mean, rstd, dx, dwp, dbp, rows, d, grid, addend);
        if (dwp) { norm_part_reduce_kernel<<<(d + 31) / 32, dim3(32, 32), 0, stream()>>>(dw, dwp, nparts, d, acc_dw); LAUNCHED("norm_part_reduce_kernel"); }
        if (dbp) { norm_part_reduce_kernel<<<(d + 31) / 32, dim3(32, 32), 0, stream()>>>(db, dbp, nparts, d, acc_db); LAUNCHED("norm_part_reduce_kernel"); }
        return;
    }
    if (dx) {
        norm_bwd_dx_scalar_kernel<LN><<<(unsigned)rows, 256, 0, stream()>>>(x, w, g, mean, rstd, dx, d, addend);
        LAUNCHED("norm_bwd_dx_scalar_kernel");
    }
    if (dw) {
        float *t = dev_alloc_t<float>(pool, (size_t)rows * d);
        norm_dw_terms_kernel<LN><<<grid_for(rows * d, 256), 256, 0, stream()>>>(x, g, mean, rstd, t, rows, d);
        LAUNCHED("norm_dw_terms_kernel");
        k_colsum_acc(dw, t, rows, d, acc_dw);
    }
    if (LN && db) k_colsum_acc(db, g, rows, d, acc_db);
}

static void rms_backward(grad_fn *fn, tensor *go) {
    tensor *x = fn->inputs[0];
    tensor *weight = fn->saved_tensors[0];
    const float *rstd = (const float *)fn->saved_tensors[1];
    int d = x->shape[x->ndim - 1];
    int64_t rows = numel_of(x) / d;
    const float *xd = (const float *)x->data + x->offset;
    const float *gd = (const float *)go->data;
    const float *wd = weight ? (const float *)weight->data + weight->offset : nullptr;
    bool acc_w = true, acc_x = true;
    const float *base = nullptr;          // a residual gradient still waiting to be copied into dx: added here instead
    float *dw = (weight && weight->requires_grad) ? grad_full(weight, &acc_w) : nullptr;
    float *dx = x->requires_grad ? grad_full_based(x, &acc_x, &base) : nullptr;   // the reference indexes dx from 0 (src/norm.c:339)
    norm_backward<false>(fn->pool, xd, wd, gd, nullptr, rstd, dx, dw, nullptr, rows, d, base ? base : (acc_x ? dx : nullptr), acc_w, true);
}

static void ln_backward(grad_fn *fn, tensor *go) {
    tensor *x = fn->inputs[0];
    tensor *weight = fn->saved_tensors[0], *bias = fn->saved_tensors[1];
    const float *mean = (const float *)fn->saved_tensors[2], *rstd = (const float *)fn->saved_tensors[3];
    int d = x->shape[x->ndim - 1];
    int64_t rows = numel_of(x) / d;
    const float *xd = (const float *)x->data + x->offset;
    const float *gd = (const float *)go->data;
    const float *wd = weight ? (const float *)weight->data + weight->offset : nullptr;
    bool acc_w = true, acc_b = true, acc_x = true;
    float *dw = (weight && weight->requires_grad) ? grad_full(weight, &acc_w) : nullptr;
    float *db = (bias && bias->requires_grad) ? grad_full(bias, &acc_b) : nullptr;
    const float *base = nullptr;
    float *dx = x->requires_grad ? grad_full_based(x, &acc_x, &base) : nullptr;
    norm_backward<true>(fn->pool, xd, wd, gd, mean, rstd, dx, dw, db, rows, d, base ? base : (acc_x ? dx : nullptr), acc_w, acc_b);
}

}  // namespace dnnb

using namespace dnnb;

extern "C" {

tensor *tensor_rms_norm(struct mem_pool *scratch, const tensor *x, const tensor *weight, float eps) {
    require_device_payloads("tensor_rms_norm", {x, weight});
    DNN_CHECK(x, "tensor_rms_norm: x is NULL");
    DNN_CHECK(x->contiguous, "tensor_rms_norm: x must be contiguous");
    int d = x->shape[x->ndim - 1];
    int64_t rows = numel_of(x) / d;
    float *rstd = dev_alloc_t<float>(scratch, (size_t)rows);
    tensor *out = tensor_scratch(scratch, x->ndim, x->shape, 0);
    const float *wd = weight ? tensor_data_ptr((tensor *)weight) : nullptr;
    norm_forward<false>((const float *)x->data + x->offset, wd, nullptr, (float *)out->data, nullptr, rstd, rows, d, eps);
    if (dnn_grad_enabled() && (x->requires_grad || (weight && weight->requires_grad))) {
        grad_fn *fn = attach(scratch, out, rms_backward, 1, 2);
        fn->inputs[0] = (tensor *)x;
        fn->saved_tensors[0] = (tensor *)weight;
        fn->saved_tensors[1] = (tensor *)rstd;
    }
    return out;
}

tensor *tensor_layer_norm(struct mem_pool *scratch, const tensor *x, const tensor *weight, const tensor *bias, float eps) {
    require_device_payloads("tensor_layer_norm", {x, weight, bias});
    DNN_CHECK(x, "tensor_layer_norm: x is NULL");
    DNN_CHECK(x->contiguous, "tensor_layer_norm: x must be contiguous");
    int d = x->shape[x->ndim - 1];
    int64_t rows = numel_of(x) / d;
    float *mean = dev_alloc_t<float>(scratch, (size_t)rows);
    float *rstd = dev_alloc_t<float>(scratch, (size_t)rows);
    tensor *out = tensor_scratch(scratch, x->ndim, x->shape, 0);
    const float *wd = weight ? tensor_data_ptr((tensor *)weight) : nullptr;
    const float *bd = bias ? tensor_data_ptr((tensor *)bias) : nullptr;
    norm_forward<true>((const float *)x->data + x->offset, wd, bd, (float *)out->data, mean, rstd, rows, d, eps);
    if (dnn_grad_enabled() && (x->requires_grad || (weight && weight->requires_grad) || (bias && bias->requires_grad))) {
        grad_fn *fn = attach(scratch, out, ln_backward, 1, 4);
        fn->inputs[0] = (tensor *)x;
        fn->saved_tensors[0] = (tensor *)weight;
        fn->saved_tensors[1] = (tensor *)bias;
        fn->saved_tensors[2] = (tensor *)mean;
        fn->saved_tensors[3] = (tensor *)rstd;
    }
    return out;
}

}  // extern "C"
