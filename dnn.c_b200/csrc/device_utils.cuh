// Launch-sizing helpers and warp/block reductions shared by the kernels.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace dnnb {

constexpr int kNumSMs = 148;   // B200

// Grid for a grid-stride loop over n items: enough CTAs to cover n once, capped
// at a few waves of the 148 SMs so large arrays reuse resident CTAs.
inline int grid_for(int64_t n, int block, int ctas_per_sm = 8) {
    int64_t need = (n + block - 1) / block;
    int64_t cap = (int64_t)kNumSMs * ctas_per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

inline bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block-wide sum; every thread gets the result.  `sh` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float *sh) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();            // protect sh from a previous use
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float r = (lane < nw) ? sh[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float *sh) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float r = (lane < nw) ? sh[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}


// Rotation of one RoPE pair (src/rope.c:60-112), roundings spelled out for the same reason as below.
__device__ __forceinline__ void rope_fwd_pair(float x, float y, float c, float s, float &ox, float &oy) {
    ox = __fmaf_rn(x, c, -__fmul_rn(y, s));
    oy = __fmaf_rn(x, s, __fmul_rn(y, c));
}
// Inverse rotation of one RoPE pair (the gradient of src/rope.c:60-112).  Roundings are spelled
// out so that every kernel that applies it -- the stand-alone RoPE backward, the in-place version
// on a fused QKV gradient and the attention backward epilogues -- produces the same bits.
__device__ __forceinline__ void rope_inv_pair(float x, float y, float c, float s, float &ox, float &oy) {
    ox = __fmaf_rn(x, c, __fmul_rn(y, s));
    oy = __fmaf_rn(y, c, -__fmul_rn(x, s));
}

}  // namespace dnnb
