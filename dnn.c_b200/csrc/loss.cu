// Cross-entropy and masked cross-entropy, forward and backward.
// replaces src/ops_activation.c:852-1145 (plain) and :1154-1410 (masked).
//
// A "slice" is one vector along the class dimension.  Forward: one CTA owns one slice and makes a
// single pass (online max / sum-of-exponentials per thread, four float4 loads in flight, merged
// across the CTA).  Backward into a fresh, packed gradient buffer is tiled the other way round
// (128 classes x a slab of slices per CTA) so that the column sums of d(logits) -- the bias
// gradient of the layer that produced the logits -- fall out of the same pass; accumulating or
// strided cases keep one CTA per slice (read logits, read-modify-write the gradient).  Rows whose
// last stride is 1 and whose start is 16-byte aligned move as float4.  The scalar loss is produced
// by a single-CTA tree sum over the per-slice terms (fixed order).
#include "common.cuh"
#include "device_utils.cuh"

namespace dnnb {

struct SliceMap {
    int nd;                         // dims other than the class dim
    int shape[DNN_MAX_DIMS];
    int lstride[DNN_MAX_DIMS];      // logits strides for those dims
    int mstride[DNN_MAX_DIMS];      // mask strides (0 where mask dim is 1 or no mask)
    int loff, moff;
    int C, cstride;                 // class count and stride along the class dim
};

__device__ __forceinline__ void slice_offsets(const SliceMap &m, int64_t s, int64_t &lo, int64_t &mo) {
    lo = m.loff; mo = m.moff;
    for (int d = m.nd - 1; d >= 0; d--) {
        int c = (int)(s % m.shape[d]); s /= m.shape[d];
        lo += (int64_t)c * m.lstride[d]; mo += (int64_t)c * m.mstride[d];
    }
}

// e^x through the special-function unit: x * log2(e) rounded once, then ex2.approx (about 2 ulp).
// Used where x <= 0: softmax terms of the loss statistics and of the gradient; the logarithm stays logf.
__device__ __forceinline__ float fast_expf(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
    return y;
}

__device__ __forceinline__ float fast_exp2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void online_add(float &mx, float &se, float v) {
    if (v > mx) { se *= expf(mx - v); mx = v; }
    se += expf(v - mx);
}
__device__ __forceinline__ void online_merge(float &mx, float &se, float omx, float ose) {
    if (omx == -INFINITY) return;
    if (mx == -INFINITY) { mx = omx; se = ose; return; }
    if (omx > mx) { se = se * expf(mx - omx) + ose; mx = omx; }
    else se += ose * expf(omx - mx);
}

__global__ void ce_fwd_kernel(const float *__restrict__ logits, const int *__restrict__ target,
                              const float *__restrict__ mask, SliceMap map,
                              float *__restrict__ max_out, float *__restrict__ se_out,
                              float *__restrict__ term_out, float *__restrict__ mval_out) {
    __shared__ float smx[32], sse[32];
    int64_t s = blockIdx.x;
    int64_t lo, mo;
    slice_offsets(map, s, lo, mo);
    float m = mask ? mask[mo] : 1.0f;
    if (mval_out && threadIdx.x == 0) mval_out[s] = m;
    if (mask && m == 0.0f) {          // skipped slice: contributes nothing
        if (threadIdx.x == 0) { term_out[s] = 0.f; max_out[s] = -INFINITY; se_out[s] = 0.f; }
        return;
    }
    const float *row = logits + lo;
    int C = map.C;
    float mx = -INFINITY, se = 0.f;
    if (map.cstride == 1 && (C & 3) == 0 && (((uintptr_t)row) & 15) == 0) {
        // Four float4 per trip, loaded before any of them is used, so that a thread keeps 64 bytes in
        // flight; one rescale per trip; exponentials through ex2 on the scores times log2(e).
        const float4 *r4 = reinterpret_cast<const float4 *>(row);
        const int n4 = C / 4, bd = blockDim.x;
        constexpr float kL2e = 1.4426950408889634f;
        float mx2 = -INFINITY;                           // running maximum times log2(e)
        for (int j = threadIdx.x; j < n4; j += 4 * bd) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                v[u] = (j + u * bd < n4) ? r4[j + u * bd] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            float cm = mx;
#pragma unroll
            for (int u = 0; u < 4; u++) cm = fmaxf(cm, fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w)));
            if (cm > mx) { const float c2 = cm * kL2e; se *= fast_exp2f(mx2 - c2); mx = cm; mx2 = c2; }
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                a0 += fast_exp2f(fmaf(v[u].x, kL2e, -mx2)); a1 += fast_exp2f(fmaf(v[u].y, kL2e, -mx2));
                a2 += fast_exp2f(fmaf(v[u].z, kL2e, -mx2)); a3 += fast_exp2f(fmaf(v[u].w, kL2e, -mx2));
            }
            se += (a0 + a1) + (a2 + a3);
        }
    } else {
        for (int j = threadIdx.x; j < C; j += blockDim.x) online_add(mx, se, row[(int64_t)j * map.cstride]);
    }
    // merge across the CTA
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float omx = __shfl_xor_sync(0xffffffffu, mx, o), ose = __shfl_xor_sync(0xffffffffu, se, o);
        online_merge(mx, se, omx, ose);
    }
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { smx[w] = mx; sse[w] = se; }
    __syncthreads();
    if (w == 0) {
        mx = lane < nw ? smx[lane] : -INFINITY;
        se = lane < nw ? sse[lane] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float omx = __shfl_xor_sync(0xffffffffu, mx, o), ose = __shfl_xor_sync(0xffffffffu, se, o);
            online_merge(mx, se, omx, ose);
        }
        if (lane == 0) {
            int t = target[s];
            float xt = row[(int64_t)t * map.cstride];
            max_out[s] = mx; se_out[s] = se;
            term_out[s] = (logf(se) + mx - xt) * m;
        }
    }
}

// loss = sum(term) * inv, inv = 1/n_slices or 1/max(sum(mask),1); also stores inv.
__global__ void ce_reduce_kernel(const float *__restrict__ term, const float *__restrict__ mval, int64_t n,
                                 float inv_n, float *__restrict__ loss_out, float *__restrict__ inv_out) {
    __shared__ float sh[32];
    float s = 0.f, ms = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { s += term[i]; if (mval) ms += mval[i]; }
    s = block_sum(s, sh);
    float inv = inv_n;
    if (mval) {
        ms = block_sum(ms, sh);
        if (ms < 1.0f) ms = 1.0f;
        inv = 1.0f / ms;
    }
    if (threadIdx.x == 0) { loss_out[0] = s * inv; inv_out[0] = inv; }
}

__global__ void ce_bwd_kernel(const float *__restrict__ logits, const int *__restrict__ target,
                              const float *__restrict__ mask, SliceMap map,
                              const float *__restrict__ max_in, const float *__restrict__ se_in,
                              const float *__restrict__ gout, const float *__restrict__ inv,
                              float *__restrict__ dlogits, int acc) {
    int64_t s = blockIdx.x;
    int64_t lo, mo;
    slice_offsets(map, s, lo, mo);
    float m = mask ? mask[mo] : 1.0f;
    float *drow = dlogits + lo;
    if (mask && m == 0.0f) {
        // a masked-out position has no gradient; a buffer that was not zero-filled gets its zeros here
        if (!acc) for (int j = threadIdx.x; j < map.C; j += blockDim.x) drow[(int64_t)j * map.cstride] = 0.f;
        return;
    }
    const float *row = logits + lo;
    float mx = max_in[s], se = se_in[s];
    int tgt = target[s];
    float scale = gout[0] * inv[0];
    if (mask) scale *= m;
    int C = map.C;
    if (map.cstride == 1 && (C & 3) == 0 && (((uintptr_t)row) & 15) == 0) {
        const float4 *r4 = reinterpret_cast<const float4 *>(row);
        float4 *d4 = reinterpret_cast<float4 *>(drow);
        for (int j = threadIdx.x; j < C / 4; j += blockDim.x) {
            float4 v = r4[j], d = acc ? d4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            int c = j * 4;
            d.x += (expf(v.x - mx) / se - (c == tgt ? 1.f : 0.f)) * scale;
            d.y += (expf(v.y - mx) / se - (c + 1 == tgt ? 1.f : 0.f)) * scale;
            d.z += (expf(v.z - mx) / se - (c + 2 == tgt ? 1.f : 0.f)) * scale;
            d.w += (expf(v.w - mx) / se - (c + 3 == tgt ? 1.f : 0.f)) * scale;
            d4[j] = d;
        }
    } else {
        for (int j = threadIdx.x; j < C; j += blockDim.x) {
            int64_t o = (int64_t)j * map.cstride;
            float r = (expf(row[o] - mx) / se - (j == tgt ? 1.f : 0.f)) * scale;
            drow[o] = acc ? drow[o] + r : r;
        }
    }
}

// The same gradient, tiled so that the column sums of what is written come for free: CTA
// (32 x 8 threads) = 128 classes x one slab of slices; a thread walks its slab 8 slices at a
// time with one float4 of classes, stores the gradient and keeps the running column sums, which
// end up in partial[slab][C].  The consumer of d(logits) is normally a linear layer whose bias
// gradient is exactly these sums.  Only for stores into a fresh buffer (acc = 0) with packed
// classes; one CTA per slice (above) serves everything else.
// Per-slice constants of the tiled kernel, computed once instead of by every thread of every CTA
// that touches the slice: where the slice starts, -max, scale / sum-of-exponentials, the scale itself
// (0 for a masked-out slice, which then writes zeros) and the target class.
struct __align__(16) CeRow { long long lo; float neg_max, k_exp, k_hot; int tgt; int pad[2]; };
__global__ void ce_rows_kernel(const int *__restrict__ target, const float *__restrict__ mask, SliceMap map,
                               const float *__restrict__ max_in, const float *__restrict__ se_in, const float *__restrict__ gout,
                               const float *__restrict__ inv, CeRow *__restrict__ rows, int64_t n_slices) {
    int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_slices) return;
    int64_t lo, mo;
    slice_offsets(map, s, lo, mo);
    const float m = mask ? mask[mo] : 1.0f;
    const bool skip = mask && m == 0.0f;
    const float scale = skip ? 0.f : (mask ? gout[0] * inv[0] * m : gout[0] * inv[0]);
    CeRow r;
    r.lo = lo; r.neg_max = skip ? 0.f : -max_in[s]; r.k_exp = skip ? 0.f : scale / se_in[s]; r.k_hot = scale;
    r.tgt = skip ? -1 : target[s]; r.pad[0] = skip ? 1 : 0; r.pad[1] = 0;
    rows[s] = r;
}

__global__ void __launch_bounds__(256)
ce_bwd_colsum_kernel(const float *__restrict__ logits, const CeRow *__restrict__ rows, float *__restrict__ dlogits,
                     float *__restrict__ partial, int C, int64_t n_slices, int slices_per) {
    __shared__ float4 tile[8][33];
    const int c = (blockIdx.x * 32 + threadIdx.x) * 4;
    const int64_t s0 = (int64_t)blockIdx.y * slices_per;
    int64_t s1 = s0 + slices_per; if (s1 > n_slices) s1 = n_slices;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < C) {
#pragma unroll 2
        for (int64_t s = s0 + threadIdx.y; s < s1; s += 8) {
            const CeRow r = rows[s];
            float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
            if (!r.pad[0]) {                                    // warp-uniform: a warp works on one slice
                const float4 v = *reinterpret_cast<const float4 *>(logits + r.lo + c);
                const int hot = r.tgt - c;                       // 0..3 when the target class is one of these four
                d.x = fmaf(fast_expf(v.x + r.neg_max), r.k_exp, hot == 0 ? -r.k_hot : 0.f);
                d.y = fmaf(fast_expf(v.y + r.neg_max), r.k_exp, hot == 1 ? -r.k_hot : 0.f);
                d.z = fmaf(fast_expf(v.z + r.neg_max), r.k_exp, hot == 2 ? -r.k_hot : 0.f);
                d.w = fmaf(fast_expf(v.w + r.neg_max), r.k_exp, hot == 3 ? -r.k_hot : 0.f);
            }
            *reinterpret_cast<float4 *>(dlogits + r.lo + c) = d;
            sum.x += d.x; sum.y += d.y; sum.z += d.z; sum.w += d.w;
        }
    }
    tile[threadIdx.y][threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; j++) { float4 v = tile[j][threadIdx.x]; t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w; }
        *reinterpret_cast<float4 *>(partial + (int64_t)blockIdx.y * C + c) = t;
    }
}

static SliceMap make_map(const tensor *logits, const tensor *mask, int dim) {
    SliceMap m;
    memset(&m, 0, sizeof m);
    m.loff = logits->offset; m.moff = mask ? mask->offset : 0;
    m.C = logits->shape[dim]; m.cstride = logits->strides[dim];
    int k = 0;
    for (int d = 0; d < logits->ndim; d++) {
        if (d == dim) continue;
        m.shape[k] = logits->shape[d];
        m.lstride[k] = logits->strides[d];
        // mask has the target's shape: dims of logits without the class dim (src/ops_activation.c:1154-1166)
        m.mstride[k] = (mask && k < mask->ndim && mask->shape[k] != 1) ? mask->strides[k] : 0;
        k++;
    }
    m.nd = k;
    return m;
}

struct CeSaved { float *max_vals, *sum_exp, *inv; };

static void ce_backward_common(grad_fn *fn, tensor *go, bool masked) {
    tensor *logits = fn->inputs[0];
    if (!wants_grad(logits)) return;
    const float *max_vals = (const float *)fn->saved_tensors[0];
    const float *sum_exp = (const float *)fn->saved_tensors[1];
    tensor *target = fn->saved_tensors[2];
    tensor *mask = masked ? fn->saved_tensors[3] : nullptr;
    int dim = *(int *)fn->saved_tensors[masked ? 4 : 3];
    const float *inv = (const float *)fn->saved_tensors[masked ? 5 : 4];
    SliceMap map = make_map(logits, mask, dim);
    int64_t n_slices = numel_of(logits) / map.C;
    if (n_slices <= 0) return;
    bool acc = true;
    float *ag = grad_rows(logits, &acc);
    // Fresh buffer, packed classes, every slice 16-byte aligned: tiled kernel that also leaves the
    // column sums of d(logits) for the layer that consumes it.
    tensor *root = logits; while (root->parent) root = root->parent;
    bool aligned = aligned16(logits->data) && aligned16(ag) && (logits->offset % 4 == 0);
    for (int k = 0; k < map.nd && aligned; k++) aligned = map.lstride[k] % 4 == 0;
    if (!acc && map.cstride == 1 && map.C % 4 == 0 && aligned && root->ndim >= 2 && root->contiguous &&
        root->shape[root->ndim - 1] == map.C && n_slices >= 64) {
        int nslabs = (int)((n_slices + 255) / 256);
        if (nslabs > 256) nslabs = 256;
        int per = (int)((n_slices + nslabs - 1) / nslabs);
        nslabs = (int)((n_slices + per - 1) / per);
        float *partial = dev_alloc_t<float>(fn->pool, (size_t)nslabs * map.C);
        float *sums = colsum_cache_reserve(map.C);
        dim3 grid((map.C / 4 + 31) / 32, nslabs), block(32, 8);
        CeRow *rows = dev_alloc_t<CeRow>(fn->pool, (size_t)n_slices);
        ce_rows_kernel<<<(unsigned)((n_slices + 255) / 256), 256, 0, stream()>>>((const int *)target->data,
            mask ? (const float *)mask->data : nullptr, map, max_vals, sum_exp, (const float *)go->data, inv, rows, n_slices);
        LAUNCHED("ce_rows_kernel");
        ce_bwd_colsum_kernel<<<grid, block, 0, stream()>>>((const float *)logits->data, rows, ag, partial, map.C, n_slices, per);
        prof_work(8.0 * n_slices * map.C);                       // read logits, write d(logits)
        LAUNCHED(masked ? "ce_masked_bwd_kernel" : "ce_bwd_kernel");
        k_colsum_finish(sums, partial, nslabs, map.C);
        // rows of the root that the slices do not cover were zero-filled: they add nothing to the sums
        colsum_cache_publish(ag, numel_of(root) / map.C, map.C);
        return;
    }
    ce_bwd_kernel<<<(unsigned)n_slices, 256, 0, stream()>>>((const float *)logits->data, (const int *)target->data,
        mask ? (const float *)mask->data : nullptr, map, max_vals, sum_exp, (const float *)go->data, inv, ag, acc ? 1 : 0);
    prof_work((acc ? 12.0 : 8.0) * n_slices * map.C);
    LAUNCHED(masked ? "ce_masked_bwd_kernel" : "ce_bwd_kernel");
}
static void cross_entropy_backward(grad_fn *fn, tensor *go) { ce_backward_common(fn, go, false); }
static void cross_entropy_masked_backward(grad_fn *fn, tensor *go) { ce_backward_common(fn, go, true); }

static tensor *ce_forward(struct mem_pool *scratch, const tensor *logits, const tensor *target, const tensor *mask, int dim) {
    int ndim = logits->ndim;
    if (dim < 0) dim += ndim;
    DNN_CHECK(dim >= 0 && dim < ndim, "tensor_cross_entropy: dim out of range");
    SliceMap map = make_map(logits, mask, dim);
    int64_t n_slices = numel_of(logits) / map.C;
    DNN_CHECK(n_slices > 0, "tensor_cross_entropy: empty logits");
    float *max_vals = dev_alloc_t<float>(scratch, (size_t)n_slices);
    float *sum_exp = dev_alloc_t<float>(scratch, (size_t)n_slices);
    float *term = dev_alloc_t<float>(scratch, (size_t)n_slices);
    float *mval = mask ? dev_alloc_t<float>(scratch, (size_t)n_slices) : nullptr;
    float *inv = dev_alloc_t<float>(scratch, 1);
    int one = 1;
    tensor *out = tensor_scratch(scratch, 1, &one, 0);
    ce_fwd_kernel<<<(unsigned)n_slices, 256, 0, stream()>>>((const float *)logits->data, (const int *)target->data,
        mask ? (const float *)mask->data : nullptr, map, max_vals, sum_exp, term, mval);
    prof_work(4.0 * n_slices * map.C);                           // one pass over the logits
    LAUNCHED(mask ? "ce_masked_fwd_kernel" : "ce_fwd_kernel");
    ce_reduce_kernel<<<1, 1024, 0, stream()>>>(term, mval, n_slices, 1.0f / (float)n_slices, (float *)out->data, inv);
    LAUNCHED("ce_reduce_kernel");
    if (dnn_grad_enabled() && logits->requires_grad) {
        int k = 0;
        grad_fn *fn = attach(scratch, out, mask ? cross_entropy_masked_backward : cross_entropy_backward, 1, mask ? 6 : 5);
        fn->inputs[0] = (tensor *)logits;
        fn->saved_tensors[k++] = (tensor *)max_vals;
        fn->saved_tensors[k++] = (tensor *)sum_exp;
        fn->saved_tensors[k++] = (tensor *)target;
        if (mask) fn->saved_tensors[k++] = (tensor *)mask;
        int *sd = host_alloc_t<int>(scratch); *sd = dim;
        fn->saved_tensors[k++] = (tensor *)sd;
        fn->saved_tensors[k++] = (tensor *)inv;
    }
    return out;
}

}  // namespace dnnb

using namespace dnnb;

extern "C" {

tensor *tensor_cross_entropy(struct mem_pool *scratch, const tensor *logits, const tensor *target, int dim) {
    require_device_payloads("tensor_cross_entropy", {logits, target});
    DNN_CHECK(logits && target, "tensor_cross_entropy: NULL argument");
    return ce_forward(scratch, logits, target, nullptr, dim);
}

tensor *tensor_cross_entropy_masked(struct mem_pool *scratch, const tensor *logits, const tensor *target,
                                    const tensor *mask, int dim) {
    require_device_payloads("tensor_cross_entropy_masked", {logits, target, mask});
    DNN_CHECK(logits && target && mask, "tensor_cross_entropy_masked: NULL argument");
    return ce_forward(scratch, logits, target, mask, dim);
}

}  // extern "C"
