// Scaled-dot-product attention (causal / prefix-LM, per-batch sequence lengths),
// forward and backward, without materialising the N x N probability matrix.
// replaces src/attention.c:39-64 (visibility rule), :259-380 (forward),
// :387-540 (backward) and :671-847 (API + tape node).
//
// The reference saves P[B,H,N,N] for backward.  Here forward keeps only the
// per-row log-sum-exp (LSE = max + log(sum)); backward recomputes
// P = exp(scale*Q.K^T - LSE) tile by tile, with D_i = sum_c dO_ic * O_ic in
// place of the reference's rowsum(P o dP) (the two are equal).
//
// This file holds the exact-fp32 kernels: 64x64 tiles staged in shared memory
// (row-major, row pitch HD+4 floats: rows stay 16-byte aligned and the rows a
// quarter-warp reads with one 128-bit load fall in different banks), 256 threads.
// A score tile is owned as rows ty+16*i x columns tx+16*j; an output tile
// ([64, d]) as rows ty+16*i (4*ty+i in the dK/dV kernel) x HD/16 adjacent
// columns, so every inner loop reads shared memory 128 bits at a time: 8 loads
// for 64 FMAs.
#include "common.cuh"
#include "device_utils.cuh"

namespace dnnb {

constexpr int TB = 64;           // tile rows (queries) and tile columns (keys)
constexpr int PS = TB + 4;       // pitch of the probability tile

struct AttnParams {
    const float *q, *k, *v;      // [B,H,N,d]
    float *o;                    // [B,H,N,d]
    float *lse;                  // [B,H,N]
    const float *dout, *dvec;    // upstream gradient, D_i
    float *dq, *dk, *dv;
    const int *seq_lens;         // device [B] or null
    int B, H, N, d;
    int prefix;                  // 0 for causal
    float scale;
    int store;                   // bit 0/1/2: dq/dk/dv are written, not added to
    // additive mask broadcast to [B,H,N,N] (src/attention.c:314-325): element (b,h,i,j) at mask[b*m_sb + h*m_sh + i*m_si + j*m_sj],
    // added to the scaled score of every visible column; null when there is none
    const float *mask;
    int64_t m_sb, m_sh, m_si, m_sj;
};
__device__ __forceinline__ float mask_at(const AttnParams &p, int b, int h, int i, int j) {
    return p.mask ? p.mask[b * p.m_sb + h * p.m_sh + i * p.m_si + j * p.m_sj] : 0.f;
}

__device__ __forceinline__ int visible_len(int i, int prefix, int nb) {
    int v = (i < prefix) ? prefix : i + 1;       // prefix == 0 gives the causal rule
    return v < nb ? v : nb;
}

// Loads rows [r0, r0+TB) x d of a [N,d] slice into shared memory (pitch HD+4),
// zero-filling rows >= nrows and columns >= d.
template <int HD>
__device__ __forceinline__ void load_tile(float *sm, const float *g, int r0, int nrows, int d) {
    constexpr int TP = HD + 4;
    if ((d & 3) == 0 && (reinterpret_cast<uintptr_t>(g) & 15) == 0) {
        constexpr int C4 = HD / 4;
        for (int idx = threadIdx.x; idx < TB * C4; idx += blockDim.x) {
            int r = idx / C4, c = (idx - r * C4) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r0 + r < nrows && c < d) v = *reinterpret_cast<const float4 *>(g + (int64_t)(r0 + r) * d + c);
            *reinterpret_cast<float4 *>(sm + r * TP + c) = v;
        }
        return;
    }
    for (int idx = threadIdx.x; idx < TB * HD; idx += blockDim.x) {
        int r = idx / HD, c = idx - r * HD;
        float v = 0.f;
        if (r0 + r < nrows && c < d) v = g[(int64_t)(r0 + r) * d + c];
        sm[r * TP + c] = v;
    }
}

// The HD/16 output columns of thread column tx: adjacent, so one row's share is one 64- or 128-bit load
// (two 128-bit loads, 64 columns apart, for HD = 128).
template <int HD> __device__ __forceinline__ int col_of(int tx, int c) {
    if (HD == 32) return 2 * tx + c;
    if (HD == 64) return 4 * tx + c;
    return (c < 4) ? 4 * tx + c : 64 + 4 * tx + (c - 4);
}
template <int HD> __device__ __forceinline__ void ld_cols(const float *row, int tx, float (&v)[HD / 16]) {
    if (HD == 32) {
        const float2 t = *reinterpret_cast<const float2 *>(row + 2 * tx);
        v[0] = t.x; v[1] = t.y;
    } else {
        const float4 t = *reinterpret_cast<const float4 *>(row + 4 * tx);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        if (HD == 128) {
            const float4 u = *reinterpret_cast<const float4 *>(row + 64 + 4 * tx);
            v[4 % (HD / 16)] = u.x; v[5 % (HD / 16)] = u.y; v[6 % (HD / 16)] = u.z; v[7 % (HD / 16)] = u.w;
        }
    }
}
__device__ __forceinline__ float f4_at(const float4 &v, int k) { return k == 0 ? v.x : k == 1 ? v.y : k == 2 ? v.z : v.w; }

// s[i][j] = sum_c A[ty+16i][c] * Bt[tx+16j][c], c ascending
template <int HD>
__device__ __forceinline__ void tile_dot(const float *A, const float *Bm, int ty, int tx, float s[4][4]) {
    constexpr int TP = HD + 4;
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) s[i][j] = 0.f;
#pragma unroll 4
    for (int c = 0; c < HD; c += 4) {
        float4 a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; i++) a[i] = *reinterpret_cast<const float4 *>(A + (ty + 16 * i) * TP + c);
#pragma unroll
        for (int j = 0; j < 4; j++) b[j] = *reinterpret_cast<const float4 *>(Bm + (tx + 16 * j) * TP + c);
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float t = s[i][j];
                t = fmaf(a[i].x, b[j].x, t); t = fmaf(a[i].y, b[j].y, t);
                t = fmaf(a[i].z, b[j].z, t); t = fmaf(a[i].w, b[j].w, t);
                s[i][j] = t;
            }
    }
}

// acc[i][c] += sum_j W[ty+16i][j] * X[j][col_of(tx,c)] over the TB rows of X, j ascending
template <int HD>
__device__ __forceinline__ void tile_apply(const float *W, const float *X, int ty, int tx, float (&acc)[4][HD / 16]) {
    constexpr int TP = HD + 4, CC = HD / 16;
#pragma unroll 2
    for (int j = 0; j < TB; j += 4) {
        float4 w[4];
        float x[4][CC];
#pragma unroll
        for (int i = 0; i < 4; i++) w[i] = *reinterpret_cast<const float4 *>(W + (ty + 16 * i) * PS + j);
#pragma unroll
        for (int jj = 0; jj < 4; jj++) ld_cols<HD>(X + (j + jj) * TP, tx, x[jj]);
#pragma unroll
        for (int jj = 0; jj < 4; jj++)
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int c = 0; c < CC; c++) acc[i][c] = fmaf(f4_at(w[i], jj), x[jj][c], acc[i][c]);
    }
}

__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- forward -----------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(256) attn_fwd_kernel(AttnParams p) {
    extern __shared__ __align__(16) float smem[];
    constexpr int TP = HD + 4;
    float *Qs = smem, *Ks = Qs + TB * TP, *Vs = Ks + TB * TP, *Ps = Vs + TB * TP;
    int b = blockIdx.z, h = blockIdx.y, i0 = blockIdx.x * TB;
    int nb = p.seq_lens ? p.seq_lens[b] : p.N;
    if (nb > p.N) nb = p.N;
    int64_t slice = ((int64_t)b * p.H + h) * p.N;
    const float *q = p.q + slice * p.d, *k = p.k + slice * p.d, *v = p.v + slice * p.d;
    float *o = p.o + slice * p.d;
    int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    constexpr int CC = HD / 16;

    if (i0 >= nb) {          // padded rows: output is zero (src/attention.c:376-377)
        for (int idx = threadIdx.x; idx < TB * p.d; idx += blockDim.x) {
            int r = idx / p.d;
            if (i0 + r < p.N) o[(int64_t)i0 * p.d + idx] = 0.f;
        }
        return;
    }
    load_tile<HD>(Qs, q, i0, nb, p.d);
    float m[4], l[4], acc[4][CC];
#pragma unroll
    for (int i = 0; i < 4; i++) { m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < CC; c++) acc[i][c] = 0.f; }
    int i_last = min(i0 + TB, nb) - 1;
    int jmax = visible_len(i_last, p.prefix, nb);           // columns any row of this tile can see
    if (p.prefix > 0 && i0 < p.prefix) jmax = max(jmax, min(p.prefix, nb));

    for (int j0 = 0; j0 < jmax; j0 += TB) {
        __syncthreads();
        load_tile<HD>(Ks, k, j0, nb, p.d);
        load_tile<HD>(Vs, v, j0, nb, p.d);
        __syncthreads();
        float s[4][4];
        tile_dot<HD>(Qs, Ks, ty, tx, s);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int row = i0 + ty + 16 * i;
            int vis = row < nb ? visible_len(row, p.prefix, nb) : 0;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                int col = j0 + tx + 16 * j;
                s[i][j] = col < vis ? s[i][j] * p.scale + mask_at(p, b, h, row, col) : -INFINITY;
                mx = fmaxf(mx, s[i][j]);
            }
            mx = half_warp_max(mx);
            float mnew = fmaxf(m[i], mx);
            float corr = (mnew == -INFINITY) ? 1.f : expf(m[i] - mnew);
            float rs = 0.f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float pe = (s[i][j] == -INFINITY) ? 0.f : expf(s[i][j] - mnew);
                Ps[(ty + 16 * i) * PS + tx + 16 * j] = pe;
                rs += pe;
            }
            rs = half_warp_sum(rs);
            l[i] = l[i] * corr + rs;
            m[i] = mnew;
#pragma unroll
            for (int c = 0; c < CC; c++) acc[i][c] *= corr;
        }
        __syncthreads();
        tile_apply<HD>(Ps, Vs, ty, tx, acc);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int row = i0 + ty + 16 * i;
        if (row >= p.N) continue;
        bool live = row < nb;
        float inv = live ? 1.f / l[i] : 0.f;
#pragma unroll
        for (int c = 0; c < CC; c++) {
            int col = col_of<HD>(tx, c);
            if (col < p.d) o[(int64_t)row * p.d + col] = live ? acc[i][c] * inv : 0.f;
        }
        if (tx == 0 && p.lse) p.lse[slice + row] = live ? m[i] + logf(l[i]) : 0.f;
    }
}

// ---- backward: D_i = sum_c dO_ic * O_ic --------------------------------------
__global__ void attn_bwd_prep_kernel(const float *__restrict__ dout, const float *__restrict__ o,
                                     float *__restrict__ dvec, int64_t rows, int d) {
    int lane = threadIdx.x & 31;
    int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    float s = 0.f;
    for (int c = lane; c < d; c += 32) s += dout[r * d + c] * o[r * d + c];
    s = warp_sum(s);
    if (lane == 0) dvec[r] = s;
}

// Recomputes P and dS for the (query tile at Qs/dOs, key tile at Ks/Vs) pair.
template <int HD>
__device__ __forceinline__ void recompute_p_ds(const AttnParams &p, const float *Qs, const float *Ks, const float *Vs,
                                               const float *dOs, const float *lse_s, const float *d_s,
                                               int i0, int j0, int nb, int ty, int tx, float *Ps, float *dSs, int b, int h) {
    float s[4][4], dp[4][4];
    tile_dot<HD>(Qs, Ks, ty, tx, s);
    tile_dot<HD>(dOs, Vs, ty, tx, dp);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int r = ty + 16 * i, row = i0 + r;
        int vis = row < nb ? visible_len(row, p.prefix, nb) : 0;
        float lse = lse_s[r], dd = d_s[r];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int col = j0 + tx + 16 * j;
            float pe = col < vis ? expf(s[i][j] * p.scale + mask_at(p, b, h, row, col) - lse) : 0.f;
            Ps[r * PS + tx + 16 * j] = pe;
            dSs[r * PS + tx + 16 * j] = pe * (dp[i][j] - dd) * p.scale;
        }
    }
}

// One CTA per key tile: dK_j += sum_i dS_ij Q_i, dV_j += sum_i P_ij dO_i.
template <int HD>
__global__ void __launch_bounds__(256) attn_bwd_dkv_kernel(AttnParams p) {
    extern __shared__ __align__(16) float smem[];
    constexpr int TP = HD + 4, TS = TB * TP;
    float *Qs = smem, *Ks = Qs + TS, *Vs = Ks + TS, *dOs = Vs + TS, *Ps = dOs + TS, *dSs = Ps + TB * PS;
    float *lse_s = dSs + TB * PS, *d_s = lse_s + TB;
    int b = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * TB;
    int nb = p.seq_lens ? p.seq_lens[b] : p.N;
    if (nb > p.N) nb = p.N;
    if (j0 >= nb) return;
    int64_t slice = ((int64_t)b * p.H + h) * p.N;
    const float *q = p.q + slice * p.d, *k = p.k + slice * p.d, *v = p.v + slice * p.d, *dout = p.dout + slice * p.d;
    int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    constexpr int CC = HD / 16;
    float dk[4][CC], dv[4][CC];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int c = 0; c < CC; c++) { dk[i][c] = 0.f; dv[i][c] = 0.f; }
    load_tile<HD>(Ks, k, j0, nb, p.d);
    load_tile<HD>(Vs, v, j0, nb, p.d);
    // first query tile that can see a key of this tile
    int i_begin = (p.prefix > 0 && j0 < p.prefix) ? 0 : (j0 / TB) * TB;
    for (int i0 = i_begin; i0 < nb; i0 += TB) {
        __syncthreads();
        load_tile<HD>(Qs, q, i0, nb, p.d);
        load_tile<HD>(dOs, dout, i0, nb, p.d);
        if (threadIdx.x < TB) {
            int row = i0 + threadIdx.x;
            lse_s[threadIdx.x] = row < nb ? p.lse[slice + row] : 0.f;
            d_s[threadIdx.x] = row < nb ? p.dvec[slice + row] : 0.f;
        }
        __syncthreads();
        recompute_p_ds<HD>(p, Qs, Ks, Vs, dOs, lse_s, d_s, i0, j0, nb, ty, tx, Ps, dSs, b, h);
        __syncthreads();
        // this thread owns key rows 4*ty+jj (adjacent: their P and dS of one query are one 128-bit load each)
        // and feature columns col_of(tx, c)
#pragma unroll 4
        for (int i = 0; i < TB; i++) {
            const float4 pj = *reinterpret_cast<const float4 *>(Ps + i * PS + 4 * ty);
            const float4 sj = *reinterpret_cast<const float4 *>(dSs + i * PS + 4 * ty);
            float go[CC], qq[CC];
            ld_cols<HD>(dOs + i * TP, tx, go);
            ld_cols<HD>(Qs + i * TP, tx, qq);
#pragma unroll
            for (int jj = 0; jj < 4; jj++)
#pragma unroll
                for (int c = 0; c < CC; c++) { dv[jj][c] = fmaf(f4_at(pj, jj), go[c], dv[jj][c]); dk[jj][c] = fmaf(f4_at(sj, jj), qq[c], dk[jj][c]); }
        }
    }
#pragma unroll
    for (int jj = 0; jj < 4; jj++) {
        int row = j0 + 4 * ty + jj;
        if (row >= nb) continue;
#pragma unroll
        for (int c = 0; c < CC; c++) {
            int col = col_of<HD>(tx, c);
            if (col >= p.d) continue;
            int64_t at = (slice + row) * p.d + col;
            if (p.dk) p.dk[at] = (p.store & 2) ? dk[jj][c] : p.dk[at] + dk[jj][c];
            if (p.dv) p.dv[at] = (p.store & 4) ? dv[jj][c] : p.dv[at] + dv[jj][c];
        }
    }
}

// One CTA per query tile: dQ_i += sum_j dS_ij K_j.
template <int HD>
__global__ void __launch_bounds__(256) attn_bwd_dq_kernel(AttnParams p) {
    extern __shared__ __align__(16) float smem[];
    constexpr int TP = HD + 4, TS = TB * TP;
    float *Qs = smem, *Ks = Qs + TS, *Vs = Ks + TS, *dOs = Vs + TS, *Ps = dOs + TS, *dSs = Ps + TB * PS;
    float *lse_s = dSs + TB * PS, *d_s = lse_s + TB;
    int b = blockIdx.z, h = blockIdx.y, i0 = blockIdx.x * TB;
    int nb = p.seq_lens ? p.seq_lens[b] : p.N;
    if (nb > p.N) nb = p.N;
    if (i0 >= nb) return;
    int64_t slice = ((int64_t)b * p.H + h) * p.N;
    const float *q = p.q + slice * p.d, *k = p.k + slice * p.d, *v = p.v + slice * p.d, *dout = p.dout + slice * p.d;
    int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    constexpr int CC = HD / 16;
    float dq[4][CC];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int c = 0; c < CC; c++) dq[i][c] = 0.f;
    load_tile<HD>(Qs, q, i0, nb, p.d);
    load_tile<HD>(dOs, dout, i0, nb, p.d);
    if (threadIdx.x < TB) {
        int row = i0 + threadIdx.x;
        lse_s[threadIdx.x] = row < nb ? p.lse[slice + row] : 0.f;
        d_s[threadIdx.x] = row < nb ? p.dvec[slice + row] : 0.f;
    }
    int i_last = min(i0 + TB, nb) - 1;
    int jmax = visible_len(i_last, p.prefix, nb);
    if (p.prefix > 0 && i0 < p.prefix) jmax = max(jmax, min(p.prefix, nb));
    for (int j0 = 0; j0 < jmax; j0 += TB) {
        __syncthreads();
        load_tile<HD>(Ks, k, j0, nb, p.d);
        load_tile<HD>(Vs, v, j0, nb, p.d);
        __syncthreads();
        recompute_p_ds<HD>(p, Qs, Ks, Vs, dOs, lse_s, d_s, i0, j0, nb, ty, tx, Ps, dSs, b, h);
        __syncthreads();
        tile_apply<HD>(dSs, Ks, ty, tx, dq);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int row = i0 + ty + 16 * i;
        if (row >= nb) continue;
#pragma unroll
        for (int c = 0; c < CC; c++) {
            int col = col_of<HD>(tx, c);
            if (col < p.d) { int64_t at = (slice + row) * p.d + col; p.dq[at] = (p.store & 1) ? dq[i][c] : p.dq[at] + dq[i][c]; }
        }
    }
}

template <int HD> static size_t fwd_smem() { return (size_t)(3 * TB * (HD + 4) + TB * PS) * 4; }
template <int HD> static size_t bwd_smem() { return (size_t)(4 * TB * (HD + 4) + 2 * TB * PS + 2 * TB) * 4; }

template <int HD>
static void attn_fwd_launch(const AttnParams &p) {
    static bool once = false;
    if (!once) {
        CUDA_OK(cudaFuncSetAttribute(attn_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fwd_smem<HD>()));
        CUDA_OK(cudaFuncSetAttribute(attn_fwd_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        once = true;
    }
    dim3 grid((p.N + TB - 1) / TB, p.H, p.B);
    attn_fwd_kernel<HD><<<grid, 256, fwd_smem<HD>(), stream()>>>(p);
    LAUNCHED("attn_fwd_kernel");
}
template <int HD>
static void attn_bwd_launch(const AttnParams &p) {
    static bool once = false;
    if (!once) {
        CUDA_OK(cudaFuncSetAttribute(attn_bwd_dkv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bwd_smem<HD>()));
        CUDA_OK(cudaFuncSetAttribute(attn_bwd_dq_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bwd_smem<HD>()));
        CUDA_OK(cudaFuncSetAttribute(attn_bwd_dkv_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        CUDA_OK(cudaFuncSetAttribute(attn_bwd_dq_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        once = true;
    }
    dim3 grid((p.N + TB - 1) / TB, p.H, p.B);
    if (p.dk || p.dv) { attn_bwd_dkv_kernel<HD><<<grid, 256, bwd_smem<HD>(), stream()>>>(p); LAUNCHED("attn_bwd_dkv_kernel"); }
    if (p.dq) { attn_bwd_dq_kernel<HD><<<grid, 256, bwd_smem<HD>(), stream()>>>(p); LAUNCHED("attn_bwd_dq_kernel"); }
}

// tensor-core kernels (attention_tc.cu)
bool attn_tc_supported(int d, const HeadView &q, const HeadView &k, const HeadView &v);
void attn_forward_tc(const HeadView &q, const HeadView &k, const HeadView &v, const HeadView &o, float *lse, const int *seq_lens,
                     int B, int H, int N, int d, int prefix, float scale);
void attn_backward_tc(const HeadView &q, const HeadView &k, const HeadView &v, const float *lse, const HeadView &dout, const float *dvec,
                      const HeadView &dq, const HeadView &dk, const HeadView &dv, const int *seq_lens,
                      int B, int H, int N, int d, int prefix, float scale, int store,
                      const float *rope_c = nullptr, const float *rope_s = nullptr);

// TF32 mode runs on the tensor core (head dims 32 and 64); the FP32 and 3xTF32 modes, and
// other head dims, run the exact kernels of this file.
static bool use_tc(const AttnParams &p) {
    return gemm_mode() == DNN_CUDA_GEMM_TF32 && p.mask == nullptr &&
           attn_tc_supported(p.d, packed_heads(p.q, p.H, p.N, p.d), packed_heads(p.k, p.H, p.N, p.d), packed_heads(p.v, p.H, p.N, p.d));
}

void attn_forward_fp32(const AttnParams &p) {
    if (p.d <= 32) attn_fwd_launch<32>(p);
    else if (p.d <= 64) attn_fwd_launch<64>(p);
    else attn_fwd_launch<128>(p);
}
void attn_backward_fp32(const AttnParams &p) {
    if (p.d <= 32) attn_bwd_launch<32>(p);
    else if (p.d <= 64) attn_bwd_launch<64>(p);
    else attn_bwd_launch<128>(p);
}

// D_i for token-major dO and O: row (b,n,h) of [B,N,H,d] -> dvec[(b*H + h)*N + n].
// d/4 lanes share a row (one float4 each), so a warp covers 128/d rows with 128-bit loads.
template <int D, bool TOKMAJOR>
__global__ void attn_bwd_prep_v4_kernel(const float4 *__restrict__ dout, const float4 *__restrict__ o,
                                        float *__restrict__ dvec, int B, int N, int H) {
    constexpr int LPR = D / 4, RPW = 32 / LPR;
    const int lane = threadIdx.x & 31, sub = lane % LPR;
    const int64_t rows = (int64_t)B * N * H;
    int64_t r = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * RPW + lane / LPR;     // (b, n, h)
    float s = 0.f;
    if (r < rows) {
        float4 a = dout[r * LPR + sub], b = o[r * LPR + sub];
        s = a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
    }
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (r < rows && sub == 0) {
        if (TOKMAJOR) {
            int h = (int)(r % H);
            int64_t bn = r / H;
            int n = (int)(bn % N), b = (int)(bn / N);
            dvec[((int64_t)b * H + h) * N + n] = s;
        } else {
            dvec[r] = s;              // rows are already (b, h, n)
        }
    }
}
// Both layouts go through the same arithmetic (same partial sums, same reduction tree), so the
// packed and the token-major path give identical D_i.
template <bool TOKMAJOR>
static void launch_prep_v4(const float *dout, const float *o, float *dvec, int B, int N, int H, int d) {
    const float4 *g4 = reinterpret_cast<const float4 *>(dout), *o4 = reinterpret_cast<const float4 *>(o);
    int64_t rows = (int64_t)B * N * H;
    if (d == 64) attn_bwd_prep_v4_kernel<64, TOKMAJOR><<<(unsigned)((rows + 15) / 16), 256, 0, stream()>>>(g4, o4, dvec, B, N, H);
    else         attn_bwd_prep_v4_kernel<32, TOKMAJOR><<<(unsigned)((rows + 31) / 32), 256, 0, stream()>>>(g4, o4, dvec, B, N, H);
    LAUNCHED("attn_bwd_prep_kernel");
}

struct AttnSaved { float *lse; const int *seq_lens_dev; int mode, prefix; float scale; tensor *out; tensor *mask; };

// Strides of an additive mask against the coordinates (b, h, i, j).  The reference looks the mask up with
// _bcast_off(mask, mask->ndim, {b,h,i,j}) (src/attention.c:317-323, src/broadcast.h:26-44): dimension k of the
// mask is indexed by the k-th coordinate, dimensions of size 1 repeat.  A 4-D mask therefore broadcasts as
// documented, while a mask of fewer dimensions is read by the LEADING coordinates (an [N,N] mask at [b][h]).
// That lookup is kept as it is; what is added is the bounds check the reference does not have.
static void set_mask(AttnParams &p, const tensor *mask) {
    p.mask = nullptr; p.m_sb = p.m_sh = p.m_si = p.m_sj = 0;
    if (!mask) return;
    DNN_CHECK(mask->ndim >= 1 && mask->ndim <= 4, "tensor_attention: mask must have 1 to 4 dims");
    const int want[4] = {p.B, p.H, p.N, p.N};
    int64_t st[4] = {0, 0, 0, 0};
    for (int k = 0; k < mask->ndim; k++) {
        DNN_CHECK(mask->shape[k] == 1 || mask->shape[k] >= want[k], "tensor_attention: mask dimension smaller than the coordinate that indexes it");
        st[k] = mask->shape[k] == 1 ? 0 : mask->strides[k];
    }
    p.mask = (const float *)mask->data + mask->offset;
    p.m_sb = st[0]; p.m_sh = st[1]; p.m_si = st[2]; p.m_sj = st[3];
}

static void attention_backward(grad_fn *fn, tensor *go) {
    tensor *q = fn->inputs[0], *k = fn->inputs[1], *v = fn->inputs[2];
    AttnSaved *sv = (AttnSaved *)fn->saved_tensors[0];
    AttnParams p;
    memset(&p, 0, sizeof p);
    p.B = q->shape[0]; p.H = q->shape[1]; p.N = q->shape[2]; p.d = q->shape[3];
    p.q = (const float *)q->data; p.k = (const float *)k->data; p.v = (const float *)v->data;
    p.o = (float *)sv->out->data; p.lse = sv->lse; p.seq_lens = sv->seq_lens_dev;
    p.prefix = sv->mode == ATTENTION_PREFIX_LM ? sv->prefix : 0; p.scale = sv->scale;
    p.dout = (const float *)go->data;
    set_mask(p, sv->mask);
    // Without seq_lens the kernels write every row of dq, dk and dv, so a gradient buffer
    // that nothing has written yet is stored to instead of zero-filled and added to.
    // Operands that share a buffer, or padded batches, keep the add.
    bool full = sv->seq_lens_dev == nullptr && q != k && q != v && k != v;
    bool aq = true, ak = true, av = true;
    p.dq = wants_grad(q) ? (full ? grad_full(q, &aq) : _grad_ensure(q)) : nullptr;
    p.dk = wants_grad(k) ? (full ? grad_full(k, &ak) : _grad_ensure(k)) : nullptr;
    p.dv = wants_grad(v) ? (full ? grad_full(v, &av) : _grad_ensure(v)) : nullptr;
    p.store = (aq ? 0 : 1) | (ak ? 0 : 2) | (av ? 0 : 4);
    int64_t rows = (int64_t)p.B * p.H * p.N;
    float *dvec = dev_alloc_t<float>(fn->pool, (size_t)rows);
    if ((p.d == 32 || p.d == 64) && aligned16(p.dout) && aligned16(p.o)) {
        launch_prep_v4<false>(p.dout, p.o, dvec, p.B, p.N, p.H, p.d);
    } else {
        attn_bwd_prep_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream()>>>(p.dout, p.o, dvec, rows, p.d);
        LAUNCHED("attn_bwd_prep_kernel");
    }
    p.dvec = dvec;
    auto pk = [&](const float *x) { return packed_heads(x, p.H, p.N, p.d); };
    if (use_tc(p)) attn_backward_tc(pk(p.q), pk(p.k), pk(p.v), p.lse, pk(p.dout), p.dvec, pk(p.dq), pk(p.dk), pk(p.dv), p.seq_lens,
                                    p.B, p.H, p.N, p.d, p.prefix, p.scale, p.store);
    else attn_backward_fp32(p);
}


// ---- attention straight from a fused QKV projection ---------------------------------------
// qkv is the [B,N,3*H*d] output of the QKV linear layer, i.e. [B,N,3,H,d].  The tensor-core
// kernels read Q, K and V through strided tensor maps and write the output token-major
// [B,N,H*d], so split_qkv_heads, merge_heads and their backward copies disappear; RoPE is
// applied to the Q and K slices of qkv in place (nothing else reads qkv: the backward of the
// projection needs its inputs, not its output).  Backward writes dQ, dK, dV straight into the
// gradient of qkv and undoes the rotation there.  Same arithmetic as the unfused op sequence
// (src/transformer.c:143-170), element for element.

// rows = B*N tokens; each token row holds 3*H*d floats; pairs of the first 2*H*d are rotated.
template <bool BWD>
__global__ void rope_qkv_kernel(float *__restrict__ qkv, const float *__restrict__ fc, const float *__restrict__ fs,
                                int64_t total2, int N, int H, int d) {
    // one thread per float4 = two adjacent pairs of q or k
    const int d4 = d >> 2, dh = d >> 1, per_tok = 2 * H * d4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total2; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t tok = i / per_tok;
        int rem = (int)(i - tok * per_tok);         // (which, h, quad)
        int quad = rem % d4;
        int n = (int)(tok % N);
        float4 *ptr = reinterpret_cast<float4 *>(qkv + tok * (int64_t)(3 * H * d)) + rem;
        float2 c = *reinterpret_cast<const float2 *>(fc + (int64_t)n * dh + 2 * quad);
        float2 sn = *reinterpret_cast<const float2 *>(fs + (int64_t)n * dh + 2 * quad);
        float4 v = *ptr, o;
        if (!BWD) {
            rope_fwd_pair(v.x, v.y, c.x, sn.x, o.x, o.y);
            rope_fwd_pair(v.z, v.w, c.y, sn.y, o.z, o.w);
        } else {
            rope_inv_pair(v.x, v.y, c.x, sn.x, o.x, o.y);
            rope_inv_pair(v.z, v.w, c.y, sn.y, o.z, o.w);
        }
        *ptr = o;
    }
}

static int g_fused_attention = -1;      // -1: not decided yet (environment DNN_CUDA_FUSED_QKV, default on)
static bool fused_attention_enabled() {
    if (g_fused_attention < 0) { const char *e = getenv("DNN_CUDA_FUSED_QKV"); g_fused_attention = (e && e[0] == '0') ? 0 : 1; }
    return g_fused_attention != 0;
}

struct FusedSaved { float *lse; const int *seq_lens_dev; int mode, prefix, H; float scale; tensor *out; const float *fc, *fs; };

static HeadView qkv_slice(float *base, int which, int N, int H, int d) {
    HeadView v; v.p = base + (int64_t)which * H * d; v.sb = (int64_t)N * 3 * H * d; v.sh = d; v.sn = (int64_t)3 * H * d; return v;
}
static HeadView token_major(float *base, int N, int H, int d) {
    HeadView v; v.p = base; v.sb = (int64_t)N * H * d; v.sh = d; v.sn = (int64_t)H * d; return v;
}
static void rope_qkv(bool bwd, float *qkv, const float *fc, const float *fs, int B, int N, int H, int d) {
    int64_t total = (int64_t)B * N * 2 * H * (d / 4);
    if (total <= 0) return;
    if (bwd) rope_qkv_kernel<true><<<grid_for(total, 256), 256, 0, stream()>>>(qkv, fc, fs, total, N, H, d);
    else     rope_qkv_kernel<false><<<grid_for(total, 256), 256, 0, stream()>>>(qkv, fc, fs, total, N, H, d);
    LAUNCHED(bwd ? "rope_qkv_bwd_kernel" : "rope_qkv_fwd_kernel");
}

static void attention_qkv_backward(grad_fn *fn, tensor *go) {
    tensor *qkv = fn->inputs[0];
    if (!wants_grad(qkv)) return;
    FusedSaved *sv = (FusedSaved *)fn->saved_tensors[0];
    const int B = qkv->shape[0], N = qkv->shape[1], H = sv->H, d = qkv->shape[2] / (3 * H);
    float *qd = (float *)qkv->data;
    const float *gd = (const float *)go->data;
    int64_t rows = (int64_t)B * N * H;
    float *dvec = dev_alloc_t<float>(fn->pool, (size_t)rows);
    launch_prep_v4<true>(gd, (const float *)sv->out->data, dvec, B, N, H, d);
    // The kernels store every row when no per-batch lengths are given.  The rotation is undone
    // in place, which is only right on a buffer that holds nothing but this op's gradient: a
    // gradient buffer that already has content gets the result through a temporary.
    bool acc = true;
    float *g_qkv = grad_full(qkv, &acc);
    int64_t numel = (int64_t)B * N * 3 * H * d;
    float *dst = acc ? dev_alloc_t<float>(fn->pool, (size_t)numel) : g_qkv;
    int store = 7;
    if (sv->seq_lens_dev) { k_fill(dst, numel, 0.0f); store = 0; }       // rows beyond a sequence's length are never written
    // In store mode the kernels rotate dQ and dK back in their epilogues; otherwise a pass over dst does it.
    const bool rot_in_kernel = sv->fc && store == 7 && (((uintptr_t)sv->fc | (uintptr_t)sv->fs) & 15) == 0;
    attn_backward_tc(qkv_slice(qd, 0, N, H, d), qkv_slice(qd, 1, N, H, d), qkv_slice(qd, 2, N, H, d), sv->lse,
                     token_major(const_cast<float *>(gd), N, H, d), dvec,
                     qkv_slice(dst, 0, N, H, d), qkv_slice(dst, 1, N, H, d), qkv_slice(dst, 2, N, H, d), sv->seq_lens_dev,
                     B, H, N, d, sv->mode == ATTENTION_PREFIX_LM ? sv->prefix : 0, sv->scale, store,
                     rot_in_kernel ? sv->fc : nullptr, rot_in_kernel ? sv->fs : nullptr);
    if (sv->fc && !rot_in_kernel) rope_qkv(true, dst, sv->fc, sv->fs, B, N, H, d);
    if (acc) k_axpy_acc(g_qkv, dst, numel);
}

// Whether a block with these sizes will take the fused path (asked before the QKV projection
// runs, so that the projection's epilogue can apply the rotation).
bool attention_from_qkv_applicable(const tensor *x, int H, int d, const tensor *fc, const tensor *fs) {
    if (!fused_attention_enabled() || gemm_mode() != DNN_CUDA_GEMM_TF32) return false;
    if (!x || x->ndim != 3 || H <= 0 || (d != 32 && d != 64)) return false;
    if (fc && fs) {
        if (!fc->contiguous || !fs->contiguous || fc->shape[0] < x->shape[1]) return false;
        const float *a = (const float *)fc->data + fc->offset, *b = (const float *)fs->data + fs->offset;
        if ((((uintptr_t)a | (uintptr_t)b) & 15) != 0) return false;
    }
    return true;
}

// Returns nullptr when the tensor-core path does not apply (mode, head size, layout); the
// caller then runs the unfused op sequence.  `rotated`: the projection that produced qkv has
// already applied RoPE to its Q and K columns.
tensor *attention_from_qkv(struct mem_pool *scratch, tensor *qkv, int H, tensor *fc, tensor *fs,
                           attention_mode mode, int prefix_len, const int *seq_lens, bool rotated) {
    if (!fused_attention_enabled() || gemm_mode() != DNN_CUDA_GEMM_TF32) return nullptr;
    if (!qkv || qkv->ndim != 3 || !qkv->contiguous || qkv->offset != 0 || qkv->parent) return nullptr;
    const int B = qkv->shape[0], N = qkv->shape[1], D3 = qkv->shape[2];
    if (H <= 0 || D3 % (3 * H) != 0) return nullptr;
    const int d = D3 / (3 * H);
    float *qd = (float *)qkv->data;
    if (!attn_tc_supported(d, qkv_slice(qd, 0, N, H, d), qkv_slice(qd, 1, N, H, d), qkv_slice(qd, 2, N, H, d))) return nullptr;
    const float *fcd = nullptr, *fsd = nullptr;
    if (fc && fs) {
        if (!fc->contiguous || !fs->contiguous || fc->shape[0] < N) return nullptr;
        fcd = (const float *)fc->data + fc->offset; fsd = (const float *)fs->data + fs->offset;
        if ((((uintptr_t)fcd | (uintptr_t)fsd) & 7) != 0) return nullptr;
    }
    if (mode == ATTENTION_PREFIX_LM) DNN_CHECK(prefix_len > 0 && prefix_len <= N, "tensor_attention: prefix_len out of range");
    if (mode == ATTENTION_CAUSAL) DNN_CHECK(prefix_len == 0, "tensor_attention: prefix_len must be 0 in causal mode");

    int shape[3] = {B, N, H * d};
    tensor *out = tensor_scratch(scratch, 3, shape, 0);
    bool needs_grad = dnn_grad_enabled() && qkv->requires_grad;
    float *lse = needs_grad ? dev_alloc_t<float>(scratch, (size_t)B * H * N) : nullptr;
    const int *lens = seq_lens ? (const int *)dev_put(scratch, seq_lens, (size_t)B * sizeof(int)) : nullptr;
    const float scale = 1.0f / sqrtf((float)d);
    if (fcd && !rotated) rope_qkv(false, qd, fcd, fsd, B, N, H, d);
    attn_forward_tc(qkv_slice(qd, 0, N, H, d), qkv_slice(qd, 1, N, H, d), qkv_slice(qd, 2, N, H, d),
                    token_major((float *)out->data, N, H, d), lse, lens, B, H, N, d,
                    mode == ATTENTION_PREFIX_LM ? prefix_len : 0, scale);
    if (needs_grad) {
        grad_fn *fn = attach(scratch, out, attention_qkv_backward, 1, 1);
        fn->inputs[0] = qkv;
        FusedSaved *sv = host_alloc_t<FusedSaved>(scratch);
        sv->lse = lse; sv->seq_lens_dev = lens; sv->mode = (int)mode; sv->prefix = prefix_len; sv->H = H;
        sv->scale = scale; sv->out = out; sv->fc = fcd; sv->fs = fsd;
        fn->saved_tensors[0] = (tensor *)sv;
    }
    return out;
}

}  // namespace dnnb

using namespace dnnb;

extern "C" {

tensor *tensor_attention_ex(struct mem_pool *scratch, tensor *q, tensor *k, tensor *v, tensor *mask,
                            attention_mode mode, int prefix_len, const int *seq_lens) {
    require_device_payloads("tensor_attention_ex", {q, k, v, mask});
    DNN_CHECK(q && k && v, "tensor_attention: NULL operand");
    DNN_CHECK(q->ndim == 4 && k->ndim == 4 && v->ndim == 4, "tensor_attention: operands must be [B,H,N,d]");
    DNN_CHECK(q->contiguous && k->contiguous && v->contiguous, "tensor_attention: operands must be contiguous");
    int B = q->shape[0], H = q->shape[1], N = q->shape[2], d = q->shape[3];
    for (int i = 0; i < 4; i++)
        DNN_CHECK(k->shape[i] == q->shape[i] && v->shape[i] == q->shape[i], "tensor_attention: shape mismatch");
    if (mode == ATTENTION_PREFIX_LM) DNN_CHECK(prefix_len > 0 && prefix_len <= N, "tensor_attention: prefix_len out of range");
    if (mode == ATTENTION_CAUSAL) DNN_CHECK(prefix_len == 0, "tensor_attention: prefix_len must be 0 in causal mode");
    // An additive mask (src/attention.c:314-325; no model of the reference passes one) is added to the scaled scores of
    // the visible columns.  It gets no gradient itself; with a mask the exact fp32 kernels run in every mode.
    DNN_CHECK(d <= 128, "tensor_attention: head dim above 128 is not supported");

    int shape[4] = {B, H, N, d};
    tensor *out = tensor_scratch(scratch, 4, shape, 0);
    bool needs_grad = dnn_grad_enabled() && (q->requires_grad || k->requires_grad || v->requires_grad);
    AttnParams p;
    memset(&p, 0, sizeof p);
    p.B = B; p.H = H; p.N = N; p.d = d;
    p.q = (const float *)q->data; p.k = (const float *)k->data; p.v = (const float *)v->data;   // offsets ignored, as in the reference
    p.o = (float *)out->data;
    p.lse = needs_grad ? dev_alloc_t<float>(scratch, (size_t)B * H * N) : nullptr;
    p.seq_lens = seq_lens ? (const int *)dev_put(scratch, seq_lens, (size_t)B * sizeof(int)) : nullptr;
    p.prefix = mode == ATTENTION_PREFIX_LM ? prefix_len : 0;
    p.scale = 1.0f / sqrtf((float)d);
    set_mask(p, mask);
    if (use_tc(p)) attn_forward_tc(packed_heads(p.q, H, N, d), packed_heads(p.k, H, N, d), packed_heads(p.v, H, N, d),
                                   packed_heads(p.o, H, N, d), p.lse, p.seq_lens, B, H, N, d, p.prefix, p.scale);
    else attn_forward_fp32(p);

    if (needs_grad) {
        grad_fn *fn = attach(scratch, out, attention_backward, 3, 1);
        fn->inputs[0] = q; fn->inputs[1] = k; fn->inputs[2] = v;
        AttnSaved *sv = host_alloc_t<AttnSaved>(scratch);
        sv->lse = p.lse; sv->seq_lens_dev = p.seq_lens; sv->mode = (int)mode; sv->prefix = prefix_len;
        sv->scale = p.scale; sv->out = out; sv->mask = mask;
        fn->saved_tensors[0] = (tensor *)sv;
    }
    return out;
}

void dnn_cuda_set_fused_attention(int on) { g_fused_attention = on ? 1 : 0; }
int dnn_cuda_get_fused_attention(void) { return fused_attention_enabled() ? 1 : 0; }

tensor *tensor_attention(struct mem_pool *scratch, tensor *q, tensor *k, tensor *v, tensor *mask) {
    require_device_payloads("tensor_attention", {q, k, v, mask});
    return tensor_attention_ex(scratch, q, k, v, mask, ATTENTION_CAUSAL, 0, nullptr);
}

}  // extern "C"
