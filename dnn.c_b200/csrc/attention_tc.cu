// Tensor-core attention for sm_100a (TF32 tcgen05.mma, TMEM accumulators, TMA loads).
//
// Same mathematics as the exact kernels in attention.cu (causal / prefix-LM rule and
// per-batch lengths of src/attention.c:39-64, no N x N matrix, P recomputed in backward
// from the saved log-sum-exp), but every product runs on the tensor core:
//
//   forward, one CTA per (batch, head, 128 query rows), key tiles of 64:
//       S = Q K^T            tcgen05.mma, both operands K-major, result in TMEM
//       softmax              4 warps, ONE THREAD PER ROW (TMEM lane = row): tcgen05.ld the
//                            row, running max / sum in registers, P rounded to TF32 and
//                            written to shared memory in the 128-byte-swizzled K-major form
//       PV = P V             tcgen05.mma, A = P from shared memory, B = V MN-major
//       O  = O*corr + PV     in registers (PV read back from TMEM)
//   backward dK/dV, one CTA per (batch, head, 128 keys), query tiles of 64, transposed
//   problem so that a TMEM lane is a KEY:
//       S^T = K Q^T, dP^T = V dO^T ; P^T, dS^T per thread ; dV += P^T dO, dK += dS^T Q
//       (dV and dK accumulate in TMEM over all query tiles)
//   backward dQ, one CTA per (batch, head, 128 query rows), key tiles of 64:
//       S = Q K^T, dP = dO V^T ; dS per thread ; dQ += dS K  (accumulates in TMEM)
//
// One extra warp per CTA issues all TMA loads and all MMAs.  Operand buffers are single
// but each is refilled as soon as the MMAs that read it have committed, one phase ahead of
// its next use, and the score accumulators are double-buffered in TMEM, so the products of
// tile it+1 and the copies for it run behind the thread work of tile it.  Two forward CTAs
// fit on an SM; the backward kernels use 8 compute warps (two threads per TMEM lane).
// All mbarrier waits are bounded; a wait that gives up sets an error code (reported by
// dnn_cuda_sync) and the CTA still frees its TMEM.  No atomics: results are reproducible.
#include "common.cuh"
#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace dnnb {

__device__ int g_attn_error = 0;

struct AttnTcParams {
    float *o, *lse;                      // forward outputs
    const float *dvec, *lse_in;          // backward inputs (D_i, LSE_i), [B,H,N]
    float *dq, *dk, *dv;
    const int *seq_lens;
    int B, H, N;
    int prefix;
    float scale;
    int store;                           // bit 0/1/2: dq/dk/dv are written, not added to
};

__device__ __forceinline__ int vis_len(int i, int prefix, int nb) {
    int v = (i < prefix) ? prefix : i + 1;
    return v < nb ? v : nb;
}

// 32 consecutive floats of row r of a K-major tile [k-blocks][rows][32], 128-byte swizzle
__device__ __forceinline__ void store_row_block(uint8_t *tile, int rows, int r, int kb, const float (&v)[32]) {
    uint8_t *row = tile + (size_t)kb * rows * 128 + (size_t)r * 128;
#pragma unroll
    for (int q = 0; q < 8; q++)
        *reinterpret_cast<float4 *>(row + ((q ^ (r & 7)) << 4)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
}

// Failure handling.  Every wait is bounded.  The first wait that gives up records a code and
// raises a per-CTA abort flag in shared memory; from then on all waits of the CTA return at
// once, the loops run to their end without touching TMEM or the tensor core (so named
// barriers still see every thread), and the CTA frees its TMEM and exits.
constexpr uint32_t kAttnSpins = 1u << 22;
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < kAttnSpins; it++) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 255) == 255) { if (*abort_flag) return false; __nanosleep(64); }
    }
    return false;
}
// control thread (one lane)
#define CTRL_WAIT(bar, parity, code)                                                     \
    if (ok && !wait_or_abort((bar), (parity), abort_flag)) { atomicCAS(&g_attn_error, 0, (code)); *abort_flag = 1; ok = false; }
// compute warps (all 32 lanes, result made warp-uniform so aligned TMEM loads stay converged)
#define WARP_WAIT(bar, parity, code)                                                     \
    do { bool mine_ = ok && wait_or_abort((bar), (parity), abort_flag);                  \
         if (ok && !mine_) { atomicCAS(&g_attn_error, 0, (code)); *abort_flag = 1; }     \
         ok = __all_sync(0xffffffffu, mine_); } while (0)

// ════════════════════════════════ forward ════════════════════════════════
template <int HD>
struct FwdCfg {
    static constexpr int BM = 128, BN = 64, KB = HD / 32;
    static constexpr int kQ = KB * BM * 128, kK = KB * BN * 128, kV = KB * BN * 128, kP = (BN / 32) * BM * 128;
    static constexpr int kSmem = kQ + kK + kV + kP + 1024 + 256;
    static constexpr int kTmemCols = 256;          // S buffers at 0 and 64, PV (HD columns) at 128
};

// Pipeline (it = key tile index):
//   control thread            S(it+1) is issued before PV(it), into the other S buffer, as soon as
//                             K(it+1) has landed; PV(it) is issued when the softmax threads have
//                             published P(it).
//   softmax thread, tile it   max over S(it) -> fold PV(it-1) into O (frees the PV accumulator and
//                             the P buffer) -> exponentials, P(it) to shared memory -> signal.
// So the tensor core works on S(it+1) and PV(it) while the threads are busy with tile it.
template <int HD>
__global__ void __launch_bounds__(160, 2)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, AttnTcParams p) {
    using Cfg = FwdCfg<HD>;
    constexpr int BM = Cfg::BM, BN = Cfg::BN, KB = Cfg::KB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem, *sK = sQ + Cfg::kQ, *sV = sK + Cfg::kK, *sP = sV + Cfg::kV;
    uint64_t *bars = (uint64_t *)(sP + Cfg::kP);
    uint64_t *bar_q = bars, *bar_k = bars + 1, *bar_v = bars + 2, *bar_s = bars + 3 /* [2] */, *bar_p = bars + 5, *bar_o = bars + 6;
    uint32_t *tmem_slot = (uint32_t *)(bars + 8);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y, i0 = blockIdx.x * BM;
    const int bh = b * p.H + h;
    int nb = p.seq_lens ? p.seq_lens[b] : p.N;
    if (nb > p.N) nb = p.N;
    const int64_t slice = (int64_t)bh * p.N;
    float *o = p.o + slice * HD;

    if (i0 >= nb) {                      // rows beyond the sequence: zero output (src/attention.c:376-377)
        for (int idx = threadIdx.x; idx < BM * HD; idx += blockDim.x) {
            int r = idx / HD;
            if (i0 + r < p.N) o[(int64_t)i0 * HD + idx] = 0.f;
        }
        return;
    }
    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1); mbar_init(bar_k, 1); mbar_init(bar_v, 1); mbar_init(&bar_s[0], 1); mbar_init(&bar_s[1], 1);
        mbar_init(bar_p, 4); mbar_init(bar_o, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_pv = tmem + 128;

    const int i_last = min(i0 + BM, nb) - 1;
    const int jmax = vis_len(i_last, p.prefix, nb);
    const int n_iter = (jmax + BN - 1) / BN;
    bool ok = true;

    if (warp == 4) {
        if (lane == 0) {
            mbar_expect_tx(bar_q, Cfg::kQ);
            for (int kb = 0; kb < KB; kb++) tma_load_3d(sQ + kb * BM * 128, &tmQ, kb * 32, i0, bh, bar_q);
            mbar_expect_tx(bar_k, Cfg::kK);
            for (int kb = 0; kb < KB; kb++) tma_load_3d(sK + kb * BN * 128, &tmK, kb * 32, 0, bh, bar_k);
            mbar_expect_tx(bar_v, Cfg::kV);
            for (int c = 0; c < KB; c++) tma_load_3d(sV + c * BN * 128, &tmV, c * 32, 0, bh, bar_v);
            const uint32_t idesc_s = make_idesc_tf32(BN, false, false), idesc_pv = make_idesc_tf32(HD, false, true);
            const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP);
            auto issue_s = [&](int it) {
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < HD / 8; kk++)
                    tc_mma_tf32(tmem + (uint32_t)((it & 1) * 64), kmajor_desc(aQ, BM, kk), kmajor_desc(aK, BN, kk), idesc_s, kk > 0);
                tc_commit(&bar_s[it & 1]);
            };
            CTRL_WAIT(bar_q, 0, 0x101)
            CTRL_WAIT(bar_k, 0, 0x102)
            if (ok) issue_s(0);
            for (int it = 0; it < n_iter && ok; it++) {
                const uint32_t ph = it & 1;
                // S(it) complete: its K tile is free, fetch K(it+1) and start S(it+1) in the other buffer.
                // (That buffer held S(it-1), which the threads finished reading before they
                // published P(it-1), and P(it-1) was awaited in the previous trip.)
                CTRL_WAIT(&bar_s[it & 1], (it >> 1) & 1, 0x103)
                if (!ok) break;
                if (it + 1 < n_iter) {
                    mbar_expect_tx(bar_k, Cfg::kK);
                    for (int kb = 0; kb < KB; kb++) tma_load_3d(sK + kb * BN * 128, &tmK, kb * 32, (it + 1) * BN, bh, bar_k);
                    CTRL_WAIT(bar_k, (it + 1) & 1, 0x104)
                if (!ok) break;
                    issue_s(it + 1);
                }
                CTRL_WAIT(bar_p, ph, 0x105)          // P(it) published, PV(it-1) consumed
                if (!ok) break;
                CTRL_WAIT(bar_v, ph, 0x106)
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < BN / 8; kk++)
                    tc_mma_tf32(tmem_pv, kmajor_desc(aP, BM, kk), mnmajor_desc(aV, BN, kk), idesc_pv, kk > 0);
                tc_commit(bar_o);
                if (it + 1 < n_iter) {
                    CTRL_WAIT(bar_o, ph, 0x107)       // V tile free
                if (!ok) break;
                    mbar_expect_tx(bar_v, Cfg::kV);
                    for (int c = 0; c < KB; c++) tma_load_3d(sV + c * BN * 128, &tmV, c * 32, (it + 1) * BN, bh, bar_v);
                }
            }
        }
    } else {
        // one thread per query row
        const int r = warp * 32 + lane, row = i0 + r;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const int vis = row < nb ? vis_len(row, p.prefix, nb) : 0;
        // the running maximum is kept in units of log2(e)*scale so that exp() is one ex2
        const float sl2 = p.scale * 1.4426950408889634f;
        float m = -INFINITY, l = 0.f, corr_prev = 1.f;
        float acc[HD];
#pragma unroll
        for (int c = 0; c < HD; c++) acc[c] = 0.f;
        auto fold_pv = [&](float corr) {          // O = O*corr + PV, PV read back from TMEM
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t t[32];
                tc_ld32(tmem_pv + lane_base + c0, t);
#pragma unroll
                for (int j = 0; j < 32; j++) acc[c0 + j] = fmaf(acc[c0 + j], corr, __uint_as_float(t[j]));
            }
        };
        for (int it = 0; it < n_iter; it++) {
            const int j0 = it * BN;
            const uint32_t tmem_s = tmem + (uint32_t)((it & 1) * 64);
            WARP_WAIT(&bar_s[it & 1], (it >> 1) & 1, 0x111);
            if (!ok) break;
            tc_fence_after();
            // pass 1: row maximum over the 64 columns of this key tile (TMEM reads are cheap,
            // so the scores are read twice instead of being kept in 64 registers)
            float mx = -INFINITY;
#pragma unroll
            for (int half = 0; half < BN / 32; half++) {
                uint32_t s[32];
                tc_ld32(tmem_s + lane_base + half * 32, s);
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (j0 + half * 32 + j < vis) mx = fmaxf(mx, __uint_as_float(s[j]) * sl2);
            }
            const float mnew = fmaxf(m, mx);
            const float corr = (mnew == -INFINITY) ? 1.f : fast_exp2(m - mnew);
            // fold the previous tile's PV (scaled by the previous correction); this also
            // proves that the tensor core is done with the P buffer
            if (it > 0) {
                WARP_WAIT(bar_o, (it - 1) & 1, 0x112);
                if (!ok) break;
                tc_fence_after();
                fold_pv(corr_prev);
            }
            corr_prev = corr;
            float rs = 0.f;
            // pass 2: probabilities, rounded to TF32, into the swizzled A-operand tile
#pragma unroll
            for (int half = 0; half < BN / 32; half++) {
                uint32_t s[32];
                float pv[32];
                tc_ld32(tmem_s + lane_base + half * 32, s);
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    float e = (j0 + half * 32 + j < vis) ? fast_exp2(fmaf(__uint_as_float(s[j]), sl2, -mnew)) : 0.f;
                    rs += e; pv[j] = to_tf32(e);
                }
                store_row_block(sP, BM, r, half, pv);
            }
            l = l * corr + rs;
            m = mnew;
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p);
        }
        if (ok && n_iter > 0) {
            WARP_WAIT(bar_o, (n_iter - 1) & 1, 0x113);
            tc_fence_after();
            if (ok) fold_pv(corr_prev);
        }
        if (ok && row < p.N) {
            const bool live = row < nb;
            const float inv = live ? 1.f / l : 0.f;
            float4 *dst = reinterpret_cast<float4 *>(o + (int64_t)row * HD);
#pragma unroll
            for (int c = 0; c < HD; c += 4)
                dst[c >> 2] = make_float4(acc[c] * inv, acc[c + 1] * inv, acc[c + 2] * inv, acc[c + 3] * inv);
            if (p.lse) p.lse[slice + row] = live ? (m + log2f(l)) * 0.6931471805599453f : 0.f;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem, Cfg::kTmemCols); }
}

// ════════════════════════ backward: dK, dV (one CTA per 128 keys) ════════════════════════
// 8 compute warps: warp w works on TMEM lane quadrant w%4 (keys) and on the 32 query columns
// w/4 of the 64-query tile.  S^T / dP^T are double-buffered in TMEM, so the products of query
// tile it+1 run while the threads turn tile it into P^T and dS^T.
template <int HD>
struct DkvCfg {
    static constexpr int BKEY = 128, BQ = 64, KB = HD / 32;
    static constexpr int kKt = KB * BKEY * 128;            // K and V tiles, K-major A operands
    static constexpr int kQk = KB * BQ * 128;              // Q / dO of one query tile, K-major B (for S^T, dP^T)
    static constexpr int kQm = KB * BQ * 128;              // the same rows, MN-major B (for dK, dV)
    static constexpr int kPt = (BQ / 32) * BKEY * 128;     // P^T and dS^T, K-major A (k = query)
    static constexpr int kSmem = 2 * kKt + 2 * kQk + 2 * kQm + 2 * kPt + 6 * BQ * 4 + 1024 + 256;
    static constexpr int kTmemCols = 512;                  // S^T 0/64, dP^T 128/192, dV 256.., dK 320..
    static constexpr int kThreads = 288;
};

template <int HD>
__global__ void __launch_bounds__(288, 1)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap tmKa, const __grid_constant__ CUtensorMap tmVa,
                       const __grid_constant__ CUtensorMap tmQk, const __grid_constant__ CUtensorMap tmGk,
                       const __grid_constant__ CUtensorMap tmQm, const __grid_constant__ CUtensorMap tmGm, AttnTcParams p) {
    using Cfg = DkvCfg<HD>;
    constexpr int BKEY = Cfg::BKEY, BQ = Cfg::BQ, KB = Cfg::KB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sK = smem, *sV = sK + Cfg::kKt, *sQk = sV + Cfg::kKt, *sGk = sQk + Cfg::kQk, *sQm = sGk + Cfg::kQk,
            *sGm = sQm + Cfg::kQm, *sPt = sGm + Cfg::kQm, *sSt = sPt + Cfg::kPt;
    float *s_lse = (float *)(sSt + Cfg::kPt), *s_d = s_lse + 2 * BQ;       // [2][BQ] each
    int *s_vis = (int *)(s_d + 2 * BQ);
    uint64_t *bars = (uint64_t *)(((uintptr_t)(s_vis + 2 * BQ) + 15) & ~(uintptr_t)15);
    uint64_t *bar_kv = bars, *bar_in1 = bars + 1, *bar_in2 = bars + 2, *bar_s = bars + 3 /* [2] */, *bar_p = bars + 5, *bar_o = bars + 6;
    uint32_t *tmem_slot = (uint32_t *)(bars + 8);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * BKEY;
    const int bh = b * p.H + h;
    int nb = p.seq_lens ? p.seq_lens[b] : p.N;
    if (nb > p.N) nb = p.N;
    if (j0 >= nb) return;
    const int64_t slice = (int64_t)bh * p.N;

    if (threadIdx.x == 0) {
        mbar_init(bar_kv, 1); mbar_init(bar_in1, 1); mbar_init(bar_in2, 1); mbar_init(&bar_s[0], 1); mbar_init(&bar_s[1], 1);
        mbar_init(bar_p, 8); mbar_init(bar_o, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_dv = tmem + 256, t_dk = tmem + 320;

    // first query tile that can see a key of this tile; all later tiles up to nb
    const int i_begin = (p.prefix > 0 && j0 < p.prefix) ? 0 : (j0 / BQ) * BQ;
    const int n_iter = (nb - i_begin + BQ - 1) / BQ;
    bool ok = true;

    if (warp == 8) {
        if (lane == 0) {
            mbar_expect_tx(bar_kv, 2 * Cfg::kKt);
            for (int kb = 0; kb < KB; kb++) {
                tma_load_3d(sK + kb * BKEY * 128, &tmKa, kb * 32, j0, bh, bar_kv);
                tma_load_3d(sV + kb * BKEY * 128, &tmVa, kb * 32, j0, bh, bar_kv);
            }
            auto load_in1 = [&](int i0) {
                mbar_expect_tx(bar_in1, 2 * Cfg::kQk);
                for (int kb = 0; kb < KB; kb++) {
                    tma_load_3d(sQk + kb * BQ * 128, &tmQk, kb * 32, i0, bh, bar_in1);
                    tma_load_3d(sGk + kb * BQ * 128, &tmGk, kb * 32, i0, bh, bar_in1);
                }
            };
            auto load_in2 = [&](int i0) {
                mbar_expect_tx(bar_in2, 2 * Cfg::kQm);
                for (int c = 0; c < KB; c++) {
                    tma_load_3d(sQm + c * BQ * 128, &tmQm, c * 32, i0, bh, bar_in2);
                    tma_load_3d(sGm + c * BQ * 128, &tmGm, c * 32, i0, bh, bar_in2);
                }
            };
            load_in1(i_begin);
            load_in2(i_begin);
            const uint32_t id_s = make_idesc_tf32(BQ, false, false), id_g = make_idesc_tf32(HD, false, true);
            const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQk = smem_u32(sQk), aGk = smem_u32(sGk),
                           aQm = smem_u32(sQm), aGm = smem_u32(sGm), aPt = smem_u32(sPt), aSt = smem_u32(sSt);
            auto issue_sdp = [&](int it) {
                const uint32_t t_st = tmem + (uint32_t)((it & 1) * 64), t_dpt = tmem + 128 + (uint32_t)((it & 1) * 64);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < HD / 8; kk++) tc_mma_tf32(t_st, kmajor_desc(aK, BKEY, kk), kmajor_desc(aQk, BQ, kk), id_s, kk > 0);
#pragma unroll
                for (int kk = 0; kk < HD / 8; kk++) tc_mma_tf32(t_dpt, kmajor_desc(aV, BKEY, kk), kmajor_desc(aGk, BQ, kk), id_s, kk > 0);
                tc_commit(&bar_s[it & 1]);
            };
            CTRL_WAIT(bar_kv, 0, 0x201)
            CTRL_WAIT(bar_in1, 0, 0x202)
            if (ok) issue_sdp(0);
            for (int it = 0; it < n_iter && ok; it++) {
                const uint32_t ph = it & 1;
                const int i_next = i_begin + (it + 1) * BQ;
                CTRL_WAIT(&bar_s[it & 1], (it >> 1) & 1, 0x203)
                if (!ok) break;
                if (it + 1 < n_iter) {
                    load_in1(i_next);
                    CTRL_WAIT(bar_in1, (it + 1) & 1, 0x204)
                if (!ok) break;
                    issue_sdp(it + 1);
                }
                CTRL_WAIT(bar_p, ph, 0x205)
                if (!ok) break;
                CTRL_WAIT(bar_in2, ph, 0x206)
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < BQ / 8; kk++) tc_mma_tf32(t_dv, kmajor_desc(aPt, BKEY, kk), mnmajor_desc(aGm, BQ, kk), id_g, (it > 0 || kk > 0));
#pragma unroll
                for (int kk = 0; kk < BQ / 8; kk++) tc_mma_tf32(t_dk, kmajor_desc(aSt, BKEY, kk), mnmajor_desc(aQm, BQ, kk), id_g, (it > 0 || kk > 0));
                tc_commit(bar_o);
                if (it + 1 < n_iter) {
                    CTRL_WAIT(bar_o, ph, 0x207)
                if (!ok) break;
                    load_in2(i_next);
                }
            }
        }
    } else {
        const int q4 = warp & 3, hq = warp >> 2;
        const int r = q4 * 32 + lane, key = j0 + r;
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        const float sl2 = p.scale * 1.4426950408889634f;
        for (int it = 0; it < n_iter; it++) {
            const int i0 = i_begin + it * BQ;
            const int buf = it & 1;
            if (threadIdx.x < BQ) {
                int row = i0 + threadIdx.x;
                bool live = row < nb;
                s_lse[buf * BQ + threadIdx.x] = live ? p.lse_in[slice + row] * 1.4426950408889634f : 0.f;    // log2 units
                s_d[buf * BQ + threadIdx.x] = live ? p.dvec[slice + row] : 0.f;
                s_vis[buf * BQ + threadIdx.x] = live ? vis_len(row, p.prefix, nb) : 0;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");        // every thread reaches this in every trip, also after an abort
            WARP_WAIT(&bar_s[buf], (it >> 1) & 1, 0x211);
            float pt[32], st[32];
            if (ok) {
                tc_fence_after();
                uint32_t s[32], dp[32];
                tc_ld32(tmem + (uint32_t)(buf * 64) + lane_base + hq * 32, s);
                tc_ld32(tmem + 128 + (uint32_t)(buf * 64) + lane_base + hq * 32, dp);
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    int q = buf * BQ + hq * 32 + j;
                    float pe = (key < s_vis[q]) ? fast_exp2(fmaf(__uint_as_float(s[j]), sl2, -s_lse[q])) : 0.f;
                    pt[j] = to_tf32(pe);
                    st[j] = to_tf32(pe * (__uint_as_float(dp[j]) - s_d[q]) * p.scale);
                }
            }
            // the previous tile's dV/dK products must have finished reading P^T / dS^T
            if (it > 0) WARP_WAIT(bar_o, (it - 1) & 1, 0x212);
            if (ok) {
                store_row_block(sPt, BKEY, r, hq, pt);
                store_row_block(sSt, BKEY, r, hq, st);
                fence_proxy_async();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_p);
            }
        }
        if (ok && n_iter > 0) {
            WARP_WAIT(bar_o, (n_iter - 1) & 1, 0x213);
            tc_fence_after();
            const int c0 = hq * 32;
            if (ok && c0 < HD) {             // warp-uniform: every lane takes part in the TMEM loads
                uint32_t a[32], c[32];
                tc_ld32(t_dv + lane_base + c0, a);
                tc_ld32(t_dk + lane_base + c0, c);
                if (p.dv && key < nb) {
                    float4 *dst = reinterpret_cast<float4 *>(p.dv + (slice + key) * HD + c0);
                    const bool st = p.store & 4;
#pragma unroll
                    for (int j = 0; j < 32; j += 4) { float4 v = st ? make_float4(0.f, 0.f, 0.f, 0.f) : dst[j >> 2];
                        v.x += __uint_as_float(a[j]); v.y += __uint_as_float(a[j + 1]); v.z += __uint_as_float(a[j + 2]); v.w += __uint_as_float(a[j + 3]); dst[j >> 2] = v; }
                }
                if (p.dk && key < nb) {
                    float4 *dst = reinterpret_cast<float4 *>(p.dk + (slice + key) * HD + c0);
                    const bool st = p.store & 2;
#pragma unroll
                    for (int j = 0; j < 32; j += 4) { float4 v = st ? make_float4(0.f, 0.f, 0.f, 0.f) : dst[j >> 2];
                        v.x += __uint_as_float(c[j]); v.y += __uint_as_float(c[j + 1]); v.z += __uint_as_float(c[j + 2]); v.w += __uint_as_float(c[j + 3]); dst[j >> 2] = v; }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) { tc_fence_after(); tmem_dealloc(tmem, Cfg::kTmemCols); }
}

// ════════════════════════ backward: dQ (one CTA per 128 query rows) ════════════════════════
template <int HD>
struct DqCfg {
    static constexpr int BM = 128, BN = 64, KB = HD / 32;
    static constexpr int kQ = KB * BM * 128;               // Q and dO tiles, K-major A
    static constexpr int kKk = KB * BN * 128;              // K / V of one key tile, K-major B
    static constexpr int kKm = KB * BN * 128;              // K of the key tile, MN-major B (for dQ)
    static constexpr int kS = (BN / 32) * BM * 128;        // dS, K-major A (k = key)
    static constexpr int kSmem = 2 * kQ + 2 * kKk + kKm + kS + 1024 + 256;
    static constexpr int kTmemCols = 512;                  // S 0/64, dP 128/192, dQ 256..
    static constexpr int kThreads = 288;
};

template <int HD>
__global__ void __launch_bounds__(288, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQa, const __grid_constant__ CUtensorMap tmGa,
                      const __grid_constant__ CUtensorMap tmKk, const __grid_constant__ CUtensorMap tmVk,
                      const __grid_constant__ CUtensorMap tmKm, AttnTcParams p) {
    using Cfg = DqCfg<HD>;
    constexpr int BM = Cfg::BM, BN = Cfg::BN, KB = Cfg::KB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem, *sG = sQ + Cfg::kQ, *sKk = sG + Cfg::kQ, *sVk = sKk + Cfg::kKk, *sKm = sVk + Cfg::kKk, *sS = sKm + Cfg::kKm;
    uint64_t *bars = (uint64_t *)(sS + Cfg::kS);
    uint64_t *bar_q = bars, *bar_in1 = bars + 1, *bar_in2 = bars + 2, *bar_s = bars + 3 /* [2] */, *bar_p = bars + 5, *bar_o = bars + 6;
    uint32_t *tmem_slot = (uint32_t *)(bars + 8);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y, i0 = blockIdx.x * BM;
    const int bh = b * p.H + h;
    int nb = p.seq_lens ? p.seq_lens[b] : p.N;
    if (nb > p.N) nb = p.N;
    if (i0 >= nb) return;
    const int64_t slice = (int64_t)bh * p.N;

    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1); mbar_init(bar_in1, 1); mbar_init(bar_in2, 1); mbar_init(&bar_s[0], 1); mbar_init(&bar_s[1], 1);
        mbar_init(bar_p, 8); mbar_init(bar_o, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_dq = tmem + 256;

    const int i_last = min(i0 + BM, nb) - 1;
    const int jmax = vis_len(i_last, p.prefix, nb);
    const int n_iter = (jmax + BN - 1) / BN;
    bool ok = true;

    if (warp == 8) {
        if (lane == 0) {
            mbar_expect_tx(bar_q, 2 * Cfg::kQ);
            for (int kb = 0; kb < KB; kb++) {
                tma_load_3d(sQ + kb * BM * 128, &tmQa, kb * 32, i0, bh, bar_q);
                tma_load_3d(sG + kb * BM * 128, &tmGa, kb * 32, i0, bh, bar_q);
            }
            auto load_in1 = [&](int j) {
                mbar_expect_tx(bar_in1, 2 * Cfg::kKk);
                for (int kb = 0; kb < KB; kb++) {
                    tma_load_3d(sKk + kb * BN * 128, &tmKk, kb * 32, j, bh, bar_in1);
                    tma_load_3d(sVk + kb * BN * 128, &tmVk, kb * 32, j, bh, bar_in1);
                }
            };
            auto load_in2 = [&](int j) {
                mbar_expect_tx(bar_in2, Cfg::kKm);
                for (int c = 0; c < KB; c++) tma_load_3d(sKm + c * BN * 128, &tmKm, c * 32, j, bh, bar_in2);
            };
            load_in1(0);
            load_in2(0);
            const uint32_t id_s = make_idesc_tf32(BN, false, false), id_q = make_idesc_tf32(HD, false, true);
            const uint32_t aQ = smem_u32(sQ), aG = smem_u32(sG), aKk = smem_u32(sKk), aVk = smem_u32(sVk), aKm = smem_u32(sKm), aS = smem_u32(sS);
            auto issue_sdp = [&](int it) {
                const uint32_t t_s = tmem + (uint32_t)((it & 1) * 64), t_dp = tmem + 128 + (uint32_t)((it & 1) * 64);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < HD / 8; kk++) tc_mma_tf32(t_s, kmajor_desc(aQ, BM, kk), kmajor_desc(aKk, BN, kk), id_s, kk > 0);
#pragma unroll
                for (int kk = 0; kk < HD / 8; kk++) tc_mma_tf32(t_dp, kmajor_desc(aG, BM, kk), kmajor_desc(aVk, BN, kk), id_s, kk > 0);
                tc_commit(&bar_s[it & 1]);
            };
            CTRL_WAIT(bar_q, 0, 0x301)
            CTRL_WAIT(bar_in1, 0, 0x302)
            if (ok) issue_sdp(0);
            for (int it = 0; it < n_iter && ok; it++) {
                const uint32_t ph = it & 1;
                const int j_next = (it + 1) * BN;
                CTRL_WAIT(&bar_s[it & 1], (it >> 1) & 1, 0x303)
                if (!ok) break;
                if (it + 1 < n_iter) {
                    load_in1(j_next);
                    CTRL_WAIT(bar_in1, (it + 1) & 1, 0x304)
                if (!ok) break;
                    issue_sdp(it + 1);
                }
                CTRL_WAIT(bar_p, ph, 0x305)
                if (!ok) break;
                CTRL_WAIT(bar_in2, ph, 0x306)
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < BN / 8; kk++) tc_mma_tf32(t_dq, kmajor_desc(aS, BM, kk), mnmajor_desc(aKm, BN, kk), id_q, (it > 0 || kk > 0));
                tc_commit(bar_o);
                if (it + 1 < n_iter) {
                    CTRL_WAIT(bar_o, ph, 0x307)
                if (!ok) break;
                    load_in2(j_next);
                }
            }
        }
    } else {
        const int q4 = warp & 3, hq = warp >> 2;
        const int r = q4 * 32 + lane, row = i0 + r;
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        const bool live = row < nb;
        const int vis = live ? vis_len(row, p.prefix, nb) : 0;
        const float lse2 = live ? p.lse_in[slice + row] * 1.4426950408889634f : 0.f, dd = live ? p.dvec[slice + row] : 0.f;
        const float sl2 = p.scale * 1.4426950408889634f;
        for (int it = 0; it < n_iter; it++) {
            const int buf = it & 1;
            const int col0 = it * BN + hq * 32;
            WARP_WAIT(&bar_s[buf], (it >> 1) & 1, 0x311);
            if (!ok) break;
            tc_fence_after();
            uint32_t s[32], dp[32];
            tc_ld32(tmem + (uint32_t)(buf * 64) + lane_base + hq * 32, s);
            tc_ld32(tmem + 128 + (uint32_t)(buf * 64) + lane_base + hq * 32, dp);
            float ds[32];
#pragma unroll
            for (int j = 0; j < 32; j++) {
                float pe = (col0 + j < vis) ? fast_exp2(fmaf(__uint_as_float(s[j]), sl2, -lse2)) : 0.f;
                ds[j] = to_tf32(pe * (__uint_as_float(dp[j]) - dd) * p.scale);
            }
            if (it > 0) WARP_WAIT(bar_o, (it - 1) & 1, 0x312);
            if (!ok) break;
            store_row_block(sS, BM, r, hq, ds);
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p);
        }
        if (ok && n_iter > 0) {
            WARP_WAIT(bar_o, (n_iter - 1) & 1, 0x313);
            tc_fence_after();
            const int c0 = hq * 32;
            if (ok && c0 < HD) {
                uint32_t a[32];
                tc_ld32(t_dq + lane_base + c0, a);
                if (live) {
                    float4 *dst = reinterpret_cast<float4 *>(p.dq + (slice + row) * HD + c0);
                    const bool st = p.store & 1;
#pragma unroll
                    for (int j = 0; j < 32; j += 4) { float4 v = st ? make_float4(0.f, 0.f, 0.f, 0.f) : dst[j >> 2];
                        v.x += __uint_as_float(a[j]); v.y += __uint_as_float(a[j + 1]); v.z += __uint_as_float(a[j + 2]); v.w += __uint_as_float(a[j + 3]); dst[j >> 2] = v; }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) { tc_fence_after(); tmem_dealloc(tmem, Cfg::kTmemCols); }
}

// ════════════════════════════════ host side ════════════════════════════════
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        CUDA_OK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q));
        DNN_CHECK(ptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available in this driver");
        fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// [BH, N, d] fp32 tensor; box = {32 floats of d, rows, 1}; rows beyond N read as zero.
static CUtensorMap map3d(const float *base, int BH, int N, int d, int box_rows, bool mn_major) {
    CUtensorMap m;
    cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)N, (cuuint64_t)BH};
    cuuint64_t strides[2] = {(cuuint64_t)d * 4, (cuuint64_t)N * d * 4};
    cuuint32_t box[3] = {32, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 3, (void *)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "dnn_b200: cuTensorMapEncodeTiled (attention) failed (%d)\n", (int)r); abort(); }
    return m;
}

bool attn_tc_supported(int d, const void *q, const void *k, const void *v) {
    return (d == 32 || d == 64) && aligned16(q) && aligned16(k) && aligned16(v);
}

struct AttnParamsHost {           // mirrors the fields of attention.cu's AttnParams that are needed here
    const float *q, *k, *v; float *o, *lse; const float *dout, *dvec; float *dq, *dk, *dv; const int *seq_lens;
    int B, H, N, d, prefix; float scale; int store;
};

template <int HD>
static void fwd_launch(const AttnParamsHost &a) {
    using Cfg = FwdCfg<HD>;
    static bool once = false;
    if (!once) { CUDA_OK(cudaFuncSetAttribute(attn_fwd_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem)); once = true; }
    int BH = a.B * a.H;
    CUtensorMap tq = map3d(a.q, BH, a.N, HD, Cfg::BM, false), tk = map3d(a.k, BH, a.N, HD, Cfg::BN, false), tv = map3d(a.v, BH, a.N, HD, Cfg::BN, true);
    AttnTcParams p; memset(&p, 0, sizeof p);
    p.o = a.o; p.lse = a.lse; p.seq_lens = a.seq_lens; p.B = a.B; p.H = a.H; p.N = a.N; p.prefix = a.prefix; p.scale = a.scale;
    dim3 grid((a.N + Cfg::BM - 1) / Cfg::BM, a.H, a.B);
    attn_fwd_tc_kernel<HD><<<grid, 160, Cfg::kSmem, stream()>>>(tq, tk, tv, p);
    LAUNCHED("attn_fwd_tc_kernel");
}

template <int HD>
static void bwd_launch(const AttnParamsHost &a) {
    int BH = a.B * a.H;
    AttnTcParams p; memset(&p, 0, sizeof p);
    p.lse_in = a.lse; p.dvec = a.dvec; p.dq = a.dq; p.dk = a.dk; p.dv = a.dv; p.seq_lens = a.seq_lens;
    p.B = a.B; p.H = a.H; p.N = a.N; p.prefix = a.prefix; p.scale = a.scale; p.store = a.store;
    static bool once = false;
    if (!once) {
        CUDA_OK(cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvCfg<HD>::kSmem));
        CUDA_OK(cudaFuncSetAttribute(attn_bwd_dq_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, DqCfg<HD>::kSmem));
        once = true;
    }
    if (a.dk || a.dv) {
        using Cfg = DkvCfg<HD>;
        CUtensorMap tka = map3d(a.k, BH, a.N, HD, Cfg::BKEY, false), tva = map3d(a.v, BH, a.N, HD, Cfg::BKEY, false);
        CUtensorMap tqk = map3d(a.q, BH, a.N, HD, Cfg::BQ, false), tgk = map3d(a.dout, BH, a.N, HD, Cfg::BQ, false);
        CUtensorMap tqm = map3d(a.q, BH, a.N, HD, Cfg::BQ, true), tgm = map3d(a.dout, BH, a.N, HD, Cfg::BQ, true);
        dim3 grid((a.N + Cfg::BKEY - 1) / Cfg::BKEY, a.H, a.B);
        attn_bwd_dkv_tc_kernel<HD><<<grid, Cfg::kThreads, Cfg::kSmem, stream()>>>(tka, tva, tqk, tgk, tqm, tgm, p);
        LAUNCHED("attn_bwd_dkv_tc_kernel");
    }
    if (a.dq) {
        using Cfg = DqCfg<HD>;
        CUtensorMap tqa = map3d(a.q, BH, a.N, HD, Cfg::BM, false), tga = map3d(a.dout, BH, a.N, HD, Cfg::BM, false);
        CUtensorMap tkk = map3d(a.k, BH, a.N, HD, Cfg::BN, false), tvk = map3d(a.v, BH, a.N, HD, Cfg::BN, false);
        CUtensorMap tkm = map3d(a.k, BH, a.N, HD, Cfg::BN, true);
        dim3 grid((a.N + Cfg::BM - 1) / Cfg::BM, a.H, a.B);
        attn_bwd_dq_tc_kernel<HD><<<grid, Cfg::kThreads, Cfg::kSmem, stream()>>>(tqa, tga, tkk, tvk, tkm, p);
        LAUNCHED("attn_bwd_dq_tc_kernel");
    }
}

void attn_forward_tc(const float *q, const float *k, const float *v, float *o, float *lse, const int *seq_lens,
                     int B, int H, int N, int d, int prefix, float scale) {
    AttnParamsHost a; memset(&a, 0, sizeof a);
    a.q = q; a.k = k; a.v = v; a.o = o; a.lse = lse; a.seq_lens = seq_lens; a.B = B; a.H = H; a.N = N; a.d = d; a.prefix = prefix; a.scale = scale;
    if (d == 32) fwd_launch<32>(a); else fwd_launch<64>(a);
}

void attn_backward_tc(const float *q, const float *k, const float *v, const float *lse, const float *dout, const float *dvec,
                      float *dq, float *dk, float *dv, const int *seq_lens, int B, int H, int N, int d, int prefix, float scale, int store) {
    AttnParamsHost a; memset(&a, 0, sizeof a);
    a.store = store;
    a.q = q; a.k = k; a.v = v; a.lse = (float *)lse; a.dout = dout; a.dvec = dvec; a.dq = dq; a.dk = dk; a.dv = dv; a.seq_lens = seq_lens;
    a.B = B; a.H = H; a.N = N; a.d = d; a.prefix = prefix; a.scale = scale;
    if (d == 32) bwd_launch<32>(a); else bwd_launch<64>(a);
}

int attn_tc_error() {
    int e = 0;
    cudaMemcpyFromSymbol(&e, g_attn_error, sizeof e);
    return e;
}

}  // namespace dnnb
