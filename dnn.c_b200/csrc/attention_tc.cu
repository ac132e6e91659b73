// Tensor-core attention for sm_100a (TF32 tcgen05.mma, TMEM accumulators, TMA loads).
//
// Same mathematics as the exact kernels in attention.cu (causal / prefix-LM rule and
// per-batch lengths of src/attention.c:39-64, no N x N matrix, P recomputed in backward
// from the saved log-sum-exp), but every product runs on the tensor core and the
// probabilities never leave tensor memory:
//
//   forward, one CTA per (batch, head, 128 query rows), key tiles of 64:
//       S = Q K^T            tcgen05.mma, both operands K-major, result in TMEM
//       softmax              4 warps, ONE THREAD PER ROW (TMEM lane = row): tcgen05.ld the
//                            row, running max / sum in registers, P rounded to TF32 and
//                            written back over S with tcgen05.st
//       PV = P V             tcgen05.mma, A = P read from TMEM, B = V MN-major
//       O  = O*corr + PV     in registers (PV read back from TMEM, two PV buffers)
//   backward dK/dV, one CTA per (batch, head, 128 keys), query tiles of 64, transposed
//   problem so that a TMEM lane is a KEY:
//       S^T = K Q^T, dP^T = V dO^T ; the threads turn them in place into P^T and dS^T ;
//       dV += P^T dO, dK += dS^T Q with A from TMEM (dV and dK accumulate in TMEM)
//   backward dQ, one CTA per (batch, head, 128 query rows), key tiles of 64:
//       S = Q K^T, dP = dO V^T ; dS written over dP ; dQ += dS K  (accumulates in TMEM)
//
// Every kernel is a pipeline of single-thread roles and compute warps: loader threads issue
// the TMA loads into two-slot rings, one thread issues the MMAs, and the compute warps do the
// per-element work.  The score accumulators are double-buffered in TMEM (triple-buffered in
// the backward kernels), so the loads and products of tile t+1 run behind the thread work of
// tile t and no latency sits between two tiles.  A slot is reloaded when the MMAs that read
// it have committed.  A TF32 tcgen05.mma of 64 columns costs the tensor core 55 to 85 cycles
// whatever its width up to 128, so the products themselves set the pace: the MMA issuer adds
// constants to prebuilt descriptors and never waits on a product it has just issued.  Operands are addressed through
// strides, so packed [B,H,N,d] heads and the [B,N,3,H,d] output of a fused QKV projection
// are read and written in place.
// All mbarrier waits are bounded; a wait that gives up sets an error code (reported by
// dnn_cuda_sync) and the CTA still frees its TMEM.  No atomics: results are reproducible.
#include "common.cuh"
#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace dnnb {

__device__ int g_attn_error = 0;

struct AttnTcParams {
    HeadView o;                          // forward output
    float *lse;                          // forward output, [B,H,N]
    const float *dvec, *lse_in;          // backward inputs (D_i, LSE_i), [B,H,N]
    HeadView dq, dk, dv;                 // p == nullptr: not wanted
    const int *seq_lens;
    int B, H, N;
    int prefix;
    float scale;
    int store;                           // bit 0/1/2: dq/dk/dv are written, not added to
    const float *rope_c, *rope_s;        // backward: [N, d/2] tables; when set, dQ and dK leave the kernel rotated back
                                         // (the gradient of the RoPE that produced Q and K), which needs store mode
    int tma_out;                         // backward: gradients leave through the copy engine (tile store / tile add)
};

__device__ __forceinline__ int vis_len(int i, int prefix, int nb) {
    int v = (i < prefix) ? prefix : i + 1;
    return v < nb ? v : nb;
}

// Failure handling.  Every wait is bounded.  The first wait that gives up records a code and
// raises a per-CTA abort flag in shared memory; from then on all waits of the CTA return at
// once, the loops run to their end without touching TMEM or the tensor core (so named
// barriers still see every thread), and the CTA frees its TMEM and exits.
// Bits of x rounded to TF32 (nearest, ties away) for a value the tensor core will read: adding half
// of the dropped range is enough, the core ignores the low 13 mantissa bits itself.  One integer add
// instead of a conversion instruction, which shares its unit with the exponentials.  Finite inputs only.
__device__ __forceinline__ uint32_t tf32_bits(float x) { return __float_as_uint(x) + 0x1000u; }
constexpr uint32_t kAttnSpins = 1u << 22;
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    uint32_t addr = smem_u32(bar);
    if (mbar_test(addr, parity)) return true;
    for (uint32_t it = 0; it < kAttnSpins; it++) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 255) == 255) { if (*abort_flag) return false; __nanosleep(64); }
    }
    return false;
}
// single-thread roles (loader, MMA issuer)
#define CTRL_WAIT(bar, parity, code)                                                     \
    if (ok && !wait_or_abort((bar), (parity), abort_flag)) { atomicCAS(&g_attn_error, 0, (code)); *abort_flag = 1; ok = false; }
// compute warps: lane 0 polls the barrier and the warp takes its answer (one poller per warp
// keeps 256 threads from hammering a shared-memory barrier that the tensor core's operand reads
// share a port with); every lane then passes the tcgen05 fence that follows the wait
#define WARP_WAIT(bar, parity, code)                                                     \
    do { int mine_ = 1;                                                                  \
         if (lane == 0) {                                                                \
             mine_ = ok && wait_or_abort((bar), (parity), abort_flag);                   \
             if (ok && !mine_) { atomicCAS(&g_attn_error, 0, (code)); *abort_flag = 1; } \
         }                                                                               \
         ok = __shfl_sync(0xffffffffu, mine_, 0) != 0; } while (0)

// Tile t of a two-slot ring uses slot t & 1; the barrier of that slot completes once per
// use, so the completion that belongs to tile t has parity (t >> 1) & 1.
__device__ __forceinline__ uint32_t use_parity(int t) { return (uint32_t)(t >> 1) & 1u; }
// The backward kernels keep THREE score buffers in TMEM (tile t uses buffer t % 3), so the
// products of tile t+1 never wait for the tensor core to finish reading tile t-1.
__device__ __forceinline__ int buf3(int t) { return t % 3; }
__device__ __forceinline__ uint32_t use_parity3(int t) { return (uint32_t)(t / 3) & 1u; }

// Undoes the rotary embedding on 32 consecutive gradient columns [c0, c0+32) of position `pos`.
template <int HD>
__device__ __forceinline__ void unrotate32(uint32_t (&a)[32], const float *__restrict__ fc, const float *__restrict__ fs, int pos, int c0) {
    const float4 *c4 = reinterpret_cast<const float4 *>(fc + (int64_t)pos * (HD / 2) + c0 / 2);
    const float4 *s4 = reinterpret_cast<const float4 *>(fs + (int64_t)pos * (HD / 2) + c0 / 2);
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const float4 c = __ldg(c4 + q), s = __ldg(s4 + q);
        const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int j = 8 * q + 2 * e;
            float ox, oy;
            rope_inv_pair(__uint_as_float(a[j]), __uint_as_float(a[j + 1]), cc[e], ss[e], ox, oy);
            a[j] = __float_as_uint(ox); a[j + 1] = __float_as_uint(oy);
        }
    }
}

// Adds (or stores) 32 consecutive floats held in registers to a row in global memory.
__device__ __forceinline__ void emit_row32(float *dst, const uint32_t (&a)[32], bool store) {
    float4 *d4 = reinterpret_cast<float4 *>(dst);
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        float4 v = store ? make_float4(0.f, 0.f, 0.f, 0.f) : d4[j >> 2];
        v.x += __uint_as_float(a[j]); v.y += __uint_as_float(a[j + 1]); v.z += __uint_as_float(a[j + 2]); v.w += __uint_as_float(a[j + 3]);
        d4[j >> 2] = v;
    }
}

// The same 32 x 32 piece (one row of 32 floats per lane) written as a 128-byte-swizzled tile for the copy engine:
// 16-byte piece j of row `lane` lands at piece j ^ (lane & 7).  One tile store (or tile add) then writes whole
// 128-byte row segments, where 32 lanes storing 16 bytes each to 32 different rows cost 32 transactions per instruction
// (measured: the dK/dV kernel spent 6-11 thousand cycles per CTA issuing those stores).
__device__ __forceinline__ void stage_tile32(uint8_t *tile, const uint32_t (&a)[32], int lane) {
#pragma unroll
    for (int j = 0; j < 8; j++)
        *reinterpret_cast<uint4 *>(tile + lane * 128 + ((j ^ (lane & 7)) << 4)) = make_uint4(a[4 * j], a[4 * j + 1], a[4 * j + 2], a[4 * j + 3]);
}

// ════════════════════════════════ forward ════════════════════════════════
template <int HD>
struct FwdCfg {
    static constexpr int BM = 128, BN = 64, KB = HD / 32;
    static constexpr int kQ = KB * BM * 128, kK = KB * BN * 128, kV = KB * BN * 128;
    static constexpr int kSmem = kQ + 2 * kK + 2 * kV + 1024 + 256;
    static constexpr int kTmemCols = 256;          // S/P buffers at 0 and 64, PV buffers (HD columns) at 128 and 128+HD
    static constexpr int kThreads = 192;           // 4 softmax warps, loader warp, MMA warp
};

// Tile t = key rows [64 t, 64 t + 64).
//   loader       K(t), V(t) into slot t&1 as soon as S(t-2) resp. PV(t-2) have committed
//   MMA thread   S(t+1) as soon as K(t+1) has landed and PV(t-1) has released the score buffer;
//                PV(t) when the threads have published P(t)
//   row thread   max over S(t) -> fold PV(t-1) into O -> exponentials, P(t) over S(t) -> signal
template <int HD>
__global__ void __launch_bounds__(192, 2)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, AttnTcParams p) {
    using Cfg = FwdCfg<HD>;
    constexpr int BM = Cfg::BM, BN = Cfg::BN, KB = Cfg::KB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem, *sK = sQ + Cfg::kQ, *sV = sK + 2 * Cfg::kK;
    uint64_t *bars = (uint64_t *)(sV + 2 * Cfg::kV);
    uint64_t *bar_q = bars, *k_full = bars + 1, *v_full = bars + 3, *bar_s = bars + 5, *bar_p = bars + 7, *bar_o = bars + 9;   // [2] each
    uint32_t *tmem_slot = (uint32_t *)(bars + 11);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // grid = (batch x heads, query tiles): CTAs are dispatched x-fastest, so all heads' LAST query tiles -- which
    // see the most keys under the causal and prefix rules -- go first and the shortest CTAs fill the tail
    const int b = (int)blockIdx.x / p.H, h = (int)blockIdx.x % p.H, i0 = (int)(gridDim.y - 1 - blockIdx.y) * BM;
    int nb = p.seq_lens ? p.seq_lens[b] : p.N;
    if (nb > p.N) nb = p.N;
    float *o = p.o.p + (int64_t)b * p.o.sb + (int64_t)h * p.o.sh;
    const int64_t slice = (int64_t)(b * p.H + h) * p.N;

    if (i0 >= nb) {                      // rows beyond the sequence: zero output (src/attention.c:376-377)
        for (int idx = threadIdx.x; idx < BM * HD; idx += blockDim.x) {
            int r = idx / HD, c = idx - r * HD;
            if (i0 + r < p.N) o[(int64_t)(i0 + r) * p.o.sn + c] = 0.f;
        }
        return;
    }
    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1);
        for (int s = 0; s < 2; s++) { mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&bar_s[s], 1); mbar_init(&bar_p[s], 4); mbar_init(&bar_o[s], 1); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int i_last = min(i0 + BM, nb) - 1;
    const int jmax = vis_len(i_last, p.prefix, nb);
    const int n_iter = (jmax + BN - 1) / BN;
    bool ok = true;

    if (warp == 4) {
        if (lane == 0) {                 // ---- loader
            mbar_expect_tx(bar_q, Cfg::kQ);
            for (int kb = 0; kb < KB; kb++) tma_load_4d(sQ + kb * BM * 128, &tmQ, kb * 32, i0, h, b, bar_q);
            for (int t = 0; t < n_iter && ok; t++) {
                const int s = t & 1;
                if (t >= 2) CTRL_WAIT(&bar_s[s], use_parity(t - 2), 0x101)
                if (!ok) break;
                mbar_expect_tx(&k_full[s], Cfg::kK);
                for (int kb = 0; kb < KB; kb++) tma_load_4d(sK + s * Cfg::kK + kb * BN * 128, &tmK, kb * 32, t * BN, h, b, &k_full[s]);
                if (t >= 2) CTRL_WAIT(&bar_o[s], use_parity(t - 2), 0x102)
                if (!ok) break;
                mbar_expect_tx(&v_full[s], Cfg::kV);
                for (int c = 0; c < KB; c++) tma_load_4d(sV + s * Cfg::kV + c * BN * 128, &tmV, c * 32, t * BN, h, b, &v_full[s]);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {                 // ---- MMA issuer
            const uint32_t idesc_s = make_idesc_tf32(BN, false, false), idesc_pv = make_idesc_tf32(HD, false, true);
            // descriptors of K=8 step 0 of every operand buffer; the issue loops only add constants
            const uint64_t dQ0 = kmajor_desc(smem_u32(sQ), BM, 0);
            const uint64_t dK0 = kmajor_desc(smem_u32(sK), BN, 0);
            const uint64_t dV0 = mnmajor_desc(smem_u32(sV), BN, 0);
            auto issue_s = [&](int t) {
                tc_fence_after();
                const uint64_t dk = dK0 + (uint64_t)((t & 1) * (Cfg::kK >> 4));
                const uint32_t d = tmem + (uint32_t)((t & 1) * 64);
#pragma unroll
                for (int kk = 0; kk < HD / 8; kk++)
                    tc_mma_tf32(d, dQ0 + kmajor_step(BM, kk), dk + kmajor_step(BN, kk), idesc_s, kk > 0);
                tc_commit(&bar_s[t & 1]);
            };
            CTRL_WAIT(bar_q, 0, 0x111)
            CTRL_WAIT(&k_full[0], 0, 0x112)
            if (ok) issue_s(0);
            for (int t = 0; t < n_iter && ok; t++) {
                if (t + 1 < n_iter) {
                    CTRL_WAIT(&k_full[(t + 1) & 1], use_parity(t + 1), 0x113)
                    // the other score buffer still holds P(t-1) until PV(t-1) has read it
                    if (t >= 1) CTRL_WAIT(&bar_o[(t - 1) & 1], use_parity(t - 1), 0x114)
                    if (!ok) break;
                    issue_s(t + 1);
                }
                CTRL_WAIT(&bar_p[t & 1], use_parity(t), 0x115)          // P(t) published, PV(t-2) folded
                CTRL_WAIT(&v_full[t & 1], use_parity(t), 0x116)
                if (!ok) break;
                tc_fence_after();
                const uint64_t dv = dV0 + (uint64_t)((t & 1) * (Cfg::kV >> 4));
                const uint32_t d_pv = tmem + 128 + (uint32_t)((t & 1) * HD), a_p = tmem + (uint32_t)((t & 1) * 64);
#pragma unroll
                for (int kk = 0; kk < BN / 8; kk++)
                    tc_mma_tf32_ts(d_pv, a_p + kk * 8, dv + mnmajor_step(kk), idesc_pv, kk > 0);
                tc_commit(&bar_o[t & 1]);
            }
        }
    } else {
        // ---- one thread per query row
        const int r = warp * 32 + lane, row = i0 + r;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const int vis = row < nb ? vis_len(row, p.prefix, nb) : 0;
        const int vis_min = __reduce_min_sync(0xffffffffu, vis);
        // the running maximum is kept in units of log2(e)*scale so that exp() is one ex2
        const float sl2 = p.scale * 1.4426950408889634f;
        float m = -INFINITY, l = 0.f, corr_prev = 1.f;
        float acc[HD];
#pragma unroll
        for (int c = 0; c < HD; c++) acc[c] = 0.f;
        auto fold_pv = [&](int t, float corr) {          // O = O*corr + PV(t), PV read back from TMEM
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t x[32];
                tc_ld32(tmem + 128 + (uint32_t)((t & 1) * HD) + lane_base + c0, x);
#pragma unroll
                for (int j = 0; j < 32; j++) acc[c0 + j] = fmaf(acc[c0 + j], corr, __uint_as_float(x[j]));
            }
        };
        for (int t = 0; t < n_iter; t++) {
            const int j0 = t * BN;
            const uint32_t tmem_s = tmem + (uint32_t)((t & 1) * 64) + lane_base;
            WARP_WAIT(&bar_s[t & 1], use_parity(t), 0x121);
            if (!ok) break;
            tc_fence_after();
            // pass 1: row maximum over the 64 columns of this key tile (TMEM reads are cheap,
            // so the scores are read twice instead of being kept in 64 registers)
            // A tile every row of the warp sees in full needs no mask tests: all but the one or two
            // diagonal tiles of a causal CTA.  The maximum is taken over the raw scores on four
            // independent chains and scaled once (the scale is positive).
            const bool full = j0 + BN <= vis_min;
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int half = 0; half < BN / 32; half++) {
                uint32_t s[32];
                tc_ld32(tmem_s + half * 32, s);
                if (full) {
#pragma unroll
                    for (int j = 0; j < 32; j++) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(s[j]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (j0 + half * 32 + j < vis) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(s[j]));
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl2;
            const float mnew = fmaxf(m, mx);
            const float corr = (mnew == -INFINITY) ? 1.f : fast_exp2(m - mnew);
            // fold the previous tile's PV (scaled by the previous correction)
            if (t > 0) {
                WARP_WAIT(&bar_o[(t - 1) & 1], use_parity(t - 1), 0x122);
                if (!ok) break;
                tc_fence_after();
                fold_pv(t - 1, corr_prev);
            }
            corr_prev = corr;
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
            // pass 2: probabilities, rounded to TF32, written over the scores
#pragma unroll
            for (int half = 0; half < BN / 32; half++) {
                uint32_t s[32];
                tc_ld32(tmem_s + half * 32, s);
                if (full) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float e = fast_exp2(fmaf(__uint_as_float(s[j]), sl2, -mnew));
                        rs4[j & 3] += e; s[j] = tf32_bits(e);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float e = (j0 + half * 32 + j < vis) ? fast_exp2(fmaf(__uint_as_float(s[j]), sl2, -mnew)) : 0.f;
                        rs4[j & 3] += e; s[j] = tf32_bits(e);
                    }
                }
                tc_st32(tmem_s + half * 32, s);
            }
            tc_wait_st();
            l = l * corr + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
            m = mnew;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_p[t & 1]);
        }
        if (ok) {
            WARP_WAIT(&bar_o[(n_iter - 1) & 1], use_parity(n_iter - 1), 0x123);
            tc_fence_after();
            if (ok) fold_pv(n_iter - 1, corr_prev);
        }
        if (ok && p.tma_out) {
            // every product has completed, so the Q tile's shared memory stages the output: one 32 x 32 tile per
            // 32 columns and warp, handed to the copy engine (rows beyond N are clipped, rows beyond the
            // sequence's length are written as zeros like before)
            const bool live = row < nb;
            const float inv = live ? 1.f / l : 0.f;
            uint8_t *st = sQ + warp * (HD / 32) * 4096;
#pragma unroll
            for (int cc = 0; cc < HD / 32; cc++) {
                uint32_t a[32];
#pragma unroll
                for (int j = 0; j < 32; j++) a[j] = __float_as_uint(acc[cc * 32 + j] * inv);
                stage_tile32(st + cc * 4096, a, lane);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                for (int cc = 0; cc < HD / 32; cc++) tma_store_4d(&tmO, st + cc * 4096, cc * 32, i0 + warp * 32, h, b, false);
                bulk_commit();
                bulk_wait<0>();
            }
            if (p.lse && row < p.N) p.lse[slice + row] = live ? (m + log2f(l)) * 0.6931471805599453f : 0.f;
        } else if (ok && row < p.N) {
            const bool live = row < nb;
            const float inv = live ? 1.f / l : 0.f;
            float4 *dst = reinterpret_cast<float4 *>(o + (int64_t)row * p.o.sn);
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
// w/4 of the 64-query tile.  Query tile t brings Q and dO twice: K-major (B operands of S^T and
// dP^T, ring 1) and MN-major (B operands of dK and dV, ring 2); the two rings are released
// by different products and filled by different threads, so each is reloaded as early as its
// own readers allow.
template <int HD>
struct DkvCfg {
    static constexpr int BKEY = 128, BQ = 64, KB = HD / 32;
    static constexpr int kKt = KB * BKEY * 128;            // K and V tiles, K-major A operands
    static constexpr int kQk = KB * BQ * 128;              // Q / dO of one query tile, K-major B (for S^T, dP^T)
    static constexpr int kQm = KB * BQ * 128;              // the same rows, MN-major B (for dK, dV)
    static constexpr int kSmem = 2 * kKt + 4 * kQk + 4 * kQm + 3 * 8 * 64 * 4 + 1024 + 256;
    static constexpr int kTmemCols = 512;                  // S^T/P^T 0,64,128 ; dP^T/dS^T 192,256,320 ; dV 384.. ; dK 448..
    static constexpr int kThreads = 352;                   // 8 compute warps, ring-1 loader, MMA warp, ring-2 loader
};

template <int HD>
__global__ void __launch_bounds__(352, 1)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap tmKa, const __grid_constant__ CUtensorMap tmVa,
                       const __grid_constant__ CUtensorMap tmQk, const __grid_constant__ CUtensorMap tmGk,
                       const __grid_constant__ CUtensorMap tmQm, const __grid_constant__ CUtensorMap tmGm,
                       const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV, AttnTcParams p) {
    using Cfg = DkvCfg<HD>;
    constexpr int BKEY = Cfg::BKEY, BQ = Cfg::BQ, KB = Cfg::KB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sK = smem, *sV = sK + Cfg::kKt, *sQk = sV + Cfg::kKt, *sGk = sQk + 2 * Cfg::kQk, *sQm = sGk + 2 * Cfg::kQk,
            *sGm = sQm + 2 * Cfg::kQm;
    float *s_lse = (float *)(sGm + 2 * Cfg::kQm), *s_d = s_lse + 8 * 64;       // [8 warps][2][32] each
    int *s_vis = (int *)(s_d + 8 * 64);
    uint64_t *bars = (uint64_t *)(((uintptr_t)(s_vis + 8 * 64) + 15) & ~(uintptr_t)15);
    uint64_t *bar_kv = bars, *in1_full = bars + 1 /*[2]*/, *in2_full = bars + 3 /*[2]*/, *bar_o = bars + 5 /*[2]*/,
             *bar_s = bars + 7 /*[3]*/, *bar_p = bars + 10 /*[3]*/;
    uint32_t *tmem_slot = (uint32_t *)(bars + 13);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // grid = (batch x heads, key tiles): the first key tiles are seen by the most queries and are dispatched first
    const int b = (int)blockIdx.x / p.H, h = (int)blockIdx.x % p.H, j0 = (int)blockIdx.y * BKEY;
    int nb = p.seq_lens ? p.seq_lens[b] : p.N;
    if (nb > p.N) nb = p.N;
    if (j0 >= nb) return;
    const int64_t slice = (int64_t)(b * p.H + h) * p.N;

    if (threadIdx.x == 0) {
        mbar_init(bar_kv, 1);
        for (int s = 0; s < 2; s++) { mbar_init(&in1_full[s], 1); mbar_init(&in2_full[s], 1); mbar_init(&bar_o[s], 1); }
        for (int s = 0; s < 3; s++) { mbar_init(&bar_s[s], 1); mbar_init(&bar_p[s], 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_dv = tmem + 384, t_dk = tmem + 448;

    // first query tile that can see a key of this tile; all later tiles up to nb
    const int i_begin = (p.prefix > 0 && j0 < p.prefix) ? 0 : (j0 / BQ) * BQ;
    const int n_iter = (nb - i_begin + BQ - 1) / BQ;
    bool ok = true;

    if (warp == 8) {
        if (lane == 0) {                 // ---- loader of K, V and ring 1 (freed by S^T/dP^T of tile t-2)
            mbar_expect_tx(bar_kv, 2 * Cfg::kKt);
            for (int kb = 0; kb < KB; kb++) {
                tma_load_4d(sK + kb * BKEY * 128, &tmKa, kb * 32, j0, h, b, bar_kv);
                tma_load_4d(sV + kb * BKEY * 128, &tmVa, kb * 32, j0, h, b, bar_kv);
            }
            for (int t = 0; t < n_iter && ok; t++) {
                const int s = t & 1, i0 = i_begin + t * BQ;
                if (t >= 2) CTRL_WAIT(&bar_s[buf3(t - 2)], use_parity3(t - 2), 0x201)
                if (!ok) break;
                mbar_expect_tx(&in1_full[s], 2 * Cfg::kQk);
                for (int kb = 0; kb < KB; kb++) {
                    tma_load_4d(sQk + s * Cfg::kQk + kb * BQ * 128, &tmQk, kb * 32, i0, h, b, &in1_full[s]);
                    tma_load_4d(sGk + s * Cfg::kQk + kb * BQ * 128, &tmGk, kb * 32, i0, h, b, &in1_full[s]);
                }
            }
        }
    } else if (warp == 10) {
        if (lane == 0) {                 // ---- loader of ring 2 (freed by dV/dK of tile t-2)
            for (int t = 0; t < n_iter && ok; t++) {
                const int s = t & 1, i0 = i_begin + t * BQ;
                if (t >= 2) CTRL_WAIT(&bar_o[s], use_parity(t - 2), 0x202)
                if (!ok) break;
                mbar_expect_tx(&in2_full[s], 2 * Cfg::kQm);
                for (int c = 0; c < KB; c++) {
                    tma_load_4d(sQm + s * Cfg::kQm + c * BQ * 128, &tmQm, c * 32, i0, h, b, &in2_full[s]);
                    tma_load_4d(sGm + s * Cfg::kQm + c * BQ * 128, &tmGm, c * 32, i0, h, b, &in2_full[s]);
                }
            }
        }
    } else if (warp == 9) {
        if (lane == 0) {                 // ---- MMA issuer
            const uint32_t id_s = make_idesc_tf32(BQ, false, false), id_g = make_idesc_tf32(HD, false, true);
            // descriptors of K=8 step 0 of every operand buffer; the issue loops only add constants
            const uint64_t dK0 = kmajor_desc(smem_u32(sK), BKEY, 0), dV0 = kmajor_desc(smem_u32(sV), BKEY, 0);
            const uint64_t dQk0 = kmajor_desc(smem_u32(sQk), BQ, 0);
            const uint64_t dGk0 = kmajor_desc(smem_u32(sGk), BQ, 0);
            const uint64_t dQm0 = mnmajor_desc(smem_u32(sQm), BQ, 0);
            const uint64_t dGm0 = mnmajor_desc(smem_u32(sGm), BQ, 0);
            auto issue_sdp = [&](int t) {
                const uint32_t t_st = tmem + (uint32_t)(buf3(t) * 64), t_dpt = t_st + 192;
                const uint64_t slot = (uint64_t)((t & 1) * (Cfg::kQk >> 4)), dq = dQk0 + slot, dg = dGk0 + slot;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < HD / 8; kk++) tc_mma_tf32(t_st, dK0 + kmajor_step(BKEY, kk), dq + kmajor_step(BQ, kk), id_s, kk > 0);
#pragma unroll
                for (int kk = 0; kk < HD / 8; kk++) tc_mma_tf32(t_dpt, dV0 + kmajor_step(BKEY, kk), dg + kmajor_step(BQ, kk), id_s, kk > 0);
                tc_commit(&bar_s[buf3(t)]);
            };
            CTRL_WAIT(bar_kv, 0, 0x211)
            CTRL_WAIT(&in1_full[0], 0, 0x212)
            if (ok) issue_sdp(0);
            for (int t = 0; t < n_iter && ok; t++) {
                if (t + 1 < n_iter) {
                    CTRL_WAIT(&in1_full[(t + 1) & 1], use_parity(t + 1), 0x213)
                    // score buffer (t+1)%3 held P^T, dS^T of tile t-2 until dV/dK(t-2) had read them
                    if (t >= 2) CTRL_WAIT(&bar_o[(t - 2) & 1], use_parity(t - 2), 0x214)
                    if (!ok) break;
                    issue_sdp(t + 1);
                }
                CTRL_WAIT(&bar_p[buf3(t)], use_parity3(t), 0x215)
                CTRL_WAIT(&in2_full[t & 1], use_parity(t), 0x216)
                if (!ok) break;
                tc_fence_after();
                const uint32_t t_pt = tmem + (uint32_t)(buf3(t) * 64), t_dst = t_pt + 192;
                const uint64_t slot2 = (uint64_t)((t & 1) * (Cfg::kQm >> 4)), dgm = dGm0 + slot2, dqm = dQm0 + slot2;
#pragma unroll
                for (int kk = 0; kk < BQ / 8; kk++)
                    tc_mma_tf32_ts(t_dv, t_pt + kk * 8, dgm + mnmajor_step(kk), id_g, (t > 0 || kk > 0));
#pragma unroll
                for (int kk = 0; kk < BQ / 8; kk++)
                    tc_mma_tf32_ts(t_dk, t_dst + kk * 8, dqm + mnmajor_step(kk), id_g, (t > 0 || kk > 0));
                tc_commit(&bar_o[t & 1]);
            }
        }
    } else {
        const int q4 = warp & 3, hq = warp >> 2;
        const int r = q4 * 32 + lane, key = j0 + r;
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        const float sl2 = p.scale * 1.4426950408889634f;
        // Per-query statistics of tile t (log-sum-exp in log2 units, negated; D times the scale; visible
        // length) are fetched one tile ahead, each lane for one of the warp's 32 queries, and handed
        // round through a strip of shared memory that belongs to this warp alone: no CTA-wide barrier.
        float *w_lse = s_lse + warp * 64, *w_d = s_d + warp * 64;                // [2][32] each
        int *w_vis = s_vis + warp * 64;
        float pre_lse = 0.f, pre_d = 0.f; int pre_vis = 0;
        auto prefetch_stats = [&](int t) {
            int row = i_begin + t * BQ + hq * 32 + lane;
            bool live = t < n_iter && row < nb;
            pre_lse = live ? -p.lse_in[slice + row] * 1.4426950408889634f : 0.f;
            pre_d = live ? p.dvec[slice + row] * p.scale : 0.f;
            pre_vis = live ? vis_len(row, p.prefix, nb) : 0;
        };
        prefetch_stats(0);
        const int key_last = j0 + q4 * 32 + 31;          // last key of this warp's lane quadrant
        for (int t = 0; t < n_iter; t++) {
            const int sb = (t & 1) * 32, buf = buf3(t);
            w_lse[sb + lane] = pre_lse; w_d[sb + lane] = pre_d; w_vis[sb + lane] = pre_vis;
            // every key of the warp visible to every query of the tile: no mask tests (all but the diagonal tiles)
            const bool full = key_last < __reduce_min_sync(0xffffffffu, pre_vis);
            prefetch_stats(t + 1);
            __syncwarp();
            WARP_WAIT(&bar_s[buf], use_parity3(t), 0x221);
            if (ok) {
                tc_fence_after();
                uint32_t s[32], dp[32];
                const uint32_t a_s = tmem + (uint32_t)(buf * 64) + lane_base + hq * 32, a_dp = a_s + 192;
                tc_ld32(a_s, s);
                tc_ld32(a_dp, dp);
                const float4 *l4 = reinterpret_cast<const float4 *>(w_lse + sb), *d4 = reinterpret_cast<const float4 *>(w_d + sb);
                const int4 *v4 = reinterpret_cast<const int4 *>(w_vis + sb);
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float4 L = l4[j >> 2], D = d4[j >> 2];
                    const float ls[4] = {L.x, L.y, L.z, L.w}, ds[4] = {D.x, D.y, D.z, D.w};
                    if (full) {
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float pe = fast_exp2(fmaf(__uint_as_float(s[j + e]), sl2, ls[e]));
                            s[j + e] = tf32_bits(pe);
                            dp[j + e] = tf32_bits(pe * fmaf(__uint_as_float(dp[j + e]), p.scale, -ds[e]));
                        }
                    } else {
                        const int4 V = v4[j >> 2];
                        const int vs[4] = {V.x, V.y, V.z, V.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float pe = (key < vs[e]) ? fast_exp2(fmaf(__uint_as_float(s[j + e]), sl2, ls[e])) : 0.f;
                            s[j + e] = tf32_bits(pe);
                            dp[j + e] = tf32_bits(pe * fmaf(__uint_as_float(dp[j + e]), p.scale, -ds[e]));
                        }
                    }
                }
                tc_st32(a_s, s);            // P^T over S^T
                tc_st32(a_dp, dp);          // dS^T over dP^T
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_p[buf]);
            }
        }
        if (ok) {
            WARP_WAIT(&bar_o[(n_iter - 1) & 1], use_parity(n_iter - 1), 0x223);
            tc_fence_after();
            const int c0 = hq * 32;
            if (ok && c0 < HD) {             // warp-uniform: every lane takes part in the TMEM loads
                uint32_t a[32], c[32];
                tc_ld32(t_dv + lane_base + c0, a);
                tc_ld32(t_dk + lane_base + c0, c);
                if (p.dk.p && key < nb && p.rope_c) unrotate32<HD>(c, p.rope_c, p.rope_s, key, c0);
                if (p.tma_out) {
                    // every product has completed (bar_o of the last tile), so the operand rings are free: two staging
                    // tiles per warp in ring 2.  Keys at or beyond the sequence's length have exact zero rows (their
                    // probabilities are zero) and only occur in add mode; rows beyond N are clipped by the copy engine.
                    uint8_t *st = sQm + (hq * 4 + q4) * 8192;
                    stage_tile32(st, a, lane);
                    stage_tile32(st + 4096, c, lane);
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (p.dv.p) tma_store_4d(&tmDV, st, c0, j0 + q4 * 32, h, b, (p.store & 4) == 0);
                        if (p.dk.p) tma_store_4d(&tmDK, st + 4096, c0, j0 + q4 * 32, h, b, (p.store & 2) == 0);
                        bulk_commit();
                        bulk_wait<0>();
                    }
                } else {
                    if (p.dv.p && key < nb)
                        emit_row32(p.dv.p + (int64_t)b * p.dv.sb + (int64_t)h * p.dv.sh + (int64_t)key * p.dv.sn + c0, a, (p.store & 4) != 0);
                    if (p.dk.p && key < nb)
                        emit_row32(p.dk.p + (int64_t)b * p.dk.sb + (int64_t)h * p.dk.sh + (int64_t)key * p.dk.sn + c0, c, (p.store & 2) != 0);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) { tc_fence_after(); tmem_dealloc(tmem, Cfg::kTmemCols); }
}

// ════════════════════════ backward: dQ (one CTA per 128 query rows) ════════════════════════
// 8 compute warps as above (lane quadrant = query rows, 32 key columns each).  Key tile t brings
// K and V K-major (B operands of S and dP, ring 1) and K MN-major (B operand of dQ, ring 2).
template <int HD>
struct DqCfg {
    static constexpr int BM = 128, BN = 64, KB = HD / 32;
    static constexpr int kQ = KB * BM * 128;               // Q and dO tiles, K-major A operands
    static constexpr int kKk = KB * BN * 128;              // K / V of one key tile, K-major B
    static constexpr int kKm = KB * BN * 128;              // K of the same tile, MN-major B
    static constexpr int kSmem = 2 * kQ + 4 * kKk + 2 * kKm + 1024 + 256;
    static constexpr int kTmemCols = 512;                  // S 0,64,128 ; dP/dS 192,256,320 ; dQ 384..
    static constexpr int kThreads = 352;
};

template <int HD>
__global__ void __launch_bounds__(352, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQa, const __grid_constant__ CUtensorMap tmGa,
                      const __grid_constant__ CUtensorMap tmKk, const __grid_constant__ CUtensorMap tmVk,
                      const __grid_constant__ CUtensorMap tmKm, AttnTcParams p) {
    using Cfg = DqCfg<HD>;
    constexpr int BM = Cfg::BM, BN = Cfg::BN, KB = Cfg::KB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem, *sG = sQ + Cfg::kQ, *sKk = sG + Cfg::kQ, *sVk = sKk + 2 * Cfg::kKk, *sKm = sVk + 2 * Cfg::kKk;
    uint64_t *bars = (uint64_t *)(sKm + 2 * Cfg::kKm);
    uint64_t *bar_qg = bars, *in1_full = bars + 1 /*[2]*/, *in2_full = bars + 3 /*[2]*/, *bar_o = bars + 5 /*[2]*/,
             *bar_s = bars + 7 /*[3]*/, *bar_p = bars + 10 /*[3]*/;
    uint32_t *tmem_slot = (uint32_t *)(bars + 13);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // grid = (batch x heads, query tiles): CTAs are dispatched x-fastest, so all heads' LAST query tiles -- which
    // see the most keys under the causal and prefix rules -- go first and the shortest CTAs fill the tail
    const int b = (int)blockIdx.x / p.H, h = (int)blockIdx.x % p.H, i0 = (int)(gridDim.y - 1 - blockIdx.y) * BM;
    int nb = p.seq_lens ? p.seq_lens[b] : p.N;
    if (nb > p.N) nb = p.N;
    if (i0 >= nb) return;
    const int64_t slice = (int64_t)(b * p.H + h) * p.N;

    if (threadIdx.x == 0) {
        mbar_init(bar_qg, 1);
        for (int s = 0; s < 2; s++) { mbar_init(&in1_full[s], 1); mbar_init(&in2_full[s], 1); mbar_init(&bar_o[s], 1); }
        for (int s = 0; s < 3; s++) { mbar_init(&bar_s[s], 1); mbar_init(&bar_p[s], 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_dq = tmem + 384;

    const int i_last = min(i0 + BM, nb) - 1;
    const int jmax = vis_len(i_last, p.prefix, nb);
    const int n_iter = (jmax + BN - 1) / BN;
    bool ok = true;

    if (warp == 8) {
        if (lane == 0) {                 // ---- loader of Q, dO and ring 1 (freed by S/dP of tile t-2)
            mbar_expect_tx(bar_qg, 2 * Cfg::kQ);
            for (int kb = 0; kb < KB; kb++) {
                tma_load_4d(sQ + kb * BM * 128, &tmQa, kb * 32, i0, h, b, bar_qg);
                tma_load_4d(sG + kb * BM * 128, &tmGa, kb * 32, i0, h, b, bar_qg);
            }
            for (int t = 0; t < n_iter && ok; t++) {
                const int s = t & 1, jt = t * BN;
                if (t >= 2) CTRL_WAIT(&bar_s[buf3(t - 2)], use_parity3(t - 2), 0x301)
                if (!ok) break;
                mbar_expect_tx(&in1_full[s], 2 * Cfg::kKk);
                for (int kb = 0; kb < KB; kb++) {
                    tma_load_4d(sKk + s * Cfg::kKk + kb * BN * 128, &tmKk, kb * 32, jt, h, b, &in1_full[s]);
                    tma_load_4d(sVk + s * Cfg::kKk + kb * BN * 128, &tmVk, kb * 32, jt, h, b, &in1_full[s]);
                }
            }
        }
    } else if (warp == 10) {
        if (lane == 0) {                 // ---- loader of ring 2 (freed by dQ of tile t-2)
            for (int t = 0; t < n_iter && ok; t++) {
                const int s = t & 1, jt = t * BN;
                if (t >= 2) CTRL_WAIT(&bar_o[s], use_parity(t - 2), 0x302)
                if (!ok) break;
                mbar_expect_tx(&in2_full[s], Cfg::kKm);
                for (int c = 0; c < KB; c++) tma_load_4d(sKm + s * Cfg::kKm + c * BN * 128, &tmKm, c * 32, jt, h, b, &in2_full[s]);
            }
        }
    } else if (warp == 9) {
        if (lane == 0) {                 // ---- MMA issuer
            const uint32_t id_s = make_idesc_tf32(BN, false, false), id_q = make_idesc_tf32(HD, false, true);
            const uint64_t dQ0 = kmajor_desc(smem_u32(sQ), BM, 0), dG0 = kmajor_desc(smem_u32(sG), BM, 0);
            const uint64_t dKk0 = kmajor_desc(smem_u32(sKk), BN, 0);
            const uint64_t dVk0 = kmajor_desc(smem_u32(sVk), BN, 0);
            const uint64_t dKm0 = mnmajor_desc(smem_u32(sKm), BN, 0);
            auto issue_sdp = [&](int t) {
                const uint32_t t_s = tmem + (uint32_t)(buf3(t) * 64), t_dp = t_s + 192;
                const uint64_t slot = (uint64_t)((t & 1) * (Cfg::kKk >> 4)), dk = dKk0 + slot, dv = dVk0 + slot;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < HD / 8; kk++) tc_mma_tf32(t_s, dQ0 + kmajor_step(BM, kk), dk + kmajor_step(BN, kk), id_s, kk > 0);
#pragma unroll
                for (int kk = 0; kk < HD / 8; kk++) tc_mma_tf32(t_dp, dG0 + kmajor_step(BM, kk), dv + kmajor_step(BN, kk), id_s, kk > 0);
                tc_commit(&bar_s[buf3(t)]);
            };
            CTRL_WAIT(bar_qg, 0, 0x311)
            CTRL_WAIT(&in1_full[0], 0, 0x312)
            if (ok) issue_sdp(0);
            for (int t = 0; t < n_iter && ok; t++) {
                if (t + 1 < n_iter) {
                    CTRL_WAIT(&in1_full[(t + 1) & 1], use_parity(t + 1), 0x313)
                    if (t >= 2) CTRL_WAIT(&bar_o[(t - 2) & 1], use_parity(t - 2), 0x314)     // dS(t-2) read by dQ(t-2)
                    if (!ok) break;
                    issue_sdp(t + 1);
                }
                CTRL_WAIT(&bar_p[buf3(t)], use_parity3(t), 0x315)
                CTRL_WAIT(&in2_full[t & 1], use_parity(t), 0x316)
                if (!ok) break;
                tc_fence_after();
                const uint32_t t_ds = tmem + 192 + (uint32_t)(buf3(t) * 64);
                const uint64_t dkm = dKm0 + (uint64_t)((t & 1) * (Cfg::kKm >> 4));
#pragma unroll
                for (int kk = 0; kk < BN / 8; kk++)
                    tc_mma_tf32_ts(t_dq, t_ds + kk * 8, dkm + mnmajor_step(kk), id_q, (t > 0 || kk > 0));
                tc_commit(&bar_o[t & 1]);
            }
        }
    } else {
        const int q4 = warp & 3, hq = warp >> 2;
        const int r = q4 * 32 + lane, row = i0 + r;
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        const bool live = row < nb;
        const int vis = live ? vis_len(row, p.prefix, nb) : 0;
        const float sl2 = p.scale * 1.4426950408889634f;
        const float lse2 = live ? p.lse_in[slice + row] * 1.4426950408889634f : 0.f;
        const float dvec_s = live ? p.dvec[slice + row] * p.scale : 0.f;
        const int vis_min = __reduce_min_sync(0xffffffffu, vis);
        for (int t = 0; t < n_iter; t++) {
            const int buf = buf3(t);
            WARP_WAIT(&bar_s[buf], use_parity3(t), 0x321);
            if (ok) {
                tc_fence_after();
                uint32_t s[32], dp[32];
                const uint32_t a_s = tmem + (uint32_t)(buf * 64) + lane_base + hq * 32, a_dp = a_s + 192;
                tc_ld32(a_s, s);
                tc_ld32(a_dp, dp);
                const int jb = t * BN + hq * 32;
                if (jb + 32 <= vis_min) {          // all 32 keys visible to every row of the warp: no mask tests
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float pe = fast_exp2(fmaf(__uint_as_float(s[j]), sl2, -lse2));
                        dp[j] = tf32_bits(pe * fmaf(__uint_as_float(dp[j]), p.scale, -dvec_s));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float pe = (jb + j < vis) ? fast_exp2(fmaf(__uint_as_float(s[j]), sl2, -lse2)) : 0.f;
                        dp[j] = tf32_bits(pe * fmaf(__uint_as_float(dp[j]), p.scale, -dvec_s));
                    }
                }
                tc_st32(a_dp, dp);          // dS over dP
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_p[buf]);
            }
        }
        if (ok) {
            WARP_WAIT(&bar_o[(n_iter - 1) & 1], use_parity(n_iter - 1), 0x323);
            tc_fence_after();
            const int c0 = hq * 32;
            if (ok && c0 < HD) {
                uint32_t a[32];
                tc_ld32(t_dq + lane_base + c0, a);
                if (live && p.rope_c) unrotate32<HD>(a, p.rope_c, p.rope_s, row, c0);
                if (live) emit_row32(p.dq.p + (int64_t)b * p.dq.sb + (int64_t)h * p.dq.sh + (int64_t)row * p.dq.sn + c0, a, (p.store & 1) != 0);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) { tc_fence_after(); tmem_dealloc(tmem, Cfg::kTmemCols); }
}

// ════════════════════════ backward: dQ, two CTAs per SM ════════════════════════
// The same work split as the kernel above, but lean enough for two CTAs to share an SM: one score
// buffer instead of three (256 TMEM columns per CTA), one slot per operand ring instead of two
// (112 KB of tiles per CTA).  Inside a CTA a tile then runs strictly in sequence -- S and dP, the
// threads' dS, dQ -- and it is the OTHER CTA's products that keep the tensor core busy meanwhile; its
// start-up (Q and dO, 64 KB) and its final dQ store hide behind the neighbour in the same way.
template <int HD>
struct Dq2Cfg {
    static constexpr int BM = 128, BN = 64, KB = HD / 32;
    static constexpr int kQ = KB * BM * 128;               // Q and dO tiles, K-major A operands
    static constexpr int kKk = KB * BN * 128;              // K / V of one key tile, K-major B
    static constexpr int kKm = KB * BN * 128;              // K of the same tile, MN-major B
    static constexpr int kTiles = 2 * kQ + 2 * kKk + kKm;
    // Two CTAs of head size 64 fit an SM only if tiles + padding + barriers stay within 113 KB each: the
    // array is declared 1024-byte aligned and up to kPad bytes of round-up are tolerated; a base further
    // off than that is reported as an error instead of running over the allocation.
    static constexpr int kPad = 768;
    static constexpr int kSmem = kTiles + kPad + 256;
    static constexpr int kTmemCols = 256;                  // S 0.. ; dP/dS 64.. ; dQ 128..
    static constexpr int kThreads = 352;
};

template <int HD>
__global__ void __launch_bounds__(352, 2)
attn_bwd_dq2_tc_kernel(const __grid_constant__ CUtensorMap tmQa, const __grid_constant__ CUtensorMap tmGa,
                       const __grid_constant__ CUtensorMap tmKk, const __grid_constant__ CUtensorMap tmVk,
                       const __grid_constant__ CUtensorMap tmKm, const __grid_constant__ CUtensorMap tmDQ, AttnTcParams p) {
    using Cfg = Dq2Cfg<HD>;
    constexpr int BM = Cfg::BM, BN = Cfg::BN, KB = Cfg::KB;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    if (smem - smem_raw > Cfg::kPad) {          // the same for every thread: nobody has touched a barrier or TMEM yet
        if (threadIdx.x == 0) atomicCAS(&g_attn_error, 0, 0x3ff);
        return;
    }
    uint8_t *sQ = smem, *sG = sQ + Cfg::kQ, *sKk = sG + Cfg::kQ, *sVk = sKk + Cfg::kKk, *sKm = sVk + Cfg::kKk;
    uint64_t *bars = (uint64_t *)(sKm + Cfg::kKm);
    // every barrier completes once per tile, so the completion that belongs to tile t has parity t & 1
    uint64_t *bar_qg = bars, *in1_full = bars + 1, *in2_full = bars + 2, *bar_o = bars + 3, *bar_s = bars + 4, *bar_p = bars + 5;
    uint32_t *tmem_slot = (uint32_t *)(bars + 6);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // grid = (batch x heads, query tiles): CTAs are dispatched x-fastest, so all heads' LAST query tiles -- which
    // see the most keys under the causal and prefix rules -- go first and the shortest CTAs fill the tail
    const int b = (int)blockIdx.x / p.H, h = (int)blockIdx.x % p.H, i0 = (int)(gridDim.y - 1 - blockIdx.y) * BM;
    int nb = p.seq_lens ? p.seq_lens[b] : p.N;
    if (nb > p.N) nb = p.N;
    if (i0 >= nb) return;
    const int64_t slice = (int64_t)(b * p.H + h) * p.N;

    if (threadIdx.x == 0) {
        mbar_init(bar_qg, 1);
        mbar_init(in1_full, 1); mbar_init(in2_full, 1); mbar_init(bar_o, 1); mbar_init(bar_s, 1); mbar_init(bar_p, 8);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_s = tmem, t_dp = tmem + 64, t_dq = tmem + 128;

    const int i_last = min(i0 + BM, nb) - 1;
    const int jmax = vis_len(i_last, p.prefix, nb);
    const int n_iter = (jmax + BN - 1) / BN;
    bool ok = true;

    if (warp == 8) {
        if (lane == 0) {                 // ---- loader of Q, dO and of K, V K-major (their slot is free when S/dP of tile t-1 are done)
            mbar_expect_tx(bar_qg, 2 * Cfg::kQ);
            for (int kb = 0; kb < KB; kb++) {
                tma_load_4d(sQ + kb * BM * 128, &tmQa, kb * 32, i0, h, b, bar_qg);
                tma_load_4d(sG + kb * BM * 128, &tmGa, kb * 32, i0, h, b, bar_qg);
            }
            for (int t = 0; t < n_iter && ok; t++) {
                const int jt = t * BN;
                if (t >= 1) CTRL_WAIT(bar_s, (uint32_t)(t - 1) & 1u, 0x341)
                if (!ok) break;
                mbar_expect_tx(in1_full, 2 * Cfg::kKk);
                for (int kb = 0; kb < KB; kb++) {
                    tma_load_4d(sKk + kb * BN * 128, &tmKk, kb * 32, jt, h, b, in1_full);
                    tma_load_4d(sVk + kb * BN * 128, &tmVk, kb * 32, jt, h, b, in1_full);
                }
            }
        }
    } else if (warp == 10) {
        if (lane == 0) {                 // ---- loader of K MN-major (free when dQ of tile t-1 is done)
            for (int t = 0; t < n_iter && ok; t++) {
                const int jt = t * BN;
                if (t >= 1) CTRL_WAIT(bar_o, (uint32_t)(t - 1) & 1u, 0x342)
                if (!ok) break;
                mbar_expect_tx(in2_full, Cfg::kKm);
                for (int c = 0; c < KB; c++) tma_load_4d(sKm + c * BN * 128, &tmKm, c * 32, jt, h, b, in2_full);
            }
        }
    } else if (warp == 9) {
        if (lane == 0) {                 // ---- MMA issuer
            const uint32_t id_s = make_idesc_tf32(BN, false, false), id_q = make_idesc_tf32(HD, false, true);
            const uint64_t dQ0 = kmajor_desc(smem_u32(sQ), BM, 0), dG0 = kmajor_desc(smem_u32(sG), BM, 0);
            const uint64_t dKk0 = kmajor_desc(smem_u32(sKk), BN, 0);
            const uint64_t dVk0 = kmajor_desc(smem_u32(sVk), BN, 0);
            const uint64_t dKm0 = mnmajor_desc(smem_u32(sKm), BN, 0);
            CTRL_WAIT(bar_qg, 0, 0x351)
            for (int t = 0; t < n_iter && ok; t++) {
                const uint32_t par = (uint32_t)t & 1u;
                CTRL_WAIT(in1_full, par, 0x353)
                if (t >= 1) CTRL_WAIT(bar_o, par ^ 1u, 0x354)          // dQ(t-1) has read dS(t-1): the score buffers are free
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < HD / 8; kk++) tc_mma_tf32(t_s, dQ0 + kmajor_step(BM, kk), dKk0 + kmajor_step(BN, kk), id_s, kk > 0);
#pragma unroll
                for (int kk = 0; kk < HD / 8; kk++) tc_mma_tf32(t_dp, dG0 + kmajor_step(BM, kk), dVk0 + kmajor_step(BN, kk), id_s, kk > 0);
                tc_commit(bar_s);
                CTRL_WAIT(bar_p, par, 0x355)
                CTRL_WAIT(in2_full, par, 0x356)
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < BN / 8; kk++)
                    tc_mma_tf32_ts(t_dq, t_dp + kk * 8, dKm0 + mnmajor_step(kk), id_q, (t > 0 || kk > 0));
                tc_commit(bar_o);
            }
        }
    } else {
        const int q4 = warp & 3, hq = warp >> 2;
        const int r = q4 * 32 + lane, row = i0 + r;
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        const bool live = row < nb;
        const int vis = live ? vis_len(row, p.prefix, nb) : 0;
        const float sl2 = p.scale * 1.4426950408889634f;
        const float lse2 = live ? p.lse_in[slice + row] * 1.4426950408889634f : 0.f;
        const float dvec_s = live ? p.dvec[slice + row] * p.scale : 0.f;
        const int vis_min = __reduce_min_sync(0xffffffffu, vis);
        for (int t = 0; t < n_iter; t++) {
            WARP_WAIT(bar_s, (uint32_t)t & 1u, 0x361);
            if (ok) {
                tc_fence_after();
                uint32_t s[32], dp[32];
                const uint32_t a_s = t_s + lane_base + hq * 32, a_dp = a_s + 64;
                tc_ld32(a_s, s);
                tc_ld32(a_dp, dp);
                const int jb = t * BN + hq * 32;
                if (jb + 32 <= vis_min) {          // all 32 keys visible to every row of the warp: no mask tests
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float pe = fast_exp2(fmaf(__uint_as_float(s[j]), sl2, -lse2));
                        dp[j] = tf32_bits(pe * fmaf(__uint_as_float(dp[j]), p.scale, -dvec_s));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float pe = (jb + j < vis) ? fast_exp2(fmaf(__uint_as_float(s[j]), sl2, -lse2)) : 0.f;
                        dp[j] = tf32_bits(pe * fmaf(__uint_as_float(dp[j]), p.scale, -dvec_s));
                    }
                }
                tc_st32(a_dp, dp);          // dS over dP
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_p);
            }
        }
        if (ok) {
            WARP_WAIT(bar_o, (uint32_t)(n_iter - 1) & 1u, 0x363);
            tc_fence_after();
            const int c0 = hq * 32;
            if (ok && c0 < HD) {
                uint32_t a[32];
                tc_ld32(t_dq + lane_base + c0, a);
                if (live && p.rope_c) unrotate32<HD>(a, p.rope_c, p.rope_s, row, c0);
                if (p.tma_out) {            // all products are done: the Q tile's shared memory stages the output (see the dK/dV kernel)
                    uint8_t *st = sQ + (hq * 4 + q4) * 4096;
                    stage_tile32(st, a, lane);
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_4d(&tmDQ, st, c0, i0 + q4 * 32, h, b, (p.store & 1) == 0);
                        bulk_commit();
                        bulk_wait<0>();
                    }
                } else if (live) {
                    emit_row32(p.dq.p + (int64_t)b * p.dq.sb + (int64_t)h * p.dq.sh + (int64_t)row * p.dq.sn + c0, a, (p.store & 1) != 0);
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

// Strided [B,H,N,d] fp32 operand as a 4-D map {d, N, H, B}; box = {32 floats of d, rows, 1, 1};
// rows beyond N read as zero.
static CUtensorMap map4d(const HeadView &v, int B, int H, int N, int d, int box_rows, bool mn_major) {
    CUtensorMap m;
    cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)v.sn * 4, (cuuint64_t)v.sh * 4, (cuuint64_t)v.sb * 4};
    cuuint32_t box[4] = {32, (cuuint32_t)box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 4, (void *)v.p, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "dnn_b200: cuTensorMapEncodeTiled (attention) failed (%d)\n", (int)r); abort(); }
    return m;
}

// The same view as the destination of 32 x 32 tile stores (rows beyond N are clipped).
static CUtensorMap map4d_out(const HeadView &v, int B, int H, int N, int d) {
    CUtensorMap m;
    cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)v.sn * 4, (cuuint64_t)v.sh * 4, (cuuint64_t)v.sb * 4};
    cuuint32_t box[4] = {32, 32, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void *)v.p, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "dnn_b200: cuTensorMapEncodeTiled (attention output) failed (%d)\n", (int)r); abort(); }
    return m;
}

static bool view_ok(const HeadView &v) {
    return aligned16(v.p) && v.sn % 4 == 0 && v.sh % 4 == 0 && v.sb % 4 == 0;
}
bool attn_tc_supported(int d, const HeadView &q, const HeadView &k, const HeadView &v) {
    return (d == 32 || d == 64) && view_ok(q) && view_ok(k) && view_ok(v);
}

struct AttnHost {
    HeadView q, k, v, o, dout, dq, dk, dv;
    float *lse; const float *dvec; const int *seq_lens;
    int B, H, N, d, prefix; float scale; int store;
    const float *rope_c, *rope_s;
};

// Visible (query, key) pairs of all heads when every sequence has its full length N: rows inside the
// prefix see the prefix, the others see themselves and everything before (src/attention.c:39-64).
// Per-batch lengths are device data here, so padding is not subtracted: with seq_lens the figure is
// an upper bound.  Used only for the work figure of the launch timeline.
static double visible_pairs(const AttnHost &a) {
    const double P = a.prefix < a.N ? a.prefix : a.N, N = a.N;
    return (double)a.B * a.H * (P * P + (N * (N + 1.0) - P * (P + 1.0)) * 0.5);
}

template <int HD>
static void fwd_launch(const AttnHost &a) {
    using Cfg = FwdCfg<HD>;
    static bool once = false;
    if (!once) {
        CUDA_OK(cudaFuncSetAttribute(attn_fwd_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
        // two CTAs per SM need the largest shared-memory carve-out; left to the driver's choice, the kernel sometimes
        // ran with room for one (forward 2.1 instead of 1.4 ms per step in one run out of several)
        CUDA_OK(cudaFuncSetAttribute(attn_fwd_tc_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        once = true;
    }
    CUtensorMap tq = map4d(a.q, a.B, a.H, a.N, HD, Cfg::BM, false), tk = map4d(a.k, a.B, a.H, a.N, HD, Cfg::BN, false),
                tv = map4d(a.v, a.B, a.H, a.N, HD, Cfg::BN, true);
    AttnTcParams p; memset(&p, 0, sizeof p);
    p.o = a.o; p.lse = a.lse; p.seq_lens = a.seq_lens; p.B = a.B; p.H = a.H; p.N = a.N; p.prefix = a.prefix; p.scale = a.scale;
    dim3 grid(a.B * a.H, (a.N + Cfg::BM - 1) / Cfg::BM);
    static int tma_epilogue = -1;
    if (tma_epilogue < 0) { const char *e = getenv("DNN_CUDA_ATTN_TMA_OUT"); tma_epilogue = (e && e[0] == '0') ? 0 : 1; }
    p.tma_out = tma_epilogue && view_ok(a.o);
    CUtensorMap to = map4d_out(p.tma_out ? a.o : a.q, a.B, a.H, a.N, HD);
    attn_fwd_tc_kernel<HD><<<grid, Cfg::kThreads, Cfg::kSmem, stream()>>>(tq, tk, tv, to, p);
    prof_work(4.0 * HD * visible_pairs(a));                      // S = Q K^T and O = P V
    LAUNCHED("attn_fwd_tc_kernel");
}

template <int HD>
static void bwd_launch(const AttnHost &a) {
    AttnTcParams p; memset(&p, 0, sizeof p);
    p.lse_in = a.lse; p.dvec = a.dvec; p.dq = a.dq; p.dk = a.dk; p.dv = a.dv; p.seq_lens = a.seq_lens;
    p.B = a.B; p.H = a.H; p.N = a.N; p.prefix = a.prefix; p.scale = a.scale; p.store = a.store;
    p.rope_c = a.rope_c; p.rope_s = a.rope_s;
    static bool once = false;
    if (!once) {
        CUDA_OK(cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvCfg<HD>::kSmem));
        CUDA_OK(cudaFuncSetAttribute(attn_bwd_dq_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, DqCfg<HD>::kSmem));
        CUDA_OK(cudaFuncSetAttribute(attn_bwd_dq2_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Dq2Cfg<HD>::kSmem));
        CUDA_OK(cudaFuncSetAttribute(attn_bwd_dq2_tc_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        once = true;
    }
    if (a.dk.p || a.dv.p) {
        using Cfg = DkvCfg<HD>;
        CUtensorMap tka = map4d(a.k, a.B, a.H, a.N, HD, Cfg::BKEY, false), tva = map4d(a.v, a.B, a.H, a.N, HD, Cfg::BKEY, false);
        CUtensorMap tqk = map4d(a.q, a.B, a.H, a.N, HD, Cfg::BQ, false), tgk = map4d(a.dout, a.B, a.H, a.N, HD, Cfg::BQ, false);
        CUtensorMap tqm = map4d(a.q, a.B, a.H, a.N, HD, Cfg::BQ, true), tgm = map4d(a.dout, a.B, a.H, a.N, HD, Cfg::BQ, true);
        dim3 grid(a.B * a.H, (a.N + Cfg::BKEY - 1) / Cfg::BKEY);
        // gradients leave as tile stores when their views can be described to the copy engine (16-byte aligned base and strides)
        static int tma_epilogue = -1;
        if (tma_epilogue < 0) { const char *e = getenv("DNN_CUDA_ATTN_TMA_OUT"); tma_epilogue = (e && e[0] == '0') ? 0 : 1; }
        p.tma_out = tma_epilogue && (!a.dk.p || view_ok(a.dk)) && (!a.dv.p || view_ok(a.dv));
        CUtensorMap tdk = map4d_out(a.dk.p && p.tma_out ? a.dk : a.k, a.B, a.H, a.N, HD), tdv = map4d_out(a.dv.p && p.tma_out ? a.dv : a.v, a.B, a.H, a.N, HD);
        attn_bwd_dkv_tc_kernel<HD><<<grid, Cfg::kThreads, Cfg::kSmem, stream()>>>(tka, tva, tqk, tgk, tqm, tgm, tdk, tdv, p);
        prof_work(6.0 * HD * visible_pairs(a));                  // dV, dP, dK (the recomputed S is not counted)
        LAUNCHED("attn_bwd_dkv_tc_kernel");
    }
    if (a.dq.p) {
        using Cfg = DqCfg<HD>;
        CUtensorMap tqa = map4d(a.q, a.B, a.H, a.N, HD, Cfg::BM, false), tga = map4d(a.dout, a.B, a.H, a.N, HD, Cfg::BM, false);
        CUtensorMap tkk = map4d(a.k, a.B, a.H, a.N, HD, Cfg::BN, false), tvk = map4d(a.v, a.B, a.H, a.N, HD, Cfg::BN, false);
        CUtensorMap tkm = map4d(a.k, a.B, a.H, a.N, HD, Cfg::BN, true);
        dim3 grid(a.B * a.H, (a.N + Cfg::BM - 1) / Cfg::BM);
        // DNN_CUDA_ATTN_DQ: 2 (default) two lean CTAs per SM, 1 one CTA per SM with three score buffers and two-slot rings
        static int lean = -1;
        if (lean < 0) { const char *e = getenv("DNN_CUDA_ATTN_DQ"); lean = (e && e[0] == '1') ? 0 : 1; }
        static int tma_epilogue = -1;
        if (tma_epilogue < 0) { const char *e = getenv("DNN_CUDA_ATTN_TMA_OUT"); tma_epilogue = (e && e[0] == '0') ? 0 : 1; }
        p.tma_out = lean && tma_epilogue && view_ok(a.dq);
        CUtensorMap tdq = map4d_out(p.tma_out ? a.dq : a.q, a.B, a.H, a.N, HD);
        if (lean) attn_bwd_dq2_tc_kernel<HD><<<grid, Dq2Cfg<HD>::kThreads, Dq2Cfg<HD>::kSmem, stream()>>>(tqa, tga, tkk, tvk, tkm, tdq, p);
        else attn_bwd_dq_tc_kernel<HD><<<grid, Cfg::kThreads, Cfg::kSmem, stream()>>>(tqa, tga, tkk, tvk, tkm, p);
        prof_work(2.0 * HD * visible_pairs(a));                  // dQ (recomputed S and dP not counted)
        LAUNCHED("attn_bwd_dq_tc_kernel");
    }
}

void attn_forward_tc(const HeadView &q, const HeadView &k, const HeadView &v, const HeadView &o, float *lse, const int *seq_lens,
                     int B, int H, int N, int d, int prefix, float scale) {
    AttnHost a; memset(&a, 0, sizeof a);
    a.q = q; a.k = k; a.v = v; a.o = o; a.lse = lse; a.seq_lens = seq_lens; a.B = B; a.H = H; a.N = N; a.d = d; a.prefix = prefix; a.scale = scale;
    if (d == 32) fwd_launch<32>(a); else fwd_launch<64>(a);
}

void attn_backward_tc(const HeadView &q, const HeadView &k, const HeadView &v, const float *lse, const HeadView &dout, const float *dvec,
                      const HeadView &dq, const HeadView &dk, const HeadView &dv, const int *seq_lens,
                      int B, int H, int N, int d, int prefix, float scale, int store, const float *rope_c, const float *rope_s) {
    AttnHost a; memset(&a, 0, sizeof a);
    a.store = store;
    DNN_CHECK(!rope_c || (store & 3) == 3, "attention backward: the fused rotation needs dQ and dK in store mode");
    a.rope_c = rope_c; a.rope_s = rope_s;
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
