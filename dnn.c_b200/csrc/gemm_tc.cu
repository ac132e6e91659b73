// TF32 tensor-core GEMM for sm_100a: tcgen05.mma with TMEM accumulators, fed by TMA.
//
//   C[M,N] (=|+=) A[M,K] * B[K,N] (+ bias[N]),  fp32 in memory, TF32 multiply, fp32 accumulate.
//
// One persistent CTA per SM walks (tile, k-split) work units.  Warp roles:
//   warp 0      one elected lane issues the TMA loads (cp.async.bulk.tensor, one
//               CTA's own tiles, no multicast) into a ring of shared-memory stages;
//   warp 1      one elected lane issues tcgen05.mma (128 x BN x 8 per instruction)
//               and commits stage / accumulator completions to mbarriers;
//   warps 2..5  epilogue: tcgen05.ld the 128 x BN accumulator from TMEM, add the bias,
//               write 32 x 32 pieces into swizzled staging tiles and hand them to the
//               copy engine (tile store, or tile add for C +=), so every global write
//               is a full 128-byte row segment.  TMEM holds two accumulators, so the
//               epilogue of one tile overlaps the main loop of the next.
// Operands may be K-major (K contiguous in memory) or MN-major (M resp. N
// contiguous); both are expressed through the shared-memory matrix descriptor
// (128-byte swizzle) and the instruction descriptor's major bits, so the same
// kernel serves A*B, A*B^T, dA and dW without transposing anything in memory.
// Tails in M, N and K need no special code: TMA zero-fills out-of-bounds boxes.
//
// X3 (3xTF32 in one pass): the stages hold the RAW fp32 tiles (the tensor core reads the upper 19 bits
// of each word, i.e. x truncated to TF32 = "big") next to a second copy that eight more warps fill
// with small = x - big as soon as a tile has landed; per K=8 step the issuing thread then runs
// As*Bb, Ab*Bs and Ab*Bb.  Nothing is split in global memory.  X3 = 1: all three into one accumulator
// (the two TMEM accumulators alternate between tiles as in the TF32 kernel).  X3 = 2: Ab*Bb into the
// first and the two small terms into the second accumulator, added by the epilogue in fp32 -- the
// tensor core truncates its accumulator on every add, and keeping the small terms out of the large
// sum leaves that bias where one TF32 product per K step puts it; the price is that the epilogue of
// a tile no longer overlaps the main loop of the next.
//
// Every mbarrier wait is bounded; a wait that runs out records an error code
// that dnn_cuda_sync() reports, and the CTA still frees its TMEM and returns.
#include "common.cuh"
#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace dnnb {

constexpr int BM = 128;            // tile rows = MMA M
constexpr int BK = 32;             // K per stage: 32 fp32 = one 128-byte swizzle row
constexpr int UMMA_K = 8;          // K per tcgen05.mma for TF32
constexpr int kGemmThreads = 192;
constexpr int kSplitWarps = 8;                  // warps that split the landed tiles of the 3xTF32 kernel
constexpr int kGemmThreadsX3 = 192 + kSplitWarps * 32;

__device__ int g_gemm_error = 0;   // 0 ok; otherwise (role << 8 | detail) of the first wait that gave up

struct TcArgs {
    float *C; int64_t ldc;             // row-major output (or split-K partials, ldc = N)
    const float *bias;
    int M, N, K;
    int accumulate;
    int a_kmajor, b_kmajor;
    int splits, kb_per_split;          // split-K: work unit = (tile, split)
    int chained;                       // the splits of a tile run one after the other on the tile's CTA and add into C
    int tiles_m, tiles_n;
    int n_fastest;                     // tile order: consecutive work units walk along N (1) or along M (0)
    int a_chunked, b_chunked;          // MN-major operand described as {32, K, extent/32}: one TMA copy per stage
    const float *resid; int64_t resid_ld;     // epilogue: C = A*B + bias + resid (row-major, same shape as C)
    const float *rope_c, *rope_s;      // epilogue rotation of the first rope_cols columns (heads of rope_d, position = row % rope_N)
    int rope_N, rope_d, rope_cols;
};

template <int BN, bool PAIR, int X3 = 0> struct TcCfg {
    static constexpr int kRowsB = PAIR ? BN / 2 : BN;             // B rows (n) this CTA loads per stage
    static constexpr int kStageA = BM * BK * 4;                   // 16 KiB
    static constexpr int kStageB = kRowsB * BK * 4;
    static constexpr int kCopies = X3 ? 2 : 1;                    // X3: the raw tile and its small part
    static constexpr int kStages = X3 ? ((kStageA + kStageB) == 49152 ? 2 : 3) : ((kStageA + kStageB) == 49152 ? 4 : 6);
    static constexpr int kStore = 4 * 2 * 4096;                   // per epilogue warp: two 32x32 fp32 staging tiles
    static constexpr int kSmem = kStages * kCopies * (kStageA + kStageB) + kStore + 1024 /*align*/ + 256 /*barriers*/;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kThreads = X3 ? kGemmThreadsX3 : kGemmThreads;
};

// small part of x for the 3xTF32 products: x minus its upper 19 bits, with half a TF32 unit added to
// the bits so that the tensor core's truncation of it rounds to nearest
__device__ __forceinline__ float tf32_small(float v) {
    float s = v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    return __uint_as_float(__float_as_uint(s) + 0x1000u);
}

// Work unit -> tile coordinates.  Units that run at the same time should share the operand that
// does not fit in L2: walking along M re-reads the A rows once per N tile, walking along N
// re-reads B once per M tile; the host picks the order whose re-read operand stays in L2.
__device__ __forceinline__ void tile_of(const TcArgs &g, int tile, int &tm, int &tn) {
    if (g.n_fastest) { tm = tile / g.tiles_n; tn = tile - tm * g.tiles_n; }
    else { tn = tile / g.tiles_m; tm = tile - tn * g.tiles_m; }
}

// The n-th work unit of a walker.  Split-K proper deals (tile, split) units round robin, so the pieces of a tile run
// on different CTAs and meet in a buffer of partials.  Chained: a walker takes whole tiles and runs their pieces
// one after the other; each piece has its own accumulator chain and the pieces meet in C itself.
__device__ __forceinline__ bool unit_at(const TcArgs &g, int n, int walker, int walkers, int num_tiles, int &tile, int &split) {
    if (g.chained) {
        tile = walker + (n / g.splits) * walkers;
        split = n % g.splits;
        return tile < num_tiles;
    }
    const int u = walker + n * walkers;
    tile = u / g.splits; split = u - tile * g.splits;
    return u < num_tiles * g.splits;
}

template <int BN, bool PAIR, int X3>
__global__ void __launch_bounds__(X3 ? kGemmThreadsX3 : kGemmThreads, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, TcArgs g) {
    using Cfg = TcCfg<BN, PAIR, X3>;
    constexpr int kStrideA = Cfg::kCopies * Cfg::kStageA, kStrideB = Cfg::kCopies * Cfg::kStageB;   // bytes per stage
    static_assert(!PAIR || BN == 256, "a CTA pair computes 256 x 256 tiles");
    // PAIR: the grid is made of clusters of two CTAs; a pair walks the work units together,
    // rank 0 (the leader) issues the MMAs for both.
    const uint32_t rank = PAIR ? cluster_rank() : 0u;
    const int walker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int walkers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    constexpr int kTileM = PAIR ? 2 * BM : BM;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sA = smem, *sB = smem + Cfg::kStages * kStrideA;
    uint8_t *sC = smem + Cfg::kStages * (kStrideA + kStrideB);
    uint64_t *bars = (uint64_t *)(sC + Cfg::kStore);
    uint64_t *full = bars, *empty = bars + Cfg::kStages, *acc_full = bars + 2 * Cfg::kStages, *acc_empty = acc_full + 2;
    uint64_t *conv = acc_empty + 2;        // X3: stage split, counted on the leader for both CTAs of a pair
    uint32_t *tmem_slot = (uint32_t *)(conv + Cfg::kStages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&conv[s], PAIR ? 2 * kSplitWarps : kSplitWarps); }
        for (int a = 0; a < 2; a++) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], PAIR ? 8 : 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {     // one warp of each CTA of the pair, collectively: the same columns in both CTAs
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Cfg::kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Cfg::kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();      // the peer's barriers are initialised before anything is sent to them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_tiles = g.tiles_m * g.tiles_n;
    const int num_kb_total = (g.K + BK - 1) / BK;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            int tile, split;
            for (int n = 0; ok && unit_at(g, n, walker, walkers, num_tiles, tile, split); n++) {
                int tm, tn;
                tile_of(g, tile, tm, tn);
                int m0 = tm * kTileM + (int)rank * BM;
                int n0 = tn * BN + (int)rank * Cfg::kRowsB;      // a pair splits B's columns between its CTAs
                int kb0 = split * g.kb_per_split, kb1 = min(kb0 + g.kb_per_split, num_kb_total);
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(&empty[stage], phase ^ 1)) { atomicCAS(&g_gemm_error, 0, 0x100 | stage); ok = false; break; }
                    // both CTAs' bytes are counted on the leader's barrier, which alone is armed; X3: every CTA
                    // counts its own bytes on its own barrier, because its own warps split the tiles next
                    constexpr bool kToLeader = PAIR && !X3;
                    if (X3) mbar_expect_tx(&full[stage], Cfg::kStageA + Cfg::kStageB);
                    else if (rank == 0) mbar_expect_tx(&full[stage], (PAIR ? 2 : 1) * (Cfg::kStageA + Cfg::kStageB));
                    const uint32_t bar = kToLeader ? map_to_rank(smem_u32(&full[stage]), 0) : smem_u32(&full[stage]);
                    auto load = [&](void *dst, const CUtensorMap *map, int x, int y) {
                        if (kToLeader) tma_load_2d_pair(dst, map, x, y, bar);
                        else tma_load_2d(dst, map, x, y, &full[stage]);
                    };
                    uint8_t *a = sA + stage * kStrideA, *b = sB + stage * kStrideB;
                    int k = kb * BK;
                    auto load3 = [&](void *dst, const CUtensorMap *map, int y, int z) {
                        if (kToLeader) tma_load_3d_pair(dst, map, 0, y, z, bar);
                        else tma_load_3d(dst, map, 0, y, z, &full[stage]);
                    };
                    if (g.a_kmajor) load(a, &tmA, k, m0);                                          // box {32 k, 128 rows}
                    else if (g.a_chunked) load3(a, &tmA, k, m0 >> 5);                              // box {32 m, 32 k, 4 chunks of m}
                    else for (int c = 0; c < BM / 32; c++) load(a + c * 4096, &tmA, m0 + c * 32, k);   // box {32 m, 32 k}
                    if (g.b_kmajor) load(b, &tmB, k, n0);
                    else if (g.b_chunked) load3(b, &tmB, k, n0 >> 5);
                    else for (int c = 0; c < Cfg::kRowsB / 32; c++) load(b + c * 4096, &tmB, n0 + c * 32, k);
                    if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // instruction descriptor: D=f32, A=B=tf32, major bits, N>>3, M>>4 (M = 256 across a pair)
            uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((g.a_kmajor ? 0u : 1u) << 15) | ((g.b_kmajor ? 0u : 1u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
            // Descriptors are built once; inside the loops only the 16-byte-granular address field
            // moves (by stage and by K=8 step), so issuing an MMA costs a few integer adds.  The
            // tensor core needs 128 cycles per instruction at N = 256 and the issuing thread has to
            // stay well under that.
            const uint32_t a_lbo = g.a_kmajor ? 16 : 4096, b_lbo = g.b_kmajor ? 16 : 4096;
            const uint32_t a_sbo = g.a_kmajor ? 1024 : 512, b_sbo = g.b_kmajor ? 1024 : 512;
            const uint32_t a_lt = g.a_kmajor ? 2 : 1, b_lt = g.b_kmajor ? 2 : 1;
            const uint64_t a_desc0 = make_smem_desc(smem_u32(sA), a_lbo, a_sbo, a_lt), b_desc0 = make_smem_desc(smem_u32(sB), b_lbo, b_sbo, b_lt);
            const uint64_t a_adv = (g.a_kmajor ? UMMA_K * 4 : 1024) >> 4, b_adv = (g.b_kmajor ? UMMA_K * 4 : 1024) >> 4;   // per K=8 step
            int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0;
            bool ok = true;
            int tile, split;
            for (int n = 0; ok && unit_at(g, n, walker, walkers, num_tiles, tile, split); n++) {
                int kb0 = split * g.kb_per_split, kb1 = min(kb0 + g.kb_per_split, num_kb_total);
                if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) { atomicCAS(&g_gemm_error, 0, 0x200 | acc); break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                const uint32_t tmem_small = X3 == 2 ? tmem_base + (uint32_t)BN : tmem_d;      // X3 == 2: acc stays 0
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!(X3 ? mbar_wait_cluster(&conv[stage], phase) : mbar_wait(&full[stage], phase))) {
                        atomicCAS(&g_gemm_error, 0, 0x300 | stage); ok = false; break;
                    }
                    tc_fence_after();
                    const uint64_t a_st = a_desc0 + (uint64_t)(stage * (kStrideA >> 4)), b_st = b_desc0 + (uint64_t)(stage * (kStrideB >> 4));
                    auto mma = [&](uint32_t d, uint64_t ad, uint64_t bd, uint32_t accum) {
                        if (PAIR) tc_mma_tf32_pair(d, ad, bd, idesc, accum);
                        else tc_mma_tf32(d, ad, bd, idesc, accum);
                    };
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        const uint64_t ad = a_st + k * a_adv, bd = b_st + k * b_adv;
                        const uint32_t first = (kb > kb0 || k > 0) ? 1u : 0u;
                        if (X3) {       // the two small terms first, then big x big
                            const uint64_t as = ad + (Cfg::kStageA >> 4), bs = bd + (Cfg::kStageB >> 4);
                            mma(tmem_small, as, bd, first);
                            mma(tmem_small, ad, bs, 1u);
                            mma(tmem_d, ad, bd, X3 == 2 ? first : 1u);
                        } else {
                            mma(tmem_d, ad, bd, first);
                        }
                    }
                    // frees the stage (in both CTAs of a pair) when these MMAs have read it
                    if (PAIR) tc_commit_pair(&empty[stage], 3); else tc_commit(&empty[stage]);
                    if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (PAIR) tc_commit_pair(&acc_full[acc], 3); else tc_commit(&acc_full[acc]);      // accumulator complete
                if (X3 == 2) acc_phase ^= 1;
                else if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else if (X3 && warp >= 6) {
        // split warps 6..13: small = x - trunc(x) of the stage that has just landed, element by element
        // (the layout of the tile does not matter), then tell the leader's MMA thread
        const int t = (int)threadIdx.x - kGemmThreads;
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        int tile, split;
        for (int n = 0; ok && unit_at(g, n, walker, walkers, num_tiles, tile, split); n++) {
            int kb0 = split * g.kb_per_split, kb1 = min(kb0 + g.kb_per_split, num_kb_total);
            for (int kb = kb0; kb < kb1; kb++) {
                if (!mbar_wait(&full[stage], phase)) { if (lane == 0) atomicCAS(&g_gemm_error, 0, 0x500 | stage); ok = false; break; }
                const float4 *ra = reinterpret_cast<const float4 *>(sA + stage * kStrideA);
                float4 *wa = reinterpret_cast<float4 *>(sA + stage * kStrideA + Cfg::kStageA);
#pragma unroll
                for (int i = 0; i < Cfg::kStageA / 16 / (kSplitWarps * 32); i++) {
                    const float4 v = ra[t + i * kSplitWarps * 32];
                    wa[t + i * kSplitWarps * 32] = make_float4(tf32_small(v.x), tf32_small(v.y), tf32_small(v.z), tf32_small(v.w));
                }
                const float4 *rb = reinterpret_cast<const float4 *>(sB + stage * kStrideB);
                float4 *wb = reinterpret_cast<float4 *>(sB + stage * kStrideB + Cfg::kStageB);
#pragma unroll
                for (int i = 0; i < Cfg::kStageB / 16 / (kSplitWarps * 32); i++) {
                    const float4 v = rb[t + i * kSplitWarps * 32];
                    wb[t + i * kSplitWarps * 32] = make_float4(tf32_small(v.x), tf32_small(v.y), tf32_small(v.z), tf32_small(v.w));
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(map_to_rank(smem_u32(&conv[stage]), 0));
                    else mbar_arrive(&conv[stage]);
                }
                if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
            }
        }
    } else {
        // epilogue warps 2..5: TMEM lanes 32*(warp%4) .. +31  <->  tile rows
        const int q = warp & 3;
        int acc = 0; uint32_t acc_phase = 0;
        uint32_t chunk = 0;
        int tile, split;
        for (int n = 0; unit_at(g, n, walker, walkers, num_tiles, tile, split); n++) {
            int tm, tn;
            tile_of(g, tile, tm, tn);
            int m0 = tm * kTileM + (int)rank * BM, n0 = tn * BN;
            int kb0 = split * g.kb_per_split;
            bool has_k = kb0 < num_kb_total;
            if (!mbar_wait(&acc_full[acc], acc_phase)) { if (lane == 0) atomicCAS(&g_gemm_error, 0, 0x400 | acc); break; }
            tc_fence_after();
            const int row0 = m0 + q * 32;
            const bool use_bias = g.bias != nullptr && split == 0;
            // chained: the first piece of a tile is stored (or added to the C that was there), every later piece is
            // added by the copy engine in L2, after this warp's earlier writes to the same rows have completed
            const bool add_to_c = g.chained ? (g.accumulate != 0 || split > 0) : (g.accumulate != 0);
            const int plane = g.chained ? 0 : split;
            if (g.chained && split > 0) {
                if (lane == 0) bulk_wait<0>();
                __syncwarp();
            }
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), r);
                const int col0 = n0 + c0;
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; j++) v[j] = has_k ? __uint_as_float(r[j]) : 0.f;
                if (X3 == 2 && has_k) {      // the small terms' accumulator
                    tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(BN + c0), r);
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] += __uint_as_float(r[j]);
                }
                if (use_bias) {
                    if (col0 + 32 <= g.N) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 bb = __ldg(reinterpret_cast<const float4 *>(g.bias + col0 + j));
                            v[j] += bb.x; v[j + 1] += bb.y; v[j + 2] += bb.z; v[j + 3] += bb.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) if (col0 + j < g.N) v[j] += g.bias[col0 + j];
                    }
                }
                if (g.resid && row0 + lane < g.M) {
                    const float *rr = g.resid + (int64_t)(row0 + lane) * g.resid_ld + col0;
                    if (col0 + 32 <= g.N) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 x = *reinterpret_cast<const float4 *>(rr + j);
                            v[j] += x.x; v[j + 1] += x.y; v[j + 2] += x.z; v[j + 3] += x.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) if (col0 + j < g.N) v[j] += rr[j];
                    }
                }
                if (g.rope_c && col0 < g.rope_cols) {         // rope_cols, rope_d are multiples of 32: the chunk lies in one head
                    const int pos = (row0 + lane) % g.rope_N, hc = col0 % g.rope_d;
                    const float4 *c4 = reinterpret_cast<const float4 *>(g.rope_c + (int64_t)pos * (g.rope_d >> 1) + (hc >> 1));
                    const float4 *s4 = reinterpret_cast<const float4 *>(g.rope_s + (int64_t)pos * (g.rope_d >> 1) + (hc >> 1));
#pragma unroll
                    for (int q4 = 0; q4 < 4; q4++) {
                        const float4 c = __ldg(c4 + q4), sn = __ldg(s4 + q4);
                        const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int j = 8 * q4 + 2 * e;
                            float ox, oy;
                            rope_fwd_pair(v[j], v[j + 1], cc[e], ss[e], ox, oy);
                            v[j] = ox; v[j + 1] = oy;
                        }
                    }
                }
                // the staging tile about to be written was handed to the copy engine two chunks ago
                if (lane == 0) bulk_wait_read<1>();
                __syncwarp();
                uint8_t *buf = sC + (q * 2 + (chunk & 1)) * 4096;
#pragma unroll
                for (int j = 0; j < 8; j++)       // 128-byte swizzle: 16-byte piece j of row `lane` lands at piece j ^ (lane & 7)
                    *reinterpret_cast<float4 *>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    if (col0 < g.N && row0 < g.M) tma_store_3d(&tmC, buf, col0, row0, plane, add_to_c);
                    bulk_commit();
                }
                chunk++;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {       // the leader's MMA warp waits for the epilogue warps of both CTAs
                if (PAIR) mbar_arrive_cluster(map_to_rank(smem_u32(&acc_empty[acc]), 0));
                else mbar_arrive(&acc_empty[acc]);
            }
            if (X3 == 2) acc_phase ^= 1;
            else if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        if (lane == 0) bulk_wait<0>();      // the staging tiles must outlive the copies that read them
    }
    // teardown: everyone meets here, also after a wait that gave up
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();      // neither CTA leaves while the other may still touch its shared memory or TMEM
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols) : "memory");
    }
}

// C (=|+=) sum_s part[s] (+ bias), fixed order
__global__ void splitk_reduce_kernel(float *__restrict__ C, int64_t ldc, const float *__restrict__ part, int64_t part_ld, int splits,
                                     int M, int N, const float *__restrict__ bias, int accumulate) {
    int64_t total = (int64_t)M * N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int m = (int)(i / N), n = (int)(i - (int64_t)m * N);
        float s = 0.f;
        for (int k = 0; k < splits; k++) s += part[((int64_t)k * M + m) * part_ld + n];
        if (bias) s += bias[n];
        float *c = C + (int64_t)m * ldc + n;
        *c = accumulate ? *c + s : s;
    }
}

// The same with four columns per thread (N, ldc multiples of 4; all pointers 16-byte aligned).
__global__ void splitk_reduce_v4_kernel(float *__restrict__ C, int64_t ldc, const float4 *__restrict__ part, int splits,
                                        int M, int N4, const float4 *__restrict__ bias, int accumulate) {
    const int64_t total = (int64_t)M * N4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / N4), n = (int)(i - (int64_t)m * N4);
        float4 s = part[i];
        for (int k = 1; k < splits; k++) {
            const float4 v = part[(int64_t)k * total + i];
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        if (bias) { const float4 b = bias[n]; s.x += b.x; s.y += b.y; s.z += b.z; s.w += b.w; }
        float4 *c = reinterpret_cast<float4 *>(C + (int64_t)m * ldc) + n;
        if (accumulate) { const float4 o = *c; s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w; }
        *c = s;
    }
}

// big = x with the 13 low mantissa bits cleared (exactly a TF32 value), small = x - big
__global__ void tf32_split_kernel(const float *__restrict__ x, float *__restrict__ big, float *__restrict__ small,
                                  int64_t rows, int64_t cols, int64_t pitch) {
    int64_t total = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / cols, c = i - r * cols;
        float v = x[r * pitch + c];
        float b = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
        big[i] = b; small[i] = v - b;
    }
}

// ---- host side ------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        CUDA_OK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        DNN_CHECK(p && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available in this driver");
        fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A tensor map is a pure function of its arguments, and a training loop asks for the same few hundred
// over and over (bump pools hand out the same addresses every step), so the encoded maps are kept in
// a small direct-mapped table per host thread; a miss costs one driver call, as before.
struct MapKey {
    const void *base; int64_t a, b, c; int32_t d, kind;
    bool operator==(const MapKey &o) const { return base == o.base && a == o.a && b == o.b && c == o.c && d == o.d && kind == o.kind; }
};
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
static constexpr int kMapSlots = 1024;
template <typename Build> static CUtensorMap cached_map(const MapKey &k, Build build) {
    static thread_local MapSlot *table = nullptr;
    if (!table) table = (MapSlot *)calloc(kMapSlots, sizeof(MapSlot));
    uint64_t h = (uint64_t)(uintptr_t)k.base * 0x9E3779B97F4A7C15ull;
    h ^= ((uint64_t)k.a + 0x7F4A7C15ull) * 0xBF58476D1CE4E5B9ull; h ^= h >> 29;
    h ^= ((uint64_t)k.b * 31 + (uint64_t)k.c * 131 + (uint64_t)k.d * 8191 + (uint64_t)k.kind) * 0x94D049BB133111EBull; h ^= h >> 32;
    MapSlot &s = table[h % kMapSlots];
    if (s.used && s.key == k) return s.map;
    s.map = build(); s.key = k; s.used = true;
    return s.map;
}

// 2-D map over a matrix whose contiguous dimension has `inner` elements and whose
// other dimension has `outer` elements `pitch` floats apart; box = {32, box_outer}.
// `raw`: the words reach shared memory unrounded (the 3xTF32 kernel splits them there).
static CUtensorMap make_map(const float *base, int64_t inner, int64_t outer, int64_t pitch, int box_outer, bool mn_major, bool raw = false) {
  return cached_map(MapKey{base, inner, outer, pitch, box_outer, (mn_major ? 1 : 0) | (raw ? 8 : 0)}, [&] {
    CUtensorMap m;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * 4};
    cuuint32_t box[2] = {32, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    // TFLOAT32: the copy engine rounds fp32 to TF32 (nearest even) on the way into shared
    // memory; the tensor core on its own would truncate, which biases every product low.
    CUresult r = encode_tiled()(&m, raw ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 2, (void *)base, dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "dnn_b200: cuTensorMapEncodeTiled failed (%d)\n", (int)r); abort(); }
    return m;
  });
}

// 3-D map {N, M, splits} over the output (or over the split-K partials); box = one 32 x 32 staging tile.
static CUtensorMap make_out_map(float *base, int64_t N, int64_t M, int64_t ldc, int splits) {
  return cached_map(MapKey{base, N, M, ldc, splits, 2}, [&] {
    CUtensorMap m;
    cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)splits};
    cuuint64_t strides[2] = {(cuuint64_t)ldc * 4, (cuuint64_t)M * (cuuint64_t)ldc * 4};
    cuuint32_t box[3] = {32, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void *)base, dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "dnn_b200: cuTensorMapEncodeTiled (output) failed (%d)\n", (int)r); abort(); }
    return m;
  });
}

// MN-major operand whose contiguous extent is a multiple of 32: 3-D map {32, outer, inner/32} with
// box {32, 32, chunks}, which lands in shared memory as [chunk][k row][32 floats] -- the layout the
// per-chunk 2-D copies produce -- with one copy instead of `chunks`.  (The split dimension cannot be
// clipped by the copy engine, hence the multiple-of-32 condition; a chunk index beyond the last
// chunk is out of bounds in the third dimension and reads zeros.)
static CUtensorMap make_chunked_map(const float *base, int64_t inner, int64_t outer, int64_t pitch, int chunks, bool raw = false) {
  return cached_map(MapKey{base, inner, outer, pitch, chunks, 3 | (raw ? 8 : 0)}, [&] {
    CUtensorMap m;
    cuuint64_t dims[3] = {32, (cuuint64_t)outer, (cuuint64_t)(inner / 32)};
    cuuint64_t strides[2] = {(cuuint64_t)pitch * 4, 128};
    cuuint32_t box[3] = {32, 32, (cuuint32_t)chunks};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode_tiled()(&m, raw ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 3, (void *)base, dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "dnn_b200: cuTensorMapEncodeTiled (chunked) failed (%d)\n", (int)r); abort(); }
    return m;
  });
}

static bool operand_ok(const float *p, int64_t rs, int64_t cs, int64_t rows, int64_t cols) {
    if (!aligned16(p)) return false;
    if (cs == 1) return rs % 4 == 0 && rs >= cols;     // contiguous along the column index
    if (rs == 1) return cs % 4 == 0 && cs >= rows;     // contiguous along the row index
    return false;
}

// Normalised problem: row-major C.  Returns false when the layout cannot be fed to TMA.
static bool normalise(const GemmArgs &in, GemmArgs &g) {
    g = in;
    if (g.batch != 1 || g.M <= 0 || g.N <= 0 || g.K <= 0) return false;
    if (g.c_cs != 1) {
        if (g.c_rs != 1 || g.bias) return false;
        // C^T = B^T A^T : swap the operands so that the output is row-major
        GemmArgs t = g;
        t.A = g.B; t.a_rs = g.b_cs; t.a_cs = g.b_rs;
        t.B = g.A; t.b_rs = g.a_cs; t.b_cs = g.a_rs;
        t.M = g.N; t.N = g.M; t.c_rs = g.c_cs; t.c_cs = 1;
        g = t;
    }
    if (!aligned16(g.C) || g.c_rs % 4 != 0 || g.c_rs < g.N) return false;
    if (g.bias && !aligned16(g.bias)) return false;
    if (!operand_ok(g.A, g.a_rs, g.a_cs, g.M, g.K)) return false;
    if (!operand_ok(g.B, g.b_rs, g.b_cs, g.K, g.N)) return false;
    return true;
}

bool gemm_tc_supported(const GemmArgs &in) {
    GemmArgs g;
    if (!normalise(in, g)) return false;
    // tiny problems are launch-bound either way; keep them on the exact kernel
    return (int64_t)g.M * g.N * g.K >= (int64_t)64 * 64 * 32;
}

struct ResidEpilogue { const float *r; int64_t ld; bool pending, honoured; };
static thread_local ResidEpilogue g_resid = {nullptr, 0, false, false};
void gemm_residual_request(const float *resid, int64_t ld) { g_resid.r = resid; g_resid.ld = ld; g_resid.pending = true; g_resid.honoured = false; }
// For a kernel outside this file that can add the residual itself: hands the pending request over and marks it honoured.
bool gemm_residual_claim(const float **resid, int64_t *ld) {
    if (!g_resid.pending) return false;
    *resid = g_resid.r; *ld = g_resid.ld;
    g_resid.pending = false; g_resid.honoured = true;
    return true;
}
bool gemm_residual_take() {
    bool h = g_resid.honoured;
    g_resid.pending = false; g_resid.honoured = false;
    return h;
}

struct RopeEpilogue { const float *fc, *fs; int N, d, cols; bool pending, honoured; };
static thread_local RopeEpilogue g_rope = {nullptr, nullptr, 0, 0, 0, false, false};
void gemm_rope_epilogue_request(const float *fc, const float *fs, int N, int d, int cols) {
    g_rope.fc = fc; g_rope.fs = fs; g_rope.N = N; g_rope.d = d; g_rope.cols = cols; g_rope.pending = true; g_rope.honoured = false;
}
bool gemm_rope_epilogue_take() {
    bool h = g_rope.honoured;
    g_rope.pending = false; g_rope.honoured = false;
    return h;
}

static float *g_scratch = nullptr;
static size_t g_scratch_cap = 0;
static float *scratch(size_t bytes) {
    if (bytes > g_scratch_cap) {
        CUDA_OK(cudaStreamSynchronize(stream()));
        if (g_scratch) CUDA_OK(cudaFree(g_scratch));
        g_scratch_cap = bytes + (bytes >> 2);
        CUDA_OK(cudaMalloc((void **)&g_scratch, g_scratch_cap));
    }
    return g_scratch;
}

// Split-K factor.  Cost model in units of one k-block of one tile: every wave of work units
// pays its k-blocks plus a fixed fill-and-drain share, and every split pays for writing and
// re-reading one partial copy of the output.
static int choose_splits(int tiles, int slots, int num_kb, int64_t M, int64_t N) {
    if (tiles >= slots || num_kb < 32) return 1;
    const double drain = 8.0;
    const double partial = (double)M * N * 8.0 / 6.0e12 / 0.5e-6;      // ~0.5 us per k-block, ~6 TB/s
    int best = 1; double best_cost = 1e30;
    int max_splits = num_kb / 8 < 32 ? num_kb / 8 : 32;
    for (int s = 1; s <= max_splits; s++) {
        int kbs = (num_kb + s - 1) / s;
        int eff = (num_kb + kbs - 1) / kbs;                            // splits that really get work
        if (eff != s) continue;
        int waves = (tiles * s + slots - 1) / slots;
        double cost = waves * (kbs + drain) + (s > 1 ? partial * s : 0.0);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
    }
    return best;
}

// Longest accumulation chain, in k-blocks of 32, that one work unit may run inside the tensor core (0: no limit).
// The tensor core adds into its fp32 accumulator with truncation, so a chain of K products is biased low by about
// 2.4e-9 x K relative (measured: 1.6e-6 at K = 768, 7.3e-6 at K = 3072).  That is invisible next to TF32 rounding,
// but it is the error floor of the 3xTF32 mode, whose main product therefore runs as split-K pieces of bounded
// length that splitk_reduce adds in fp32 with round-to-nearest, in fixed order.
static thread_local int g_chain_kb = 0;

template <int BN, bool PAIR, int X3>
static void launch_tc(const GemmArgs &g, bool a_kmajor, bool b_kmajor) {
    using Cfg = TcCfg<BN, PAIR, X3>;
    constexpr int kTileM = PAIR ? 2 * BM : BM;
    static bool once = false;
    if (!once) {
        CUDA_OK(cudaFuncSetAttribute(gemm_tf32_kernel<BN, PAIR, X3>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
        once = true;
    }
    // A(m,k): K-major -> matrix [M rows][K contiguous]; MN-major -> [K rows][M contiguous]
    const bool a_chunked = !a_kmajor && g.M % 32 == 0, b_chunked = !b_kmajor && g.N % 32 == 0;
    CUtensorMap tmA = a_kmajor ? make_map(g.A, g.K, g.M, g.a_rs, BM, false, X3 != 0)
                    : a_chunked ? make_chunked_map(g.A, g.M, g.K, g.a_cs, BM / 32, X3 != 0) : make_map(g.A, g.M, g.K, g.a_cs, 32, true, X3 != 0);
    CUtensorMap tmB = b_kmajor ? make_map(g.B, g.K, g.N, g.b_cs, Cfg::kRowsB, false, X3 != 0)
                    : b_chunked ? make_chunked_map(g.B, g.N, g.K, g.b_rs, Cfg::kRowsB / 32, X3 != 0) : make_map(g.B, g.N, g.K, g.b_rs, 32, true, X3 != 0);
    TcArgs t;
    t.a_chunked = a_chunked ? 1 : 0; t.b_chunked = b_chunked ? 1 : 0;
    t.M = g.M; t.N = g.N; t.K = g.K; t.a_kmajor = a_kmajor; t.b_kmajor = b_kmajor;
    t.tiles_m = (g.M + kTileM - 1) / kTileM; t.tiles_n = (g.N + BN - 1) / BN;
    int tiles = t.tiles_m * t.tiles_n;
    int num_kb = (g.K + BK - 1) / BK;
    // Tile order.  Walking along M streams all of A once per N tile; that is free while A stays
    // in L2 (about half of the 126 MB is a safe share) and otherwise costs tiles_n passes over
    // A from HBM.  When A is too large and B is not, walk along N instead.
    const double a_bytes = 4.0 * g.M * g.K, b_bytes = 4.0 * g.K * g.N, l2_share = 48e6;
    t.n_fastest = (t.tiles_n > 1 && a_bytes > l2_share && b_bytes <= l2_share) ? 1 : 0;
    const int slots = PAIR ? kNumSMs / 2 : kNumSMs;      // work units in flight: one per CTA, or per CTA pair
    // split-K when the output has too few tiles to fill the SMs and K is long
    int splits = choose_splits(tiles, slots, num_kb, g.M, g.N);
    bool chained = false;
    if (g_chain_kb > 0 && (num_kb + splits - 1) / splits > g_chain_kb) {
        // Pieces only because of the chain limit, with enough tiles to fill the SMs anyway: a tile's pieces run back to
        // back on its CTA and add into C through L2 (fixed order, so still deterministic) instead of meeting in a
        // buffer of partials that another kernel sums.
        chained = splits == 1;
        splits = (num_kb + g_chain_kb - 1) / g_chain_kb;
    }
    t.kb_per_split = (num_kb + splits - 1) / splits;
    splits = (num_kb + t.kb_per_split - 1) / t.kb_per_split;
    t.splits = splits;
    t.chained = chained ? 1 : 0;
    t.resid = nullptr; t.resid_ld = 0;
    if (g_resid.pending && splits == 1 && !g.accumulate && aligned16(g_resid.r) && g_resid.ld % 4 == 0) {
        t.resid = g_resid.r; t.resid_ld = g_resid.ld;
        g_resid.pending = false; g_resid.honoured = true;
    }
    t.rope_c = t.rope_s = nullptr; t.rope_N = t.rope_d = t.rope_cols = 0;
    if (g_rope.pending && splits == 1 && !g.accumulate && g.M % g_rope.N == 0 && g_rope.cols <= g.N &&
        g_rope.cols % 32 == 0 && g_rope.d % 32 == 0 && (((uintptr_t)g_rope.fc | (uintptr_t)g_rope.fs) & 15) == 0) {
        t.rope_c = g_rope.fc; t.rope_s = g_rope.fs; t.rope_N = g_rope.N; t.rope_d = g_rope.d; t.rope_cols = g_rope.cols;
        g_rope.pending = false; g_rope.honoured = true;
    }
    if (splits == 1 || chained) { t.C = g.C; t.ldc = g.c_rs; t.bias = g.bias; t.accumulate = g.accumulate ? 1 : 0; }
    else { t.ldc = (g.N + 3) & ~(int64_t)3;      // rows of the partials padded to 16 bytes: the copy engine's stride rule
           t.C = scratch((size_t)splits * g.M * t.ldc * 4); t.bias = nullptr; t.accumulate = 0; }
    int units = chained ? tiles : tiles * splits;
    int walkers = units < slots ? units : slots;
    CUtensorMap tmC = make_out_map(t.C, g.N, g.M, t.ldc, chained ? 1 : splits);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(PAIR ? 2 * walkers : walkers);
    cfg.blockDim = dim3(Cfg::kThreads);
    cfg.dynamicSmemBytes = Cfg::kSmem;
    cfg.stream = stream();
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = PAIR ? 2 : 1; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    prof_begin(0);
    CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_tf32_kernel<BN, PAIR, X3>, tmA, tmB, tmC, t));
    prof_work(2.0 * g.M * g.N * g.K);
    LAUNCHED(X3 ? "gemm_3xtf32_kernel" : "gemm_tf32_kernel");
    prof_end(0, 2.0 * g.M * g.N * g.K);
    if (splits > 1 && !chained) {
        const bool v4 = g.N % 4 == 0 && g.c_rs % 4 == 0 && ((uintptr_t)g.C & 15) == 0 && ((uintptr_t)t.C & 15) == 0 &&
                        (!g.bias || ((uintptr_t)g.bias & 15) == 0);
        if (v4)
            splitk_reduce_v4_kernel<<<grid_for((int64_t)g.M * (g.N / 4), 256), 256, 0, stream()>>>(
                g.C, g.c_rs, (const float4 *)t.C, splits, g.M, g.N / 4, (const float4 *)g.bias, g.accumulate ? 1 : 0);
        else
            splitk_reduce_kernel<<<grid_for((int64_t)g.M * g.N, 256), 256, 0, stream()>>>(g.C, g.c_rs, t.C, t.ldc, splits, g.M, g.N, g.bias,
                                                                                         g.accumulate ? 1 : 0);
        LAUNCHED("splitk_reduce_kernel");
    }
}

template <int X3> static void run_tc_as(const GemmArgs &g) {
    bool a_k = g.a_cs == 1, b_k = g.b_rs == 1;
    // a [M,1]-shaped or [1,K]-shaped operand satisfies both; prefer K-major
    static int pair_ok = -1;
    if (pair_ok < 0) { const char *e = getenv("DNN_CUDA_GEMM_PAIR"); pair_ok = (e && e[0] == '0') ? 0 : 1; }
    if (g.N > 128 && g.M > 128 && pair_ok) launch_tc<256, true, X3>(g, a_k, b_k);
    else if (g.N > 128) launch_tc<256, false, X3>(g, a_k, b_k);
    else launch_tc<128, false, X3>(g, a_k, b_k);
}
static void run_tc(const GemmArgs &g) { run_tc_as<0>(g); }

// Packed copies big/small of an operand, laid out row-major over its contiguous dimension.
static void split_operand(const float *p, int64_t rs, int64_t cs, int64_t rows, int64_t cols, float *big, float *small,
                          int64_t &nrs, int64_t &ncs) {
    int64_t outer, inner, pitch;
    if (cs == 1) { outer = rows; inner = cols; pitch = rs; nrs = cols; ncs = 1; }
    else { outer = cols; inner = rows; pitch = cs; nrs = 1; ncs = rows; }
    tf32_split_kernel<<<grid_for(outer * inner, 256), 256, 0, stream()>>>(p, big, small, outer, inner, pitch);
    LAUNCHED("tf32_split_kernel");
}

void gemm_tc(const GemmArgs &in, bool split3) {
    GemmArgs g;
    bool ok = normalise(in, g);
    DNN_CHECK(ok, "gemm_tc called with an unsupported layout");
    if (!split3) { run_tc(g); return; }
    static int chain = -1, fused = -1;
    if (chain < 0) { const char *e = getenv("DNN_CUDA_3X_CHAIN_KB"); chain = e ? atoi(e) : 16; }
    if (fused < 0) { const char *e = getenv("DNN_CUDA_3X_FUSED"); fused = e ? atoi(e) : 1; }
    const bool exact_mode = gemm_mode() == DNN_CUDA_GEMM_3XTF32;
    // One launch: raw tiles, split in shared memory, three products per K step.  Where the precision policy of the
    // TF32 mode chose 3xTF32, all three go into one accumulator: that removes the operand rounding, which is all
    // that is asked there.  In the exact mode the small terms get the second accumulator: with everything in one,
    // the tensor core truncates the large sum three times per K step instead of once, and through a deep model
    // that bias alone (measured 1.4e-5 .. 1.8e-5 on the gradients of the 64-image vision-LM step) exceeds 1e-5.
    // DNN_CUDA_3X_FUSED: 1 as described (default), 0 the three launches with operands split in global memory.
    if (fused) {
        g_chain_kb = exact_mode ? chain : 0;
        if (exact_mode) run_tc_as<2>(g); else run_tc_as<1>(g);     // a requested rotation or residual rides in the epilogue
        g_chain_kb = 0;
        return;
    }
    g_rope.pending = false;            // an epilogue rotation cannot be split over the three partial products
    g_resid.pending = false;           // nor can a residual be added three times
    // 3xTF32: x = big + small with big exactly TF32; A*B ~= Ab*Bb + Ab*Bs + As*Bb, fp32 accumulation.
    int64_t a_inner = g.a_cs == 1 ? g.K : g.M, a_outer = g.a_cs == 1 ? g.M : g.K;
    int64_t b_inner = g.b_cs == 1 ? g.N : g.K, b_outer = g.b_cs == 1 ? g.K : g.N;
    if (a_inner % 4 || b_inner % 4) { gemm_simt(in); return; }     // ragged inner extents: exact kernel
    size_t na = (size_t)a_inner * a_outer, nb = (size_t)b_inner * b_outer;
    static float *buf = nullptr; static size_t cap = 0;
    size_t need = (2 * na + 2 * nb) * 4 + 1024;
    if (need > cap) {
        CUDA_OK(cudaStreamSynchronize(stream()));
        if (buf) CUDA_OK(cudaFree(buf));
        cap = need + (need >> 2);
        CUDA_OK(cudaMalloc((void **)&buf, cap));
    }
    auto al = [](size_t n) { return (n + 63) & ~(size_t)63; };
    float *Ab = buf, *As = Ab + al(na), *Bb = As + al(na), *Bs = Bb + al(nb);
    int64_t ars, acs, brs, bcs;
    split_operand(g.A, g.a_rs, g.a_cs, g.M, g.K, Ab, As, ars, acs);
    split_operand(g.B, g.b_rs, g.b_cs, g.K, g.N, Bb, Bs, brs, bcs);
    GemmArgs t = g;
    t.a_rs = ars; t.a_cs = acs; t.b_rs = brs; t.b_cs = bcs;
    // smallest terms first so that they are not lost against a large accumulator
    t.A = As; t.B = Bb; t.bias = nullptr; run_tc(t);
    t.accumulate = true;
    t.A = Ab; t.B = Bs; run_tc(t);
    g_chain_kb = gemm_mode() == DNN_CUDA_GEMM_3XTF32 ? chain : 0;      // only the exact mode is after the last 1e-5
    t.A = Ab; t.B = Bb; t.bias = g.bias; run_tc(t);
    g_chain_kb = 0;
}

int gemm_tc_error() {
    int e = 0;
    cudaMemcpyFromSymbol(&e, g_gemm_error, sizeof e);
    return e;
}

}  // namespace dnnb
