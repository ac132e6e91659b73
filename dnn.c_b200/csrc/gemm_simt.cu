// fp32 FMA GEMM with arbitrary element strides on every operand.
//
// This is the exact-fp32 path (DNN_CUDA_GEMM_FP32) and the path for shapes the
// tensor-core kernel cannot take (row pitches that are not multiples of 16
// bytes, e.g. a [128,10] weight).  64x64 output tile, K step 16, 256 threads,
// 4x4 outputs per thread, operands staged through shared memory with the
// thread->element mapping chosen so that the unit-stride dimension of each
// operand is the one adjacent threads walk.
#include "common.cuh"
#include "device_utils.cuh"
#include <vector>

namespace dnnb {

constexpr int SBM = 64, SBN = 64, SBK = 16;

__global__ void __launch_bounds__(256)
gemm_simt_kernel(GemmArgs g) {
    __shared__ float As[SBK][SBM + 4];
    __shared__ float Bs[SBK][SBN + 4];
    int tid = threadIdx.x;
    int bz = blockIdx.z;
    const float *A = g.A + (int64_t)bz * g.a_bs;
    const float *B = g.B + (int64_t)bz * g.b_bs;
    float *C = g.C + (int64_t)bz * g.c_bs;
    int m0 = blockIdx.y * SBM, n0 = blockIdx.x * SBN;
    int ty = tid >> 4, tx = tid & 15;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    bool a_kfast = (g.a_cs == 1);      // K contiguous in A
    bool b_nfast = (g.b_cs == 1);      // N contiguous in B
    for (int k0 = 0; k0 < g.K; k0 += SBK) {
#pragma unroll
        for (int t = 0; t < 4; t++) {
            int idx = tid + t * 256;
            int m, k;
            if (a_kfast) { k = idx & (SBK - 1); m = idx >> 4; } else { m = idx & (SBM - 1); k = idx >> 6; }
            int gm = m0 + m, gk = k0 + k;
            As[k][m] = (gm < g.M && gk < g.K) ? A[(int64_t)gm * g.a_rs + (int64_t)gk * g.a_cs] : 0.f;
            int n;
            if (b_nfast) { n = idx & (SBN - 1); k = idx >> 6; } else { k = idx & (SBK - 1); n = idx >> 4; }
            int gn = n0 + n; gk = k0 + k;
            Bs[k][n] = (gn < g.N && gk < g.K) ? B[(int64_t)gk * g.b_rs + (int64_t)gn * g.b_cs] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < SBK; k++) {
            float4 av = *reinterpret_cast<const float4 *>(&As[k][ty * 4]);
            float4 bv = *reinterpret_cast<const float4 *>(&Bs[k][tx * 4]);
            float a[4] = {av.x, av.y, av.z, av.w}, b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int gm = m0 + ty * 4 + i;
        if (gm >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int gn = n0 + tx * 4 + j;
            if (gn >= g.N) continue;
            float v = acc[i][j];
            if (g.bias) v += g.bias[gn];
            float *c = C + (int64_t)gm * g.c_rs + (int64_t)gn * g.c_cs;
            *c = g.accumulate ? *c + v : v;
        }
    }
}

void gemm_simt(const GemmArgs &g) {
    if (g.M <= 0 || g.N <= 0 || g.batch <= 0) return;
    GemmArgs a = g;
    // gridDim.z is limited to 65535: chunk very large batch counts
    for (int b0 = 0; b0 < g.batch; b0 += 65535) {
        int nb = g.batch - b0 < 65535 ? g.batch - b0 : 65535;
        a.A = g.A + (int64_t)b0 * g.a_bs; a.B = g.B + (int64_t)b0 * g.b_bs; a.C = g.C + (int64_t)b0 * g.c_bs;
        dim3 grid((g.N + SBN - 1) / SBN, (g.M + SBM - 1) / SBM, nb);
        gemm_simt_kernel<<<grid, 256, 0, stream()>>>(a);
        LAUNCHED("gemm_simt_kernel");
    }
}

// ---- products with at most four output rows (a decoding step: one token per sequence) ----------------------
// Such a product reads its whole weight matrix to produce a few thousand numbers: it is bound by the bandwidth at which
// W streams in, and a 64- or 128-row tile kernel gives it a handful of CTAs (9 for a [1,768] x [768,2304] product).
// Two fp32 kernels that put every SM on the stream instead:
//   W with N contiguous ([K,N], a linear layer's weight): a thread owns four adjacent columns and walks a slice of K
//     (x staged in shared memory), the slices' partial sums are added in fixed order by gemv_reduce_kernel;
//   W with K contiguous ([N,K], the tied vocabulary projection): a warp owns one output column.
constexpr int kGemvRows = 4, kGemvSlice = 256, kGemvSplits = 128;

template <int MM>
__global__ void __launch_bounds__(128)
gemv_kn_kernel(const float *__restrict__ x, int64_t x_rs, const float *__restrict__ W, int64_t w_rs, float *__restrict__ part,
               int N, int K, int k_per_split, int vec, const float *__restrict__ W2 = nullptr, float *__restrict__ part2 = nullptr) {
    __shared__ float xs[MM][kGemvSlice];
    if (blockIdx.z == 1) { W = W2; part = part2; }            // a second product of the same x in the same launch
    const int k0 = blockIdx.y * k_per_split, k1 = min(K, k0 + k_per_split);
    for (int i = threadIdx.x; i < MM * (k1 - k0); i += blockDim.x) {
        int m = i / (k1 - k0), k = i - m * (k1 - k0);
        xs[m][k] = x[(int64_t)m * x_rs + k0 + k];
    }
    __syncthreads();
    const int n = (blockIdx.x * 128 + threadIdx.x) * 4;
    if (n >= N) return;
    float acc[MM][4];
#pragma unroll
    for (int m = 0; m < MM; m++) { acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f; }
    if (vec) {
#pragma unroll 8
        for (int k = k0; k < k1; k++) {
            const float4 w = __ldg(reinterpret_cast<const float4 *>(W + (int64_t)k * w_rs + n));
#pragma unroll
            for (int m = 0; m < MM; m++) {
                const float xv = xs[m][k - k0];
                acc[m][0] = fmaf(xv, w.x, acc[m][0]); acc[m][1] = fmaf(xv, w.y, acc[m][1]);
                acc[m][2] = fmaf(xv, w.z, acc[m][2]); acc[m][3] = fmaf(xv, w.w, acc[m][3]);
            }
        }
    } else {
        for (int k = k0; k < k1; k++) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (n + j >= N) break;
                const float w = W[(int64_t)k * w_rs + n + j];
#pragma unroll
                for (int m = 0; m < MM; m++) acc[m][j] = fmaf(xs[m][k - k0], w, acc[m][j]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MM; m++)
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (n + j < N) part[((int64_t)blockIdx.y * MM + m) * N + n + j] = acc[m][j];
}

// A warp per output: lane l adds slices l, l + 32, ... in order, then the 32 sums meet in a fixed shuffle tree, so the result
// does not depend on timing.  (One thread per output walked up to 128 dependent loads; eight lanes still a dozen.)
__global__ void gemv_reduce_kernel(float *__restrict__ C, int64_t c_rs, const float *__restrict__ part, int splits, int M, int N,
                                   const float *__restrict__ bias, int accumulate, const float *__restrict__ resid, int64_t resid_ld) {
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), l = threadIdx.x & 31;
    if (i >= M * N) return;                                        // whole warps leave together
    const int m = i / N, n = i - m * N;
    float s = 0.f;
    for (int k = l; k < splits; k += 32) s += part[((int64_t)k * M + m) * N + n];
    s = warp_sum(s);
    if (l != 0) return;
    if (bias) s += bias[n];
    if (resid) s += resid[(int64_t)m * resid_ld + n];          // x + (a W + b), the value a separate add would give
    float *c = C + (int64_t)m * c_rs + n;
    *c = accumulate ? *c + s : s;
}

// out = silu(g) * u for two products of the same x that are still in slices (gate and up projection of a SwiGLU layer):
// a warp per output adds the slices of both in the order of gemv_reduce_kernel and applies tensor_swiglu's arithmetic.
__global__ void gemv_reduce_swiglu_kernel(float *__restrict__ out, const float *__restrict__ pg, const float *__restrict__ pu, int splits,
                                          int M, int N, const float *__restrict__ bg, const float *__restrict__ bu) {
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), l = threadIdx.x & 31;
    if (i >= M * N) return;
    const int m = i / N, n = i - m * N;
    float g = 0.f, u = 0.f;
    for (int k = l; k < splits; k += 32) { g += pg[((int64_t)k * M + m) * N + n]; u += pu[((int64_t)k * M + m) * N + n]; }
    g = warp_sum(g); u = warp_sum(u);
    if (l != 0) return;
    if (bg) g += bg[n];
    if (bu) u += bu[n];
    out[(int64_t)m * N + n] = (g / (1.0f + expf(-g))) * u;
}

template <int MM>
__global__ void __launch_bounds__(256)
gemv_nk_kernel(const float *__restrict__ x, int64_t x_rs, const float *__restrict__ W, int64_t w_cs, float *__restrict__ C, int64_t c_rs,
               int N, int K, const float *__restrict__ bias, int accumulate, int vec) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    const float *w = W + (int64_t)n * w_cs;
    float acc[MM];
#pragma unroll
    for (int m = 0; m < MM; m++) acc[m] = 0.f;
    if (vec) {
        for (int k = lane * 4; k < K; k += 128) {
            const float4 wv = __ldg(reinterpret_cast<const float4 *>(w + k));
#pragma unroll
            for (int m = 0; m < MM; m++) {
                const float4 xv = *reinterpret_cast<const float4 *>(x + (int64_t)m * x_rs + k);
                acc[m] = fmaf(xv.x, wv.x, acc[m]); acc[m] = fmaf(xv.y, wv.y, acc[m]);
                acc[m] = fmaf(xv.z, wv.z, acc[m]); acc[m] = fmaf(xv.w, wv.w, acc[m]);
            }
        }
    } else {
        for (int k = lane; k < K; k += 32)
#pragma unroll
            for (int m = 0; m < MM; m++) acc[m] = fmaf(x[(int64_t)m * x_rs + k], w[k], acc[m]);
    }
#pragma unroll
    for (int m = 0; m < MM; m++) {
        float s = warp_sum(acc[m]);
        if (lane == 0) {
            if (bias) s += bias[n];
            float *c = C + (int64_t)m * c_rs + n;
            *c = accumulate ? *c + s : s;
        }
    }
}

// out[M,N] = silu(x Wg + bg) * (x Wu + bu) for at most four rows: both products in one launch, one reduction.
// Wg, Wu: [K,N] row-major with N a multiple of 4 and 16-byte aligned; returns false when the shapes do not qualify.
bool gemv_swiglu(const float *x, int64_t x_rs, int M, const float *Wg, const float *bg, const float *Wu, const float *bu,
                 int K, int N, float *out) {
    if (M < 1 || M > kGemvRows || K < 64 || N < 64 || N % 4 != 0 || ((reinterpret_cast<uintptr_t>(Wg) | reinterpret_cast<uintptr_t>(Wu)) & 15) != 0) return false;
    const int blocks_n = (N + 511) / 512;
    int splits = (2 * kNumSMs + blocks_n - 1) / blocks_n;          // the launch holds two products
    if (splits > kGemvSplits) splits = kGemvSplits;
    int kps = (K + splits - 1) / splits;
    if (kps > kGemvSlice) kps = kGemvSlice;
    if (kps < 8) kps = 8;
    splits = (K + kps - 1) / kps;
    static float *part = nullptr; static size_t cap = 0;
    const size_t one = (size_t)splits * M * N, need = 2 * one * sizeof(float);
    if (need > cap) {
        CUDA_OK(cudaStreamSynchronize(stream()));
        if (part) CUDA_OK(cudaFree(part));
        cap = need + (need >> 1);
        CUDA_OK(cudaMalloc((void **)&part, cap));
    }
    dim3 grid(blocks_n, splits, 2);
    switch (M) {
        case 1: gemv_kn_kernel<1><<<grid, 128, 0, stream()>>>(x, x_rs, Wg, N, part, N, K, kps, 1, Wu, part + one); break;
        case 2: gemv_kn_kernel<2><<<grid, 128, 0, stream()>>>(x, x_rs, Wg, N, part, N, K, kps, 1, Wu, part + one); break;
        case 3: gemv_kn_kernel<3><<<grid, 128, 0, stream()>>>(x, x_rs, Wg, N, part, N, K, kps, 1, Wu, part + one); break;
        default: gemv_kn_kernel<4><<<grid, 128, 0, stream()>>>(x, x_rs, Wg, N, part, N, K, kps, 1, Wu, part + one); break;
    }
    prof_work(8.0 * K * N);
    LAUNCHED("gemv_kn_kernel");
    gemv_reduce_swiglu_kernel<<<(M * N + 7) / 8, 256, 0, stream()>>>(out, part, part + one, splits, M, N, bg, bu);
    LAUNCHED("gemv_reduce_swiglu_kernel");
    return true;
}

static bool gemv_applicable(const GemmArgs &g) {
    return g.batch == 1 && g.M >= 1 && g.M <= kGemvRows && g.a_cs == 1 && g.c_cs == 1 && g.K >= 64 && g.N >= 64 &&
           (g.b_cs == 1 || g.b_rs == 1);
}

static void gemv(const GemmArgs &g) {
    if (g.b_cs == 1) {                                            // [K,N], N contiguous
        const int blocks_n = (g.N + 511) / 512;
        int splits = (4 * kNumSMs + blocks_n - 1) / blocks_n;
        if (splits > kGemvSplits) splits = kGemvSplits;
        int kps = (g.K + splits - 1) / splits;
        if (kps > kGemvSlice) kps = kGemvSlice;
        if (kps < 8) kps = 8;
        splits = (g.K + kps - 1) / kps;
        static float *part = nullptr; static size_t cap = 0;
        const size_t need = (size_t)splits * g.M * g.N * sizeof(float);
        if (need > cap) {
            CUDA_OK(cudaStreamSynchronize(stream()));
            if (part) CUDA_OK(cudaFree(part));
            cap = need + (need >> 1);
            CUDA_OK(cudaMalloc((void **)&part, cap));
        }
        const int vec = (g.N % 4 == 0 && g.b_rs % 4 == 0 && (reinterpret_cast<uintptr_t>(g.B) & 15) == 0) ? 1 : 0;
        dim3 grid(blocks_n, splits);
        switch (g.M) {
            case 1: gemv_kn_kernel<1><<<grid, 128, 0, stream()>>>(g.A, g.a_rs, g.B, g.b_rs, part, g.N, g.K, kps, vec); break;
            case 2: gemv_kn_kernel<2><<<grid, 128, 0, stream()>>>(g.A, g.a_rs, g.B, g.b_rs, part, g.N, g.K, kps, vec); break;
            case 3: gemv_kn_kernel<3><<<grid, 128, 0, stream()>>>(g.A, g.a_rs, g.B, g.b_rs, part, g.N, g.K, kps, vec); break;
            default: gemv_kn_kernel<4><<<grid, 128, 0, stream()>>>(g.A, g.a_rs, g.B, g.b_rs, part, g.N, g.K, kps, vec); break;
        }
        prof_work(4.0 * g.K * g.N);
        LAUNCHED("gemv_kn_kernel");
        const float *resid = nullptr; int64_t resid_ld = 0;
        if (!g.accumulate) gemm_residual_claim(&resid, &resid_ld);     // a pending request of matmul_add_residual
        gemv_reduce_kernel<<<(g.M * g.N + 7) / 8, 256, 0, stream()>>>(g.C, g.c_rs, part, splits, g.M, g.N, g.bias, g.accumulate ? 1 : 0,
                                                                              resid, resid_ld);
        LAUNCHED("gemv_reduce_kernel");
        return;
    }
    const int vec = (g.K % 4 == 0 && g.b_cs % 4 == 0 && g.a_rs % 4 == 0 && ((reinterpret_cast<uintptr_t>(g.B) | reinterpret_cast<uintptr_t>(g.A)) & 15) == 0) ? 1 : 0;
    const int grid = (g.N + 7) / 8;
    switch (g.M) {
        case 1: gemv_nk_kernel<1><<<grid, 256, 0, stream()>>>(g.A, g.a_rs, g.B, g.b_cs, g.C, g.c_rs, g.N, g.K, g.bias, g.accumulate ? 1 : 0, vec); break;
        case 2: gemv_nk_kernel<2><<<grid, 256, 0, stream()>>>(g.A, g.a_rs, g.B, g.b_cs, g.C, g.c_rs, g.N, g.K, g.bias, g.accumulate ? 1 : 0, vec); break;
        case 3: gemv_nk_kernel<3><<<grid, 256, 0, stream()>>>(g.A, g.a_rs, g.B, g.b_cs, g.C, g.c_rs, g.N, g.K, g.bias, g.accumulate ? 1 : 0, vec); break;
        default: gemv_nk_kernel<4><<<grid, 256, 0, stream()>>>(g.A, g.a_rs, g.B, g.b_cs, g.C, g.c_rs, g.N, g.K, g.bias, g.accumulate ? 1 : 0, vec); break;
    }
    prof_work(4.0 * g.K * g.N);
    LAUNCHED("gemv_nk_kernel");
}

// Which product of an op a GEMM is: the precision policy of TF32 mode can send each kind to 3xTF32.
static thread_local int g_role = GEMM_ROLE_FORWARD;
void gemm_set_role(int role) { g_role = role; }
static unsigned g_roles_3x = 0;
static double g_max_flop_3x = 4e9;          // TF32 mode: CONVOLUTION products of at most this many FLOP take the 3xTF32 path
static double g_simt_max_flop = 8e9;        // 3xTF32 mode: products of at most this many FLOP take the fp32 FMA kernel
static bool g_policy_env_read = false;
void gemm_set_policy(unsigned roles_3x, double max_flop_3x) { g_roles_3x = roles_3x; g_max_flop_3x = max_flop_3x; g_policy_env_read = true; }
void gemm_get_policy(unsigned *roles_3x, double *max_flop_3x) { *roles_3x = g_roles_3x; *max_flop_3x = g_max_flop_3x; }
void gemm_set_exact_policy(double simt_max_flop) { g_simt_max_flop = simt_max_flop; }
double gemm_get_exact_policy() { return g_simt_max_flop; }

// DNN_CUDA_TF32_3X_SHAPES="role:N:K,role:N:K,...": single GEMM shapes (role 0/1/2, output columns N, reduction K of
// the product as the op states it) that take the 3xTF32 path; a measurement aid for choosing the policy.
struct ShapeRule { int role, N, K; };
static std::vector<ShapeRule> g_shape_rules;
static bool g_shapes_read = false;
static void read_shape_rules() {
    g_shapes_read = true;
    g_shape_rules.clear();
    const char *e = getenv("DNN_CUDA_TF32_3X_SHAPES");
    while (e && *e) {
        ShapeRule r;
        int used = 0;
        if (sscanf(e, "%d:%d:%d%n", &r.role, &r.N, &r.K, &used) == 3) g_shape_rules.push_back(r);
        e += used;
        while (*e && *e != ',') e++;
        if (*e == ',') e++;
    }
}
void gemm_reread_env() { g_shapes_read = false; }

void gemm(const GemmArgs &g) {
    if (gemv_applicable(g)) { gemv(g); return; }          // a few output rows: bandwidth-bound on W, exact fp32 in every mode
    int mode = gemm_mode();
    if (mode == DNN_CUDA_GEMM_FP32 || !gemm_tc_supported(g)) { gemm_simt(g); return; }
    if (!g_policy_env_read) {
        g_policy_env_read = true;
        if (const char *e = getenv("DNN_CUDA_TF32_3X_ROLES")) g_roles_3x = (unsigned)atoi(e);
        if (const char *e = getenv("DNN_CUDA_TF32_3X_MAX_GFLOP")) g_max_flop_3x = atof(e) * 1e9;
        if (const char *e = getenv("DNN_CUDA_3X_SIMT_MAX_GFLOP")) g_simt_max_flop = atof(e) * 1e9;
    }
    if (!g_shapes_read) read_shape_rules();
    // Precision policy.
    // TF32 mode: a convolution lowered to a GEMM has a short reduction (C*k*k = 9 .. 288) or a narrow output (32 .. 64
    // channels), so it uses a fraction of the tensor core and is bound by the traffic of its column matrix: two more
    // products cost little.  And the gradients of a CNN are what TF32 rounding hurts most -- with random labels and
    // fresh weights they are what is left after 512 per-sample gradients cancel (measured on the MNIST-shaped CNN:
    // 1.7e-2 on the filter gradients in plain TF32, 2.9e-4 with 3xTF32 products).  So convolution GEMMs of at most
    // 4 GFLOP take the 3xTF32 path; so does any GEMM with a long reduction into a small output (a filter gradient),
    // and whatever dnn_cuda_set_tf32_policy names by role.
    // 3xTF32 mode: products of at most 8 GFLOP take the fp32 FMA kernel -- 3xTF32 leaves about 5e-7 per element
    // (operand remainders rounded to TF32, the small x small term dropped), which small models whose gradients cancel
    // heavily amplify past 1e-5.
    const double flop = 2.0 * g.M * g.N * g.K * (g.batch > 0 ? g.batch : 1);
    if (mode == DNN_CUDA_GEMM_3XTF32 && flop <= g_simt_max_flop) { gemm_simt(g); return; }
    const int role = g_role & 3;
    const bool conv = (g_role & GEMM_ROLE_CONV) != 0;
    bool small_long = (int64_t)g.M * g.N <= 65536 && g.K >= 1024;
    bool by_policy = ((g_roles_3x >> role) & 1u) || (conv && flop <= g_max_flop_3x);
    bool by_shape = false;
    for (const ShapeRule &r : g_shape_rules) if (r.role == role && r.N == g.N && r.K == g.K) by_shape = true;
    gemm_tc(g, mode == DNN_CUDA_GEMM_3XTF32 || small_long || by_policy || by_shape);
}

}  // namespace dnnb
