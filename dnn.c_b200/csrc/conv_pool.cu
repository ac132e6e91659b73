// conv2d (im2col + GEMM) and avg_pool2d, forward and backward.
// replaces src/conv.c:50-919 and src/ops_pool.c:118-381 of the reference.
//
// conv2d.  The reference has two paths with different OUTPUT MEMORY LAYOUTS and
// both are reproduced:
//   * 3x3 / stride 1 / pad 1 takes a Winograd F(2x2,3x3) path and writes true
//     NCHW (src/conv.c:719-800).  Here: im2col + GEMM into an (M, out_C) buffer
//     followed by a permute to NCHW; Winograd is an exact algebraic rewrite, so
//     the results agree to rounding.
//   * every other geometry takes im2col + GEMM and writes the GEMM result
//     (M, out_C), M = (n, oh, ow), straight into the tensor that is DECLARED
//     [N, out_C, H_out, W_out] (src/conv.c:847-863), and its backward reads the
//     upstream gradient the same way (:437-506).  Kept bit-for-bit in layout.
// Both paths sum the bias gradient with NCHW indexing (src/conv.c:418-435,555-570).
// The column matrix is stored (K, M) like the reference's and kept for backward.
#include "common.cuh"
#include "device_utils.cuh"

namespace dnnb {

struct ConvGeom { int N, C, H, W, out_C, kH, kW, stride, pad, H_out, W_out, M, K; };

// col[k][m], k = (c, kh, kw), m = (n, oh, ow).  Row k of the column matrix is, image by image, a shifted
// (and strided) copy of one input plane, so the index arithmetic is split by what it depends on:
//   blockIdx.y = c (taps kernel) or k (row kernel)   decoded once per CTA;
//   threadIdx.x = one output position of a plane      decoded once per thread into the source offset of every
//                                                     filter tap (-1: padding);
//   threadIdx.y + blockIdx.x = the image n            the only thing the inner loop changes.
// Consecutive lanes own consecutive positions, so every load and every store of a warp is one run of
// consecutive floats (a 128-byte line per instruction).  An earlier version gave each thread four positions
// and one 128-bit store; its four gather loads per store were 16 bytes apart from lane to lane, four L1
// wavefronts each, and the kernel ran at half the bandwidth of this one.
// Taps kernel (kH*kW <= 9): a CTA row reads its plane once (from L1 after the first tap) and writes all kH*kW rows.
__global__ void __launch_bounds__(256) im2col_taps_kernel(const float *__restrict__ x, float *__restrict__ col, ConvGeom g) {
    const int c = blockIdx.y, KK = g.kH * g.kW, HoWo = g.H_out * g.W_out;
    const int64_t plane = (int64_t)g.H * g.W;
    for (int o = threadIdx.x; o < HoWo; o += blockDim.x) {
        const int oh = o / g.W_out, ow = o - oh * g.W_out;
        int off[9];
#pragma unroll
        for (int t = 0; t < 9; t++) {
            const int kh = t / g.kW, kw = t - kh * g.kW;
            const int ih = oh * g.stride - g.pad + kh, iw = ow * g.stride - g.pad + kw;
            off[t] = (t < KK && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) ? ih * g.W + iw : -1;
        }
        for (int n = blockIdx.x * blockDim.y + threadIdx.y; n < g.N; n += gridDim.x * blockDim.y) {
            const float *src = x + ((int64_t)n * g.C + c) * plane;
            float *dst = col + (int64_t)c * KK * g.M + (int64_t)n * HoWo + o;
            float v[9];
#pragma unroll
            for (int t = 0; t < 9; t++) v[t] = off[t] >= 0 ? __ldg(src + off[t]) : 0.f;
#pragma unroll
            for (int t = 0; t < 9; t++) if (t < KK) dst[(int64_t)t * g.M] = v[t];
        }
    }
}
// Row kernel (any filter size): one CTA row per row k of the column matrix.
__global__ void __launch_bounds__(256) im2col_row_kernel(const float *__restrict__ x, float *__restrict__ col, ConvGeom g) {
    const int k = blockIdx.y;
    const int kw = k % g.kW, kh = (k / g.kW) % g.kH, c = k / (g.kW * g.kH);
    const int HoWo = g.H_out * g.W_out;
    const int64_t plane = (int64_t)g.H * g.W;
    for (int o = threadIdx.x; o < HoWo; o += blockDim.x) {
        const int oh = o / g.W_out, ow = o - oh * g.W_out;
        const int ih = oh * g.stride - g.pad + kh, iw = ow * g.stride - g.pad + kw;
        const int off = (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) ? ih * g.W + iw : -1;
        float *dst = col + (int64_t)k * g.M + o;
        for (int n = blockIdx.x * blockDim.y + threadIdx.y; n < g.N; n += gridDim.x * blockDim.y)
            dst[(int64_t)n * HoWo] = off >= 0 ? __ldg(x + ((int64_t)n * g.C + c) * plane + off) : 0.f;
    }
}
// Thread block (bx, by): bx lanes over the positions of a plane, by images side by side; grid.x over the images.
static void conv_launch_shape(int positions, int N, int rows, dim3 &grid, dim3 &block) {
    int bx = ((positions + 31) / 32) * 32;
    if (bx > 256) bx = 256;
    const int by = 256 / bx;
    int gx = (N + by - 1) / by;
    const int cap = (kNumSMs * 16 + rows - 1) / rows;          // a few waves in total
    if (gx > cap) gx = cap < 1 ? 1 : cap;
    grid = dim3(gx, rows); block = dim3(bx, by);
}
static void run_im2col(const float *x, float *col, const ConvGeom &g) {
    dim3 grid, block;
    if (g.kH * g.kW <= 9 && g.C <= 65535) {
        conv_launch_shape(g.H_out * g.W_out, g.N, g.C, grid, block);
        im2col_taps_kernel<<<grid, block, 0, stream()>>>(x, col, g);
    } else {
        DNN_CHECK(g.K <= 65535, "conv2d: C * kH * kW above 65535 is not supported");
        conv_launch_shape(g.H_out * g.W_out, g.N, g.K, grid, block);
        im2col_row_kernel<<<grid, block, 0, stream()>>>(x, col, g);
    }
    prof_work(4.0 * ((double)g.N * g.C * g.H * g.W + (double)g.K * g.M));
    LAUNCHED("im2col_kernel");
}

// dx[n,c,ih,iw] (=|+=) sum over the windows (kh,kw,oh,ow) that read this pixel of dcol[k][m]; gather form,
// fixed order (kh, then kw), no atomics.  Same split of the index arithmetic and the same lane layout as im2col:
// blockIdx.y = c, a thread owns one pixel of a plane and decodes, once, for each of the (at most 9) filter taps
// the position of the column-matrix element that tap contributed (-1: none); the inner loop over images is
// loads of consecutive floats per warp and adds.  kH*kW <= 9.
template <bool ACC>
__global__ void __launch_bounds__(256) col2im_taps_kernel(const float *__restrict__ dcol, float *__restrict__ dx, ConvGeom g) {
    const int c = blockIdx.y, HW = g.H * g.W, HoWo = g.H_out * g.W_out, KK = g.kH * g.kW;
    for (int p = threadIdx.x; p < HW; p += blockDim.x) {
        const int ih = p / g.W, iw = p - ih * g.W;
        int pos[9];
#pragma unroll
        for (int t = 0; t < 9; t++) {
            pos[t] = -1;
            if (t >= KK) continue;
            const int kh = t / g.kW, kw = t - kh * g.kW;
            const int a = ih + g.pad - kh, b = iw + g.pad - kw;
            if (a < 0 || b < 0 || a % g.stride || b % g.stride) continue;
            const int oh = a / g.stride, ow = b / g.stride;
            if (oh >= g.H_out || ow >= g.W_out) continue;
            pos[t] = oh * g.W_out + ow;
        }
        for (int n = blockIdx.x * blockDim.y + threadIdx.y; n < g.N; n += gridDim.x * blockDim.y) {
            const float *src = dcol + (int64_t)c * KK * g.M + (int64_t)n * HoWo;      // tap t: + t * M
            float s = 0.f;
#pragma unroll
            for (int t = 0; t < 9; t++) if (pos[t] >= 0) s += __ldg(src + (int64_t)t * g.M + pos[t]);
            float *dst = dx + ((int64_t)n * g.C + c) * HW + p;
            *dst = ACC ? *dst + s : s;
        }
    }
}
// Any geometry.
template <bool ACC>
__global__ void col2im_kernel(const float *__restrict__ dcol, float *__restrict__ dx, ConvGeom g) {
    int64_t total = (int64_t)g.N * g.C * g.H * g.W;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        int iw = (int)(idx % g.W); int64_t t = idx / g.W; int ih = (int)(t % g.H); t /= g.H; int c = (int)(t % g.C); int n = (int)(t / g.C);
        float s = 0.f;
        for (int kh = 0; kh < g.kH; kh++) {
            int a = ih + g.pad - kh;
            if (a < 0 || a % g.stride) continue;
            int oh = a / g.stride;
            if (oh >= g.H_out) continue;
            for (int kw = 0; kw < g.kW; kw++) {
                int b = iw + g.pad - kw;
                if (b < 0 || b % g.stride) continue;
                int ow = b / g.stride;
                if (ow >= g.W_out) continue;
                int k = (c * g.kH + kh) * g.kW + kw;
                int m = (n * g.H_out + oh) * g.W_out + ow;
                s += dcol[(int64_t)k * g.M + m];
            }
        }
        dx[idx] = ACC ? dx[idx] + s : s;
    }
}
static void run_col2im(const float *dcol, float *dx, const ConvGeom &g, bool accumulate) {
    const int HW = g.H * g.W;
    if (g.kH * g.kW <= 9 && g.C <= 65535) {
        dim3 grid, block;
        conv_launch_shape(HW, g.N, g.C, grid, block);
        if (accumulate) col2im_taps_kernel<true><<<grid, block, 0, stream()>>>(dcol, dx, g);
        else col2im_taps_kernel<false><<<grid, block, 0, stream()>>>(dcol, dx, g);
    } else {
        const int grid = grid_for((int64_t)g.N * g.C * HW, 256);
        if (accumulate) col2im_kernel<true><<<grid, 256, 0, stream()>>>(dcol, dx, g);
        else col2im_kernel<false><<<grid, 256, 0, stream()>>>(dcol, dx, g);
    }
    prof_work(4.0 * ((accumulate ? 2.0 : 1.0) * g.N * g.C * g.H * g.W + (double)g.K * g.M));
    LAUNCHED("col2im_kernel");
}

// (M, out_C) <-> NCHW, per image a [HW, OC] <-> [OC, HW] transpose through a padded 32 x 32 shared-memory
// tile, so that both the reads and the writes are full 128-byte rows.
//   TO_NCHW:  dst[n, oc, hw] = src[(n*HW + hw), oc];   otherwise  dst[(n*HW + hw), oc] = src[n, oc, hw].
template <bool TO_NCHW>
__global__ void __launch_bounds__(256) conv_permute_kernel(float *__restrict__ dst, const float *__restrict__ src, int OC, int HW) {
    __shared__ float tile[32][33];
    const int n = blockIdx.z;
    const int64_t img = (int64_t)n * OC * HW;
    // rows/cols of the SOURCE matrix of this image: [R, Cc] row-major -> destination [Cc, R]
    const int R = TO_NCHW ? HW : OC, Cc = TO_NCHW ? OC : HW;
    const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;         // 32 x 8
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
        const int r = r0 + ty + i, c = c0 + tx;
        if (r < R && c < Cc) tile[ty + i][tx] = src[img + (int64_t)r * Cc + c];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
        const int c = c0 + ty + i, r = r0 + tx;
        if (r < R && c < Cc) dst[img + (int64_t)c * R + r] = tile[tx][ty + i];
    }
}
template <bool TO_NCHW>
static void run_permute(float *dst, const float *src, int N, int OC, int HW) {
    const int R = TO_NCHW ? HW : OC, Cc = TO_NCHW ? OC : HW;
    for (int n0 = 0; n0 < N; n0 += 65535) {
        const int nb = N - n0 < 65535 ? N - n0 : 65535;
        const int64_t off = (int64_t)n0 * OC * HW;
        conv_permute_kernel<TO_NCHW><<<dim3((Cc + 31) / 32, (R + 31) / 32, nb), 256, 0, stream()>>>(dst + off, src + off, OC, HW);
        prof_work(8.0 * nb * OC * HW);
        LAUNCHED("conv_permute_kernel");
    }
}

// dbias[oc] += sum_{n,hw} g[(n*OC + oc)*HW + hw].  CTA (oc, s) sums the images n = s, s + S, ... of its
// channel into part[oc*S + s]; conv_dbias_final_kernel adds the S partials in order (fixed order).  The CTA's
// rows (one per image, HW floats each) are walked as one list of 128-bit pieces, four independent loads in
// flight per thread; rows that are not a multiple of four floats long take the scalar loop.
__global__ void __launch_bounds__(256) conv_dbias_kernel(float *__restrict__ part, const float *__restrict__ g, int N, int OC, int HW) {
    __shared__ float sh[32];
    const int oc = blockIdx.x, S = gridDim.y;
    const int64_t img = (int64_t)OC * HW;
    const int rows = (N - (int)blockIdx.y + S - 1) / S;               // images n = blockIdx.y + r * S
    const float *base = g + (int64_t)blockIdx.y * img + (int64_t)oc * HW;
    const int64_t row_pitch = (int64_t)S * img;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (HW % 4 == 0 && (((uintptr_t)g) & 15) == 0) {
        const int w4 = HW >> 2, items = rows * w4;
        auto piece = [&](int i) { const int r = i / w4, c4 = i - r * w4;
                                  return __ldg(reinterpret_cast<const float4 *>(base + (int64_t)r * row_pitch) + c4); };
        int i = threadIdx.x;
        for (; i + 3 * 256 < items; i += 4 * 256) {
            const float4 a = piece(i), b = piece(i + 256), c = piece(i + 512), d = piece(i + 768);
            s0 += (a.x + a.y) + (a.z + a.w); s1 += (b.x + b.y) + (b.z + b.w);
            s2 += (c.x + c.y) + (c.z + c.w); s3 += (d.x + d.y) + (d.z + d.w);
        }
        for (; i < items; i += 256) { const float4 a = piece(i); s0 += (a.x + a.y) + (a.z + a.w); }
    } else {
        for (int r = 0; r < rows; r++)
            for (int hw = threadIdx.x; hw < HW; hw += blockDim.x) s0 += __ldg(base + (int64_t)r * row_pitch + hw);
    }
    const float s = block_sum((s0 + s1) + (s2 + s3), sh);
    if (threadIdx.x == 0) part[oc * S + blockIdx.y] = s;
}
__global__ void conv_dbias_final_kernel(float *__restrict__ db, const float *__restrict__ part, int OC, int S) {
    int oc = blockIdx.x * blockDim.x + threadIdx.x;
    if (oc >= OC) return;
    float s = 0.f;
    for (int i = 0; i < S; i++) s += part[oc * S + i];
    db[oc] += s;
}
// Filters whose row length K = C*kH*kW is not a multiple of 4 floats (the first layer of an image model:
// 1 x 3 x 3 = 9) cannot be described to the copy engine.  They are copied into rows padded to Kp floats
// (zeros behind K), the GEMMs run on the padded rows, and the filter gradient is added back without the pad.
__global__ void conv_pad_rows_kernel(float *__restrict__ dst, const float *__restrict__ src, int rows, int K, int Kp) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * Kp) return;
    int r = i / Kp, k = i - r * Kp;
    dst[i] = k < K ? src[r * K + k] : 0.f;
}
__global__ void conv_unpad_add_kernel(float *__restrict__ dst, const float *__restrict__ src, int rows, int K, int Kp) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * K) return;
    int r = i / K, k = i - r * K;
    dst[i] += src[r * Kp + k];
}
static const float *padded_filters(struct mem_pool *pool, const float *w, int out_C, int K, int Kp) {
    float *wp = dev_alloc_t<float>(pool, (size_t)out_C * Kp);
    conv_pad_rows_kernel<<<(out_C * Kp + 255) / 256, 256, 0, stream()>>>(wp, w, out_C, K, Kp);
    LAUNCHED("conv_pad_rows_kernel");
    return wp;
}

struct ConvSaved { ConvGeom g; float *col; tensor *bias; int nchw; };

static void conv2d_backward(grad_fn *fn, tensor *go) {
    tensor *input = fn->inputs[0], *weight = fn->inputs[1];
    ConvSaved *sv = (ConvSaved *)fn->saved_tensors[0];
    const ConvGeom &g = sv->g;
    tensor *bias = sv->bias;
    const float *gd = (const float *)go->data;
    const float *wd = (const float *)weight->data + weight->offset;
    int HW = g.H_out * g.W_out;

    // Gradient buffers first: an activation's gradient comes from the same pool
    // as the temporaries below and must survive the release at the end.
    float *wg = weight->requires_grad ? _grad_ensure(weight) : nullptr;
    bool acc_x = true;
    float *xg = input->requires_grad ? grad_full(input, &acc_x) : nullptr;      // col2im writes every pixel: a fresh buffer is stored to
    if (bias && bias->requires_grad) {
        float *bg = _grad_ensure(bias);
        int S = g.N < 32 ? g.N : 32;
        float *part = dev_alloc_t<float>(fn->pool, (size_t)g.out_C * S);
        conv_dbias_kernel<<<dim3(g.out_C, S), 256, 0, stream()>>>(part, gd, g.N, g.out_C, HW);
        LAUNCHED("conv_dbias_kernel");
        conv_dbias_final_kernel<<<(g.out_C + 127) / 128, 128, 0, stream()>>>(bg, part, g.out_C, S);
        LAUNCHED("conv_dbias_final_kernel");
    }
    size_t mark = mem_pool_mark(fn->pool);
    const int Kp = (g.K + 3) & ~3;
    const bool padded = Kp != g.K && gemm_mode() != DNN_CUDA_GEMM_FP32;
    const float *wk = padded ? padded_filters(fn->pool, wd, g.out_C, g.K, Kp) : wd;
    const int wpitch = padded ? Kp : g.K;
    const float *g_mc = gd;                 // upstream gradient read as (M, out_C)
    if (sv->nchw) {
        float *tmp = dev_alloc_t<float>(fn->pool, (size_t)g.M * g.out_C);
        run_permute<false>(tmp, gd, g.N, g.out_C, HW);
        g_mc = tmp;
    }
    if (wg) {
        GemmArgs a;     // dW[oc,k] += sum_m g_mc[m,oc] * col[k,m]
        a.A = g_mc; a.a_rs = 1; a.a_cs = g.out_C; a.a_bs = 0;
        a.B = sv->col; a.b_rs = 1; a.b_cs = g.M; a.b_bs = 0;
        float *dwp = padded ? dev_alloc_t<float>(fn->pool, (size_t)g.out_C * Kp) : nullptr;
        a.C = padded ? dwp : wg + weight->offset; a.c_rs = wpitch; a.c_cs = 1; a.c_bs = 0;
        a.bias = nullptr; a.M = g.out_C; a.N = g.K; a.K = g.M; a.batch = 1; a.accumulate = !padded;
        gemm_set_role(GEMM_ROLE_DW | GEMM_ROLE_CONV);
        gemm(a);
        gemm_set_role(GEMM_ROLE_FORWARD);
        if (padded) {
            conv_unpad_add_kernel<<<(g.out_C * g.K + 255) / 256, 256, 0, stream()>>>(wg + weight->offset, dwp, g.out_C, g.K, Kp);
            LAUNCHED("conv_unpad_add_kernel");
        }
    }
    if (xg) {
        float *dcol = dev_alloc_t<float>(fn->pool, (size_t)g.K * g.M);
        GemmArgs a;     // dcol[k,m] = sum_oc W[oc,k] * g_mc[m,oc]
        a.A = wk; a.a_rs = 1; a.a_cs = wpitch; a.a_bs = 0;
        a.B = g_mc; a.b_rs = 1; a.b_cs = g.out_C; a.b_bs = 0;
        a.C = dcol; a.c_rs = g.M; a.c_cs = 1; a.c_bs = 0;
        a.bias = nullptr; a.M = g.K; a.N = g.M; a.K = g.out_C; a.batch = 1; a.accumulate = false;
        gemm_set_role(GEMM_ROLE_DA | GEMM_ROLE_CONV);
        gemm(a);
        gemm_set_role(GEMM_ROLE_FORWARD);
        run_col2im(dcol, xg + input->offset, g, acc_x);
    }
    mem_pool_release(fn->pool, mark);
}

// ---- avg_pool2d ------------------------------------------------------------------
// Any window geometry: one thread per output element.
__global__ void avgpool_fwd_kernel(const float *__restrict__ x, float *__restrict__ out,
                                   int64_t planes, int H, int W, int H_out, int W_out, int k, int stride, float inv_k2) {
    int64_t total = planes * H_out * W_out;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        int ow = (int)(idx % W_out); int64_t t = idx / W_out; int oh = (int)(t % H_out); int64_t pl = t / H_out;
        const float *xp = x + pl * H * W + (int64_t)(oh * stride) * W + ow * stride;
        float s = 0.f;
        for (int di = 0; di < k; di++)
            for (int dj = 0; dj < k; dj++) s += xp[di * W + dj];
        out[idx] = s * inv_k2;
    }
}
// 2 x 2 windows, stride 2, W a multiple of 4 (the pooling of the image models).  A thread owns two
// neighbouring outputs of a plane: its position is decoded once, then it walks the planes with two
// 128-bit loads (the two input rows of its windows) and one 64-bit store per plane.  Sums run in the
// reference's order (row by row inside a window, src/ops_pool.c:293-313).
__global__ void __launch_bounds__(256) avgpool_fwd_k2_kernel(const float *__restrict__ x, float *__restrict__ out,
                                                             int planes, int H, int W, int H_out, int W_out) {
    const int pairs = H_out * (W_out >> 1);                 // W_out is even because W % 4 == 0
    const int64_t in_plane = (int64_t)H * W, out_plane = (int64_t)H_out * W_out;
    for (int e = threadIdx.x; e < pairs; e += blockDim.x) {
        const int oh = e / (W_out >> 1), ow = (e - oh * (W_out >> 1)) * 2;
        const int in_off = (2 * oh) * W + 2 * ow, out_off = oh * W_out + ow;
        for (int pl = blockIdx.x * blockDim.y + threadIdx.y; pl < planes; pl += gridDim.x * blockDim.y) {
            const float *xp = x + pl * in_plane + in_off;
            const float4 a = __ldg(reinterpret_cast<const float4 *>(xp)), b = __ldg(reinterpret_cast<const float4 *>(xp + W));
            float2 o;
            o.x = (((a.x + a.y) + b.x) + b.y) * 0.25f;
            o.y = (((a.z + a.w) + b.z) + b.w) * 0.25f;
            *reinterpret_cast<float2 *>(out + pl * out_plane + out_off) = o;
        }
    }
}
// Any window geometry, gather form: every input element sums the windows that cover it.
template <bool ACC>
__global__ void avgpool_bwd_kernel(const float *__restrict__ g, float *__restrict__ dx,
                                   int64_t planes, int H, int W, int H_out, int W_out, int k, int stride, float inv_k2) {
    int64_t total = planes * H * W;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        int iw = (int)(idx % W); int64_t t = idx / W; int ih = (int)(t % H); int64_t pl = t / H;
        // windows (oh, ow) with oh*stride <= ih < oh*stride + k
        int oh_lo = ih - k + 1 <= 0 ? 0 : (ih - k + stride) / stride;
        int oh_hi = ih / stride; if (oh_hi > H_out - 1) oh_hi = H_out - 1;
        int ow_lo = iw - k + 1 <= 0 ? 0 : (iw - k + stride) / stride;
        int ow_hi = iw / stride; if (ow_hi > W_out - 1) ow_hi = W_out - 1;
        float s = 0.f;
        for (int oh = oh_lo; oh <= oh_hi; oh++)
            for (int ow = ow_lo; ow <= ow_hi; ow++) s += g[pl * H_out * W_out + (int64_t)oh * W_out + ow] * inv_k2;
        dx[idx] = ACC ? dx[idx] + s : s;
    }
}
// Windows that do not overlap (stride == k) and W a multiple of 4: every input element belongs to at most
// one window.  A thread owns four neighbouring input elements of a plane, decodes once which output each
// of them reads (or none, past the last full window), and walks the planes with one 128-bit store each.
template <bool ACC>
__global__ void __launch_bounds__(256) avgpool_bwd_tiles_kernel(const float *__restrict__ g, float *__restrict__ dx, int planes,
                                                                int H, int W, int H_out, int W_out, int k, float inv_k2) {
    const int n4 = (H * W) >> 2;
    const int64_t in_plane = (int64_t)H * W, out_plane = (int64_t)H_out * W_out;
    for (int e = threadIdx.x; e < n4; e += blockDim.x) {
        int src[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int p = 4 * e + j, ih = p / W, iw = p - ih * W;
            const int oh = ih / k, ow = iw / k;
            src[j] = (oh < H_out && ow < W_out) ? oh * W_out + ow : -1;
        }
        for (int pl = blockIdx.x * blockDim.y + threadIdx.y; pl < planes; pl += gridDim.x * blockDim.y) {
            const float *gp = g + pl * out_plane;
            float4 v;
            v.x = src[0] >= 0 ? __ldg(gp + src[0]) * inv_k2 : 0.f; v.y = src[1] >= 0 ? __ldg(gp + src[1]) * inv_k2 : 0.f;
            v.z = src[2] >= 0 ? __ldg(gp + src[2]) * inv_k2 : 0.f; v.w = src[3] >= 0 ? __ldg(gp + src[3]) * inv_k2 : 0.f;
            float4 *dst = reinterpret_cast<float4 *>(dx + pl * in_plane + 4 * e);
            if (ACC) { const float4 o = *dst; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
            *dst = v;
        }
    }
}

// Thread block (bx, by): bx threads cover the positions of a plane, by planes side by side.
static void plane_launch_shape(int positions, int64_t planes, dim3 &grid, dim3 &block) {
    int bx = ((positions + 31) / 32) * 32;
    if (bx > 256) bx = 256;
    const int by = 256 / bx;
    int64_t gx = (planes + by - 1) / by;
    const int64_t cap = (int64_t)kNumSMs * 16;
    if (gx > cap) gx = cap;
    grid = dim3((unsigned)gx); block = dim3(bx, by);
}

static void avg_pool2d_backward(grad_fn *fn, tensor *go) {
    tensor *x = fn->inputs[0];
    int k = *(int *)fn->saved_tensors[0], stride = *(int *)fn->saved_tensors[1];
    if (!x->requires_grad) return;
    int N = x->shape[0], C = x->shape[1], H = x->shape[2], W = x->shape[3];
    int H_out = (H - k) / stride + 1, W_out = (W - k) / stride + 1;
    // every input element is written (elements no window covers get a zero contribution), so a fresh
    // gradient buffer is stored to; indexed from 0 with packed NCHW strides, as the reference does
    bool acc = true;
    float *xg = x->contiguous ? grad_full(x, &acc) : _grad_ensure(x);
    int64_t planes = (int64_t)N * C;
    const float inv = 1.0f / (float)(k * k);
    const float *gd = (const float *)go->data;
    if (stride == k && W % 4 == 0 && aligned16(xg) && planes < (1 << 30)) {
        dim3 grid, block;
        plane_launch_shape(H * W / 4, planes, grid, block);
        if (acc) avgpool_bwd_tiles_kernel<true><<<grid, block, 0, stream()>>>(gd, xg, (int)planes, H, W, H_out, W_out, k, inv);
        else avgpool_bwd_tiles_kernel<false><<<grid, block, 0, stream()>>>(gd, xg, (int)planes, H, W, H_out, W_out, k, inv);
    } else {
        const int grid = grid_for(planes * H * W, 256);
        if (acc) avgpool_bwd_kernel<true><<<grid, 256, 0, stream()>>>(gd, xg, planes, H, W, H_out, W_out, k, stride, inv);
        else avgpool_bwd_kernel<false><<<grid, 256, 0, stream()>>>(gd, xg, planes, H, W, H_out, W_out, k, stride, inv);
    }
    prof_work(4.0 * ((acc ? 2.0 : 1.0) * planes * H * W + (double)planes * H_out * W_out));
    LAUNCHED("avgpool_bwd_kernel");
}

}  // namespace dnnb

using namespace dnnb;

extern "C" {

tensor *tensor_conv2d(struct mem_pool *scratch, tensor *input, tensor *weight, tensor *bias, int stride, int pad) {
    require_device_payloads("tensor_conv2d", {input, weight, bias});
    DNN_CHECK(input && weight, "conv2d: NULL operand");
    DNN_CHECK(input->ndim == 4, "conv2d: input must be (N, C, H, W)");
    DNN_CHECK(weight->ndim == 4, "conv2d: weight must be (out_C, in_C, kH, kW)");
    DNN_CHECK(input->shape[1] == weight->shape[1], "conv2d: in_channels mismatch");
    DNN_CHECK(input->contiguous && weight->contiguous, "conv2d: input and weight must be contiguous");
    DNN_CHECK(!bias || (bias->ndim == 1 && bias->shape[0] == weight->shape[0]), "conv2d: bias shape");
    DNN_CHECK(stride > 0, "conv2d: stride must be positive");
    ConvGeom g;
    g.N = input->shape[0]; g.C = input->shape[1]; g.H = input->shape[2]; g.W = input->shape[3];
    g.out_C = weight->shape[0]; g.kH = weight->shape[2]; g.kW = weight->shape[3];
    g.stride = stride; g.pad = pad;
    g.H_out = (g.H + 2 * pad - g.kH) / stride + 1;
    g.W_out = (g.W + 2 * pad - g.kW) / stride + 1;
    DNN_CHECK(g.H_out > 0 && g.W_out > 0, "conv2d: kernel larger than padded input");
    g.M = g.N * g.H_out * g.W_out; g.K = g.C * g.kH * g.kW;
    int shape[4] = {g.N, g.out_C, g.H_out, g.W_out};
    tensor *out = tensor_scratch(scratch, 4, shape, 0);
    bool nchw = (g.kH == 3 && g.kW == 3 && stride == 1 && pad == 1);
    bool needs_grad = dnn_grad_enabled() && (input->requires_grad || weight->requires_grad || (bias && bias->requires_grad));

    size_t mark = mem_pool_mark(scratch);
    float *col = dev_alloc_t<float>(scratch, (size_t)g.K * g.M);
    run_im2col((const float *)input->data + input->offset, col, g);
    float *mc = nchw ? dev_alloc_t<float>(scratch, (size_t)g.M * g.out_C) : (float *)out->data;
    GemmArgs a;         // mc[m,oc] = sum_k col[k,m] * W[oc,k] + bias[oc]
    a.A = col; a.a_rs = 1; a.a_cs = g.M; a.a_bs = 0;
    const int Kp = (g.K + 3) & ~3;
    const bool padded = Kp != g.K && gemm_mode() != DNN_CUDA_GEMM_FP32;
    const float *wsrc = (const float *)weight->data + weight->offset;
    a.B = padded ? padded_filters(scratch, wsrc, g.out_C, g.K, Kp) : wsrc; a.b_rs = 1; a.b_cs = padded ? Kp : g.K; a.b_bs = 0;
    a.C = mc; a.c_rs = g.out_C; a.c_cs = 1; a.c_bs = 0;
    a.bias = bias ? (const float *)bias->data + bias->offset : nullptr;
    a.M = g.M; a.N = g.out_C; a.K = g.K; a.batch = 1; a.accumulate = false;
    gemm_set_role(GEMM_ROLE_FORWARD | GEMM_ROLE_CONV);
    gemm(a);
    gemm_set_role(GEMM_ROLE_FORWARD);
    if (nchw) {
        run_permute<true>((float *)out->data, mc, g.N, g.out_C, g.H_out * g.W_out);
    }
    if (needs_grad) {
        grad_fn *fn = attach(scratch, out, conv2d_backward, 2, 1);
        fn->inputs[0] = input; fn->inputs[1] = weight;
        ConvSaved *sv = host_alloc_t<ConvSaved>(scratch);
        sv->g = g; sv->col = col; sv->bias = bias; sv->nchw = nchw ? 1 : 0;
        fn->saved_tensors[0] = (tensor *)sv;
    } else {
        mem_pool_release(scratch, mark);     // nothing kept: give the column matrix back
    }
    return out;
}

tensor *tensor_avg_pool2d(struct mem_pool *scratch, const tensor *x, int k, int stride) {
    require_device_payloads("tensor_avg_pool2d", {x});
    DNN_CHECK(x, "avg_pool2d: NULL input");
    DNN_CHECK(x->ndim == 4, "avg_pool2d: input must be (N, C, H, W)");
    DNN_CHECK(k > 0, "avg_pool2d: kernel size must be positive");
    if (stride <= 0) stride = k;
    int N = x->shape[0], C = x->shape[1], H = x->shape[2], W = x->shape[3];
    int H_out = (H - k) / stride + 1, W_out = (W - k) / stride + 1;
    DNN_CHECK(H_out > 0 && W_out > 0, "avg_pool2d: kernel too large for input");
    int shape[4] = {N, C, H_out, W_out};
    tensor *out = tensor_scratch(scratch, 4, shape, 0);
    const float *xd = (const float *)x->data + x->offset;
    if (!x->contiguous) {
        float *tmp = dev_alloc_t<float>(scratch, (size_t)numel_of(x));
        k_gather(tmp, (const float *)x->data, view_of(x), numel_of(x));
        xd = tmp;
    }
    int64_t planes = (int64_t)N * C;
    if (k == 2 && stride == 2 && W % 4 == 0 && aligned16(xd) && aligned16(out->data) && planes < (1 << 30)) {
        dim3 grid, block;
        plane_launch_shape(H_out * (W_out / 2), planes, grid, block);
        avgpool_fwd_k2_kernel<<<grid, block, 0, stream()>>>(xd, (float *)out->data, (int)planes, H, W, H_out, W_out);
    } else {
        avgpool_fwd_kernel<<<grid_for(planes * H_out * W_out, 256), 256, 0, stream()>>>(xd, (float *)out->data, planes, H, W,
                                                                                        H_out, W_out, k, stride, 1.0f / (float)(k * k));
    }
    prof_work(4.0 * ((double)planes * H * W + (double)planes * H_out * W_out));
    LAUNCHED("avgpool_fwd_kernel");
    if (dnn_grad_enabled() && x->requires_grad) {
        grad_fn *fn = attach(scratch, out, avg_pool2d_backward, 1, 2);
        fn->inputs[0] = (tensor *)x;
        int *ks = host_alloc_t<int>(scratch), *ss = host_alloc_t<int>(scratch);
        *ks = k; *ss = stride;
        fn->saved_tensors[0] = (tensor *)ks; fn->saved_tensors[1] = (tensor *)ss;
    }
    return out;
}

}  // extern "C"
