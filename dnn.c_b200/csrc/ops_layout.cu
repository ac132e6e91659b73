// Layout and indexing ops: rotary embedding, head split / merge, embedding
// gather and scatter-add.  All HBM-bound copies with 128-bit accesses.
// replaces src/rope.c:60-171, src/multihead.c:74-348, src/embedding.c:18-110.
#include "common.cuh"
#include "device_utils.cuh"
#include <vector>

namespace dnnb {

// ---- RoPE --------------------------------------------------------------------
// x viewed as [outer, N, d]; pair k of position n rotates by (cos,sin)[n, k].
// Forward rotates x in place.  Backward adds the inverse rotation of g to dx.
// One thread handles one float4 = two adjacent pairs.
template <bool BWD>
__global__ void rope_kernel(float *__restrict__ dst, const float *__restrict__ g,
                            const float *__restrict__ fc, const float *__restrict__ fs,
                            int64_t total4, int N, int d, int acc) {
    int d4 = d >> 2, dh = d >> 1;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (int64_t)gridDim.x * blockDim.x) {
        int q = (int)(i % d4);
        int n = (int)((i / d4) % N);
        float2 c = *reinterpret_cast<const float2 *>(fc + (int64_t)n * dh + 2 * q);
        float2 s = *reinterpret_cast<const float2 *>(fs + (int64_t)n * dh + 2 * q);
        if (!BWD) {
            float4 v = reinterpret_cast<float4 *>(dst)[i];
            float4 o;
            rope_fwd_pair(v.x, v.y, c.x, s.x, o.x, o.y);
            rope_fwd_pair(v.z, v.w, c.y, s.y, o.z, o.w);
            reinterpret_cast<float4 *>(dst)[i] = o;
        } else {
            float4 v = reinterpret_cast<const float4 *>(g)[i];
            float4 o = acc ? reinterpret_cast<float4 *>(dst)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            float rx, ry, rz, rw;
            rope_inv_pair(v.x, v.y, c.x, s.x, rx, ry);
            rope_inv_pair(v.z, v.w, c.y, s.y, rz, rw);
            o.x += rx; o.y += ry; o.z += rz; o.w += rw;
            reinterpret_cast<float4 *>(dst)[i] = o;
        }
    }
}
template <bool BWD>
__global__ void rope_pair_kernel(float *__restrict__ dst, const float *__restrict__ g,
                                 const float *__restrict__ fc, const float *__restrict__ fs,
                                 int64_t pairs, int N, int d, int acc) {
    int dh = d >> 1;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += (int64_t)gridDim.x * blockDim.x) {
        int k = (int)(i % dh);
        int n = (int)((i / dh) % N);
        float c = fc[(int64_t)n * dh + k], s = fs[(int64_t)n * dh + k];
        if (!BWD) {
            float a = dst[2 * i], b = dst[2 * i + 1];
            rope_fwd_pair(a, b, c, s, dst[2 * i], dst[2 * i + 1]);
        } else {
            float a = g[2 * i], b = g[2 * i + 1];
            float r0, r1;
            rope_inv_pair(a, b, c, s, r0, r1);
            if (acc) { r0 += dst[2 * i]; r1 += dst[2 * i + 1]; }
            dst[2 * i] = r0; dst[2 * i + 1] = r1;
        }
    }
}

static void rope_run(bool bwd, float *dst, const float *g, const float *fc, const float *fs, int64_t numel, int N, int d, int acc = 1) {
    if (numel <= 0) return;
    bool vec = d % 4 == 0 && aligned16(dst) && (!g || aligned16(g)) && (((uintptr_t)fc | (uintptr_t)fs) & 7) == 0;
    if (vec) {
        int64_t n4 = numel / 4;
        if (bwd) rope_kernel<true><<<grid_for(n4, 256), 256, 0, stream()>>>(dst, g, fc, fs, n4, N, d, acc);
        else     rope_kernel<false><<<grid_for(n4, 256), 256, 0, stream()>>>(dst, g, fc, fs, n4, N, d, acc);
    } else {
        int64_t np = numel / 2;
        if (bwd) rope_pair_kernel<true><<<grid_for(np, 256), 256, 0, stream()>>>(dst, g, fc, fs, np, N, d, acc);
        else     rope_pair_kernel<false><<<grid_for(np, 256), 256, 0, stream()>>>(dst, g, fc, fs, np, N, d, acc);
    }
    LAUNCHED(bwd ? "rope_bwd_kernel" : "rope_fwd_kernel");
}

static void rope_backward(grad_fn *fn, tensor *go) {
    tensor *x = fn->inputs[0];
    tensor *fc = fn->saved_tensors[0], *fs = fn->saved_tensors[1];
    if (!wants_grad(x)) return;
    int d = x->shape[x->ndim - 1], N = x->shape[x->ndim - 2];
    bool acc = true;
    float *grad = x->contiguous ? grad_full(x, &acc) : _grad_ensure(x);
    rope_run(true, grad + x->offset, (const float *)go->data + go->offset,
             (const float *)fc->data + fc->offset, (const float *)fs->data + fs->offset, numel_of(x), N, d, acc);
}

// ---- [B,P,Q,dk] <-> strided permutations ---------------------------------------
// The packed side is indexed (b,p,q,i) row-major; the strided side at
// b*sb + p*sp + q*sq + i.  MODE 0: packed <- strided.  1: strided = packed.  2: strided += packed.
template <int MODE, typename V>
__global__ void permute_kernel(float *__restrict__ packed_or_dst, float *__restrict__ strided,
                               int64_t total, int P, int Q, int dkv, int64_t sb, int64_t sp, int64_t sq) {
    constexpr int W = sizeof(V) / 4;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        int i = (int)(idx % dkv);
        int64_t r = idx / dkv;
        int q = (int)(r % Q); r /= Q;
        int p = (int)(r % P);
        int64_t b = r / P;
        V *pk = reinterpret_cast<V *>(packed_or_dst) + idx;
        V *st = reinterpret_cast<V *>(strided + b * sb + p * sp + q * sq + (int64_t)i * W);
        if (MODE == 0) *pk = *st;
        else if (MODE == 1) *st = *pk;
        else {
            V a = *st, c = *pk;
            float *af = reinterpret_cast<float *>(&a); const float *cf = reinterpret_cast<const float *>(&c);
#pragma unroll
            for (int k = 0; k < W; k++) af[k] += cf[k];
            *st = a;
        }
    }
}

template <int MODE>
static void permute(const char *name, float *packed, float *strided, int64_t B, int P, int Q, int dk,
                    int64_t sb, int64_t sp, int64_t sq) {
    int64_t n = B * P * Q * dk;
    if (n <= 0) return;
    bool vec = dk % 4 == 0 && aligned16(packed) && aligned16(strided) && sb % 4 == 0 && sp % 4 == 0 && sq % 4 == 0;
    if (vec) permute_kernel<MODE, float4><<<grid_for(n / 4, 256), 256, 0, stream()>>>(packed, strided, n / 4, P, Q, dk / 4, sb, sp, sq);
    else     permute_kernel<MODE, float><<<grid_for(n, 256), 256, 0, stream()>>>(packed, strided, n, P, Q, dk, sb, sp, sq);
    LAUNCHED(name);
}

static void split_qkv_heads_backward(grad_fn *fn, tensor *go) {
    tensor *qkv = fn->inputs[0];
    int B = qkv->shape[0], N = qkv->shape[1], D = qkv->shape[2];
    int which = *(int *)fn->saved_tensors[0];
    int H = go->shape[1], dk = go->shape[3];
    float *ig = _grad_ensure(qkv);
    // packed g is [B,H,N,dk]; destination [B,N,3,H,dk]
    permute<2>("split_qkv_bwd_kernel", (float *)go->data + go->offset, ig + qkv->offset + (int64_t)which * H * dk,
               B, H, N, dk, (int64_t)N * D, dk, D);
}

static void merge_heads_backward(grad_fn *fn, tensor *go) {
    tensor *in = fn->inputs[0];
    int B = in->shape[0], H = in->shape[1], N = in->shape[2], dk = in->shape[3];
    float *ig = _grad_ensure(in);
    // packed g is [B,N,H,dk]; destination [B,H,N,dk]; overwrites (src/multihead.c:177)
    permute<1>("merge_heads_bwd_kernel", (float *)go->data + go->offset, ig + in->offset,
               B, N, H, dk, (int64_t)H * N * dk, dk, (int64_t)N * dk);
}

static void split_heads_backward(grad_fn *fn, tensor *go) {
    tensor *in = fn->inputs[0];
    int B = in->shape[0], N = in->shape[1], D = in->shape[2];
    int H = *(int *)fn->saved_tensors[0];
    int dk = D / H;
    float *ig = _grad_ensure(in);
    // packed g is [B,H,N,dk]; destination [B,N,H*dk]; overwrites (src/multihead.c:92)
    permute<1>("split_heads_bwd_kernel", (float *)go->data + go->offset, ig + in->offset,
               B, H, N, dk, (int64_t)N * D, dk, D);
}

// ---- embedding -------------------------------------------------------------------
__global__ void embedding_fwd_kernel(float *__restrict__ out, const float *__restrict__ table, const int *__restrict__ ids,
                                     int n_ids, int d, int vocab, int64_t t_s0, int64_t t_s1, int vec) {
    int row = blockIdx.x;
    if (row >= n_ids) return;
    int id = ids[row];
    bool ok = id >= 0 && id < vocab;       // the reference asserts; an invalid id yields zeros here
    if (vec) {
        const float4 *src = reinterpret_cast<const float4 *>(table + (int64_t)id * t_s0);
        float4 *dst = reinterpret_cast<float4 *>(out + (int64_t)row * d);
        for (int j = threadIdx.x; j < d / 4; j += blockDim.x) dst[j] = ok ? src[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x)
            out[(int64_t)row * d + j] = ok ? table[(int64_t)id * t_s0 + (int64_t)j * t_s1] : 0.f;
    }
}

// Scatter-add with duplicate ids, deterministic and in the order of the reference's serial loop
// (src/embedding.c:37-43): the occurrences of every id are bucketed (count, scan, fill), and one
// CTA per id adds the rows of its occurrences in ascending position.  The only atomics are integer
// counters whose final values do not depend on the order of arrival.
__global__ void emb_count_kernel(const int *__restrict__ ids, int n, int vocab, int *__restrict__ count) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int id = ids[i];
    if (id >= 0 && id < vocab) atomicAdd(&count[id], 1);
}
// start[v] = sum of count[0..v).  One CTA of 1024 threads walks the vocabulary in tiles of 1024 with coalesced
// loads; inside a tile the counts are scanned with warp shuffles (lanes, then the 32 warp totals), and a running
// total carries over from tile to tile.
__global__ void __launch_bounds__(1024) emb_scan_kernel(const int *__restrict__ count, int vocab, int *__restrict__ start) {
    __shared__ int warp_tot[32];
    __shared__ int tile_total;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int carry = 0;                                        // the same value in every thread
    for (int base = 0; base < vocab; base += 1024) {
        const int v = base + threadIdx.x;
        const int c = v < vocab ? count[v] : 0;
        int incl = c;
        for (int o = 1; o < 32; o <<= 1) { int t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
        if (lane == 31) warp_tot[wid] = incl;
        __syncthreads();
        if (wid == 0) {
            int w = warp_tot[lane], wi = w;
            for (int o = 1; o < 32; o <<= 1) { int t = __shfl_up_sync(0xffffffffu, wi, o); if (lane >= o) wi += t; }
            warp_tot[lane] = wi - w;                      // exclusive prefix of the warp totals
            if (lane == 31) tile_total = wi;
        }
        __syncthreads();
        if (v < vocab) start[v] = carry + warp_tot[wid] + incl - c;
        carry += tile_total;
        __syncthreads();                                  // warp_tot and tile_total are rewritten by the next tile
    }
}
__global__ void emb_fill_kernel(const int *__restrict__ ids, int n, int vocab, const int *__restrict__ start,
                                int *__restrict__ cursor, int *__restrict__ list) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int id = ids[i];
    if (id >= 0 && id < vocab) list[start[id] + atomicAdd(&cursor[id], 1)] = i;
}
// One CTA per POSITION; the CTA whose position is the first occurrence of its id does the id's work and
// the others leave at once, so the grid is as large as the batch, not as the vocabulary, and no CTA is
// launched for a table row nobody looked up.  The bucket of an id is in arrival order: it is sorted in
// shared memory (rank = number of smaller positions; positions are distinct), then the rows of the
// upstream gradient are added in ascending position -- the order of the reference's serial loop
// (src/embedding.c:37-43) -- in registers, with one 128-bit read-modify-write of the table row at the end.
constexpr int kEmbBucket = 1024;       // occurrences of one id that are sorted in shared memory
__global__ void __launch_bounds__(128) embedding_bwd_kernel(float *__restrict__ tg, const float *__restrict__ g,
                                                            const int *__restrict__ ids, const int *__restrict__ count,
                                                            const int *__restrict__ start, const int *__restrict__ list,
                                                            int vocab, int d, int64_t g_s0, int64_t t_s0, int64_t t_s1, int vec) {
    __shared__ int sorted[kEmbBucket];
    __shared__ int sh[4];
    const int me = blockIdx.x, id = ids[me];
    if (id < 0 || id >= vocab) return;
    const int k = count[id];
    const int *mine = list + start[id];
    if (k == 1) { if (threadIdx.x == 0) sorted[0] = me; }
    else if (k <= kEmbBucket) {
        int leader = 1;
        for (int j = threadIdx.x; j < k; j += blockDim.x) {
            const int p = __ldg(mine + j);
            if (p < me) leader = 0;
        }
        if (!__syncthreads_and(leader)) return;                  // an earlier position of this id does the work
        for (int j = threadIdx.x; j < k; j += blockDim.x) {
            const int p = __ldg(mine + j);
            int rank = 0;
            for (int q = 0; q < k; q++) rank += __ldg(mine + q) < p;
            sorted[rank] = p;
        }
    } else {
        int leader = 1;
        for (int j = threadIdx.x; j < k; j += blockDim.x) if (__ldg(mine + j) < me) leader = 0;
        if (!__syncthreads_and(leader)) return;
    }
    __syncthreads();
    float *row = tg + (int64_t)id * t_s0;
    if (k <= kEmbBucket) {
        if (vec) {
            float4 *r4 = reinterpret_cast<float4 *>(row);
            for (int c = threadIdx.x; c < d / 4; c += blockDim.x) {
                float4 a = r4[c];
                for (int it = 0; it < k; it++) {
                    const float4 x = __ldg(reinterpret_cast<const float4 *>(g + (int64_t)sorted[it] * g_s0) + c);
                    a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
                }
                r4[c] = a;
            }
        } else {
            for (int c = threadIdx.x; c < d; c += blockDim.x) {
                float a = row[(int64_t)c * t_s1];
                for (int it = 0; it < k; it++) a += g[(int64_t)sorted[it] * g_s0 + c];
                row[(int64_t)c * t_s1] = a;
            }
        }
        return;
    }
    // a bucket too long for shared memory: the next position to add is the smallest one above the last
    int last = -1;
    for (int it = 0; it < k; it++) {
        int best = 0x7fffffff;
        for (int j = threadIdx.x; j < k; j += blockDim.x) { int p = mine[j]; if (p > last && p < best) best = p; }
        for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
        if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = best;
        __syncthreads();
        best = sh[0];
        for (int w = 1; w < (int)(blockDim.x >> 5); w++) best = min(best, sh[w]);
        __syncthreads();
        last = best;
        const float *gr = g + (int64_t)last * g_s0;
        if (vec) {
            const float4 *g4 = reinterpret_cast<const float4 *>(gr);
            float4 *r4 = reinterpret_cast<float4 *>(row);
            for (int c = threadIdx.x; c < d / 4; c += blockDim.x) {
                float4 a = r4[c], x = g4[c];
                r4[c] = make_float4(a.x + x.x, a.y + x.y, a.z + x.z, a.w + x.w);
            }
        } else {
            for (int c = threadIdx.x; c < d; c += blockDim.x) row[(int64_t)c * t_s1] += gr[c];
        }
    }
}

static void embedding_backward(grad_fn *fn, tensor *go) {
    tensor *table = fn->inputs[0];
    tensor *ids = fn->saved_tensors[0];
    if (!wants_grad(table)) return;
    int n = ids->shape[0], d = table->shape[1], vocab = table->shape[0];
    if (n <= 0 || vocab <= 0) return;
    float *tg = _grad_ensure(table);
    const int *idp = (const int *)ids->data;
    int *count = (int *)dev_alloc(fn->pool, (size_t)vocab * 2 * sizeof(int), true);      // count | cursor, zeroed
    int *cursor = count + vocab;
    int *start = (int *)dev_alloc(fn->pool, (size_t)vocab * sizeof(int), false);
    int *list = (int *)dev_alloc(fn->pool, (size_t)n * sizeof(int), false);
    emb_count_kernel<<<(n + 255) / 256, 256, 0, stream()>>>(idp, n, vocab, count);
    LAUNCHED("emb_count_kernel");
    emb_scan_kernel<<<1, 1024, 0, stream()>>>(count, vocab, start);
    LAUNCHED("emb_scan_kernel");
    emb_fill_kernel<<<(n + 255) / 256, 256, 0, stream()>>>(idp, n, vocab, start, cursor, list);
    LAUNCHED("emb_fill_kernel");
    const float *gd = (const float *)go->data;
    int vec = table->strides[1] == 1 && d % 4 == 0 && table->strides[0] % 4 == 0 && go->strides[0] % 4 == 0 &&
              aligned16(tg) && aligned16(gd);
    embedding_bwd_kernel<<<n, 128, 0, stream()>>>(tg, gd, idp, count, start, list, vocab, d, go->strides[0], table->strides[0],
                                                  table->strides[1], vec);
    prof_work(8.0 * n * d);                                      // read the upstream rows; the touched table rows are at most as many again
    LAUNCHED("embedding_bwd_kernel");
}

}  // namespace dnnb

using namespace dnnb;

extern "C" {

tensor *tensor_rope(struct mem_pool *scratch, tensor *x, const tensor *freqs_cos, const tensor *freqs_sin) {
    require_device_payloads("tensor_rope", {x, freqs_cos, freqs_sin});
    DNN_CHECK(x && freqs_cos && freqs_sin, "tensor_rope: NULL argument");
    DNN_CHECK(x->contiguous && freqs_cos->contiguous && freqs_sin->contiguous, "tensor_rope: operands must be contiguous");
    DNN_CHECK(x->ndim >= 2, "tensor_rope: x must have at least 2 dims");
    int d = x->shape[x->ndim - 1], N = x->shape[x->ndim - 2];
    DNN_CHECK(d % 2 == 0, "tensor_rope: last dim must be even");
    DNN_CHECK(freqs_cos->ndim == 2 && freqs_cos->shape[0] == N && freqs_cos->shape[1] == d / 2, "tensor_rope: cos table shape");
    DNN_CHECK(freqs_sin->ndim == 2 && freqs_sin->shape[0] == N && freqs_sin->shape[1] == d / 2, "tensor_rope: sin table shape");
    rope_run(false, (float *)x->data + x->offset, nullptr, (const float *)freqs_cos->data + freqs_cos->offset,
             (const float *)freqs_sin->data + freqs_sin->offset, numel_of(x), N, d);
    // The result shares x's payload but is its own autograd node with its own
    // gradient buffer (src/rope.c:117-126).
    tensor *out = (tensor *)_mem_pool_alloc(scratch, sizeof(tensor), x);
    out->parent = nullptr; out->grad_fn = nullptr; out->grad = nullptr;
    if (dnn_grad_enabled() && x->requires_grad) {
        grad_fn *fn = attach(scratch, out, rope_backward, 1, 2);
        fn->inputs[0] = x;
        fn->saved_tensors[0] = (tensor *)freqs_cos;
        fn->saved_tensors[1] = (tensor *)freqs_sin;
    }
    return out;
}

void tensor_rope_freqs_init(struct mem_pool *params, tensor **freqs_cos, tensor **freqs_sin,
                            int dim, int max_seq_len, float base) {
    DNN_CHECK(dim > 0 && dim % 2 == 0 && max_seq_len > 0, "tensor_rope_freqs_init: bad dims");
    if (base == 0.0f) base = 10000.0f;
    int dh = dim / 2;
    int shape[2] = {max_seq_len, dh};
    *freqs_cos = tensor_zeros(params, 2, shape, 0);
    *freqs_sin = tensor_zeros(params, 2, shape, 0);
    // Tables are computed on the host with libm, exactly as the reference does
    // (src/rope.c:163-169), then uploaded: bit-identical tables.
    std::vector<float> c((size_t)max_seq_len * dh), s((size_t)max_seq_len * dh);
    for (int k = 0; k < dh; k++) {
        float theta = powf(base, -2.0f * k / (float)dim);
        for (int n = 0; n < max_seq_len; n++) {
            float angle = (float)n * theta;
            c[(size_t)n * dh + k] = cosf(angle);
            s[(size_t)n * dh + k] = sinf(angle);
        }
    }
    dnn_cuda_upload(*freqs_cos, c.data(), c.size() * 4);
    dnn_cuda_upload(*freqs_sin, s.data(), s.size() * 4);
}

tensor *tensor_split_heads(struct mem_pool *scratch, tensor *t, int H) {
    require_device_payloads("tensor_split_heads", {t});
    DNN_CHECK(t->ndim == 3, "split_heads: input must be 3D [B, N, H*d_k]");
    DNN_CHECK(t->contiguous, "split_heads: input must be contiguous");
    int B = t->shape[0], N = t->shape[1], D = t->shape[2];
    DNN_CHECK(H > 0 && D % H == 0, "split_heads: D must be divisible by H");
    int dk = D / H;
    int shape[4] = {B, H, N, dk};
    tensor *out = tensor_scratch(scratch, 4, shape, 0);
    permute<0>("split_heads_fwd_kernel", (float *)out->data, (float *)t->data + t->offset, B, H, N, dk, (int64_t)N * D, dk, D);
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, out, split_heads_backward, 1, 1);
        fn->inputs[0] = t;
        int *h = host_alloc_t<int>(scratch); *h = H;
        fn->saved_tensors[0] = (tensor *)h;
    }
    return out;
}

tensor *tensor_merge_heads(struct mem_pool *scratch, tensor *t) {
    require_device_payloads("tensor_merge_heads", {t});
    DNN_CHECK(t->ndim == 4, "merge_heads: input must be 4D [B, H, N, d_k]");
    DNN_CHECK(t->contiguous, "merge_heads: input must be contiguous");
    int B = t->shape[0], H = t->shape[1], N = t->shape[2], dk = t->shape[3];
    int shape[3] = {B, N, H * dk};
    tensor *out = tensor_scratch(scratch, 3, shape, 0);
    permute<0>("merge_heads_fwd_kernel", (float *)out->data, (float *)t->data + t->offset, B, N, H, dk,
               (int64_t)H * N * dk, dk, (int64_t)N * dk);
    if (dnn_grad_enabled() && t->requires_grad) {
        grad_fn *fn = attach(scratch, out, merge_heads_backward, 1, 0);
        fn->inputs[0] = t;
    }
    return out;
}

void tensor_split_qkv_heads(struct mem_pool *scratch, tensor *qkv, int H,
                            tensor **Qh_out, tensor **Kh_out, tensor **Vh_out) {
    require_device_payloads("tensor_split_qkv_heads", {qkv});
    DNN_CHECK(qkv->ndim == 3, "split_qkv_heads: qkv must be 3D [B,N,3*H*d_k]");
    DNN_CHECK(qkv->contiguous, "split_qkv_heads: qkv must be contiguous");
    int B = qkv->shape[0], N = qkv->shape[1], D = qkv->shape[2];
    DNN_CHECK(D % (3 * H) == 0, "split_qkv_heads: D must be 3*H*d_k");
    int dk = D / (3 * H);
    int shape[4] = {B, H, N, dk};
    tensor *outs[3];
    for (int i = 0; i < 3; i++) outs[i] = tensor_scratch(scratch, 4, shape, 0);
    for (int i = 0; i < 3; i++)
        permute<0>("split_qkv_fwd_kernel", (float *)outs[i]->data, (float *)qkv->data + qkv->offset + (int64_t)i * H * dk,
                   B, H, N, dk, (int64_t)N * D, dk, D);
    if (dnn_grad_enabled() && qkv->requires_grad) {
        for (int i = 0; i < 3; i++) {
            grad_fn *fn = attach(scratch, outs[i], split_qkv_heads_backward, 1, 1);
            fn->inputs[0] = qkv;
            int *idx = host_alloc_t<int>(scratch); *idx = i;
            fn->saved_tensors[0] = (tensor *)idx;
        }
    }
    *Qh_out = outs[0]; *Kh_out = outs[1]; *Vh_out = outs[2];
}

tensor *tensor_embedding(struct mem_pool *scratch, const tensor *table, const tensor *ids) {
    require_device_payloads("tensor_embedding", {table, ids});
    DNN_CHECK(table && ids, "embedding: NULL argument");
    DNN_CHECK(table->ndim == 2, "embedding: table must be 2D");
    DNN_CHECK(ids->ndim == 1, "embedding: ids must be 1D");
    DNN_CHECK(table->contiguous, "embedding: table must be contiguous");
    int vocab = table->shape[0], d = table->shape[1], n = ids->shape[0];
    int shape[2] = {n, d};
    tensor *out = tensor_scratch(scratch, 2, shape, 0);
    if (n > 0) {
        const float *td = (const float *)table->data;     // the reference ignores table->offset here
        int vec = d % 4 == 0 && aligned16(td) && aligned16(out->data) && table->strides[1] == 1 && table->strides[0] % 4 == 0;
        embedding_fwd_kernel<<<n, 128, 0, stream()>>>((float *)out->data, td, (const int *)ids->data, n, d, vocab,
                                                      table->strides[0], table->strides[1], vec);
        LAUNCHED("embedding_fwd_kernel");
    }
    if (dnn_grad_enabled() && table->requires_grad) {
        grad_fn *fn = attach(scratch, out, embedding_backward, 1, 1);
        fn->inputs[0] = (tensor *)table;
        fn->saved_tensors[0] = (tensor *)ids;
    }
    return out;
}

}  // extern "C"
