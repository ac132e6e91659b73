// Evaluation-only generation for the decoder LM and the vision LM: KV cache, cached transformer
// block, sampling helpers, decoder_lm_generate and vision_lm_generate.  replaces
// src/transformer.c:28-112,211-416, src/gpt.c:220-421 and src/vlm.c:436-611 of the reference.
//
// No tape is built (generation runs with gradients off).  The cache lives in device memory as
// [B,H,max_seq,d]; a step projects the new tokens, rotates Q and K at their absolute positions,
// appends K and V to the cache with one strided device copy each, and runs attention of the new
// queries against everything cached.  That attention has N_new queries (usually one) against S
// keys, so it is a small bandwidth-bound kernel of its own: one CTA per query row, scores in
// shared memory.  Differences from the reference that do not change a token: the prompt is
// pre-filled in one pass instead of token by token; logits travel to the host once per token for
// the reference's own sampling arithmetic and random stream.
#include "common.cuh"
#include "device_utils.cuh"
#include <vector>

namespace dnnb {

constexpr int kEosId = 258;      // TOKENIZER_EOS_ID of the reference (include/tokenizer.h:24)

// One CTA per (query i, head, batch).  visible(i) = first index the query may NOT see.
// q: [B,H,Nn,d] packed; k,v: cache with row stride d and head/batch strides; out: [B,H,Nn,d] packed.
__global__ void attn_cached_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                   float *__restrict__ out, int H, int Nn, int S, int d, int64_t k_sb, int64_t k_sh,
                                   int old_seq, int prefix, float scale) {
    extern __shared__ float sc[];                 // S scores, then 32 floats of reduction scratch
    float *red = sc + S;
    const int i = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int gq = old_seq + i;
    int vis = (prefix > 0 && gq < prefix) ? prefix : gq + 1;
    if (vis > S) vis = S;
    const float *qr = q + (((int64_t)b * H + h) * Nn + i) * d;
    const float *kb = k + (int64_t)b * k_sb + (int64_t)h * k_sh;
    const float *vb = v + (int64_t)b * k_sb + (int64_t)h * k_sh;
    float mx = -INFINITY;
    for (int j = threadIdx.x; j < vis; j += blockDim.x) {
        const float *kr = kb + (int64_t)j * d;
        float s = 0.f;
        for (int c = 0; c < d; c++) s += qr[c] * kr[c];
        s *= scale;
        sc[j] = s;
        mx = fmaxf(mx, s);
    }
    mx = block_max(mx, red);
    float se = 0.f;
    for (int j = threadIdx.x; j < vis; j += blockDim.x) { float e = expf(sc[j] - mx); sc[j] = e; se += e; }
    se = block_sum(se, red);
    __syncthreads();
    const float inv = 1.0f / se;
    float *orow = out + (((int64_t)b * H + h) * Nn + i) * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < vis; j++) acc += sc[j] * vb[(int64_t)j * d + c];
        orow[c] = acc * inv;
    }
}

// One decoding step of one block's attention for ONE new token per sequence, with the position read from device
// memory so that the launch does not depend on it (and a whole token step can be replayed as a graph).  CTA (h, b):
// takes the token's q, k, v from the fused projection [B, 3*H*d], rotates q and k at position pos (the arithmetic
// of tensor_rope), appends k and v to the cache at row pos, attends over rows 0..pos and writes the head's d outputs
// token-major into out[B, H*d] -- what split_qkv_heads, two rope passes, two cache copies, attn_cached_kernel and
// merge_heads do in seven launches, with the same arithmetic per element.
constexpr int kDecodeGroups = 16;      // key groups of the output sum (256 threads / (d / 4) column groups at d = 64)
__global__ void __launch_bounds__(256) decode_attn_kernel(const float *__restrict__ qkv, const float *__restrict__ fc, const float *__restrict__ fs,
                                   float *__restrict__ kc, float *__restrict__ vc, int64_t c_sb, int64_t c_sh,
                                   float *__restrict__ out, const int *__restrict__ pos_dev, int H, int d, int max_seq, float scale) {
    extern __shared__ __align__(16) float sc[];   // q (d, padded to 4), scores (max_seq, padded), reduction scratch (32), output partials (groups x d)
    const int dp = (d + 3) & ~3, sp = (max_seq + 3) & ~3;
    float *qs = sc, *scr = sc + dp, *red = scr + sp, *part = red + 32;
    const int h = blockIdx.x, b = blockIdx.y;
    const int pos = *pos_dev;
    if (pos < 0 || pos >= max_seq) return;        // a full cache is refused on the host; nothing is written out of range
    const int S = pos + 1;
    const float *tok = qkv + (int64_t)b * 3 * H * d + (int64_t)h * d;
    float *kb = kc + (int64_t)b * c_sb + (int64_t)h * c_sh, *vb = vc + (int64_t)b * c_sb + (int64_t)h * c_sh;
    const int dh = d >> 1;
    for (int m = threadIdx.x; m < dh; m += blockDim.x) {
        float q0 = tok[2 * m], q1 = tok[2 * m + 1], k0 = tok[(int64_t)H * d + 2 * m], k1 = tok[(int64_t)H * d + 2 * m + 1];
        if (fc) {
            const float c = fc[(int64_t)pos * dh + m], sn = fs[(int64_t)pos * dh + m];
            float ox, oy;
            rope_fwd_pair(q0, q1, c, sn, ox, oy); q0 = ox; q1 = oy;
            rope_fwd_pair(k0, k1, c, sn, ox, oy); k0 = ox; k1 = oy;
        }
        qs[2 * m] = q0; qs[2 * m + 1] = q1;
        kb[(int64_t)pos * d + 2 * m] = k0; kb[(int64_t)pos * d + 2 * m + 1] = k1;
    }
    if ((d & 1) && threadIdx.x == 0) {            // an odd last element has no partner and is not rotated
        qs[d - 1] = tok[d - 1];
        kb[(int64_t)pos * d + d - 1] = tok[(int64_t)H * d + d - 1];
    }
    for (int c = threadIdx.x; c < d; c += blockDim.x) vb[(int64_t)pos * d + c] = tok[(int64_t)2 * H * d + c];
    __syncthreads();                              // this CTA's own cache row is read back below
    // scores: a thread per key; with d a multiple of 4 its row is read as independent 128-bit loads
    const bool v4 = (d & 3) == 0 && ((c_sb | c_sh) & 3) == 0 && ((reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc)) & 15) == 0;
    float mx = -INFINITY;
    for (int j = threadIdx.x; j < S; j += blockDim.x) {
        const float *kr = kb + (int64_t)j * d;
        float s = 0.f;
        if (v4) {
            const float4 *k4 = reinterpret_cast<const float4 *>(kr), *q4 = reinterpret_cast<const float4 *>(qs);
#pragma unroll 8
            for (int c = 0; c < (d >> 2); c++) {
                const float4 kv = k4[c], qv = q4[c];
                s += qv.x * kv.x; s += qv.y * kv.y; s += qv.z * kv.z; s += qv.w * kv.w;
            }
        } else {
            for (int c = 0; c < d; c++) s += qs[c] * kr[c];
        }
        s *= scale;
        scr[j] = s;
        mx = fmaxf(mx, s);
    }
    mx = block_max(mx, red);
    float se = 0.f;
    for (int j = threadIdx.x; j < S; j += blockDim.x) { float e = expf(scr[j] - mx); scr[j] = e; se += e; }
    se = block_sum(se, red);
    __syncthreads();
    const float inv = 1.0f / se;
    float *orow = out + (int64_t)b * H * d + (int64_t)h * d;
    const int d4 = d >> 2;
    int groups = v4 && d4 > 0 ? (int)blockDim.x / d4 : 0;
    if (groups > kDecodeGroups) groups = kDecodeGroups;
    if (groups >= 2) {
        // output: thread (cg, kg) sums keys kg, kg + groups, ... for four adjacent columns; the groups' sums are added in order
        const int cg = threadIdx.x % d4, kg = threadIdx.x / d4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (kg < groups) {
#pragma unroll 4
            for (int j = kg; j < S; j += groups) {
                const float p = scr[j];
                const float4 v = *reinterpret_cast<const float4 *>(vb + (int64_t)j * d + 4 * cg);
                acc.x += p * v.x; acc.y += p * v.y; acc.z += p * v.z; acc.w += p * v.w;
            }
            *reinterpret_cast<float4 *>(part + (int64_t)kg * d + 4 * cg) = acc;
        }
        __syncthreads();
        for (int c = threadIdx.x; c < d; c += blockDim.x) {
            float a = 0.f;
            for (int g = 0; g < groups; g++) a += part[(int64_t)g * d + c];
            orow[c] = a * inv;
        }
    } else {
        for (int c = threadIdx.x; c < d; c += blockDim.x) {
            float acc = 0.f;
            for (int j = 0; j < S; j++) acc += scr[j] * vb[(int64_t)j * d + c];
            orow[c] = acc * inv;
        }
    }
}
__global__ void bump_pos_kernel(int *pos) { *pos += 1; }

}  // namespace dnnb

using namespace dnnb;

// One token through one block with the position in device memory (see decode_attn_kernel): x [B, 1, d_model].
static tensor *block_decode_step(struct mem_pool *scratch, transformer_block *block, const tensor *x, kv_cache *cache, const int *pos_dev) {
    const int B = x->shape[0], H = block->n_heads, d = block->d_k;
    tensor *h = rms_norm_forward(scratch, block->attn_norm, x);
    tensor *qkv = linear_forward(scratch, block->qkv_proj, h);
    int shape[3] = {B, 1, H * d};
    tensor *merged = tensor_scratch(scratch, 3, shape, 0);
    const bool rope = block->freqs_cos && block->freqs_sin;
    const tensor *kc = cache->k_cache, *vc = cache->v_cache;
    const size_t smem = ((size_t)d + cache->max_seq + 8 + 32 + (size_t)kDecodeGroups * d) * sizeof(float);
    DNN_CHECK(smem <= 200 * 1024, "decode step: sequence too long for the score buffer");
    static size_t smem_set = 0;
    if (smem > 48 * 1024 && smem > smem_set) {
        CUDA_OK(cudaFuncSetAttribute(decode_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        smem_set = 200 * 1024;
    }
    decode_attn_kernel<<<dim3(H, B), 256, smem, stream()>>>(
        (const float *)qkv->data + qkv->offset,
        rope ? (const float *)block->freqs_cos->data + block->freqs_cos->offset : nullptr,
        rope ? (const float *)block->freqs_sin->data + block->freqs_sin->offset : nullptr,
        (float *)kc->data + kc->offset, (float *)vc->data + vc->offset, kc->strides[0], kc->strides[1],
        (float *)merged->data, pos_dev, H, d, cache->max_seq, 1.0f / sqrtf((float)d));
    LAUNCHED("decode_attn_kernel");
    // the two residual additions ride in the reduction of the projection that feeds them: x + (a W + b)
    tensor *x1 = matmul_add_residual(scratch, merged, block->out_proj->weight, 0, block->out_proj->bias, x);
    h = rms_norm_forward(scratch, block->ffn_norm, x1);
    swiglu_ffn *f = block->ffn;
    // gate and up projection in one launch, SwiGLU in their reduction, when the weights are plain [K,N] matrices
    const tensor *wg = f->gate_proj->weight, *wu = f->up_proj->weight, *bg = f->gate_proj->bias, *bu = f->up_proj->bias;
    tensor *hidden = nullptr;
    if (wg->ndim == 2 && wu->ndim == 2 && wg->contiguous && wu->contiguous && wg->shape[0] == wu->shape[0] && wg->shape[1] == wu->shape[1] &&
        (!bg || bg->contiguous) && (!bu || bu->contiguous) && h->contiguous) {
        int fs[3] = {B, 1, wg->shape[1]};
        hidden = tensor_scratch(scratch, 3, fs, 0);
        if (!gemv_swiglu((const float *)h->data + h->offset, wg->shape[0], B, (const float *)wg->data + wg->offset,
                         bg ? (const float *)bg->data + bg->offset : nullptr, (const float *)wu->data + wu->offset,
                         bu ? (const float *)bu->data + bu->offset : nullptr, wg->shape[0], wg->shape[1], (float *)hidden->data))
            hidden = nullptr;
    }
    if (!hidden) {
        tensor *gate = linear_forward(scratch, f->gate_proj, h);
        tensor *up = linear_forward(scratch, f->up_proj, h);
        hidden = tensor_swiglu(scratch, gate, up);
    }
    return matmul_add_residual(scratch, hidden, f->down_proj->weight, 0, f->down_proj->bias, x1);
}

// Cached token steps until max_len or end-of-sequence; output[cur - 1] is the last token so far and the caches hold
// everything before it.
static void decode_tokens(struct mem_pool *scratch_pool, struct mem_pool *data_pool, decoder_lm *lm, std::vector<kv_cache *> &caches,
                          tensor *single, int *output, int &cur, int max_len, float temperature, std::vector<float> &logits_host) {
    const int V = lm->vocab_size, D = lm->d_model;
    int one_shape[1] = {1};
    // Token steps.  The position lives in device memory (decode_attn_kernel), the scratch pool hands out the
    // same addresses for every token, and the token id arrives in a fixed buffer, so nothing in a step
    // depends on a host value that changes: the first step runs eagerly (and grows whatever buffers need
    // growing), the second is recorded with stream capture, and every later token is one graph launch
    // between the upload of its id and the read-back of its logits.  DNN_CUDA_GEN_GRAPH=0: every step eager.
    const char *ge = getenv("DNN_CUDA_GEN_GRAPH");
    const bool want_graph = !(ge && ge[0] == '0');
    tensor *pos_t = tensor_zeros_data(data_pool, 1, one_shape);
    const int *pos_dev = (const int *)pos_t->data;
    int pos_host = caches[0]->seq_len;
    DNN_CHECK(dnn_cuda_upload(pos_t, &pos_host, sizeof(int)) == 0, "generate: upload failed");
    cudaGraph_t graph = nullptr; cudaGraphExec_t exec = nullptr;
    const float *logits_dev = nullptr;
    long long graph_kernels = 0;
    auto token_step = [&]() {                  // the kernels of one token; returns where its logits land
        tensor *emb = embedding_forward(scratch_pool, nullptr, lm->embed, single);
        int hs[3] = {1, 1, D};
        tensor *h = tensor_reshape(scratch_pool, emb, 3, hs);
        for (int i = 0; i < lm->n_layers; i++) h = block_decode_step(scratch_pool, lm->blocks[i], h, caches[(size_t)i], pos_dev);
        tensor *logits = decoder_lm_lm_head_forward(scratch_pool, lm, rms_norm_forward(scratch_pool, lm->norm, h));
        bump_pos_kernel<<<1, 1, 0, stream()>>>((int *)pos_t->data);
        LAUNCHED("bump_pos_kernel");
        return (const float *)logits->data + logits->offset;
    };
    int steps = 0;
    while (cur < max_len) {
        DNN_CHECK(caches[0]->seq_len < caches[0]->max_seq, "generate: cache full");
        DNN_CHECK(!lm->blocks[0]->freqs_cos || caches[0]->seq_len < lm->blocks[0]->freqs_cos->shape[0],
                  "generate: position beyond the rotary tables (decoder_lm_enable_rope max_seq_len)");
        DNN_CHECK(dnn_cuda_upload(single, &output[cur - 1], sizeof(int)) == 0, "generate: upload failed");
        if (exec) {
            DNN_CHECK(cudaGraphLaunch(exec, stream()) == cudaSuccess, "generate: graph launch failed");
            add_launches(graph_kernels);
        } else if (want_graph && steps == 1) {
            const long long before = dnn_cuda_launch_count();
            cudaError_t e = cudaStreamBeginCapture(stream(), cudaStreamCaptureModeThreadLocal);
            DNN_CHECK(e == cudaSuccess, "generate: cudaStreamBeginCapture failed");
            logits_dev = token_step();
            e = cudaStreamEndCapture(stream(), &graph);
            graph_kernels = dnn_cuda_launch_count() - before;
            add_launches(-graph_kernels);                  // recorded, not run
            mem_pool_reset(scratch_pool);
            if (e == cudaSuccess && graph && cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess) {
                DNN_CHECK(cudaGraphLaunch(exec, stream()) == cudaSuccess, "generate: graph launch failed");
                add_launches(graph_kernels);
            } else {                                       // recording refused: this and all later steps run eagerly
                cudaGetLastError();
                if (graph) { cudaGraphDestroy(graph); graph = nullptr; }
                exec = nullptr;
                logits_dev = token_step();
            }
        } else {
            logits_dev = token_step();
        }
        DNN_CHECK(dnn_cuda_memcpy_d2h(logits_host.data(), logits_dev, (size_t)V * sizeof(float)) == 0, "generate: cannot read logits");
        int next = temperature == 0.0f ? decoder_lm_argmax_token(logits_host.data(), V)
                                       : decoder_lm_sample_with_temp(logits_host.data(), V, temperature);
        if (!exec) mem_pool_reset(scratch_pool);
        for (int i = 0; i < lm->n_layers; i++) caches[(size_t)i]->seq_len += 1;
        steps++;
        output[cur++] = next;
        if (next == kEosId) break;
    }
    dnn_cuda_sync();
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    mem_pool_reset(scratch_pool);

}

extern "C" {

kv_cache *kv_cache_create(struct mem_pool *params_pool, int B, int H, int max_seq, int d_k) {
    DNN_CHECK(B > 0 && H > 0 && max_seq > 0 && d_k > 0, "kv_cache_create: sizes must be positive");
    kv_cache *kvc = host_alloc_t<kv_cache>(params_pool);
    int shape[4] = {B, H, max_seq, d_k};
    kvc->k_cache = tensor_zeros(params_pool, 4, shape, 0);
    kvc->v_cache = tensor_zeros(params_pool, 4, shape, 0);
    kvc->seq_len = 0;
    kvc->max_seq = max_seq;
    return kvc;
}

void kv_cache_append(kv_cache *kvc, const tensor *K_new, const tensor *V_new) {
    DNN_CHECK(kvc && K_new && V_new, "kv_cache_append: NULL argument");
    DNN_CHECK(K_new->ndim == 4 && V_new->ndim == 4, "kv_cache_append: inputs must be 4D [B, H, N, d_k]");
    DNN_CHECK(K_new->contiguous && V_new->contiguous, "kv_cache_append: inputs must be contiguous");
    int B = K_new->shape[0], H = K_new->shape[1], Nn = K_new->shape[2], D = K_new->shape[3];
    DNN_CHECK(B == kvc->k_cache->shape[0] && H == kvc->k_cache->shape[1] && D == kvc->k_cache->shape[3], "kv_cache_append: shape mismatch");
    DNN_CHECK(Nn == V_new->shape[2], "kv_cache_append: K/V seq len mismatch");
    DNN_CHECK(kvc->seq_len + Nn <= kvc->max_seq, "kv_cache_append: cache full");
    size_t row = (size_t)Nn * D * 4, pitch = (size_t)kvc->max_seq * D * 4;
    const tensor *src[2] = {K_new, V_new};
    tensor *dst[2] = {kvc->k_cache, kvc->v_cache};
    for (int t = 0; t < 2; t++)
        CUDA_OK(cudaMemcpy2DAsync((float *)dst[t]->data + dst[t]->offset + (size_t)kvc->seq_len * D, pitch,
                                  (const float *)src[t]->data + src[t]->offset, row, row, (size_t)B * H,
                                  cudaMemcpyDeviceToDevice, stream()));
    kvc->seq_len += Nn;
}

tensor *kv_cache_get_K(struct mem_pool *scratch, kv_cache *kvc) {
    DNN_CHECK(kvc && kvc->seq_len > 0, "kv_cache_get_K: empty cache");
    return tensor_slice(scratch, kvc->k_cache, 2, 0, kvc->seq_len);
}
tensor *kv_cache_get_V(struct mem_pool *scratch, kv_cache *kvc) {
    DNN_CHECK(kvc && kvc->seq_len > 0, "kv_cache_get_V: empty cache");
    return tensor_slice(scratch, kvc->v_cache, 2, 0, kvc->seq_len);
}

tensor *transformer_block_forward_cached_ex(struct mem_pool *scratch, transformer_block *block, const tensor *x, kv_cache *cache,
                                            attention_mode mode, int prefix_len) {
    DNN_CHECK(block && x && cache, "cached forward: NULL argument");
    DNN_CHECK(x->contiguous && x->ndim >= 2 && x->shape[x->ndim - 1] == block->d_model, "cached forward: x must be contiguous [.., N, d_model]");
    DNN_CHECK(!dnn_grad_enabled() || !x->requires_grad, "cached forward is evaluation-only: enter dnn_no_grad first");
    const int B = x->shape[0], Nn = x->shape[x->ndim - 2], H = block->n_heads, d = block->d_k;
    if (mode == ATTENTION_PREFIX_LM) DNN_CHECK(cache->seq_len == 0, "prefix-LM prefill requires an empty cache");
    DNN_CHECK(d <= 1024, "cached forward: head size too large");

    tensor *h = rms_norm_forward(scratch, block->attn_norm, x);
    tensor *qkv = linear_forward(scratch, block->qkv_proj, h);
    tensor *q, *k, *v;
    tensor_split_qkv_heads(scratch, qkv, H, &q, &k, &v);
    if (block->freqs_cos && block->freqs_sin) {          // new tokens sit at positions [seq_len, seq_len + Nn)
        tensor *fc = tensor_slice(scratch, block->freqs_cos, 0, cache->seq_len, Nn);
        tensor *fs = tensor_slice(scratch, block->freqs_sin, 0, cache->seq_len, Nn);
        q = tensor_rope(scratch, q, fc, fs);
        k = tensor_rope(scratch, k, fc, fs);
    }
    kv_cache_append(cache, k, v);
    const int S = cache->seq_len, old_seq = S - Nn;
    int shape[4] = {B, H, Nn, d};
    tensor *att = tensor_scratch(scratch, 4, shape, 0);
    size_t smem = ((size_t)S + 32) * sizeof(float);
    DNN_CHECK(smem <= 200 * 1024, "cached forward: sequence too long for the score buffer");
    static size_t smem_set = 0;
    if (smem > 48 * 1024 && smem > smem_set) {
        CUDA_OK(cudaFuncSetAttribute(attn_cached_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        smem_set = 200 * 1024;
    }
    const tensor *kc = cache->k_cache, *vc = cache->v_cache;
    attn_cached_kernel<<<dim3(Nn, H, B), 128, smem, stream()>>>(
        (const float *)q->data + q->offset, (const float *)kc->data + kc->offset, (const float *)vc->data + vc->offset,
        (float *)att->data, H, Nn, S, d, kc->strides[0], kc->strides[1], old_seq,
        mode == ATTENTION_PREFIX_LM ? prefix_len : 0, 1.0f / sqrtf((float)d));
    LAUNCHED("attn_cached_kernel");
    tensor *merged = tensor_merge_heads(scratch, att);
    tensor *proj = linear_forward(scratch, block->out_proj, merged);
    tensor *x1 = tensor_add(scratch, x, proj);
    h = rms_norm_forward(scratch, block->ffn_norm, x1);
    tensor *ffn = swiglu_ffn_forward(scratch, block->ffn, h);
    return tensor_add(scratch, x1, ffn);
}

tensor *transformer_block_forward_cached(struct mem_pool *scratch, transformer_block *block, const tensor *x, kv_cache *cache) {
    return transformer_block_forward_cached_ex(scratch, block, x, cache, ATTENTION_CAUSAL, 0);
}

// ── sampling on host logits, the reference's arithmetic and random stream (src/gpt.c:220-256) ──
int decoder_lm_argmax_token(const float *logits, int vocab_size) {
    int best = 0;
    float best_val = logits[0];
    for (int i = 1; i < vocab_size; i++)
        if (logits[i] > best_val) { best_val = logits[i]; best = i; }
    return best;
}

int decoder_lm_sample_with_temp(const float *logits, int vocab_size, float temp) {
    float inv_temp = 1.0f / temp, mx = -INFINITY;
    for (int i = 0; i < vocab_size; i++) { float v = logits[i] * inv_temp; if (v > mx) mx = v; }
    float sum = 0.0f;
    for (int i = 0; i < vocab_size; i++) sum += expf(logits[i] * inv_temp - mx);
    float r = dnn_rng_uniform(dnn_get_rng()), cum = 0.0f;
    for (int i = 0; i < vocab_size; i++) {
        cum += expf(logits[i] * inv_temp - mx) / sum;
        if (r < cum) return i;
    }
    return vocab_size - 1;
}

int *decoder_lm_generate(struct mem_pool *scratch_pool, struct mem_pool *data_pool, decoder_lm *lm, const tensor *prompt_ids,
                         int max_new_tokens, float temperature, int use_cache, int *n_out) {
    DNN_CHECK(lm && prompt_ids && n_out, "generate: NULL argument");
    DNN_CHECK(prompt_ids->ndim == 2 && prompt_ids->shape[0] == 1 && prompt_ids->contiguous, "generate: prompt_ids must be contiguous [1, N]");
    DNN_CHECK(max_new_tokens > 0 && temperature >= 0.0f, "generate: bad max_new_tokens / temperature");
    const int prompt_len = prompt_ids->shape[1], max_len = prompt_len + max_new_tokens, V = lm->vocab_size, D = lm->d_model;
    int *output = host_alloc_t<int>(data_pool, (size_t)max_len);                    // host ids, as in the reference
    DNN_CHECK(dnn_cuda_download(prompt_ids, output, (size_t)prompt_len * sizeof(int)) == 0, "generate: cannot read the prompt");
    int cur = prompt_len;
    std::vector<float> logits_host((size_t)V);
    dnn_grad_ctx ng = dnn_no_grad_enter();

    auto pick = [&](const tensor *logits, int row) {                               // logits [1, rows, V]
        const float *src = (const float *)logits->data + logits->offset + (size_t)row * V;
        DNN_CHECK(dnn_cuda_memcpy_d2h(logits_host.data(), src, (size_t)V * sizeof(float)) == 0, "generate: cannot read logits");
        return temperature == 0.0f ? decoder_lm_argmax_token(logits_host.data(), V)
                                   : decoder_lm_sample_with_temp(logits_host.data(), V, temperature);
    };

    if (use_cache && lm->n_layers > 0) {
        const int d_k = lm->blocks[0]->d_k, H = lm->blocks[0]->n_heads;
        size_t mark = mem_pool_mark(data_pool);                                     // caches are released at the end, output stays
        std::vector<kv_cache *> caches((size_t)lm->n_layers);
        for (int i = 0; i < lm->n_layers; i++) caches[(size_t)i] = kv_cache_create(data_pool, 1, H, max_len, d_k);
        int one_shape[1] = {1};
        tensor *single = tensor_zeros_data(data_pool, 1, one_shape);
        // prefill: the whole prompt in one pass (the reference feeds it token by token; same keys, same logits)
        {
            int pshape[1] = {prompt_len};
            tensor *pid = tensor_zeros_data(data_pool, 1, pshape);
            DNN_CHECK(dnn_cuda_upload(pid, output, (size_t)prompt_len * sizeof(int)) == 0, "generate: upload failed");
            tensor *emb = embedding_forward(scratch_pool, nullptr, lm->embed, pid);
            int hs[3] = {1, prompt_len, D};
            tensor *h = tensor_reshape(scratch_pool, emb, 3, hs);
            for (int i = 0; i < lm->n_layers; i++) h = transformer_block_forward_cached(scratch_pool, lm->blocks[i], h, caches[(size_t)i]);
            tensor *last = tensor_slice(scratch_pool, h, 1, prompt_len - 1, 1);
            tensor *lastc = tensor_contiguous(scratch_pool, last);
            tensor *logits = decoder_lm_lm_head_forward(scratch_pool, lm, rms_norm_forward(scratch_pool, lm->norm, lastc));
            int next = pick(logits, 0);
            mem_pool_reset(scratch_pool);
            output[cur++] = next;
            if (next == kEosId) goto done_cached;
        }
        decode_tokens(scratch_pool, data_pool, lm, caches, single, output, cur, max_len, temperature, logits_host);
done_cached:
        dnn_cuda_sync();
        mem_pool_release(data_pool, mark);
    } else {
        while (cur < max_len) {
            size_t mark = mem_pool_mark(data_pool);
            int ishape[2] = {1, cur};
            tensor *ids = tensor_zeros_data(data_pool, 2, ishape);
            DNN_CHECK(dnn_cuda_upload(ids, output, (size_t)cur * sizeof(int)) == 0, "generate: upload failed");
            tensor *logits = decoder_lm_forward(scratch_pool, lm, ids);
            int next = pick(logits, cur - 1);
            mem_pool_reset(scratch_pool);
            mem_pool_release(data_pool, mark);
            output[cur++] = next;
            if (next == kEosId) break;
        }
    }
    dnn_no_grad_exit(ng);
    *n_out = cur;
    return output;
}

// vision_lm_generate (src/vlm.c:436-611 of the reference): batch 1, image [1,C,H,W] or pre-patched
// [1,I,C*P*P].  With a cache the image tokens and the prompt are pre-filled together under the
// prefix-LM mask and the image embeddings go in WITHOUT the learned image positions (the reference's
// cached path calls vision_lm_image_embeds directly, src/vlm.c:505); without a cache every token
// reruns vision_lm_forward, which adds them.  Both behaviours are kept.
int *vision_lm_generate(struct mem_pool *scratch_pool, struct mem_pool *data_pool, vision_lm *vlm, const tensor *image,
                        const tensor *prompt_ids, int max_new_tokens, float temperature, int use_cache, int *n_out) {
    DNN_CHECK(vlm && image && prompt_ids && n_out, "vision_lm_generate: NULL argument");
    DNN_CHECK((image->ndim == 4 || image->ndim == 3) && image->shape[0] == 1 && image->contiguous,
              "vision_lm_generate: image must be contiguous [1,C,H,W] or [1,patches,patch_dim]");
    DNN_CHECK(prompt_ids->ndim == 2 && prompt_ids->shape[0] == 1 && prompt_ids->contiguous, "vision_lm_generate: prompt_ids must be contiguous [1, T]");
    DNN_CHECK(max_new_tokens > 0 && temperature >= 0.0f, "vision_lm_generate: bad max_new_tokens / temperature");
    decoder_lm *lm = vlm->lm;
    const int prompt_len = prompt_ids->shape[1], max_len = prompt_len + max_new_tokens;
    const int V = vlm->vocab_size, I = vlm->n_img_tokens;
    // the image moves to the data pool so that it survives the scratch resets between tokens
    tensor *img_keep = tensor_zeros_data(data_pool, image->ndim, image->shape);
    CUDA_OK(cudaMemcpyAsync(img_keep->data, (const float *)image->data + image->offset, (size_t)numel_of(image) * sizeof(float),
                            cudaMemcpyDeviceToDevice, stream()));
    int *output = host_alloc_t<int>(data_pool, (size_t)max_len);
    DNN_CHECK(dnn_cuda_download(prompt_ids, output, (size_t)prompt_len * sizeof(int)) == 0, "vision_lm_generate: cannot read the prompt");
    int cur = prompt_len;
    std::vector<float> logits_host((size_t)V);
    dnn_grad_ctx ng = dnn_no_grad_enter();

    auto pick = [&](const tensor *logits, int row) {
        const float *src = (const float *)logits->data + logits->offset + (size_t)row * V;
        DNN_CHECK(dnn_cuda_memcpy_d2h(logits_host.data(), src, (size_t)V * sizeof(float)) == 0, "vision_lm_generate: cannot read logits");
        return temperature == 0.0f ? decoder_lm_argmax_token(logits_host.data(), V)
                                   : decoder_lm_sample_with_temp(logits_host.data(), V, temperature);
    };

    if (use_cache && lm->n_layers > 0) {
        const int d_k = lm->blocks[0]->d_k, H = lm->blocks[0]->n_heads;
        size_t mark = mem_pool_mark(data_pool);
        std::vector<kv_cache *> caches((size_t)lm->n_layers);
        for (int i = 0; i < lm->n_layers; i++) caches[(size_t)i] = kv_cache_create(data_pool, 1, H, I + max_len, d_k);
        int one_shape[1] = {1};
        tensor *single = tensor_zeros_data(data_pool, 1, one_shape);
        int next;
        {   // prefill: image tokens and prompt in one prefix-LM pass
            tensor *img = vision_lm_image_embeds(scratch_pool, vlm, img_keep);
            tensor *txt = decoder_lm_token_embeds(scratch_pool, lm, prompt_ids);
            tensor *h = tensor_cat(scratch_pool, img, txt, 1);
            for (int i = 0; i < lm->n_layers; i++)
                h = transformer_block_forward_cached_ex(scratch_pool, lm->blocks[i], h, caches[(size_t)i], ATTENTION_PREFIX_LM, I);
            tensor *lastc = tensor_contiguous(scratch_pool, tensor_slice(scratch_pool, h, 1, I + prompt_len - 1, 1));
            tensor *logits = decoder_lm_lm_head_forward(scratch_pool, lm, rms_norm_forward(scratch_pool, lm->norm, lastc));
            next = pick(logits, 0);
            mem_pool_reset(scratch_pool);
            output[cur++] = next;
        }
        if (next != kEosId) decode_tokens(scratch_pool, data_pool, lm, caches, single, output, cur, max_len, temperature, logits_host);
        dnn_cuda_sync();
        mem_pool_release(data_pool, mark);
    } else {
        while (cur < max_len) {
            size_t mark = mem_pool_mark(data_pool);
            int ishape[2] = {1, cur};
            tensor *ids = tensor_zeros_data(data_pool, 2, ishape);
            DNN_CHECK(dnn_cuda_upload(ids, output, (size_t)cur * sizeof(int)) == 0, "vision_lm_generate: upload failed");
            tensor *logits = vision_lm_forward(scratch_pool, vlm, img_keep, ids);
            int next = pick(logits, I + cur - 1);
            mem_pool_reset(scratch_pool);
            mem_pool_release(data_pool, mark);
            output[cur++] = next;
            if (next == kEosId) break;
        }
    }
    dnn_no_grad_exit(ng);
    *n_out = cur;
    return output;
}

}  // extern "C"
