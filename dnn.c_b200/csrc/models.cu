// Model glue for the training path: transformer block, decoder LM, vision LM.
// Host code only; it composes the ops in the same order as the reference so
// that the autograd tape (and therefore every accumulation order between
// ops) is the same.
// replaces src/transformer.c:113-207, src/gpt.c:16-216,431-496, src/vlm.c:20-430.
#include "common.cuh"
#include <vector>
#include <string>

using namespace dnnb;

namespace {

// Fills a contiguous tensor with N(0, std) drawn from the default host RNG.
void init_normal(tensor *t, float std) {
    int64_t n = numel_of(t);
    std::vector<float> h((size_t)n);
    for (int64_t i = 0; i < n; i++) h[i] = dnn_rng_normal(dnn_get_rng()) * std;
    dnn_cuda_upload(t, h.data(), (size_t)n * 4);
    dnn_cuda_sync();
}
void init_zero(tensor *t) { k_fill((float *)t->data + t->offset, numel_of(t), 0.0f); }

void init_linears(module *m, float std, float residual_std) {
    for (module_item *it = m->items_head; it; it = it->next) {
        if (it->kind != MODULE_ITEM_CHILD) continue;
        module *child = it->as.child;
        if (strcmp(child->type_name, "linear") == 0) {
            linear *l = (linear *)child;
            bool residual = strstr(it->name, "out_proj") || strstr(it->name, "down_proj");
            if (l->weight && l->weight->contiguous) init_normal(l->weight, residual ? residual_std : std);
            init_zero(l->bias);
        } else {
            init_linears(child, std, residual_std);
        }
    }
}

struct StepTail { float gn; };

// backward -> [all-reduce] -> clip / norm -> AdamW; shared by every *_train_step
float finish_step(struct mem_pool *scratch, tensor *loss, adamw_opt *opt, float grad_clip, bool dp) {
    // data parallel: from the second step on the buckets of the gradient exchange are sent while
    // backward still runs; the first step (gradient buffers not allocated yet) exchanges afterwards
    if (dp) {
        int rc = dnn_cuda_dp_backward(scratch, loss, opt->params, opt->n_params);
        DNN_CHECK(rc == 0, "data-parallel gradient all-reduce failed");
    } else {
        dnn_backward(scratch, loss);
    }
    float gn = grad_clip > 0.0f ? clip_grad_norm(opt->params, opt->n_params, grad_clip)
                                : grad_norm(opt->params, opt->n_params);
    adamw_step(opt);
    return gn;
}

tensor *lm_step(struct mem_pool *scratch, decoder_lm *lm, const tensor *input_ids, const tensor *target,
                adamw_opt *opt, float grad_clip, float *gn_out, bool dp) {
    DNN_CHECK(lm && input_ids && target && opt, "train_step: NULL argument");
    DNN_CHECK(input_ids->ndim == 2 && input_ids->contiguous, "train_step: input_ids must be contiguous [B, N]");
    DNN_CHECK(input_ids->shape[1] >= 2, "train_step: need N >= 2");
    int N = input_ids->shape[1];
    adamw_zero_grad(opt);
    tensor *logits = decoder_lm_forward(scratch, lm, input_ids);
    tensor *shifted = tensor_slice(scratch, logits, 1, 0, N - 1);       // view [B, N-1, V]
    tensor *loss = tensor_cross_entropy(scratch, shifted, target, 2);
    float gn = finish_step(scratch, loss, opt, grad_clip, dp);
    if (gn_out) *gn_out = gn;
    return loss;
}

}  // namespace

extern "C" {

// ── transformer block (src/transformer.c:113-207) ────────────────────────
transformer_block *transformer_block_create(struct mem_pool *pool, int d_model, int n_heads, int d_k, int intermediate_size) {
    DNN_CHECK(d_model > 0 && n_heads > 0 && d_k > 0 && intermediate_size > 0, "transformer_block_create: sizes must be positive");
    DNN_CHECK(d_model == n_heads * d_k, "transformer_block_create: d_model must equal n_heads * d_k");
    transformer_block *b = host_alloc_t<transformer_block>(pool);
    module_init(&b->base, pool, "transformer_block");
    b->d_model = d_model; b->n_heads = n_heads; b->d_k = d_k;
    b->qkv_proj = linear_create(pool, d_model, 3 * n_heads * d_k);
    module_add_child(&b->base, "qkv_proj", &b->qkv_proj->base);
    b->out_proj = linear_create(pool, n_heads * d_k, d_model);
    module_add_child(&b->base, "out_proj", &b->out_proj->base);
    b->attn_norm = rms_norm_create(pool, d_model, 1e-5f);
    module_add_child(&b->base, "attn_norm", &b->attn_norm->base);
    b->ffn_norm = rms_norm_create(pool, d_model, 1e-5f);
    module_add_child(&b->base, "ffn_norm", &b->ffn_norm->base);
    b->ffn = swiglu_ffn_create(pool, d_model, intermediate_size);
    module_add_child(&b->base, "ffn", &b->ffn->base);
    b->freqs_cos = b->freqs_sin = nullptr;
    return b;
}

tensor *transformer_block_forward_ex(struct mem_pool *scratch, transformer_block *block, const tensor *x,
                                     attention_mode mode, int prefix_len, const int *seq_lens) {
    DNN_CHECK(block && x && x->ndim >= 2, "transformer_block_forward: bad input");
    DNN_CHECK(x->shape[x->ndim - 1] == block->d_model, "transformer_block_forward: last dim must be d_model");
    // attention sub-layer, pre-norm
    tensor *h = rms_norm_forward(scratch, block->attn_norm, x);
    // Tensor-core path: attention reads Q, K, V in place from qkv and writes token-major output;
    // the QKV projection applies RoPE to its Q and K columns in its epilogue.
    bool rope = block->freqs_cos && block->freqs_sin;
    bool fused = attention_from_qkv_applicable(h, block->n_heads, block->d_k, rope ? block->freqs_cos : nullptr,
                                               rope ? block->freqs_sin : nullptr);
    if (fused && rope)
        gemm_rope_epilogue_request((const float *)block->freqs_cos->data + block->freqs_cos->offset,
                                   (const float *)block->freqs_sin->data + block->freqs_sin->offset,
                                   h->shape[1], block->d_k, 2 * block->n_heads * block->d_k);
    tensor *qkv = linear_forward(scratch, block->qkv_proj, h);
    bool rotated = gemm_rope_epilogue_take();
    tensor *merged = fused ? attention_from_qkv(scratch, qkv, block->n_heads, rope ? block->freqs_cos : nullptr,
                                                rope ? block->freqs_sin : nullptr, mode, prefix_len, seq_lens, rotated)
                           : nullptr;
    DNN_CHECK(merged || !rotated, "transformer_block_forward: the projection rotated Q and K but the fused attention path refused");
    if (!merged) {
        tensor *q, *k, *v;
        tensor_split_qkv_heads(scratch, qkv, block->n_heads, &q, &k, &v);
        if (rope) {
            int N = q->shape[2];
            tensor *fc = tensor_slice(scratch, block->freqs_cos, 0, 0, N);
            tensor *fs = tensor_slice(scratch, block->freqs_sin, 0, 0, N);
            q = tensor_rope(scratch, q, fc, fs);
            k = tensor_rope(scratch, k, fc, fs);
        }
        tensor *att = tensor_attention_ex(scratch, q, k, v, nullptr, mode, prefix_len, seq_lens);
        merged = tensor_merge_heads(scratch, att);
    }
    // The two residual additions run in the epilogue of the projection that feeds them
    // (x + (a W + b), same roundings as the separate add) unless the op-by-op block is asked for.
    const bool fuse_residual = dnn_cuda_get_fused_attention() != 0;
    tensor *x1;
    if (fuse_residual) {
        x1 = matmul_add_residual(scratch, merged, block->out_proj->weight, 0, block->out_proj->bias, x);
    } else {
        tensor *proj = linear_forward(scratch, block->out_proj, merged);
        x1 = tensor_add(scratch, x, proj);
    }
    // feed-forward sub-layer, pre-norm
    h = rms_norm_forward(scratch, block->ffn_norm, x1);
    if (!fuse_residual) {
        tensor *ffn = swiglu_ffn_forward(scratch, block->ffn, h);
        return tensor_add(scratch, x1, ffn);
    }
    swiglu_ffn *f = block->ffn;
    tensor *gate = linear_forward(scratch, f->gate_proj, h);
    tensor *up = linear_forward(scratch, f->up_proj, h);
    tensor *hidden = tensor_swiglu(scratch, gate, up);
    return matmul_add_residual(scratch, hidden, f->down_proj->weight, 0, f->down_proj->bias, x1);
}

tensor *transformer_block_forward(struct mem_pool *scratch, transformer_block *block, const tensor *x) {
    return transformer_block_forward_ex(scratch, block, x, ATTENTION_CAUSAL, 0, nullptr);
}

// ── decoder LM (src/gpt.c) ────────────────────────────────────────────────
decoder_lm *decoder_lm_create(struct mem_pool *pool, int vocab_size, int d_model, int n_layers, int n_heads,
                              int d_k, int intermediate_size) {
    DNN_CHECK(vocab_size > 0 && d_model > 0 && n_layers > 0, "decoder_lm_create: sizes must be positive");
    DNN_CHECK(d_model == n_heads * d_k, "decoder_lm_create: d_model must equal n_heads * d_k");
    decoder_lm *lm = host_alloc_t<decoder_lm>(pool);
    module_init(&lm->base, pool, "decoder_lm");
    lm->d_model = d_model; lm->vocab_size = vocab_size; lm->n_layers = n_layers;
    lm->embed = embedding_create(pool, vocab_size, d_model);
    module_add_child(&lm->base, "embed", &lm->embed->base);
    lm->blocks = host_alloc_t<transformer_block *>(pool, n_layers);
    for (int i = 0; i < n_layers; i++) {
        lm->blocks[i] = transformer_block_create(pool, d_model, n_heads, d_k, intermediate_size);
        std::string nm = "blocks." + std::to_string(i);
        char *name = (char *)_mem_pool_alloc(pool, nm.size() + 1, nm.c_str());
        module_add_child(&lm->base, name, &lm->blocks[i]->base);
    }
    lm->norm = rms_norm_create(pool, d_model, 1e-5f);
    module_add_child(&lm->base, "norm", &lm->norm->base);
    // tied head: no weight of its own, only a bias (src/gpt.c:51-59)
    lm->lm_head = host_alloc_t<linear>(pool);
    module_init(&lm->lm_head->base, pool, "linear");
    lm->lm_head->in_features = d_model; lm->lm_head->out_features = vocab_size;
    lm->lm_head->weight = nullptr;
    lm->lm_head->bias = tensor_zeros(pool, 1, &vocab_size, 1);
    module_param(&lm->lm_head->base, "bias", lm->lm_head->bias);
    module_add_child(&lm->base, "lm_head", &lm->lm_head->base);
    return lm;
}

tensor *decoder_lm_token_embeds(struct mem_pool *scratch, decoder_lm *lm, const tensor *input_ids) {
    DNN_CHECK(lm && input_ids && input_ids->ndim == 2 && input_ids->contiguous, "token_embeds: input_ids must be contiguous [B, N]");
    int shape[3] = {input_ids->shape[0], input_ids->shape[1], lm->d_model};
    tensor *flat = tensor_flatten(scratch, (tensor *)input_ids);
    tensor *h = embedding_forward(scratch, nullptr, lm->embed, flat);
    return tensor_reshape(scratch, h, 3, shape);
}

tensor *decoder_lm_hidden_from_embeds_ex(struct mem_pool *scratch, decoder_lm *lm, const tensor *embeds,
                                         attention_mode mode, int prefix_len, const int *seq_lens) {
    DNN_CHECK(lm && embeds && embeds->ndim == 3 && embeds->shape[2] == lm->d_model, "hidden_from_embeds: embeds must be [B, S, D]");
    tensor *h = (tensor *)embeds;
    for (int i = 0; i < lm->n_layers; i++)
        h = transformer_block_forward_ex(scratch, lm->blocks[i], h, mode, prefix_len, seq_lens);
    return rms_norm_forward(scratch, lm->norm, h);
}
tensor *decoder_lm_hidden_from_embeds(struct mem_pool *scratch, decoder_lm *lm, const tensor *embeds) {
    return decoder_lm_hidden_from_embeds_ex(scratch, lm, embeds, ATTENTION_CAUSAL, 0, nullptr);
}
tensor *decoder_lm_lm_head_forward(struct mem_pool *scratch, decoder_lm *lm, const tensor *h) {
    return tensor_matmul_add(scratch, h, lm->embed->weight, 1, lm->lm_head->bias);
}
tensor *decoder_lm_forward_embeds_ex(struct mem_pool *scratch, decoder_lm *lm, const tensor *embeds,
                                     attention_mode mode, int prefix_len, const int *seq_lens) {
    tensor *h = decoder_lm_hidden_from_embeds_ex(scratch, lm, embeds, mode, prefix_len, seq_lens);
    return decoder_lm_lm_head_forward(scratch, lm, h);
}
tensor *decoder_lm_forward_embeds(struct mem_pool *scratch, decoder_lm *lm, const tensor *embeds) {
    return decoder_lm_forward_embeds_ex(scratch, lm, embeds, ATTENTION_CAUSAL, 0, nullptr);
}
tensor *decoder_lm_forward(struct mem_pool *scratch, decoder_lm *lm, const tensor *input_ids) {
    return decoder_lm_forward_embeds(scratch, lm, decoder_lm_token_embeds(scratch, lm, input_ids));
}

// target[b, :] = input_ids[b, 1:], as one strided device copy (src/gpt.c:155-174)
tensor *decoder_lm_shift_targets(struct mem_pool *pool, const tensor *input_ids) {
    DNN_CHECK(input_ids->ndim == 2 && input_ids->contiguous && input_ids->shape[1] >= 2, "shift_targets: input_ids must be contiguous [B, N>=2]");
    int B = input_ids->shape[0], N = input_ids->shape[1];
    int shape[2] = {B, N - 1};
    tensor *t = tensor_zeros_data(pool, 2, shape);
    CUDA_OK(cudaMemcpy2DAsync(t->data, (size_t)(N - 1) * 4, (const int *)input_ids->data + input_ids->offset + 1, (size_t)N * 4,
                              (size_t)(N - 1) * 4, B, cudaMemcpyDeviceToDevice, stream()));
    return t;
}

tensor *decoder_lm_train_step(struct mem_pool *scratch, decoder_lm *lm, const tensor *input_ids, const tensor *target,
                              adamw_opt *opt, float grad_clip, float *grad_norm_out) {
    return lm_step(scratch, lm, input_ids, target, opt, grad_clip, grad_norm_out, false);
}
tensor *dnn_cuda_dp_decoder_lm_train_step(struct mem_pool *scratch, decoder_lm *lm, const tensor *input_ids,
                                          const tensor *target, adamw_opt *opt, float grad_clip, float *grad_norm_out) {
    return lm_step(scratch, lm, input_ids, target, opt, grad_clip, grad_norm_out, dnn_cuda_dp_world_size() > 1);
}

// ── whole-step CUDA graph ────────────────────────────────────────────────
// The step's kernels, memsets and copies are recorded once with stream capture and replayed as
// one graph launch.  That works because nothing in a step depends on host values that change:
// the pools hand out the same addresses every time, the tape is only needed while recording, and
// the optimiser tail reads learning rate and bias corrections from device memory (optim.cu).
struct dnn_cuda_step_graph {
    cudaGraph_t graph; cudaGraphExec_t exec;
    OptGraph *og; adamw_opt *opt; tensor *loss;
    cudaGraphNode_t state_copy; // the node that brings learning rate and bias corrections in
    long long kernels;          // kernel launches recorded in the graph
};

dnn_cuda_step_graph *dnn_cuda_graph_capture_decoder_lm_step(struct mem_pool *scratch, decoder_lm *lm, const tensor *input_ids,
                                                            const tensor *target, adamw_opt *opt, float grad_clip) {
    DNN_CHECK(lm && input_ids && target && opt, "graph capture: NULL argument");
    DNN_CHECK(input_ids->ndim == 2 && input_ids->contiguous && input_ids->shape[1] >= 2, "graph capture: input_ids must be contiguous [B, N >= 2]");
    DNN_CHECK(dnn_cuda_dp_world_size() <= 1, "graph capture: not available with data parallelism");
    CUDA_OK(cudaStreamSynchronize(stream()));
    dnn_cuda_step_graph *sg = new dnn_cuda_step_graph();
    sg->opt = opt;
    sg->og = opt_graph_prepare(opt, grad_clip);
    const int N = input_ids->shape[1];
    const long long launches_before = dnn_cuda_launch_count();
    cudaError_t e = cudaStreamBeginCapture(stream(), cudaStreamCaptureModeThreadLocal);
    DNN_CHECK(e == cudaSuccess, "graph capture: cudaStreamBeginCapture failed");
    adamw_zero_grad(opt);
    tensor *logits = decoder_lm_forward(scratch, lm, input_ids);
    tensor *shifted = tensor_slice(scratch, logits, 1, 0, N - 1);
    sg->loss = tensor_cross_entropy(scratch, shifted, target, 2);
    dnn_backward(scratch, sg->loss);
    opt_graph_launch(sg->og, opt);
    e = cudaStreamEndCapture(stream(), &sg->graph);
    sg->kernels = dnn_cuda_launch_count() - launches_before;
    add_launches(-sg->kernels);                      // recorded, not run
    if (e != cudaSuccess || !sg->graph) {
        // typically a buffer that had to grow while recording: one eager step of the same shapes first
        fprintf(stderr, "dnn_b200: step graph capture failed (%s); run one eager training step of the same shapes before capturing\n",
                cudaGetErrorString(e));
        cudaGetLastError();
        opt_graph_destroy(sg->og);
        delete sg;
        return nullptr;
    }
    // find the copy node of the optimiser state: every replay redirects it to its own pinned slot
    size_t n_nodes = 0;
    CUDA_OK(cudaGraphGetNodes(sg->graph, nullptr, &n_nodes));
    std::vector<cudaGraphNode_t> nodes(n_nodes);
    CUDA_OK(cudaGraphGetNodes(sg->graph, nodes.data(), &n_nodes));
    sg->state_copy = nullptr;
    for (cudaGraphNode_t nd : nodes) {
        cudaGraphNodeType ty;
        CUDA_OK(cudaGraphNodeGetType(nd, &ty));
        if (ty != cudaGraphNodeTypeMemcpy) continue;
        cudaMemcpy3DParms mp;
        CUDA_OK(cudaGraphMemcpyNodeGetParams(nd, &mp));
        if (mp.dstPtr.ptr == opt_graph_state_dev(sg->og)) { sg->state_copy = nd; break; }
    }
    DNN_CHECK(sg->state_copy, "graph capture: the optimiser-state copy node was not recorded");
    e = cudaGraphInstantiate(&sg->exec, sg->graph, 0);
    DNN_CHECK(e == cudaSuccess, "graph capture: cudaGraphInstantiate failed");
    return sg;
}

int dnn_cuda_graph_replay(dnn_cuda_step_graph *sg, float *loss_out, float *grad_norm_out) {
    if (!sg) return -1;
    const void *state = opt_graph_advance(sg->og, sg->opt);
    if (cudaGraphExecMemcpyNodeSetParams1D(sg->exec, sg->state_copy, const_cast<void *>(opt_graph_state_dev(sg->og)), state,
                                           opt_graph_state_bytes(), cudaMemcpyHostToDevice) != cudaSuccess) return -3;
    if (cudaGraphLaunch(sg->exec, stream()) != cudaSuccess) return -2;
    opt_graph_launched(sg->og);
    add_launches(sg->kernels);
    int rc = 0;
    if (loss_out) rc |= dnn_cuda_memcpy_d2h(loss_out, (const float *)sg->loss->data + sg->loss->offset, sizeof(float));
    if (grad_norm_out) rc |= dnn_cuda_memcpy_d2h(grad_norm_out, opt_graph_norm(sg->og), sizeof(float));
    return rc;
}

void dnn_cuda_graph_destroy(dnn_cuda_step_graph *sg) {
    if (!sg) return;
    cudaStreamSynchronize(stream());
    if (sg->exec) cudaGraphExecDestroy(sg->exec);
    if (sg->graph) cudaGraphDestroy(sg->graph);
    opt_graph_destroy(sg->og);
    delete sg;
}

void decoder_lm_enable_rope(struct mem_pool *pool, decoder_lm *lm, int max_seq_len, float base) {
    DNN_CHECK(lm && max_seq_len > 0, "enable_rope: bad argument");
    int d_k = lm->blocks[0]->d_k;
    DNN_CHECK(d_k % 2 == 0, "enable_rope: head dim must be even");
    tensor *fc, *fs;
    tensor_rope_freqs_init(pool, &fc, &fs, d_k, max_seq_len, base);
    for (int i = 0; i < lm->n_layers; i++) { lm->blocks[i]->freqs_cos = fc; lm->blocks[i]->freqs_sin = fs; }
}

// src/gpt.c:431-477: embedding ~ N(0, 1/sqrt(D)); linear weights the same, with
// out_proj / down_proj scaled by 1/sqrt(2L); biases zero.  Draw order: the
// embedding first, then linears in registration order.
void decoder_lm_init_weights(decoder_lm *lm) {
    DNN_CHECK(lm, "init_weights: lm is NULL");
    float std = 1.0f / sqrtf((float)lm->d_model);
    float residual_std = std / sqrtf(2.0f * (float)lm->n_layers);
    init_normal(lm->embed->weight, std);
    init_linears(&lm->base, std, residual_std);
}
long long decoder_lm_num_parameters(decoder_lm *lm) { return module_num_parameters(&lm->base); }

// ── vision LM (src/vlm.c) ─────────────────────────────────────────────────
vision_lm *vision_lm_create(struct mem_pool *pool, int vocab_size, int d_model, int n_layers, int n_heads, int d_k,
                            int intermediate_size, int image_channels, int image_h, int image_w, int patch_size, int use_image_pos) {
    DNN_CHECK(image_h > 0 && image_w > 0 && patch_size > 0, "vision_lm_create: image sizes must be positive");
    DNN_CHECK(image_h % patch_size == 0 && image_w % patch_size == 0, "vision_lm_create: image must divide into patches");
    vision_lm *v = host_alloc_t<vision_lm>(pool);
    module_init(&v->base, pool, "vision_lm");
    v->vocab_size = vocab_size; v->d_model = d_model; v->image_channels = image_channels;
    v->image_h = image_h; v->image_w = image_w; v->patch_size = patch_size;
    v->patch_h = image_h / patch_size; v->patch_w = image_w / patch_size;
    v->n_img_tokens = v->patch_h * v->patch_w; v->use_image_pos = use_image_pos;
    v->patch_embed = conv2d_create(pool, image_channels, d_model, patch_size, patch_size, 0);
    module_add_child(&v->base, "patch_embed", &v->patch_embed->base);
    v->img_proj = linear_create(pool, image_channels * patch_size * patch_size, d_model);
    module_add_child(&v->base, "img_proj", &v->img_proj->base);
    v->lm = decoder_lm_create(pool, vocab_size, d_model, n_layers, n_heads, d_k, intermediate_size);
    module_add_child(&v->base, "lm", &v->lm->base);
    if (use_image_pos) {
        int shape[3] = {1, v->n_img_tokens, d_model};
        v->image_pos = tensor_zeros(pool, 3, shape, 1);
        module_param(&v->base, "image_pos", v->image_pos);
    }
    return v;
}

void vision_lm_init_weights(vision_lm *v) {
    DNN_CHECK(v, "vision_lm_init_weights: NULL");
    decoder_lm_init_weights(v->lm);
    init_normal(v->patch_embed->weight, sqrtf(1.0f / (float)(v->image_channels * v->patch_size * v->patch_size)));
    init_zero(v->patch_embed->bias);
    if (v->image_pos) init_normal(v->image_pos, 0.02f);
}
void vision_lm_enable_rope(struct mem_pool *pool, vision_lm *v, int max_text_len, float base) {
    decoder_lm_enable_rope(pool, v->lm, v->n_img_tokens + max_text_len, base);
}
long long vision_lm_num_parameters(vision_lm *v) { return module_num_parameters(&v->base); }

tensor *vision_lm_image_embeds(struct mem_pool *scratch, vision_lm *v, const tensor *images) {
    DNN_CHECK(v && images && images->contiguous, "image_embeds: images must be contiguous");
    int B = images->shape[0];
    if (images->ndim == 3) {            // pre-patched [B, I, C*P*P]
        DNN_CHECK(images->shape[1] == v->n_img_tokens, "image_embeds: patch count mismatch");
        DNN_CHECK(images->shape[2] == v->image_channels * v->patch_size * v->patch_size, "image_embeds: patch dim mismatch");
        return linear_forward(scratch, v->img_proj, images);
    }
    DNN_CHECK(images->ndim == 4 && images->shape[1] == v->image_channels && images->shape[2] == v->image_h &&
              images->shape[3] == v->image_w, "image_embeds: images must be [B, C, H, W]");
    tensor *x = conv2d_forward(scratch, v->patch_embed, images);
    x = tensor_transpose(scratch, x, 1, 2);
    x = tensor_transpose(scratch, x, 2, 3);
    x = tensor_contiguous(scratch, x);
    int shape[3] = {B, v->n_img_tokens, v->d_model};
    return tensor_reshape(scratch, x, 3, shape);
}

tensor *vision_lm_build_embeds(struct mem_pool *scratch, vision_lm *v, const tensor *images, const tensor *text_ids) {
    DNN_CHECK(v && images && text_ids && images->shape[0] == text_ids->shape[0], "build_embeds: batch mismatch");
    tensor *img = vision_lm_image_embeds(scratch, v, images);
    if (v->use_image_pos && v->image_pos) img = tensor_add(scratch, img, v->image_pos);
    tensor *txt = decoder_lm_token_embeds(scratch, v->lm, text_ids);
    return tensor_cat(scratch, img, txt, 1);
}

tensor *vision_lm_forward(struct mem_pool *scratch, vision_lm *v, const tensor *images, const tensor *text_ids) {
    tensor *e = vision_lm_build_embeds(scratch, v, images, text_ids);
    return decoder_lm_forward_embeds_ex(scratch, v->lm, e, ATTENTION_PREFIX_LM, v->n_img_tokens, nullptr);
}
tensor *vision_lm_forward_text_logits(struct mem_pool *scratch, vision_lm *v, const tensor *images, const tensor *text_ids) {
    tensor *logits = vision_lm_forward(scratch, v, images, text_ids);
    return tensor_slice(scratch, logits, 1, v->n_img_tokens, text_ids->shape[1]);
}
tensor *vision_lm_shift_targets(struct mem_pool *pool, const tensor *text_ids) { return decoder_lm_shift_targets(pool, text_ids); }

tensor *vision_lm_train_step(struct mem_pool *scratch, vision_lm *v, const tensor *images, const tensor *input_ids,
                             const tensor *target_ids, adamw_opt *opt, float grad_clip, float *grad_norm_out) {
    DNN_CHECK(v && images && input_ids && target_ids && opt, "vision_lm_train_step: NULL argument");
    DNN_CHECK(input_ids->ndim == 2 && target_ids->ndim == 2 && input_ids->shape[0] == target_ids->shape[0] &&
              input_ids->shape[1] == target_ids->shape[1], "vision_lm_train_step: ids/targets must both be [B, T]");
    adamw_zero_grad(opt);
    tensor *logits = vision_lm_forward_text_logits(scratch, v, images, input_ids);
    tensor *loss = tensor_cross_entropy(scratch, logits, target_ids, 2);
    float gn = finish_step(scratch, loss, opt, grad_clip, false);
    if (grad_norm_out) *grad_norm_out = gn;
    return loss;
}

tensor *vision_lm_loss_padded(struct mem_pool *scratch, vision_lm *v, const tensor *images, const tensor *input_ids,
                              const tensor *target_ids, const tensor *loss_mask, const int *text_lens) {
    DNN_CHECK(v && images && input_ids && target_ids && loss_mask && text_lens, "vision_lm_loss_padded: NULL argument");
    DNN_CHECK(input_ids->ndim == 2 && target_ids->ndim == 2 && loss_mask->ndim == 2, "vision_lm_loss_padded: ids, targets, mask must be [B, Tmax]");
    DNN_CHECK(input_ids->shape[1] == target_ids->shape[1] && input_ids->shape[1] == loss_mask->shape[1], "vision_lm_loss_padded: seq len mismatch");
    int B = input_ids->shape[0], Tmax = input_ids->shape[1], I = v->n_img_tokens;
    int *lens = host_alloc_t<int>(scratch, B);
    for (int b = 0; b < B; b++) lens[b] = I + (text_lens[b] > Tmax ? Tmax : text_lens[b]);
    tensor *e = vision_lm_build_embeds(scratch, v, images, input_ids);
    tensor *logits = decoder_lm_forward_embeds_ex(scratch, v->lm, e, ATTENTION_PREFIX_LM, I, lens);
    tensor *text = tensor_slice(scratch, logits, 1, I, Tmax);
    return tensor_cross_entropy_masked(scratch, text, target_ids, loss_mask, 2);
}

tensor *vision_lm_train_step_padded(struct mem_pool *scratch, vision_lm *v, const tensor *images, const tensor *input_ids,
                                    const tensor *target_ids, const tensor *loss_mask, const int *text_lens,
                                    adamw_opt *opt, float grad_clip, float *grad_norm_out) {
    DNN_CHECK(opt, "vision_lm_train_step_padded: opt is NULL");
    adamw_zero_grad(opt);
    tensor *loss = vision_lm_loss_padded(scratch, v, images, input_ids, target_ids, loss_mask, text_lens);
    float gn = finish_step(scratch, loss, opt, grad_clip, false);
    if (grad_norm_out) *grad_norm_out = gn;
    return loss;
}
// The same step with the gradient exchange between backward and clipping (the place of a DDP hook in
// src/vlm.c:348-381).  Every rank normalises its loss by its own mask sum; the gradients are averaged.
tensor *dnn_cuda_dp_vision_lm_train_step_padded(struct mem_pool *scratch, vision_lm *v, const tensor *images, const tensor *input_ids,
                                                const tensor *target_ids, const tensor *loss_mask, const int *text_lens,
                                                adamw_opt *opt, float grad_clip, float *grad_norm_out) {
    DNN_CHECK(opt, "dnn_cuda_dp_vision_lm_train_step_padded: opt is NULL");
    adamw_zero_grad(opt);
    tensor *loss = vision_lm_loss_padded(scratch, v, images, input_ids, target_ids, loss_mask, text_lens);
    float gn = finish_step(scratch, loss, opt, grad_clip, dnn_cuda_dp_world_size() > 1);
    if (grad_norm_out) *grad_norm_out = gn;
    return loss;
}

tensor *vision_lm_train_step_masked(struct mem_pool *scratch, vision_lm *v, const tensor *images, const tensor *input_ids,
                                    const tensor *target_ids, const tensor *loss_mask, adamw_opt *opt,
                                    float grad_clip, float *grad_norm_out) {
    DNN_CHECK(v && images && input_ids && target_ids && loss_mask && opt, "vision_lm_train_step_masked: NULL argument");
    adamw_zero_grad(opt);
    tensor *logits = vision_lm_forward_text_logits(scratch, v, images, input_ids);
    tensor *loss = tensor_cross_entropy_masked(scratch, logits, target_ids, loss_mask, 2);
    float gn = finish_step(scratch, loss, opt, grad_clip, false);
    if (grad_norm_out) *grad_norm_out = gn;
    return loss;
}

}  // extern "C"
