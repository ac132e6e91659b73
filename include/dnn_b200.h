/* dnn_b200.h — the C API of the dnn.c training hot path, served by CUDA kernels.
 *
 * Every type and function below has the same name, argument meaning and
 * x86-64 struct layout as the public interface of masc-it/dnn.c, so a caller
 * written against that library re-links against libdnn_b200.so unchanged.
 * The difference is where payloads live: `tensor.data` and `tensor.grad`
 * point into device memory (HBM); structs, shapes, tape nodes and saved
 * scalars stay in host memory inside the pool's `buffer`.  Host code that
 * wants to read or write payload bytes goes through dnn_cuda_upload() /
 * dnn_cuda_download() in dnn_cuda.h.
 *
 * The comment above each group names the reference interface it replaces
 * (path within the reference project : lines).
 */
#ifndef DNN_B200_H
#define DNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ───────────────────────── bump pools ─────────────────────────
 * replaces include/pool.h:6-21 and src/pool.c:8-57.
 * `buffer` holds host-side metadata; a device arena of the same capacity is
 * attached to the pool (keyed by `buffer`) and follows reset/mark/release. */
typedef struct mem_pool {
    char   *buffer;
    size_t  capacity;
    size_t  offset;
} mem_pool;

mem_pool mem_pool_create(size_t capacity);
void     mem_pool_destroy(mem_pool *pool);
void     mem_pool_reset(mem_pool *pool);
size_t   mem_pool_mark(mem_pool *pool);
void     mem_pool_release(mem_pool *pool, size_t mark);
/* host-side allocations: zero-filled (src == NULL) or copied from src */
void    *_mem_pool_alloc(struct mem_pool *pool, size_t bytes, const void *src);
void    *_mem_pool_alloc_nz(struct mem_pool *pool, size_t bytes);

/* replaces include/context.h:6-20 and src/context.c:5-35 */
typedef struct dnn_ctx {
    mem_pool *params;    /* weights, grads of weights, optimizer state */
    mem_pool *scratch;   /* activations, tape, activation grads; reset per step */
    mem_pool *data;      /* batch tensors */
} dnn_ctx;

int  dnn_ctx_init(dnn_ctx *ctx, size_t params_sz, size_t scratch_sz, size_t data_sz);
void dnn_ctx_reset_step(dnn_ctx *ctx);
void dnn_ctx_destroy(dnn_ctx *ctx);

/* ───────────────────────── host RNG ─────────────────────────
 * replaces include/rng.h:12-34 and src/rng.c:6-78 (xorshift128+ seeded by
 * SplitMix64; used for weight init, always on the host). */
typedef struct dnn_rng { uint64_t s[2]; } dnn_rng;
dnn_rng  dnn_rng_seed(uint64_t seed);
float    dnn_rng_uniform(dnn_rng *rng);
float    dnn_rng_normal(dnn_rng *rng);
int      dnn_rng_uniform_int(dnn_rng *rng, int n);
dnn_rng *dnn_get_rng(void);
void     dnn_seed(uint64_t seed);

/* ───────────────────────── tensors ─────────────────────────
 * replaces include/tensor.h:9-54 and src/tensor.c.  sizeof(tensor) == 120. */
#define DNN_MAX_DIMS 8
typedef struct grad_fn grad_fn;

typedef struct tensor {
    void    *data;                      /* device pointer (fp32 or int32 payload) */
    float   *grad;                      /* device pointer, lazily allocated, NULL until then */
    int      shape[DNN_MAX_DIMS];
    int      strides[DNN_MAX_DIMS];     /* in elements */
    int      ndim;
    unsigned int requires_grad : 1;
    unsigned int contiguous    : 1;
    unsigned int grad_fresh    : 1;     /* library-internal, in the same 32-bit unit as the two flags
                                           above: grad is allocated but not yet written (see _grad_ensure) */
    int      offset;                    /* in elements, from data */
    struct tensor *parent;              /* non-NULL for views */
    grad_fn *grad_fn;
    struct mem_pool *pool;              /* NULL for views */
} tensor;

tensor *tensor_zeros(struct mem_pool *pool, int ndim, const int *shape, int requires_grad);
tensor *tensor_zeros_data(struct mem_pool *pool, int ndim, const int *shape);
tensor *tensor_randn(struct mem_pool *pool, int ndim, const int *shape, int requires_grad);
tensor *tensor_uniform(struct mem_pool *pool, int ndim, const int *shape, int requires_grad, float bound);
tensor *tensor_scratch(struct mem_pool *pool, int ndim, const int *shape, int requires_grad);

tensor *tensor_slice(struct mem_pool *scratch, tensor *t, int dim, int start, int len);
tensor *tensor_transpose(struct mem_pool *scratch, tensor *t, int d1, int d2);
tensor *tensor_reshape(struct mem_pool *scratch, tensor *t, int ndim, const int *shape);
tensor *tensor_flatten(struct mem_pool *scratch, tensor *t);
tensor *tensor_contiguous(struct mem_pool *scratch, tensor *t);

float  *tensor_data_ptr(tensor *t);     /* device pointer: data + offset */
int     tensor_numel(const tensor *t);
int     tensor_ndim(const tensor *t);
int     tensor_shape(const tensor *t, int dim);
int     tensor_is_contiguous(const tensor *t);
int     tensor_requires_grad(const tensor *t);
void    tensor_set_requires_grad(tensor *t, int req);
int     tensor_is_leaf(const tensor *t);
void    tensor_retain_grad(tensor *t);
void    tensor_zero_grad(tensor *t);
float  *tensor_grad(const tensor *t);   /* device pointer or NULL */
tensor *tensor_root(tensor *t);
void    tensor_print(const tensor *t);  /* downloads up to 16 values */

/* ───────────────────────── autograd ─────────────────────────
 * replaces include/autograd.h:6-23, src/autograd_int.h:7-10, src/autograd.c.
 * sizeof(grad_fn) == 48. */
struct grad_fn {
    void     (*backward)(grad_fn *fn, tensor *grad_output);
    struct mem_pool *pool;
    tensor  **inputs;
    int       n_inputs;
    tensor  **saved_tensors;
    int       n_saved;
};
typedef struct { int _prev; } dnn_grad_ctx;

int          dnn_grad_enabled(void);
dnn_grad_ctx dnn_no_grad_enter(void);
void         dnn_no_grad_exit(dnn_grad_ctx ctx);
void         dnn_backward(struct mem_pool *scratch, tensor *loss);
grad_fn     *_grad_fn_create(struct mem_pool *pool);
float       *_grad_ensure(tensor *t);

/* ───────────────────────── ops ─────────────────────────
 * replaces include/ops.h:7-74.  Every op allocates its result in `scratch`,
 * launches on the library's compute stream and returns without waiting. */
tensor *tensor_add(struct mem_pool *scratch, const tensor *a, const tensor *b);              /* src/ops_elem.c:110-175 */
tensor *tensor_cat(struct mem_pool *scratch, const tensor *a, const tensor *b, int dim);     /* src/ops_elem.c:903-945 */
tensor *tensor_matmul(struct mem_pool *scratch, const tensor *a, const tensor *b);           /* src/ops_matrix.c:310-461 */
tensor *tensor_matmul_add(struct mem_pool *scratch, const tensor *a, const tensor *b,
                          int trans_b, const tensor *bias);                                   /* src/ops_matrix.c:964-1206 */
tensor *tensor_relu(struct mem_pool *scratch, const tensor *t);                              /* src/ops_activation.c:37-69 */
tensor *tensor_silu(struct mem_pool *scratch, const tensor *t);                              /* src/ops_activation.c:165-199 */
tensor *tensor_swiglu(struct mem_pool *scratch, const tensor *gate, const tensor *up);       /* src/ops_activation.c:283-333 */

/* The rest of include/ops.h: not used by the training path of the models, provided so that
 * programs written against the reference link unchanged.  Broadcasting as tensor_add. */
tensor *tensor_sub(struct mem_pool *scratch, const tensor *a, const tensor *b);              /* src/ops_elem.c:234-285 */
tensor *tensor_mul(struct mem_pool *scratch, const tensor *a, const tensor *b);              /* src/ops_elem.c:340-391 */
tensor *tensor_div(struct mem_pool *scratch, const tensor *a, const tensor *b);              /* src/ops_elem.c:452-500 */
tensor *tensor_neg(struct mem_pool *scratch, const tensor *t);                               /* src/ops_elem.c:588-625 */
tensor *tensor_pow(struct mem_pool *scratch, const tensor *t, float exp);                    /* src/ops_elem.c:526-570 */
tensor *tensor_triu(struct mem_pool *scratch, int N, int diagonal);                          /* src/ops_elem.c:643-658; 0 / -inf mask */
tensor *tensor_sigmoid(struct mem_pool *scratch, const tensor *t);                           /* src/ops_activation.c:94-125 */
tensor *tensor_softmax(struct mem_pool *scratch, const tensor *t, int dim);                  /* src/ops_activation.c:434-560 */
tensor *tensor_causal_softmax(struct mem_pool *scratch, const tensor *t);                    /* src/ops_activation.c:683-800 */
tensor *tensor_dropout(struct mem_pool *scratch, const tensor *t, float p);                  /* src/ops_activation.c:1446-1500; identity when gradients are off */
tensor *tensor_sum(struct mem_pool *scratch, const tensor *t, int dim);                      /* src/ops_reduce.c:57-136; keeps the reduced dim as 1 */
tensor *tensor_mean(struct mem_pool *scratch, const tensor *t, int dim);                     /* src/ops_reduce.c:138-153 */
tensor *tensor_cross_entropy(struct mem_pool *scratch, const tensor *logits,
                             const tensor *target, int dim);                                  /* src/ops_activation.c:948-1145 */
tensor *tensor_cross_entropy_masked(struct mem_pool *scratch, const tensor *logits,
                                    const tensor *target, const tensor *mask, int dim);       /* src/ops_activation.c:1245-1410 */
tensor *tensor_embedding(struct mem_pool *scratch, const tensor *table, const tensor *ids);  /* src/embedding.c:63-110 */
tensor *tensor_avg_pool2d(struct mem_pool *scratch, const tensor *x, int k, int stride);     /* src/ops_pool.c:249-381 */

/* replaces include/norm.h:19-36 (src/norm.c:178-277, 404-495) */
tensor *tensor_layer_norm(struct mem_pool *scratch, const tensor *x,
                          const tensor *weight, const tensor *bias, float eps);
tensor *tensor_rms_norm(struct mem_pool *scratch, const tensor *x,
                        const tensor *weight, float eps);

/* replaces include/attention.h:20-57 (src/attention.c:671-781) */
typedef enum attention_mode {
    ATTENTION_CAUSAL    = 0,
    ATTENTION_PREFIX_LM = 1
} attention_mode;
tensor *tensor_attention_ex(struct mem_pool *scratch, tensor *Q, tensor *K, tensor *V,
                            tensor *mask, attention_mode mode, int prefix_len,
                            const int *seq_lens /* host array [B] or NULL */);
tensor *tensor_attention(struct mem_pool *scratch, tensor *Q, tensor *K, tensor *V, tensor *mask);

/* replaces include/multihead.h:19-35 (src/multihead.c) */
tensor *tensor_split_heads(struct mem_pool *scratch, tensor *t, int H);
tensor *tensor_merge_heads(struct mem_pool *scratch, tensor *t);
void    tensor_split_qkv_heads(struct mem_pool *scratch, tensor *qkv, int H,
                               tensor **Qh_out, tensor **Kh_out, tensor **Vh_out);

/* replaces include/rope.h:27-47 (src/rope.c:92-171) */
tensor *tensor_rope(struct mem_pool *scratch, tensor *x,
                    const tensor *freqs_cos, const tensor *freqs_sin);
void    tensor_rope_freqs_init(struct mem_pool *params, tensor **freqs_cos, tensor **freqs_sin,
                               int dim, int max_seq_len, float base);

/* replaces include/conv.h:20-22 (src/conv.c:687-919) */
tensor *tensor_conv2d(struct mem_pool *scratch, tensor *input, tensor *weight, tensor *bias,
                      int stride, int pad);

/* ───────────────────────── optimiser ─────────────────────────
 * replaces include/optim.h (src/optim.c:67-316).  sizeof(adamw_opt) == 56. */
typedef struct adamw_opt {
    tensor  **params;
    int       n_params;
    float     lr;
    float     beta1, beta2;
    float     eps;
    float     weight_decay;
    int       t;
    tensor  **m, **v;
} adamw_opt;

adamw_opt *adamw_create(struct mem_pool *params_pool, tensor **params, int n_params, float lr,
                        float beta1, float beta2, float eps, float weight_decay);
void       adamw_free(adamw_opt *opt);
void       adamw_step(adamw_opt *opt);
void       adamw_step_with_lr_multipliers(adamw_opt *opt, const float *lr_mults);
void       adamw_zero_grad(adamw_opt *opt);
float      grad_norm(tensor **params, int n_params);                     /* one device->host sync */
float      clip_grad_norm(tensor **params, int n_params, float max_norm); /* one device->host sync */

#define LR_SCHEDULE_CONSTANT              0
#define LR_SCHEDULE_LINEAR_WARMUP_COSINE  1
#define LR_SCHEDULE_LINEAR_WARMUP         2
#define LR_SCHEDULE_COSINE                3
#define LR_SCHEDULE_STEP                  4
#define LR_SCHEDULE_EXPONENTIAL           5
typedef struct {
    struct adamw_opt *opt;
    int    schedule;
    float  base_lr;
    float  min_lr;
    int    warmup_iters;
    int    total_iters;
    int    step_size;
    float  gamma;
    int    t;
} lr_scheduler;
lr_scheduler *lr_scheduler_create(struct mem_pool *params_pool, struct adamw_opt *opt, int schedule,
                                  float base_lr, int warmup_iters, int total_iters, float min_lr,
                                  int step_size, float gamma);
void  lr_scheduler_step(lr_scheduler *sched);
float lr_scheduler_get_lr(const lr_scheduler *sched);
void  lr_scheduler_reset(lr_scheduler *sched);
void  lr_scheduler_destroy(lr_scheduler *sched);

/* ───────────────────────── modules and layers ─────────────────────────
 * replaces include/module.h and include/nn.h (src/module.c, src/nn.c).
 * sizeof(module) == 72, sizeof(linear) == 96. */
typedef enum module_item_kind { MODULE_ITEM_PARAM = 1, MODULE_ITEM_CHILD = 2 } module_item_kind;
typedef struct module_item {
    struct module_item *next;
    module_item_kind    kind;
    const char         *name;
    union { tensor *param; struct module *child; } as;
} module_item;
typedef struct module {
    struct mem_pool *pool;
    const char      *type_name;
    struct module   *parent;
    module_item     *items_head;
    module_item     *items_tail;
    int              n_items;
    int              n_direct_params;
    int              n_children;
    tensor         **flat_params;
    int              n_flat;
} module;

void      module_init(module *m, struct mem_pool *pool, const char *type_name);
void      module_param(module *m, const char *name, tensor *t);
void      module_add_child(module *m, const char *name, module *child);
tensor  **module_parameters(module *m, int *n_out);
long long module_num_parameters(module *m);
void      module_zero_grad(module *m);
tensor   *module_find_param(module *m, const char *name);
#define MODULE_STATE_MAX_NAME 4096
void      module_save(module *m, const char *path);               /* "DNNM" v1 file, weights only */
void      module_load(module *m, const char *path, int strict);

typedef struct linear     { module base; tensor *weight; tensor *bias; int in_features; int out_features; } linear;
typedef struct swiglu_ffn { module base; linear *gate_proj; linear *up_proj; linear *down_proj;
                            int d_model; int intermediate_size; } swiglu_ffn;
typedef struct layer_norm { module base; tensor *weight; tensor *bias; float eps; int d; } layer_norm;
typedef struct rms_norm   { module base; tensor *weight; float eps; int d; } rms_norm;
typedef struct embedding  { module base; tensor *weight; int vocab_size; int d_model; } embedding;
typedef struct conv2d     { module base; tensor *weight; tensor *bias; int in_channels; int out_channels;
                            int kernel_size; int stride; int padding; } conv2d;

linear     *linear_create(struct mem_pool *params, int in_features, int out_features);
tensor     *linear_forward(struct mem_pool *scratch, linear *l, const tensor *input);
swiglu_ffn *swiglu_ffn_create(struct mem_pool *params, int d_model, int intermediate_size);
tensor     *swiglu_ffn_forward(struct mem_pool *scratch, swiglu_ffn *ffn, const tensor *x);
layer_norm *layer_norm_create(struct mem_pool *params, int d, float eps);
tensor     *layer_norm_forward(struct mem_pool *scratch, layer_norm *ln, const tensor *x);
rms_norm   *rms_norm_create(struct mem_pool *params, int d, float eps);
tensor     *rms_norm_forward(struct mem_pool *scratch, rms_norm *rn, const tensor *x);
embedding  *embedding_create(struct mem_pool *params, int vocab_size, int d_model);
tensor     *embedding_forward(struct mem_pool *scratch, struct mem_pool *data, embedding *emb, const tensor *ids);
conv2d     *conv2d_create(struct mem_pool *params, int in_channels, int out_channels,
                          int kernel_size, int stride, int padding);
tensor     *conv2d_forward(struct mem_pool *scratch, conv2d *c, const tensor *input);

/* ───────────────────────── models (training path) ─────────────────────────
 * replaces the training entry points of include/transformer.h, include/gpt.h
 * and include/vlm.h (src/transformer.c:113-207, src/gpt.c:16-216,431-496,
 * src/vlm.c:20-430).  KV-cache generation and sampling are not provided. */
typedef struct {
    module      base;
    linear     *qkv_proj;
    linear     *out_proj;
    int         n_heads;
    int         d_k;
    int         d_model;
    rms_norm   *attn_norm;
    rms_norm   *ffn_norm;
    swiglu_ffn *ffn;
    tensor     *freqs_cos;
    tensor     *freqs_sin;
} transformer_block;

transformer_block *transformer_block_create(struct mem_pool *params_pool, int d_model, int n_heads,
                                            int d_k, int intermediate_size);
tensor *transformer_block_forward_ex(struct mem_pool *scratch, transformer_block *block, const tensor *x,
                                     attention_mode mode, int prefix_len, const int *seq_lens);
tensor *transformer_block_forward(struct mem_pool *scratch, transformer_block *block, const tensor *x);

/* KV cache and cached block forward for generation (evaluation only, no tape).
 * replaces include/transformer.h:26-128 (src/transformer.c:28-112,211-416).
 * k_cache / v_cache are [B, H, max_seq, d_k] device tensors. */
typedef struct {
    tensor *k_cache;
    tensor *v_cache;
    int     seq_len;
    int     max_seq;
} kv_cache;
kv_cache *kv_cache_create(struct mem_pool *params_pool, int B, int H, int max_seq, int d_k);
void      kv_cache_append(kv_cache *kvc, const tensor *K_new, const tensor *V_new);
tensor   *kv_cache_get_K(struct mem_pool *scratch, kv_cache *kvc);
tensor   *kv_cache_get_V(struct mem_pool *scratch, kv_cache *kvc);
tensor *transformer_block_forward_cached_ex(struct mem_pool *scratch, transformer_block *block, const tensor *x,
                                            kv_cache *cache, attention_mode mode, int prefix_len);
tensor *transformer_block_forward_cached(struct mem_pool *scratch, transformer_block *block, const tensor *x,
                                         kv_cache *cache);

typedef struct {
    module              base;
    embedding          *embed;
    transformer_block **blocks;
    int                 n_layers;
    rms_norm           *norm;
    linear             *lm_head;     /* weight == NULL: tied to embed->weight */
    int                 d_model;
    int                 vocab_size;
} decoder_lm;

decoder_lm *decoder_lm_create(struct mem_pool *params_pool, int vocab_size, int d_model,
                              int n_layers, int n_heads, int d_k, int intermediate_size);
tensor *decoder_lm_token_embeds(struct mem_pool *scratch, decoder_lm *lm, const tensor *input_ids);
tensor *decoder_lm_hidden_from_embeds_ex(struct mem_pool *scratch, decoder_lm *lm, const tensor *embeds,
                                         attention_mode mode, int prefix_len, const int *seq_lens);
tensor *decoder_lm_hidden_from_embeds(struct mem_pool *scratch, decoder_lm *lm, const tensor *embeds);
tensor *decoder_lm_lm_head_forward(struct mem_pool *scratch, decoder_lm *lm, const tensor *h);
tensor *decoder_lm_forward_embeds_ex(struct mem_pool *scratch, decoder_lm *lm, const tensor *embeds,
                                     attention_mode mode, int prefix_len, const int *seq_lens);
tensor *decoder_lm_forward_embeds(struct mem_pool *scratch, decoder_lm *lm, const tensor *embeds);
tensor *decoder_lm_forward(struct mem_pool *scratch, decoder_lm *lm, const tensor *input_ids);
tensor *decoder_lm_shift_targets(struct mem_pool *pool, const tensor *input_ids);
tensor *decoder_lm_train_step(struct mem_pool *scratch_pool, decoder_lm *lm, const tensor *input_ids,
                              const tensor *target, adamw_opt *opt, float grad_clip, float *grad_norm_out);
/* Generation (src/gpt.c:220-421): sampling helpers work on HOST logits with the reference's
 * arithmetic and random stream; decoder_lm_generate returns host token ids (prompt + new) allocated
 * from data_pool, batch 1, stops at token 258 (the reference tokenizer's end-of-sequence id). */
int  decoder_lm_argmax_token(const float *logits, int vocab_size);
int  decoder_lm_sample_with_temp(const float *logits, int vocab_size, float temp);
int *decoder_lm_generate(struct mem_pool *scratch_pool, struct mem_pool *data_pool, decoder_lm *lm,
                         const tensor *prompt_ids, int max_new_tokens, float temperature, int use_cache, int *n_out);
void    decoder_lm_enable_rope(struct mem_pool *params_pool, decoder_lm *lm, int max_seq_len, float base);
void    decoder_lm_init_weights(decoder_lm *lm);
long long decoder_lm_num_parameters(decoder_lm *lm);

typedef struct vision_lm {
    module      base;
    decoder_lm *lm;
    conv2d     *patch_embed;
    linear     *img_proj;
    tensor     *image_pos;
    int use_image_pos;
    int image_channels;
    int image_h;
    int image_w;
    int patch_size;
    int patch_h;
    int patch_w;
    int n_img_tokens;
    int d_model;
    int vocab_size;
} vision_lm;

vision_lm *vision_lm_create(struct mem_pool *params_pool, int vocab_size, int d_model, int n_layers,
                            int n_heads, int d_k, int intermediate_size, int image_channels,
                            int image_h, int image_w, int patch_size, int use_image_pos);
void    vision_lm_init_weights(vision_lm *vlm);
void    vision_lm_enable_rope(struct mem_pool *params_pool, vision_lm *vlm, int max_text_len, float base);
long long vision_lm_num_parameters(vision_lm *vlm);
tensor *vision_lm_image_embeds(struct mem_pool *scratch, vision_lm *vlm, const tensor *images);
tensor *vision_lm_build_embeds(struct mem_pool *scratch, vision_lm *vlm, const tensor *images, const tensor *text_ids);
tensor *vision_lm_forward(struct mem_pool *scratch, vision_lm *vlm, const tensor *images, const tensor *text_ids);
tensor *vision_lm_forward_text_logits(struct mem_pool *scratch, vision_lm *vlm, const tensor *images, const tensor *text_ids);
tensor *vision_lm_shift_targets(struct mem_pool *pool, const tensor *text_ids);
tensor *vision_lm_train_step(struct mem_pool *scratch_pool, vision_lm *vlm, const tensor *images,
                             const tensor *input_ids, const tensor *target_ids, adamw_opt *opt,
                             float grad_clip, float *grad_norm_out);
tensor *vision_lm_loss_padded(struct mem_pool *scratch_pool, vision_lm *vlm, const tensor *images,
                              const tensor *input_ids, const tensor *target_ids,
                              const tensor *loss_mask, const int *text_lens);
tensor *vision_lm_train_step_padded(struct mem_pool *scratch_pool, vision_lm *vlm, const tensor *images,
                                    const tensor *input_ids, const tensor *target_ids,
                                    const tensor *loss_mask, const int *text_lens, adamw_opt *opt,
                                    float grad_clip, float *grad_norm_out);
tensor *vision_lm_train_step_masked(struct mem_pool *scratch_pool, vision_lm *vlm, const tensor *images,
                                    const tensor *input_ids, const tensor *target_ids,
                                    const tensor *loss_mask, adamw_opt *opt,
                                    float grad_clip, float *grad_norm_out);

/* Generation with the vision LM, batch 1 (replaces src/vlm.c:436-611).  Returns host token ids
 * (prompt + new) allocated from data_pool; *n_out = their count.  As in the reference, the cached
 * path feeds the image embeddings without the learned image positions, the uncached path with them. */
int *vision_lm_generate(struct mem_pool *scratch_pool, struct mem_pool *data_pool, vision_lm *vlm,
                        const tensor *image, const tensor *prompt_ids, int max_new_tokens,
                        float temperature, int use_cache, int *n_out);

#ifdef __cplusplus
}
#endif
#endif /* DNN_B200_H */
