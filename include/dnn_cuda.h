/* dnn_cuda.h — the device-side additions to the dnn.c C API.
 *
 * The reference library (masc-it/dnn.c) is CPU only, so it has no counterpart
 * for most of these calls; each comment says which host-side idiom of the
 * reference the call stands in for.  All functions return 0 on success and a
 * negative value on failure unless stated otherwise; dnn_cuda_last_error()
 * describes the last failure.  Shape and pool-capacity violations inside the
 * dnn.c entry points keep the reference's behaviour (message + abort()).
 */
#ifndef DNN_CUDA_H
#define DNN_CUDA_H

#include "dnn_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Select the device this process drives and create its compute stream.
 * Optional: the first pool or tensor call does dnn_cuda_init(0) itself.
 * There is no CPU fallback: without a usable CUDA device the library prints a
 * message and aborts on the first call that needs device memory. */
int  dnn_cuda_init(int device);
/* 1 if a CUDA device can be used, 0 otherwise.  Never aborts. */
int  dnn_cuda_available(void);
/* Wait for all queued work.  Stands in for "the op has returned" in the
 * reference, where every op is synchronous. */
int  dnn_cuda_sync(void);
const char *dnn_cuda_last_error(void);
/* cudaStream_t of the compute stream, as an opaque pointer. */
void *dnn_cuda_stream(void);

/* Payload transfer.  Stand in for the reference idiom of dereferencing
 * t->data / t->grad on the host (src/gpt.c:165-172 builds batches that way,
 * examples read ((float*)loss->data)[0]).  `bytes` is counted from the
 * tensor's first element (data + offset); the tensor must be contiguous.
 * upload is asynchronous when `host_src` is pinned; download waits. */
int  dnn_cuda_upload(tensor *t, const void *host_src, size_t bytes);
int  dnn_cuda_download(const tensor *t, void *host_dst, size_t bytes);
int  dnn_cuda_download_grad(const tensor *t, void *host_dst, size_t bytes);
/* Raw copies for callers that hold device pointers (opt->m[i]->data etc.). */
int  dnn_cuda_memcpy_h2d(void *dev_dst, const void *host_src, size_t bytes);
int  dnn_cuda_memcpy_d2h(void *host_dst, const void *dev_src, size_t bytes);
/* Pinned host memory for end-to-end loops (batch staging). */
void *dnn_cuda_host_alloc(size_t bytes);
void  dnn_cuda_host_free(void *p);

/* Arithmetic mode of matmul / matmul_add / conv GEMMs and attention.
 *   DNN_CUDA_GEMM_FP32   fp32 FMA kernels (exact-order-free fp32; parity mode)
 *   DNN_CUDA_GEMM_TF32   tcgen05 tensor-core GEMM, TF32 inputs, fp32 accumulate
 *   DNN_CUDA_GEMM_3XTF32 tcgen05 GEMM with the big/small TF32 split (3 MMAs)
 * Replaces the reference's compile-time HAVE_CBLAS / NO_CBLAS switch
 * (src/ops_matrix.c:19-25). */
#define DNN_CUDA_GEMM_FP32   0
#define DNN_CUDA_GEMM_TF32   1
#define DNN_CUDA_GEMM_3XTF32 2
int  dnn_cuda_set_gemm_mode(int mode);
int  dnn_cuda_get_gemm_mode(void);

/* Precision policy: which GEMMs leave the arithmetic of the selected mode for a more exact one.
 * TF32 mode (dnn_cuda_set_tf32_policy):
 *   roles_3x    GEMM kinds that take the 3xTF32 path: bit 0 forward products (Y = A B), bit 1 activation
 *               gradients (dA = dY B^T), bit 2 weight gradients (dW = A^T dY) -- of matmul, matmul_add and
 *               conv2d.  Default 0.  roles_3x = 3 ("strict") is what brings every parameter gradient of a
 *               12-block transformer within 1e-3 of the reference (plain TF32: up to 1.9e-3); such a product
 *               takes three times the tensor-core time of a TF32 one (one kernel that splits the raw
 *               operand tiles in shared memory), the step about 1.7 times as long.
 *   max_flop_3x every GEMM of a CONVOLUTION (forward, input gradient, filter gradient) of at most this many FLOP
 *               (2 M N K) takes the 3xTF32 path.  Default 4e9: with reductions of 9 .. 288 and 32 .. 64 output
 *               channels these products use a fraction of the tensor core and are bound by the traffic of the
 *               column matrix, and a CNN's gradients are the ones TF32 rounding hurts most.
 *   Independently, a GEMM with at most 64 Ki outputs and a reduction of 1024 or more (the filter gradient of
 *   a small convolution) always takes the 3xTF32 path.
 * 3xTF32 mode (dnn_cuda_set_exact_policy):
 *   simt_max_flop  every GEMM of at most this many FLOP takes the fp32 FMA kernel.  Default 8e9.
 * Environment: DNN_CUDA_TF32_3X_ROLES, DNN_CUDA_TF32_3X_MAX_GFLOP, DNN_CUDA_3X_SIMT_MAX_GFLOP.
 * Switches for measuring against earlier forms of a kernel, read once at the first launch: DNN_CUDA_3X_FUSED=0
 * (3xTF32 as three launches over operands split in global memory), DNN_CUDA_ATTN_DQ=1 (attention dQ with one
 * CTA per SM), DNN_CUDA_ATTN_TMA_OUT=0 (attention outputs and gradients stored by the threads instead of the
 * copy engine), DNN_CUDA_GEMM_PAIR=0 (no CTA pairs).  None of them changes a result beyond rounding.
 * No counterpart in the reference. */
int  dnn_cuda_set_tf32_policy(unsigned roles_3x, double max_flop_3x);
int  dnn_cuda_get_tf32_policy(unsigned *roles_3x, double *max_flop_3x);
int  dnn_cuda_set_exact_policy(double simt_max_flop);
double dnn_cuda_get_exact_policy(void);

/* Transformer blocks in TF32 mode with head size 32 or 64 run attention straight from the
 * fused QKV projection: Q, K and V are read in place from its [B,N,3,H,d] output, RoPE is
 * applied there, and the result is written token-major, which removes the head split / merge
 * copies of the reference's block (src/transformer.c:143-170) without changing any value.
 * The same switch covers the block's two residual additions, which then run in the epilogue of
 * the output / down projection instead of as separate passes.
 * `on` = 0 forces the reference's op-by-op sequence (default 1; environment
 * DNN_CUDA_FUSED_QKV=0 does the same).  No counterpart in the reference. */
void dnn_cuda_set_fused_attention(int on);
int  dnn_cuda_get_fused_attention(void);

/* Optimiser state on disk (AdamW moments m and v, step counter t, hyper-parameters).  The
 * reference's state files hold weights only (module_save / module_load, src/module.c:208-339),
 * so its runs cannot be resumed; module_save + dnn_cuda_optimizer_save written at the same step
 * and loaded into a freshly created model and optimiser continue the run bit for bit.
 * 0 on success; -1 bad argument, -2 cannot open, -3 I/O error or mismatch with `opt`.
 * No counterpart in the reference. */
int  dnn_cuda_optimizer_save(const adamw_opt *opt, const char *path);
int  dnn_cuda_optimizer_load(adamw_opt *opt, const char *path);
/* The whole resume state in one file: the optimiser state above plus the LR scheduler's own step count
 * (`sched` may be NULL) and the state of the calling thread's default host random generator, from which
 * dropout masks are drawn (src/ops_activation.c:1460).  load restores all three and sets opt->lr to the
 * scheduler's value at the restored step, so a run that uses an LR schedule and dropout continues bit
 * for bit.  Same return codes.  No counterpart in the reference. */
int  dnn_cuda_train_state_save(const adamw_opt *opt, const lr_scheduler *sched, const char *path);
int  dnn_cuda_train_state_load(adamw_opt *opt, lr_scheduler *sched, const char *path);

/* Whole training step as one CUDA graph.  capture records zero_grad + forward + cross entropy +
 * backward + gradient clipping + AdamW of decoder_lm_train_step (src/gpt.c:178-216) on the
 * given tensors WITHOUT running it; replay runs the recorded step: it advances opt->t, uses the
 * current opt->lr (so lr_scheduler_step between replays works), and, where asked, copies the loss
 * and the pre-clip gradient norm back (that copy waits for the step).
 * Rules: run at least one eager decoder_lm_train_step of the same shapes first (buffers that grow
 * on demand must have their final size, parameters must own gradient buffers); new batches are
 * written into the SAME input_ids / target tensors with dnn_cuda_upload; the scratch pool may be
 * reset and used between replays, but not while a replay is in flight; data-parallel runs are not
 * captured.  Replays may be queued back to back without reading anything back: each one carries its
 * own copy of the learning rate and bias corrections (a ring of eight pinned slots; the ninth queued
 * replay waits on the host for the first to finish).  capture returns NULL with a message when
 * recording fails.  Results equal the eager step bit for bit.  No counterpart in the reference
 * (whose ops run synchronously on the host). */
typedef struct dnn_cuda_step_graph dnn_cuda_step_graph;
dnn_cuda_step_graph *dnn_cuda_graph_capture_decoder_lm_step(struct mem_pool *scratch_pool, decoder_lm *lm,
                                                            const tensor *input_ids, const tensor *target,
                                                            adamw_opt *opt, float grad_clip);
int  dnn_cuda_graph_replay(dnn_cuda_step_graph *g, float *loss_out, float *grad_norm_out);
void dnn_cuda_graph_destroy(dnn_cuda_step_graph *g);

/* Device-side timing on the compute stream (CUDA events): start records an event,
 * stop records a second one, waits for it and returns the milliseconds between. */
int   dnn_cuda_timer_start(void);
float dnn_cuda_timer_stop_ms(void);
/* Per-kernel-class profiling for roofline reports.  While enabled, every launch of
 * the tensor-core GEMM and of AdamW is bracketed by events.  read() waits for the
 * stream and returns, for class 0 (GEMM) or 1 (AdamW): launches, summed device
 * milliseconds and summed algorithmic work (FLOP for GEMM, bytes for AdamW). */
int   dnn_cuda_profile_enable(int on);
int   dnn_cuda_profile_read(int kernel_class, long long *launches, double *ms, double *work);
/* dnn_cuda_profile_enable(2) records a timeline instead: one event after EVERY kernel launch of the
 * library (launches are serialised on the compute stream, so the time between two events is the later
 * kernel's duration).  dnn_cuda_profile_kernels waits for the stream and sums the timeline by kernel
 * name: launches, device milliseconds and, where the launch site states it, the algorithmic work
 * (bytes for memory-bound kernels, FLOP for GEMM and attention; 0 where not stated).  Returns the
 * number of distinct names and fills up to `cap` rows.  The events cost time: run the timeline in a
 * pass of its own, not in a timed region. */
typedef struct dnn_cuda_kernel_time { char name[56]; long long launches; double ms; double work; } dnn_cuda_kernel_time;
int   dnn_cuda_profile_kernels(dnn_cuda_kernel_time *rows, int cap);

/* Column sums without any allocation:  out[c] += sum over r of g[r*cols + c]
 * (the bias gradient of matmul_add / add).  No counterpart in the reference: this
 * variant exists for callers that must not allocate device memory at the time of
 * the call -- programs that have given all of HBM to their own arenas, loops that
 * cannot afford the device-wide synchronisation an allocation implies, hosts whose
 * policy forbids allocating after start-up.  The partial sums go to a 4 MiB array
 * that is compiled into the library and stays resident on every GPU that loads it.
 *   - `out` (cols floats) and `g` (rows x cols floats, row-major) are device pointers
 *     supplied by the caller; the work is queued on the library's compute stream.
 *   - Limit: cols <= 8192 (any number of rows).  Wider inputs return -2 and
 *     dnn_cuda_colsum_acc_static_error() says why; nothing is launched.
 *   - The first call on a device resolves the array's device address; make that
 *     first call before starting any stream capture.
 *   - All calls share the one array.  Each call rewrites the part it reads, so no
 *     clearing is needed between calls, but two calls that overlap on the GPU (for
 *     example from different streams or processes' threads) race on it.
 * Returns 0 on success, negative on failure (-1 bad argument, -2 too wide, -3 no usable device, -4 the array's
 * address could not be resolved, -5 a launch failed); the message is kept per calling thread.  Never aborts. */
int   dnn_cuda_colsum_acc_static(float *out, const float *g, long long rows, int cols);
const char *dnn_cuda_colsum_acc_static_error(void);

/* Kernels launched by this library since process start (for benchmarks). */
long long dnn_cuda_launch_count(void);
/* Bytes of the pool's device arena in use / high-water mark since creation. */
size_t dnn_cuda_pool_device_used(const mem_pool *pool);
size_t dnn_cuda_pool_device_peak(const mem_pool *pool);

/* Padded vision-LM batches assembled on the device, with upload prefetch.  Replaces the per-sample
 * host loops at the end of imagenet_vlm_dl_next_batch (src/imagenet_vlm.c:598-647) and convert_pixels
 * (src/imagenet_vlm.c:31-46): a loader hands over RAW samples -- the stored token ids (no BOS) and the
 * uint8 HWC pixels, or the ready float patches of a version-3 shard -- and the device writes
 * input_ids (BOS + text + PAD), target_ids (text + PAD), loss_mask (1 on the first stored_len slots)
 * and the normalised NCHW image (val = px/255; (val - mean[c]) / std[c], optional horizontal flip),
 * bit-identical to the reference.
 *   create   : `slots` staging buffers (pinned host + device) for up to max_bs samples of H x W x C
 *              and texts of at most t_max - 1 stored ids; float_patches = 1 for version-3 payloads
 *              (H*W*C floats per sample, copied as they are).  mean/std: C floats (NULL = 0 / 1).
 *   put      : copies sample `index` of the batch being built in `slot` into pinned memory.  Returns
 *              -1 when stored_len + 1 > t_max, like the reference.  Waits only if the previous upload
 *              of this slot is still reading the memory.
 *   submit   : queues ONE host-to-device copy of the slot's first `bs` samples on a copy stream.
 *   assemble : on the compute stream, after the upload: writes the batch tensors (device tensors
 *              from dnn.c pools; img [>=bs,C,H,W] or [>=bs,patches,patch_dim], the others [>=bs,T])
 *              and fills the host arrays text_lens (stored_len + 1) and label_ids (may be NULL).
 *              Returns the number of samples, -1 for a geometry mismatch or a text longer than T.
 * Per slot the order is put..., submit, assemble; different slots overlap freely, so slot k+1 can be
 * filled and uploaded while the step that consumes slot k runs.  Errors: dnn_cuda_vlm_stager_error(). */
typedef struct dnn_cuda_vlm_stager dnn_cuda_vlm_stager;
dnn_cuda_vlm_stager *dnn_cuda_vlm_stager_create(int slots, int max_bs, int t_max, int H, int W, int C,
                                                int float_patches, const float *mean, const float *std);
void dnn_cuda_vlm_stager_destroy(dnn_cuda_vlm_stager *s);
int  dnn_cuda_vlm_stager_put(dnn_cuda_vlm_stager *s, int slot, int index, const int *text, int stored_len,
                             const void *image, int flip, int label);
int  dnn_cuda_vlm_stager_submit(dnn_cuda_vlm_stager *s, int slot, int bs);
int  dnn_cuda_vlm_stager_assemble(dnn_cuda_vlm_stager *s, int slot, tensor *img, tensor *input_ids,
                                  tensor *target_ids, tensor *loss_mask, int *text_lens, int *label_ids);
const char *dnn_cuda_vlm_stager_error(void);

/* Data-parallel gradient exchange (one process per GPU).  The reference has
 * no multi-process path; these follow the place where a DDP hook would sit in
 * src/gpt.c:201-206, between dnn_backward() and clip_grad_norm().
 *   unique_id : fills 128 bytes on rank 0; the caller broadcasts them.
 *   init      : joins the NCCL communicator.
 *   allreduce : averages param->grad over ranks, in place, bucketed on a
 *               second stream; params with grad == NULL are skipped, which
 *               must be the same set on every rank. */
int  dnn_cuda_dp_unique_id(void *out_128_bytes);
int  dnn_cuda_dp_init(int rank, int world_size, const void *id_128_bytes);
int  dnn_cuda_dp_allreduce_grads(tensor **params, int n_params);
int  dnn_cuda_dp_world_size(void);
/* Host-only: how dnn_cuda_dp_allreduce_grads would cut n gradient buffers (address, bytes)
 * into all-reduce buckets; returns the bucket count and fills up to `cap` of them. */
int  dnn_cuda_dp_plan_buckets(const size_t *addrs, const size_t *bytes, int n, size_t bucket_bytes,
                              size_t *out_addrs, size_t *out_bytes, int cap);
int  dnn_cuda_dp_finalize(void);
const char *dnn_cuda_dp_last_error(void);
/* dnn_backward(scratch, loss) followed by the exchange of the gradients of `params`: what a loop that
 * calls the ops itself puts between its forward pass and adamw_step (the MNIST loop of the reference,
 * examples/mnist/mnist_train.c:99-114, has dnn_backward at that place).  With the overlap enabled and the
 * gradient buffers already allocated (from the second step on) buckets are exchanged while backward
 * still runs.  Before the first exchange, and whenever a rank's bucket plan changes, the ranks compare a
 * fingerprint of their plans; -5 means they differ (nothing was exchanged, dnn_cuda_dp_last_error() says
 * why).  With one rank this is dnn_backward. */
int  dnn_cuda_dp_backward(struct mem_pool *scratch_pool, tensor *loss, tensor **params, int n_params);
/* decoder_lm_train_step with the all-reduce between backward and clipping. */
tensor *dnn_cuda_dp_decoder_lm_train_step(struct mem_pool *scratch_pool, decoder_lm *lm,
                                          const tensor *input_ids, const tensor *target,
                                          adamw_opt *opt, float grad_clip, float *grad_norm_out);
/* vision_lm_train_step_padded (src/vlm.c:348-381) with the all-reduce between backward and clipping;
 * parameters outside the graph (img_proj.* for [B,C,H,W] images) have no gradient on any rank and are
 * skipped by the exchange and by AdamW alike. */
tensor *dnn_cuda_dp_vision_lm_train_step_padded(struct mem_pool *scratch_pool, vision_lm *v, const tensor *images,
                                                const tensor *input_ids, const tensor *target_ids, const tensor *loss_mask,
                                                const int *text_lens, adamw_opt *opt, float grad_clip, float *grad_norm_out);

#ifdef __cplusplus
}
#endif
#endif /* DNN_CUDA_H */
