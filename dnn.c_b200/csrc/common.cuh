// Internal declarations shared by every translation unit of libdnn_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cstdint>
#include <cmath>
#include <initializer_list>
#include "dnn_b200.h"
#include "dnn_cuda.h"

namespace dnnb {

// Reference-style failure: print and abort (the reference uses assert()).
#define DNN_CHECK(cond, msg)                                                        \
    do { if (!(cond)) { fprintf(stderr, "dnn_b200: %s (%s:%d)\n", msg, __FILE__, __LINE__); \
                        abort(); } } while (0)

void cuda_fail(cudaError_t e, const char *what, const char *file, int line);
#define CUDA_OK(expr)                                                               \
    do { cudaError_t _e = (expr); if (_e != cudaSuccess) ::dnnb::cuda_fail(_e, #expr, __FILE__, __LINE__); } while (0)

// Compute stream of this process (creates the runtime on first use; aborts
// with a clear message when no CUDA device is usable).
cudaStream_t stream();
// Counts one kernel launch and checks the launch error.
void launched(const char *name);
void add_launches(long long n);
#define LAUNCHED(name) ::dnnb::launched(name)

// True when p points into the device arena of one of this process's pools.
bool dev_ptr_in_arena(const void *p);
// Every op reads its operands' payloads on the device.  A tensor whose `data` is host memory -- a struct the
// caller filled in by hand around a malloc'd buffer, as CPU callers of dnn.c may -- would hand a host pointer to
// a kernel; this check stops with a message instead (payloads inside a pool arena pass with a range compare,
// other pointers are looked up once through cudaPointerGetAttributes).  NULL tensors are skipped.
void require_device_payloads(const char *op, std::initializer_list<const tensor *> ts);
// Device allocation from the arena attached to `pool` (256-byte aligned).
void *dev_alloc(struct mem_pool *pool, size_t bytes, bool zero);
// Device scratch valid until the pool is reset / released.
template <typename T> inline T *dev_alloc_t(struct mem_pool *pool, size_t n, bool zero = false) {
    return (T *)dev_alloc(pool, n * sizeof(T), zero);
}
// Host-side metadata allocation (zero-filled).
template <typename T> inline T *host_alloc_t(struct mem_pool *pool, size_t n = 1) {
    return (T *)_mem_pool_alloc(pool, n * sizeof(T), nullptr);
}
// Copies a small host array into the scratch arena of `pool` (ordered on the
// compute stream) and returns the device pointer.
void *dev_put(struct mem_pool *pool, const void *host, size_t bytes);

int gemm_mode();
// Profiling hooks (no-ops unless dnn_cuda_profile_enable(1)): bracket one launch.
// Algorithmic work (bytes or FLOP) of the NEXT launch, for the per-launch timeline (dnn_cuda_profile_enable(2)).
void prof_work(double work);
void prof_begin(int kernel_class);
void prof_end(int kernel_class, double work);

inline int64_t numel_of(const tensor *t) {
    int64_t n = 1;
    for (int i = 0; i < t->ndim; i++) n *= t->shape[i];
    return n;
}
inline bool wants_grad(const tensor *t) { return t->grad_fn || t->requires_grad; }

// Logical shape + strides of a tensor, passed to kernels by value.
struct View {
    int ndim;
    int shape[DNN_MAX_DIMS];
    int strides[DNN_MAX_DIMS];
    int offset;
};
inline View view_of(const tensor *t) {
    View v; v.ndim = t->ndim; v.offset = t->offset;
    for (int i = 0; i < DNN_MAX_DIMS; i++) { v.shape[i] = i < t->ndim ? t->shape[i] : 1;
                                             v.strides[i] = i < t->ndim ? t->strides[i] : 0; }
    return v;
}
// View of `t` broadcast to (out_ndim, out_shape): leading dims and size-1 dims
// get stride 0 (src/broadcast.h:30-50 computes the same offsets per element).
View bcast_view(const tensor *t, int out_ndim, const int *out_shape);
int  bcast_shape(int na, const int *sa, int nb, const int *sb, int *out);   // src/broadcast.c

// A [B,H,N,d] operand of attention addressed through strides (in floats): element (b,h,n,c)
// lives at p[b*sb + h*sh + n*sn + c].  Packed heads and the [B,N,3,H,d] output of a fused
// QKV projection are both of this form.
struct HeadView {
    float *p;
    int64_t sb, sh, sn;
};
inline HeadView packed_heads(const float *p, int H, int N, int d) {
    HeadView v; v.p = const_cast<float *>(p); v.sb = (int64_t)H * N * d; v.sh = (int64_t)N * d; v.sn = d; return v;
}

// Attention computed straight from the [B,N,3*H*d] output of a fused QKV projection (attention.cu).
// Returns nullptr when the tensor-core path does not apply.
tensor *attention_from_qkv(struct mem_pool *scratch, tensor *qkv, int H, tensor *fc, tensor *fs,
                           attention_mode mode, int prefix_len, const int *seq_lens, bool rotated);
bool attention_from_qkv_applicable(const tensor *x, int H, int d, const tensor *fc, const tensor *fs);

// dnn_backward tells `fn` when a leaf's gradient has received its last contribution (autograd.cu).
void set_leaf_ready_observer(void (*fn)(tensor *leaf));
// Data-parallel exchange overlapped with backward (dp.cu): begin before dnn_backward, finish after.
bool dp_overlap_begin(tensor **params, int n_params);
int  dp_overlap_finish();

// Optimiser tail of a captured training step (optim.cu).
struct OptGraph;
OptGraph *opt_graph_prepare(adamw_opt *opt, float grad_clip);
void opt_graph_launch(OptGraph *og, adamw_opt *opt);
const void *opt_graph_advance(OptGraph *og, adamw_opt *opt);
void opt_graph_launched(OptGraph *og);
const void *opt_graph_state_dev(const OptGraph *og);
size_t opt_graph_state_bytes();
const float *opt_graph_norm(const OptGraph *og);
void opt_graph_destroy(OptGraph *og);

// Gradient destinations.  The reference zero-fills every gradient buffer when it is created
// and every backward adds to it.  Adding to zeros equals storing, so a buffer that is still
// "fresh" (allocated, never written) may be overwritten by an op that covers ALL of it; this
// saves the memset and the read half of the read-modify-write on most activation gradients.
//   grad_full(t, acc)  for ops that write the whole logical extent of t: returns the root's
//                      gradient buffer; acc=false means "store, the buffer is fresh".
//   grad_rows(t, acc)  same, and also for a view that is one packed slab [lo, hi) of every
//                      leading-dim block of its root (a slice along dim 1): the part of the
//                      fresh buffer outside the slabs is zeroed, the slabs are stored to.
//   _grad_ensure(t)    for everything else: the buffer is zero-filled if it was fresh.
//   grad_settle(t)     before a gradient is READ (norm, clip, AdamW, all-reduce, download).
//   grad_defer_copy(t, src)   "t's gradient := src" without doing the copy yet (t fresh and spanning
//                      its root; returns false otherwise).  The next op that writes t's gradient
//                      through grad_full_based() adds src while it writes and the copy never runs;
//                      every other access (any helper above, dnn_backward reaching t's node, the
//                      end of dnn_backward) performs the copy first.  src must stay valid and
//                      unchanged until the end of the backward pass.
//   grad_full_based(t, acc, base)  grad_full that accepts such a pending source: *base != nullptr
//                      means "store base + contribution".
float *grad_full(tensor *t, bool *accumulate);
float *grad_rows(tensor *t, bool *accumulate);
void   grad_settle(tensor *t);
bool   grad_defer_copy(tensor *t, const float *src);
float *grad_full_based(tensor *t, bool *accumulate, const float **base);
void   grad_settle_all_deferred();

// Attaches a tape node to `out` (src/autograd.c:29-33 + the per-op boilerplate).
grad_fn *attach(struct mem_pool *scratch, tensor *out, void (*bw)(grad_fn *, tensor *),
                int n_inputs, int n_saved);

// ---- kernel-side entry points used across files -------------------------
// column sums left behind by the kernel that wrote a gradient buffer (kernels_common.cu)
float *colsum_cache_reserve(int C);
void colsum_cache_publish(const float *src, int64_t rows, int C);
void colsum_cache_forget(const void *buffer);          // nullptr: forget whatever is cached
void k_colsum_finish(float *sums, const float *partial, int nparts, int C);
void k_colsum_finish2(float *sums0, const float *part0, float *sums1, const float *part1, int nparts, int C);
void k_fill(float *p, int64_t n, float v);
void k_axpy_acc(float *dst, const float *src, int64_t n);                 // dst += src
void k_copy(float *dst, const float *src, int64_t n);
// dst[view(i)] (=|+=) src[i] and dst[i] = src[view(i)] for i in [0, n)
void k_gather(float *dst, const float *src, const View &sv, int64_t n);
void k_scatter(float *dst, const View &dv, const float *src, int64_t n, bool accumulate);
// column sums: out[c] += sum_r g[r*C + c]
void k_colsum_acc(float *out, const float *g, int64_t rows, int C, bool accumulate = true);

// General strided GEMM:  C[m,n] (=|+=) sum_k A[m,k]*B[k,n] (+ bias[n])
struct GemmArgs {
    const float *A; int64_t a_rs, a_cs, a_bs;
    const float *B; int64_t b_rs, b_cs, b_bs;
    float *C;       int64_t c_rs, c_cs, c_bs;
    const float *bias;     // may be null; indexed by n
    int M, N, K, batch;
    bool accumulate;
};
void gemm(const GemmArgs &g);          // dispatches on gemm_mode(), the precision policy and layout
// Role of the next gemm() calls of this thread, for the precision policy (dnn_cuda_set_tf32_policy).
enum { GEMM_ROLE_FORWARD = 0, GEMM_ROLE_DA = 1, GEMM_ROLE_DW = 2, GEMM_ROLE_CONV = 4 /* flag: the product of a convolution */ };
void gemm_set_role(int role);
void gemm_set_policy(unsigned roles_3x, double max_flop_3x);
void gemm_get_policy(unsigned *roles_3x, double *max_flop_3x);
void gemm_set_exact_policy(double simt_max_flop);
double gemm_get_exact_policy();
void gemm_reread_env();                // the next gemm() reads DNN_CUDA_TF32_3X_SHAPES again

// One-shot epilogue request for the next tensor-core GEMM on this thread: rotate (RoPE) the
// pairs of the first `cols` output columns, which are heads of size d; row r is position r % N.
// The GEMM that honours it clears it; gemm_rope_epilogue_take() tells whether that happened
// (and clears a request nobody honoured, so that the caller can run the rotation itself).
// Same protocol for a residual: the next tensor-core GEMM computes C = A*B + bias + resid.
void gemm_residual_request(const float *resid, int64_t ld);
bool gemm_residual_take();
bool gemm_residual_claim(const float **resid, int64_t *ld);
// out[M,N] = silu(x Wg + bg) * (x Wu + bu) for at most four rows (gemm_simt.cu); false when the shapes do not qualify
bool gemv_swiglu(const float *x, int64_t x_rs, int M, const float *Wg, const float *bg, const float *Wu, const float *bu,
                 int K, int N, float *out);
// x + (a*b + bias) with the addition done in the GEMM epilogue when possible (ops_matrix.cu);
// equal to tensor_add(scratch, x, tensor_matmul_add(scratch, a, b, trans_b, bias)) bit for bit.
tensor *matmul_add_residual(struct mem_pool *scratch, const tensor *a, const tensor *b, int trans_b, const tensor *bias, const tensor *x);
void gemm_rope_epilogue_request(const float *fc, const float *fs, int N, int d, int cols);
bool gemm_rope_epilogue_take();
void gemm_simt(const GemmArgs &g);
bool gemm_tc_supported(const GemmArgs &g);
void gemm_tc(const GemmArgs &g, bool split3);
int  attn_tc_error();
int  norm_error();               // nonzero when a staged row copy of the norm backward never landed
int  gemm_tc_error();            // nonzero when a bounded wait inside the tensor-core kernel gave up

}  // namespace dnnb
