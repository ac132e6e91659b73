// Column sums with a fixed, statically reserved scratch buffer.
//
// dnn_cuda_colsum_acc_static() computes out[c] += sum_r g[r*cols + c] -- the bias
// gradient of matmul_add / add -- like the library's internal column-sum, but it
// never allocates: the per-row-block partial sums live in a file-scope __device__
// array that is part of the loaded module.  It exists for callers that are not
// allowed to allocate device memory when they call in: a host program that has
// already handed the whole GPU to its own arenas (the dnn.c pools are sized that
// way), a latency-critical loop that cannot take cudaMalloc's implicit device-wide
// synchronisation, or an embedding application whose policy forbids allocation
// after start-up.  The price is a hard size limit and a buffer that every GPU
// loading the library holds until the process exits.
#include "common.cuh"
#include "device_utils.cuh"

namespace dnnb {

constexpr int kStaticMaxCols  = 8192;     // widest matrix accepted
constexpr int kStaticMaxParts = 128;      // row blocks whose partial sums are kept
// 128 x 8192 floats = 4 MiB per device, resident for the life of the process.
static __device__ __align__(256) float g_static_partials[kStaticMaxParts * kStaticMaxCols];

// partial[p][c] = sum of rows [p*rows_per, (p+1)*rows_per) of column c
__global__ void colsum_static_partial_kernel(const float *__restrict__ g, float *__restrict__ partial,
                                             long long rows, int cols, int rows_per) {
    __shared__ float tile[32][33];
    int c = blockIdx.x * 32 + threadIdx.x;
    long long r0 = (long long)blockIdx.y * rows_per;
    long long r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
    float s = 0.f;
    if (c < cols)
        for (long long r = r0 + threadIdx.y; r < r1; r += blockDim.y) s += g[r * cols + c];
    tile[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < cols) {
        float t = 0.f;
#pragma unroll
        for (int j = 0; j < 32; j++) t += tile[j][threadIdx.x];
        partial[(long long)blockIdx.y * cols + c] = t;
    }
}
// out[c] += partial[0][c] + partial[1][c] + ... in that order
__global__ void colsum_static_final_kernel(float *__restrict__ out, const float *__restrict__ partial, int nparts, int cols) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float s = 0.f;
    for (int p = 0; p < nparts; p++) s += partial[(long long)p * cols + c];
    out[c] += s;
}

// Device address of g_static_partials, resolved once per device.  In host code the
// array's name is only a handle for the runtime; the kernels need the address that
// cudaGetSymbolAddress returns for the device that is current.
constexpr int kMaxDevices = 64;
static float *g_static_ptr[kMaxDevices] = {nullptr};

// Last failure of the calling thread (the entry point may be called from several host threads).
static thread_local char g_static_error[256] = "";
static int static_fail(int code, const char *fmt, const char *detail = "") {
    snprintf(g_static_error, sizeof g_static_error, fmt, detail);
    return code;
}

}  // namespace dnnb

using namespace dnnb;

extern "C" {

const char *dnn_cuda_colsum_acc_static_error(void) { return g_static_error; }

int dnn_cuda_colsum_acc_static(float *out, const float *g, long long rows, int cols) {
    if (!out || !g) return static_fail(-1, "colsum_acc_static: NULL pointer");
    if (rows < 0 || cols <= 0) return static_fail(-1, "colsum_acc_static: rows must be >= 0 and cols > 0");
    if (cols > kStaticMaxCols) {
        snprintf(g_static_error, sizeof g_static_error,
                 "colsum_acc_static: %d columns exceed the static scratch limit of %d; use the pooled path", cols, kStaticMaxCols);
        return -2;
    }
    if (rows == 0) return 0;
    // stream() aborts the process when no device can be used; this entry point reports instead
    if (!dnn_cuda_available()) return static_fail(-3, "colsum_acc_static: no usable CUDA device");
    cudaStream_t st = stream();
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return static_fail(-3, "colsum_acc_static: cannot identify the current device");
    if (!g_static_ptr[dev]) {
        // one-time set-up for this device (the device is current here)
        float *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_static_partials);
        if (e != cudaSuccess || !p) return static_fail(-4, "colsum_acc_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_static_ptr[dev] = p;
    }
    float *partial = g_static_ptr[dev];
    int nparts = (int)((rows + 255) / 256);
    if (nparts > kStaticMaxParts) nparts = kStaticMaxParts;
    int rows_per = (int)((rows + nparts - 1) / nparts);
    nparts = (int)((rows + rows_per - 1) / rows_per);
    // Every partial the second kernel reads is written by the first one in this same
    // call, so nothing left over from an earlier call has to be cleared.
    dim3 grid((cols + 31) / 32, nparts), block(32, 32);
    colsum_static_partial_kernel<<<grid, block, 0, st>>>(g, partial, rows, cols, rows_per);
    if ((e = cudaGetLastError()) != cudaSuccess) return static_fail(-5, "colsum_acc_static: launch failed: %s", cudaGetErrorString(e));
    colsum_static_final_kernel<<<(cols + 127) / 128, 128, 0, st>>>(out, partial, nparts, cols);
    if ((e = cudaGetLastError()) != cudaSuccess) return static_fail(-5, "colsum_acc_static: launch failed: %s", cudaGetErrorString(e));
    add_launches(2);
    return 0;
}

}  // extern "C"
