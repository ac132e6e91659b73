// Padded vision-LM batches assembled on the device, with the upload of the next batch running
// beside the training step.  replaces the per-sample host loops at the end of
// imagenet_vlm_dl_next_batch and convert_pixels (src/imagenet_vlm.c:598-647, 31-46): the reference
// expands every uint8 pixel to a normalised float on the host and writes BOS / text / PAD rows,
// targets and the loss mask element by element into host tensors.
//
// Here the loader hands over raw samples (stored token ids, uint8 HWC pixels or ready float
// patches).  They are packed into a pinned slot, one asynchronous copy on a copy stream moves the
// slot's used prefix to the device (a quarter of the bytes of a float image), and two small kernels
// on the compute stream write the batch tensors.  Slots form a ring: while slot k is being trained
// on, slot k+1 is filled and uploaded.  Events order the three parties (host packing, copy stream,
// compute stream), so no call here blocks unless its slot is still in use.
//
// Arithmetic of the pixel path: val = px * (1/255); out = (val - mean[c]) / std[c], each operation
// rounded to fp32 on its own like the reference's scalar loop, so the images are bit-identical.
#include "common.cuh"
#include "device_utils.cuh"
#include <vector>

namespace dnnb {

constexpr int kBosId = 257, kPadId = 259;      // include/tokenizer.h:23-25 of the reference

// One thread per (row, position).  text: [max_bs][t_max] stored ids, lens: stored lengths.
__global__ void vlm_text_rows_kernel(const int *__restrict__ text, const int *__restrict__ lens, int t_store,
                                     int *__restrict__ input_ids, int64_t in_stride, int *__restrict__ target_ids, int64_t tg_stride,
                                     float *__restrict__ mask, int64_t mk_stride, int bs, int t_batch) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= bs * t_batch) return;
    const int b = i / t_batch, t = i - b * t_batch;
    const int len = lens[b];
    const int *row = text + (int64_t)b * t_store;
    input_ids[b * in_stride + t] = t == 0 ? kBosId : (t <= len ? row[t - 1] : kPadId);
    target_ids[b * tg_stride + t] = t < len ? row[t] : kPadId;
    mask[b * mk_stride + t] = t < len ? 1.0f : 0.0f;
}

struct Norm3 { float mean[4], std[4]; };

__device__ __forceinline__ float norm_px(uint32_t px, float mean, float stdv) {
    return __fdiv_rn(__fsub_rn(__fmul_rn((float)px, 1.0f / 255.0f), mean), stdv);
}

// uint8 [bs][H][W][3] -> float [bs][3][H][W].  One thread per four output columns: 12 source bytes
// (three aligned words; read right-to-left when the sample is flipped) become one float4 per channel.
__global__ void vlm_pixels_c3_kernel(const uint8_t *__restrict__ px, const int *__restrict__ flips, float *__restrict__ img,
                                     int64_t img_stride, int bs, int H, int W, Norm3 nm) {
    const int wq = W >> 2;
    const int64_t total = (int64_t)bs * H * wq;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int q = (int)(i % wq);
        const int h = (int)((i / wq) % H);
        const int b = (int)(i / ((int64_t)wq * H));
        const int flip = flips[b];
        const int w0 = q * 4;
        const int ws0 = flip ? W - 4 - w0 : w0;                          // first source column of the group
        const uint32_t *src = reinterpret_cast<const uint32_t *>(px + ((int64_t)b * H + h) * W * 3 + (int64_t)ws0 * 3);
        const uint32_t a = src[0], bb = src[1], c = src[2];
        uint32_t v[12];
#pragma unroll
        for (int k = 0; k < 4; k++) { v[k] = (a >> (8 * k)) & 255u; v[4 + k] = (bb >> (8 * k)) & 255u; v[8 + k] = (c >> (8 * k)) & 255u; }
        float *dst = img + b * img_stride + (int64_t)h * W + w0;
#pragma unroll
        for (int ch = 0; ch < 3; ch++) {
            float o[4];
#pragma unroll
            for (int k = 0; k < 4; k++) o[k] = norm_px(v[(flip ? 3 - k : k) * 3 + ch], nm.mean[ch], nm.std[ch]);
            *reinterpret_cast<float4 *>(dst + (int64_t)ch * H * W) = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
}

// Any channel count / width: one thread per output element.
__global__ void vlm_pixels_any_kernel(const uint8_t *__restrict__ px, const int *__restrict__ flips, float *__restrict__ img,
                                      int64_t img_stride, int bs, int H, int W, int C, Norm3 nm) {
    const int64_t total = (int64_t)bs * C * H * W;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int w = (int)(i % W);
        const int h = (int)((i / W) % H);
        const int c = (int)((i / ((int64_t)W * H)) % C);
        const int b = (int)(i / ((int64_t)W * H * C));
        const int ws = flips[b] ? W - 1 - w : w;
        img[b * img_stride + ((int64_t)c * H + h) * W + w] =
            norm_px(px[(((int64_t)b * H + h) * W + ws) * C + c], nm.mean[c], nm.std[c]);
    }
}

}  // namespace dnnb

using namespace dnnb;

// Slot layout, identical in pinned host memory and on the device:
//   [lens: max_bs int][flips: max_bs int][text: max_bs * t_max int][images: max_bs * image_bytes]
struct dnn_cuda_vlm_stager {
    int slots, max_bs, t_max, H, W, C, float_patches;
    size_t image_bytes, image_off, slot_bytes;
    Norm3 nm;
    cudaStream_t copy_stream;
    struct Slot {
        uint8_t *host, *dev;
        cudaEvent_t uploaded, consumed;        // copy stream done reading host / compute stream done reading dev
        bool upload_pending, consume_pending;
        int bs;                                // samples submitted
        std::vector<int> labels, lens;         // host copies; lens as of the last submit
    };
    std::vector<Slot> slot;
};

static thread_local const char *g_stager_error = "";
static int stager_fail(const char *why, int code) { g_stager_error = why; return code; }

extern "C" {

const char *dnn_cuda_vlm_stager_error(void) { return g_stager_error; }

dnn_cuda_vlm_stager *dnn_cuda_vlm_stager_create(int slots, int max_bs, int t_max, int H, int W, int C, int float_patches,
                                                const float *mean, const float *std) {
    if (slots < 1 || max_bs < 1 || t_max < 2 || H < 1 || W < 1 || C < 1 || (!float_patches && C > 4)) {
        stager_fail("stager_create: bad geometry (uint8 pixels support up to 4 channels)", 0);
        return nullptr;
    }
    stream();                                   // brings the runtime up; aborts without a usable device
    auto *s = new dnn_cuda_vlm_stager();
    s->slots = slots; s->max_bs = max_bs; s->t_max = t_max; s->H = H; s->W = W; s->C = C; s->float_patches = float_patches;
    s->image_bytes = (size_t)H * W * C * (float_patches ? sizeof(float) : 1);
    s->image_off = ((size_t)max_bs * (2 + (size_t)t_max) * sizeof(int) + 255) & ~(size_t)255;
    s->slot_bytes = s->image_off + (size_t)max_bs * s->image_bytes;
    for (int c = 0; c < 4; c++) { s->nm.mean[c] = (mean && c < C) ? mean[c] : 0.f; s->nm.std[c] = (std && c < C) ? std[c] : 1.f; }
    CUDA_OK(cudaStreamCreateWithFlags(&s->copy_stream, cudaStreamNonBlocking));
    s->slot.resize((size_t)slots);
    for (auto &sl : s->slot) {
        CUDA_OK(cudaHostAlloc((void **)&sl.host, s->slot_bytes, cudaHostAllocDefault));
        CUDA_OK(cudaMalloc((void **)&sl.dev, s->slot_bytes));
        CUDA_OK(cudaEventCreateWithFlags(&sl.uploaded, cudaEventDisableTiming));
        CUDA_OK(cudaEventCreateWithFlags(&sl.consumed, cudaEventDisableTiming));
        sl.upload_pending = sl.consume_pending = false;
        sl.bs = 0;
        sl.labels.assign((size_t)max_bs, 0);
        sl.lens.assign((size_t)max_bs, 0);
        memset(sl.host, 0, s->image_off);
    }
    return s;
}

void dnn_cuda_vlm_stager_destroy(dnn_cuda_vlm_stager *s) {
    if (!s) return;
    cudaStreamSynchronize(s->copy_stream);
    cudaStreamSynchronize(stream());
    for (auto &sl : s->slot) {
        cudaFreeHost(sl.host); cudaFree(sl.dev);
        cudaEventDestroy(sl.uploaded); cudaEventDestroy(sl.consumed);
    }
    cudaStreamDestroy(s->copy_stream);
    delete s;
}

int dnn_cuda_vlm_stager_put(dnn_cuda_vlm_stager *s, int slot, int index, const int *text, int stored_len,
                            const void *image, int flip, int label) {
    if (!s || slot < 0 || slot >= s->slots || index < 0 || index >= s->max_bs || !text || !image)
        return stager_fail("stager_put: bad slot, index or pointer", -2);
    if (stored_len < 0 || stored_len + 1 > s->t_max)                      // src/imagenet_vlm.c:583
        return stager_fail("stager_put: text does not fit t_max", -1);
    auto &sl = s->slot[(size_t)slot];
    if (sl.upload_pending) { CUDA_OK(cudaEventSynchronize(sl.uploaded)); sl.upload_pending = false; }   // the copy still reads this memory
    int *lens = reinterpret_cast<int *>(sl.host), *flips = lens + s->max_bs, *txt = flips + s->max_bs;
    lens[index] = stored_len;
    flips[index] = flip ? 1 : 0;
    memcpy(txt + (size_t)index * s->t_max, text, (size_t)stored_len * sizeof(int));
    memcpy(sl.host + s->image_off + (size_t)index * s->image_bytes, image, s->image_bytes);
    sl.labels[(size_t)index] = label;
    return 0;
}

int dnn_cuda_vlm_stager_submit(dnn_cuda_vlm_stager *s, int slot, int bs) {
    if (!s || slot < 0 || slot >= s->slots || bs < 1 || bs > s->max_bs) return stager_fail("stager_submit: bad slot or batch size", -2);
    auto &sl = s->slot[(size_t)slot];
    if (sl.consume_pending) { CUDA_OK(cudaStreamWaitEvent(s->copy_stream, sl.consumed, 0)); sl.consume_pending = false; }
    CUDA_OK(cudaMemcpyAsync(sl.dev, sl.host, s->image_off + (size_t)bs * s->image_bytes, cudaMemcpyHostToDevice, s->copy_stream));
    CUDA_OK(cudaEventRecord(sl.uploaded, s->copy_stream));
    sl.upload_pending = true;
    sl.bs = bs;
    memcpy(sl.lens.data(), sl.host, (size_t)bs * sizeof(int));
    return 0;
}

int dnn_cuda_vlm_stager_assemble(dnn_cuda_vlm_stager *s, int slot, tensor *img, tensor *input_ids, tensor *target_ids,
                                 tensor *loss_mask, int *text_lens, int *label_ids) {
    if (!s || slot < 0 || slot >= s->slots || !img || !input_ids || !target_ids || !loss_mask)
        return stager_fail("stager_assemble: bad slot or NULL tensor", -2);
    auto &sl = s->slot[(size_t)slot];
    const int bs = sl.bs;
    if (bs < 1) return stager_fail("stager_assemble: nothing was submitted to this slot", -2);
    const int t_batch = input_ids->shape[1];
    if (input_ids->ndim != 2 || target_ids->ndim != 2 || loss_mask->ndim != 2 || target_ids->shape[1] != t_batch ||
        loss_mask->shape[1] != t_batch || input_ids->shape[0] < bs || target_ids->shape[0] < bs || loss_mask->shape[0] < bs ||
        input_ids->strides[1] != 1 || target_ids->strides[1] != 1 || loss_mask->strides[1] != 1)
        return stager_fail("stager_assemble: ids, targets and mask must be [>=bs, T] with unit inner stride", -1);
    const int *lens = sl.lens.data();
    for (int b = 0; b < bs; b++)
        if (lens[b] + 1 > t_batch) return stager_fail("stager_assemble: a text does not fit the batch width", -1);   // src/imagenet_vlm.c:583
    bool img_ok = img->shape[0] >= bs && img->strides[img->ndim - 1] == 1;
    if (s->float_patches) {                                               // src/imagenet_vlm.c:633-639
        const int p = 16, n_patches = (s->H / p) * (s->W / p), patch_dim = s->C * p * p;
        img_ok = img_ok && s->H % p == 0 && s->W % p == 0 && img->ndim == 3 && img->shape[1] == n_patches && img->shape[2] == patch_dim &&
                 img->strides[1] == patch_dim;
    } else {                                                              // src/imagenet_vlm.c:643
        img_ok = img_ok && img->ndim == 4 && img->shape[1] == s->C && img->shape[2] == s->H && img->shape[3] == s->W &&
                 img->strides[2] == s->W && img->strides[1] == s->H * s->W;
    }
    if (!img_ok) return stager_fail("stager_assemble: image tensor does not match the sample geometry", -1);

    cudaStream_t st = stream();
    CUDA_OK(cudaStreamWaitEvent(st, sl.uploaded, 0));
    const int *d_lens = reinterpret_cast<const int *>(sl.dev), *d_flips = d_lens + s->max_bs, *d_text = d_flips + s->max_bs;
    {
        const int n = bs * t_batch;
        vlm_text_rows_kernel<<<(n + 255) / 256, 256, 0, st>>>(
            d_text, d_lens, s->t_max, (int *)input_ids->data + input_ids->offset, input_ids->strides[0],
            (int *)target_ids->data + target_ids->offset, target_ids->strides[0],
            (float *)loss_mask->data + loss_mask->offset, loss_mask->strides[0], bs, t_batch);
        LAUNCHED("vlm_text_rows_kernel");
    }
    float *img_d = (float *)img->data + img->offset;
    const uint8_t *d_img = sl.dev + s->image_off;
    if (s->float_patches) {
        CUDA_OK(cudaMemcpy2DAsync(img_d, (size_t)img->strides[0] * sizeof(float), d_img, s->image_bytes, s->image_bytes, (size_t)bs,
                                  cudaMemcpyDeviceToDevice, st));
    } else if (s->C == 3 && s->W % 4 == 0 && img->strides[0] % 4 == 0 && ((uintptr_t)img_d & 15) == 0) {
        const int64_t n = (int64_t)bs * s->H * (s->W / 4);
        vlm_pixels_c3_kernel<<<grid_for(n, 256), 256, 0, st>>>(d_img, d_flips, img_d, img->strides[0], bs, s->H, s->W, s->nm);
        LAUNCHED("vlm_pixels_c3_kernel");
    } else {
        const int64_t n = (int64_t)bs * s->C * s->H * s->W;
        vlm_pixels_any_kernel<<<grid_for(n, 256), 256, 0, st>>>(d_img, d_flips, img_d, img->strides[0], bs, s->H, s->W, s->C, s->nm);
        LAUNCHED("vlm_pixels_any_kernel");
    }
    CUDA_OK(cudaEventRecord(sl.consumed, st));
    sl.consume_pending = true;
    for (int b = 0; b < bs; b++) {
        if (text_lens) text_lens[b] = lens[b] + 1;
        if (label_ids) label_ids[b] = sl.labels[(size_t)b];
    }
    return bs;
}

}  // extern "C"
