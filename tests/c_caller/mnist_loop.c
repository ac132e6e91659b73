/* A C caller of the dnn.c API, compiled against include/ and linked with libdnn_b200.so by
 * tests/test_gpu_c_caller.py.  It is the training loop of the reference's MNIST example
 * (examples/mnist/mnist_train.c:99-114: forward, cross entropy, dnn_backward, read the loss,
 * adamw_step, adamw_zero_grad, reset scratch) on a synthetic batch.  The only lines a CPU caller would
 * not have are the payload transfers: dnn_cuda_upload where the example memcpy's into bx->data, and
 * dnn_cuda_download where it reads ((float *)loss->data)[0].
 *
 *     mnist_loop <batch> <steps>      prints one loss per step, then "ok"
 */
#include <stdio.h>
#include <stdlib.h>
#include "dnn.h"
#include "dnn_cuda.h"

int main(int argc, char **argv) {
    int batch = argc > 1 ? atoi(argv[1]) : 32, steps = argc > 2 ? atoi(argv[2]) : 3;
    dnn_ctx ctx;
    if (dnn_ctx_init(&ctx, (size_t)64 << 20, (size_t)1 << 30, (size_t)16 << 20) != 0) return 2;
    dnn_seed(2);
    conv2d *c1 = conv2d_create(ctx.params, 1, 32, 3, 1, 1);
    conv2d *c2 = conv2d_create(ctx.params, 32, 64, 3, 1, 1);
    linear *f1 = linear_create(ctx.params, 3136, 128);
    linear *f2 = linear_create(ctx.params, 128, 10);
    module *layers[4] = {&c1->base, &c2->base, &f1->base, &f2->base};
    tensor *params[16];
    int n_params = 0;
    for (int l = 0; l < 4; l++) {
        int n = 0;
        tensor **p = module_parameters(layers[l], &n);
        for (int i = 0; i < n; i++) params[n_params++] = p[i];
    }
    adamw_opt *opt = adamw_create(ctx.params, params, n_params, 1e-3f, 0.9f, 0.999f, 1e-8f, 0.01f);

    /* synthetic batch from the library's own generator, built on the host like the example's bx / by */
    float *hx = malloc((size_t)batch * 784 * sizeof(float));
    int *hy = malloc((size_t)batch * sizeof(int));
    dnn_rng r = dnn_rng_seed(7);
    for (int i = 0; i < batch * 784; i++) hx[i] = dnn_rng_uniform(&r);
    for (int i = 0; i < batch; i++) hy[i] = dnn_rng_uniform_int(&r, 10);

    for (int s = 0; s < steps; s++) {
        int xs[4] = {batch, 1, 28, 28}, ys[1] = {batch}, flat[2] = {batch, 3136};
        tensor *bx = tensor_zeros_data(ctx.data, 4, xs), *by = tensor_zeros_data(ctx.data, 1, ys);
        if (dnn_cuda_upload(bx, hx, (size_t)batch * 784 * sizeof(float)) != 0) return 3;
        if (dnn_cuda_upload(by, hy, (size_t)batch * sizeof(int)) != 0) return 3;
        tensor *h = tensor_avg_pool2d(ctx.scratch, tensor_relu(ctx.scratch, conv2d_forward(ctx.scratch, c1, bx)), 2, 2);
        h = tensor_avg_pool2d(ctx.scratch, tensor_relu(ctx.scratch, conv2d_forward(ctx.scratch, c2, h)), 2, 2);
        h = tensor_reshape(ctx.scratch, h, 2, flat);
        h = tensor_relu(ctx.scratch, linear_forward(ctx.scratch, f1, h));
        tensor *logits = linear_forward(ctx.scratch, f2, h);
        tensor *loss = tensor_cross_entropy(ctx.scratch, logits, by, 1);
        dnn_backward(ctx.scratch, loss);
        float loss_val = 0.0f;
        if (dnn_cuda_download(loss, &loss_val, sizeof loss_val) != 0) return 4;
        printf("%.9g\n", loss_val);
        adamw_step(opt);
        adamw_zero_grad(opt);
        dnn_ctx_reset_step(&ctx);
    }
    if (dnn_cuda_sync() != 0) { fprintf(stderr, "%s\n", dnn_cuda_last_error()); return 5; }
    dnn_ctx_destroy(&ctx);
    free(hx); free(hy);
    printf("ok\n");
    return 0;
}
