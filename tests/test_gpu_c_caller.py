"""GPU: a C program written against the reference's API (the MNIST training loop of
examples/mnist/mnist_train.c:99-114), compiled with gcc against include/ and linked with libdnn_b200.so,
runs on the device and prints the same losses as the same loop driven through ctypes."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT
from oracle import dnn_oracle as O

pytestmark = pytest.mark.gpu


def test_c_training_loop_links_and_runs(binding, tmp_path):
    exe = str(tmp_path / "mnist_loop")
    libdir = os.path.join(ROOT, "dnn.c_b200")
    cc = subprocess.run(["gcc", "-std=gnu11", "-Wall", "-Werror", "-I" + os.path.join(ROOT, "include"),
                         os.path.join(ROOT, "tests", "c_caller", "mnist_loop.c"), "-o", exe, "-L" + libdir, "-l:libdnn_b200.so",
                         "-Wl,-rpath," + libdir, "-lm"], capture_output=True, text=True)
    assert cc.returncode == 0, cc.stderr
    batch, steps = 32, 3
    run = subprocess.run([exe, str(batch), str(steps)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    lines = run.stdout.split()
    assert lines[-1] == "ok" and len(lines) == steps + 1
    got = [np.float32(x) for x in lines[:steps]]
    assert got[-1] < got[0], "the loss did not go down"

    # the same loop through ctypes: same seed, same creation order, same synthetic batch
    d = binding.Dnn(binding.B200_LIB, params_mb=64, scratch_mb=1024, data_mb=16)
    lib = d.lib
    lib.dnn_seed(2)
    c1, c2 = lib.conv2d_create(d.params, 1, 32, 3, 1, 1), lib.conv2d_create(d.params, 32, 64, 3, 1, 1)
    f1, f2 = lib.linear_create(d.params, 3136, 128), lib.linear_create(d.params, 128, 10)
    params = []
    for m in (c1, c2, f1, f2):
        params += d.parameters(m)
    arr = (binding.TensorP * len(params))(*params)
    opt = lib.adamw_create(d.params, arr, len(params), 1e-3, 0.9, 0.999, 1e-8, 0.01)
    r = O.Rng(7)
    hx = np.array([r.uniform() for _ in range(batch * 784)], np.float32).reshape(batch, 1, 28, 28)
    hy = np.array([r.uniform_int(10) for _ in range(batch)], np.int32)
    want = []
    for s in range(steps):
        x, y = d.tensor(hx, d.data), d.tensor(hy, d.data)
        h = lib.tensor_avg_pool2d(d.scratch, lib.tensor_relu(d.scratch, lib.conv2d_forward(d.scratch, c1, x)), 2, 2)
        h = lib.tensor_avg_pool2d(d.scratch, lib.tensor_relu(d.scratch, lib.conv2d_forward(d.scratch, c2, h)), 2, 2)
        h = lib.tensor_reshape(d.scratch, h, 2, binding.ints([batch, 3136]))
        h = lib.tensor_relu(d.scratch, lib.linear_forward(d.scratch, f1, h))
        loss = lib.tensor_cross_entropy(d.scratch, lib.linear_forward(d.scratch, f2, h), y, 1)
        lib.dnn_backward(d.scratch, loss)
        want.append(np.float32(d.scalar(loss)))
        lib.adamw_step(opt); lib.adamw_zero_grad(opt)
        d.reset_step()
    d.close()
    assert got == want, (got, want)
