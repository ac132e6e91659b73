"""GPU: what the library does with tensors it did not create.

CPU callers of dnn.c may fill a `tensor` struct in by hand around a malloc'd payload (pool == NULL) and read
`((float *)y->data)[0]` after an op (bench/bench_ops.c:388-474 of the reference).  Here payloads live in device
memory, so such a tensor is refused at the op's entry with a message that names dnn_cuda_upload -- before any
kernel could be given the host pointer -- and a stray `fresh` bit in a hand-built struct is ignored."""
import ctypes as C
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

CHILD = r"""
import ctypes as C, sys
import numpy as np
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
from conftest import load_binding
B = load_binding()
d = B.Dnn(B.B200_LIB, params_mb=16, scratch_mb=64, data_mb=16)
host = np.ones((4, 8), np.float32)
t = B.Tensor()
t.data = host.ctypes.data                      # host memory, pool == NULL: the CPU caller's idiom
t.shape[0], t.shape[1], t.strides[0], t.strides[1], t.ndim, t.flags = 4, 8, 8, 1, 2, 2
print("calling", flush=True)
d.lib.tensor_relu(d.scratch, C.byref(t))
print("returned", flush=True)
"""


def test_host_payload_is_refused_with_a_message(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD.format(root=ROOT))
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=300)
    assert "calling" in r.stdout and "returned" not in r.stdout
    assert r.returncode != 0
    assert "dnn_cuda_upload" in r.stderr and "host memory" in r.stderr


def test_fresh_bit_of_a_hand_built_tensor_is_ignored(gpu, binding):
    """A caller-made struct with every flag bit set -- including the library's `fresh` bit, which shares a
    32-bit unit with the reference's two public flags -- and a gradient buffer of the caller's own (device
    memory that no dnn.c pool handed out, pre-filled with 5): backward must ADD to that buffer, as the
    reference would.  Only gradient buffers the library allocated itself can be `fresh` (stored to)."""
    import torch
    lib = gpu.lib
    x_np = np.linspace(-1, 1, 32, dtype=np.float32).reshape(4, 8)
    owner = gpu.tensor(x_np, gpu.data)
    mine = torch.full((4, 8), 5.0, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    t = binding.Tensor()
    C.memmove(C.byref(t), owner, C.sizeof(binding.Tensor))
    t.grad = mine.data_ptr()
    t.flags = 0xFFFFFFFF
    y = lib.tensor_relu(gpu.scratch, C.byref(t))
    gpu.backward_from(y, np.ones((4, 8), np.float32))
    gpu.sync()
    got = mine.cpu().numpy()
    assert np.array_equal(got, 5.0 + (x_np > 0)), got
    gpu.reset_step()
