"""CPU: the host-side logic of data parallelism.

* bucket planning (pure host code of libdnn_b200.so);
* the exchange semantics with two real processes over gloo: each rank computes the
  gradients of its half of the batch with the numpy oracle, the ranks average them,
  and the result must equal the single-process gradients of the whole batch -- which
  is what dnn_cuda_dp_decoder_lm_train_step promises (NCCL average of per-rank
  mean-loss gradients, then identical clip + AdamW on every rank)."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

from conftest import ROOT, load_binding

B = load_binding()


def test_bucket_planner_merges_neighbours_and_cuts_buckets():
    lib = C.CDLL(B.B200_LIB)
    f = lib.dnn_cuda_dp_plan_buckets
    f.restype = C.c_int
    f.argtypes = [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.c_int, C.c_size_t, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.c_int]
    # three buffers back to back (256-byte allocator padding), one far away, given out of order
    addrs = [0x10000 + 1024, 0x10000, 0x90000, 0x10000 + 1024 + 4096]
    sizes = [4000, 1000, 512, 300]          # 1000 -> padded to 1024; 4000 -> padded to 4096
    n = len(addrs)
    oa, ob = (C.c_size_t * 16)(), (C.c_size_t * 16)()
    k = f((C.c_size_t * n)(*addrs), (C.c_size_t * n)(*sizes), n, 1 << 20, oa, ob, 16)
    assert k == 2
    assert (oa[0], ob[0]) == (0x10000, 1024 + 4096 + 300)
    assert (oa[1], ob[1]) == (0x90000, 512)
    # a small bucket size cuts the merged range
    k = f((C.c_size_t * n)(*addrs), (C.c_size_t * n)(*sizes), n, 2048, oa, ob, 16)
    assert k == 4 and [ob[i] for i in range(3)] == [2048, 2048, 1024 + 4096 + 300 - 4096]
    assert f((C.c_size_t * 0)(), (C.c_size_t * 0)(), 0, 1024, oa, ob, 16) == 0


WORKER = r"""
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
from oracle import dnn_oracle as O
import models
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
cfg = dict(models.lm_config("tiny"), B=4)
ids, tgt = models.lm_inputs(cfg)
rng = np.random.default_rng(11)
names = O.lm_param_names(cfg["L"])
shapes = {{"embed.weight": (cfg["V"], cfg["D"]), "lm_head.bias": (cfg["V"],), "norm.weight": (cfg["D"],)}}
D, F = cfg["D"], cfg["F"]
leaf = {{"qkv_proj.weight": (D, 3 * D), "qkv_proj.bias": (3 * D,), "out_proj.weight": (D, D), "out_proj.bias": (D,),
        "attn_norm.weight": (D,), "ffn_norm.weight": (D,), "ffn.gate_proj.weight": (D, F), "ffn.gate_proj.bias": (F,),
        "ffn.up_proj.weight": (D, F), "ffn.up_proj.bias": (F,), "ffn.down_proj.weight": (F, D), "ffn.down_proj.bias": (D,)}}
P = {{}}
for n in names:
    shp = shapes.get(n) or leaf[n.split(".", 2)[2]]
    P[n] = np.ones(shp, np.float32) if n.endswith("norm.weight") else (rng.standard_normal(shp) * 0.05).astype(np.float32)
per = cfg["B"] // world
lo = rank * per
loss, G = O.lm_loss_and_grads(P, ids[lo:lo + per], tgt[lo:lo + per], cfg["L"], cfg["H"])
flat = torch.from_numpy(np.concatenate([G[n].reshape(-1) for n in names]).astype(np.float64))
dist.all_reduce(flat)            # sum, then the average the NCCL path asks for
flat /= world
if rank == 0:
    loss_all, G_all = O.lm_loss_and_grads(P, ids, tgt, cfg["L"], cfg["H"])
    want = np.concatenate([G_all[n].reshape(-1) for n in names]).astype(np.float64)
    err = np.linalg.norm(flat.numpy() - want) / np.linalg.norm(want)
    print("DP_ERR", err)
    assert err < 1e-6, err
dist.destroy_process_group()
"""


def test_two_rank_average_equals_full_batch_gradients(tmp_path):
    import subprocess
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    port = 29650 + os.getpid() % 200
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "DP_ERR" in outs[0]
