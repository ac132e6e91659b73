"""CPU: the C-ABI library loads, exports every function the headers declare,
keeps the reference's struct layouts, and its host-only logic (RNG, LR
schedule, bump pools, bucket planning) matches the oracle.  No GPU work."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from conftest import ROOT, load_binding
from oracle import dnn_oracle as O

B = load_binding()


@pytest.fixture(scope="module")
def lib():
    assert os.path.exists(B.B200_LIB), "libdnn_b200.so is not built (python dnn.c_b200/build.py)"
    return C.CDLL(B.B200_LIB)


def declared_functions():
    names = set()
    for h in ("dnn_b200.h", "dnn_cuda.h"):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
        for m in re.finditer(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\(", text):
            names.add(m.group(1))
    return sorted(n for n in names if n not in ("defined", "sizeof", "void"))


def test_every_declared_symbol_is_exported(lib):
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_tables_are_exported(lib):
    for n in list(B.API) + list(B.CUDA_API):
        assert hasattr(lib, n), n


def test_struct_layouts_match_reference():
    # sizes and offsets measured on the reference build (x86-64, LP64)
    assert C.sizeof(B.Tensor) == 120 and C.sizeof(B.GradFn) == 48 and C.sizeof(B.MemPool) == 24 and C.sizeof(B.AdamW) == 56
    offs = {f: getattr(B.Tensor, f).offset for f in ("data", "grad", "shape", "strides", "ndim", "flags", "offset", "parent", "grad_fn", "pool")}
    assert offs == dict(data=0, grad=8, shape=16, strides=48, ndim=80, flags=84, offset=88, parent=96, grad_fn=104, pool=112)


def test_shim_headers_compile(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "dnn.h"\n#include "dnn_cuda.h"\n_Static_assert(sizeof(tensor)==120,"t");_Static_assert(sizeof(grad_fn)==48,"g");'
                   '_Static_assert(sizeof(module)==72,"m");_Static_assert(sizeof(linear)==96,"l");_Static_assert(sizeof(adamw_opt)==56,"a");int main(void){return 0;}\n')
    rc = os.system("gcc -std=gnu11 -I%s -c %s -o %s" % (os.path.join(ROOT, "include"), src, tmp_path / "t.o"))
    assert rc == 0


def test_host_rng_matches_oracle(lib):
    class Rng(C.Structure):
        _fields_ = [("s", C.c_uint64 * 2)]
    lib.dnn_rng_seed.restype, lib.dnn_rng_seed.argtypes = Rng, [C.c_uint64]
    lib.dnn_rng_uniform_int.restype, lib.dnn_rng_uniform_int.argtypes = C.c_int, [C.POINTER(Rng), C.c_int]
    lib.dnn_rng_uniform.restype, lib.dnn_rng_uniform.argtypes = C.c_float, [C.POINTER(Rng)]
    for seed in (0, 4, 12345):
        r, o = lib.dnn_rng_seed(seed), O.Rng(seed)
        assert (r.s[0], r.s[1]) == (o.s0, o.s1)
        for n in (256, 32000, 10, 1):
            assert [lib.dnn_rng_uniform_int(C.byref(r), n) for _ in range(50)] == [o.uniform_int(n) for _ in range(50)]
        assert [lib.dnn_rng_uniform(C.byref(r)) for _ in range(20)] == [float(o.uniform()) for _ in range(20)]


def _ctx(lib):
    for n in ("dnn_ctx_init", "dnn_ctx_destroy", "_mem_pool_alloc", "mem_pool_mark", "mem_pool_release", "mem_pool_reset",
              "lr_scheduler_create", "lr_scheduler_step", "lr_scheduler_get_lr", "lr_scheduler_reset"):
        getattr(lib, n).restype, getattr(lib, n).argtypes = B.API[n]
    ctx = B.DnnCtx()
    assert lib.dnn_ctx_init(C.byref(ctx), 1 << 20, 1 << 20, 1 << 20) == 0
    return ctx


def test_pools_bump_mark_release_without_a_device(lib):
    ctx = _ctx(lib)
    p = ctx.scratch
    a = lib._mem_pool_alloc(p, 100, None)
    mark = lib.mem_pool_mark(p)
    b = lib._mem_pool_alloc(p, 40, None)
    assert b >= a + 100 and p.contents.offset >= 140
    assert bytes((C.c_char * 40).from_address(b)) == b"\0" * 40
    lib.mem_pool_release(p, mark)
    assert p.contents.offset == mark
    src = (C.c_char * 8)(*b"abcdefgh")
    c = lib._mem_pool_alloc(p, 8, C.cast(src, C.c_void_p))
    assert bytes((C.c_char * 8).from_address(c)) == b"abcdefgh"
    lib.mem_pool_reset(p)
    assert p.contents.offset == 0
    lib.dnn_ctx_destroy(C.byref(ctx))


@pytest.mark.parametrize("schedule,warmup,total,step,gamma", [(0, 0, 100, 0, 0.0), (1, 10, 100, 0, 0.0), (2, 5, 50, 0, 0.0),
                                                                (3, 0, 40, 0, 0.0), (4, 3, 100, 7, 0.5), (5, 0, 30, 0, 0.9)])
def test_lr_schedules_match_oracle(lib, schedule, warmup, total, step, gamma):
    ctx = _ctx(lib)
    opt = B.AdamW()
    s = lib.lr_scheduler_create(ctx.params, C.byref(opt), schedule, 6e-4, warmup, total, -1.0, step, gamma)
    for t in range(60):
        want = O.lr_schedule(schedule, 6e-4, -1.0, warmup, total, step, gamma, t)
        assert abs(opt.lr - want) <= 2e-7 * abs(want) + 1e-12, (t, opt.lr, want)
        lib.lr_scheduler_step(s)
    lib.dnn_ctx_destroy(C.byref(ctx))


def test_lr_schedules_equal_the_reference_bit_for_bit(lib):
    """The schedules are host arithmetic (src/optim.c:104-189): the library's learning rates over 130 steps
    of eight scheduler set-ups, lr_scheduler_get_lr and lr_scheduler_reset must equal the vectors the
    unmodified reference produced (tests/golden/ops.npz) exactly.  Needs no device."""
    from cases import CASES
    from golden_util import check
    case = [c for c in CASES if c.name == "lr_schedules"][0]
    ctx = _ctx(lib)

    class Host:
        pass
    h = Host()
    h.lib, h.params = lib, ctx.params
    got = case.run(h, case.make(None))
    golden = np.load(os.path.join(ROOT, "tests", "golden", "ops.npz"))
    for k, v in got.items():
        key = "lr_schedules/" + k
        check(key, v, golden[key], golden[key + "#"], 0, exact=True)
    lib.dnn_ctx_destroy(C.byref(ctx))


def test_no_device_is_reported_not_faked(lib):
    lib.dnn_cuda_available.restype = C.c_int
    import torch
    assert bool(lib.dnn_cuda_available()) == torch.cuda.is_available()
