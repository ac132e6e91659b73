import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def load_binding():
    """The package directory is `dnn.c_b200` (not an importable name), so its
    modules are loaded by path."""
    name = "dnnc_b200_binding"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "dnn.c_b200", "binding.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libdnn_ref.so")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    # The reference's dgamma accumulation races under OpenMP (src/norm.c:299-321).
    os.environ.setdefault("OMP_NUM_THREADS", "1")


@pytest.fixture(scope="session")
def binding():
    return load_binding()


@pytest.fixture(scope="session")
def gpu(binding):
    """The CUDA library with a context.  Fails (does not skip) when the
    extension is missing: there is no CPU path to fall back to."""
    assert os.path.exists(binding.B200_LIB), "libdnn_b200.so is not built"
    d = binding.Dnn(binding.B200_LIB, params_mb=1024, scratch_mb=6144, data_mb=256)
    yield d
    d.close()


@pytest.fixture(scope="session")
def ref(binding):
    """The unmodified reference library, when oracle/_ref holds a build of it."""
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libdnn_ref.so not built (needs the reference sources)")
    d = binding.Dnn(REF_LIB, params_mb=256, scratch_mb=2048, data_mb=64)
    yield d
    d.close()
