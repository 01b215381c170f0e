import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from __graft_entry__ import load_package  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    from oracle.inkq_oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own compiled kernels, when oracle/_ref/ is present and runs on this host."""
    from oracle.inkq_oracle import Reference
    if Reference.available_path()[0] is None:
        pytest.skip("oracle/_ref not built on this machine")
    return Reference()


@pytest.fixture(scope="session")
def golden():
    d = os.path.join(ROOT, "tests", "golden")
    return lambda name: np.load(os.path.join(d, name))


@pytest.fixture(scope="session")
def gpu(pkg):
    """A context on cuda:0.  GPU tests fail loudly when the library or the device is missing."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    pkg.build()
    torch.cuda.set_device(0)
    ctx = pkg.Context(0, torch.cuda.current_stream().cuda_stream)
    yield ctx
    ctx.close()


def f16(a):
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


def rel_err(got, ref):
    """max |got-ref| / max(|ref|, 1e-3 * rms(ref)): the fp32 agreement measure of this project."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    floor = 1e-3 * np.sqrt(np.mean(ref * ref)) + 1e-30
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), floor)))
