import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import cg_oracle
    cg_oracle.build()
    cg_oracle.lib()
    return cg_oracle


@pytest.fixture(scope="session")
def host_model():
    """Host build of the product's per-stream coder loops (tests/host_model/coder_host.cpp)."""
    d = os.path.join(ROOT, "tests", "host_model")
    src = os.path.join(d, "coder_host.cpp")
    hdr = os.path.join(ROOT, "cachegen_b200", "csrc", "cg_coder.cuh")
    so = os.path.join(d, "libcoder_host.so")
    if not os.path.exists(so) or os.path.getmtime(so) < max(os.path.getmtime(src), os.path.getmtime(hdr)):
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-o", so, src])
    lib = ctypes.CDLL(so)
    p, i, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    lib.hm_encode_stream.restype = i64
    lib.hm_encode_stream.argtypes = [p, i, p, i, p, i64, i]
    lib.hm_decode_stream.restype = None
    lib.hm_decode_stream.argtypes = [p, i, p, i64, i, p, i]
    lib.hm_decode_pair.restype = i
    lib.hm_decode_pair.argtypes = [p, p, i, p, i64, p, i64, i, p, i, i]
    lib.hm_fast_levels_for.restype = i
    lib.hm_fast_levels_for.argtypes = [i, i]
    return lib


@pytest.fixture(scope="session")
def golden_cpu():
    return np.load(os.path.join(ROOT, "tests", "golden", "ref_python_cpu.npz"))
