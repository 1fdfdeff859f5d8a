"""Every function declared in include/*.h is exported by its library (no compute calls)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADERS = {"orion_sched.h": "liborion_sched.so", "orion_capture.h": "liborion_capture.so", "orion_kernels.h": "liborion_kernels.so"}


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text)
    return sorted(set(n for n in names if n not in ("defined",)))


@pytest.mark.parametrize("header", sorted(HEADERS))
def test_library_exports_every_declared_symbol(header, built):
    names = _declared(header)
    assert len(names) >= 5
    lib = ctypes.CDLL(built[HEADERS[header]])
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, "not exported by %s: %s" % (HEADERS[header], missing)


def test_reference_entry_points_are_present(built):
    sched = ctypes.CDLL(built["liborion_sched.so"])
    for name in ("sched_init", "setup", "setup_change", "schedule", "reset"):
        assert hasattr(sched, name)
    cap = ctypes.CDLL(built["liborion_capture.so"])
    for name in ("block", "stop", "cudaLaunchKernel", "cudaMemcpyAsync", "cudaMalloc", "cublasSgemm_v2",
                 "cublasSgemmStridedBatched", "cudnnConvolutionForward", "cudnnBatchNormalizationForwardInference",
                 "cudnnBackendExecute", "cublasGemmEx", "cublasLtMatmul", "cudaLaunchKernelExC"):
        assert hasattr(cap, name), name


def test_kernel_entry_points_reject_bad_arguments_without_a_gpu(built):
    lib = ctypes.CDLL(built["liborion_kernels.so"])
    # dtype 7 does not exist; argument checks run before any CUDA call
    rc = lib.ob200_conv2d_fprop_ex(None, None, None, None, None, None, 0, 7, 1, 8, 8, 8, 8, 1, 1, 1, 1, 0, 0, 1, 1, 128, 1, None,
                                   None, 8, None)
    assert rc < 0
    bn, splits = ctypes.c_int(), ctypes.c_int()
    lib.ob200_plan_conv.argtypes = [ctypes.c_int, ctypes.c_longlong] + [ctypes.c_int] * 5 + [ctypes.POINTER(ctypes.c_int)] * 2
    assert lib.ob200_plan_conv(0, 196, 512, 3, 3, 512, 148, ctypes.byref(bn), ctypes.byref(splits)) == 0
    assert bn.value in (64, 128) and 1 <= splits.value <= 16
