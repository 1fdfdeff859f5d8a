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
                 "cudnnBackendExecute", "cublasGemmEx", "cublasLtMatmul", "cudaLaunchKernelExC", "cudaMallocAsync", "cudaFreeAsync",
                 "cudaMallocManaged", "cudaGraphLaunch"):
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


def _plan(lib, dtype, M, Kout, R, S, C, ctas):
    bn, splits, sk = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib.ob200_plan_schedule.argtypes = [ctypes.c_int, ctypes.c_longlong] + [ctypes.c_int] * 5 + [ctypes.POINTER(ctypes.c_int)] * 3
    assert lib.ob200_plan_schedule(dtype, M, Kout, R, S, C, ctas, ctypes.byref(bn), ctypes.byref(splits), ctypes.byref(sk)) == 0
    return bn.value, splits.value, sk.value


def test_schedule_planning_host_logic(built):
    """Which schedule a problem gets is host arithmetic: checked here for the ResNet-50 shapes without a GPU."""
    lib = ctypes.CDLL(built["liborion_kernels.so"])
    # deep tiles with a ragged last wave at training batch size: stream-K (196 tiles of 36 k-blocks on 148 CTAs)
    assert _plan(lib, 0, 32 * 28 * 28, 128, 3, 3, 128, 148) == (128, 1, 1)
    # shallow 1x1 layer (2 k-blocks per tile): one unit per tile, wide tiles, never cut
    assert _plan(lib, 0, 32 * 56 * 56, 256, 1, 1, 64, 148) == (128, 1, 0)
    # batch-4 inference, few deep tiles: split-K over the idle SMs, chains of at least four k-blocks
    bn, splits, sk = _plan(lib, 0, 4 * 7 * 7, 512, 3, 3, 512, 148)
    assert sk == 0 and bn == 64 and 2 <= splits <= 16 and 144 // splits >= 4
    # narrow outputs take narrow tiles; a small SM quota never over-splits
    assert _plan(lib, 0, 32 * 56 * 56, 64, 1, 1, 256, 148)[0] == 64
    for ctas in (1, 8, 37, 148):
        for (M, Kout, R, C) in [(12544, 64, 3, 64), (784, 1024, 1, 256), (196, 2048, 1, 512), (100352, 64, 7, 4)]:
            bn, splits, sk = _plan(lib, 0, M, Kout, R, R, C, ctas)
            nk = R * ((R * C + 31) // 32)
            assert bn in (64, 128) and 1 <= splits <= max(1, nk) and sk in (0, 1)
            tiles = ((M + 127) // 128) * ((Kout + bn - 1) // bn)
            if sk:
                assert splits == 1 and tiles * 4 >= ctas and nk >= 8
            else:
                assert tiles * splits <= max(tiles, ctas)
    # bad arguments are rejected
    assert lib.ob200_plan_schedule(0, 0, 64, 1, 1, 64, 148, None, None, None) < 0
