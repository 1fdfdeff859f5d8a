"""The allocation-free convolution entry point (ob200_conv2d_fprop_noalloc).

It exists for callers that cannot call cudaMalloc when they need a convolution — for
example while a stream is being captured, from inside an allocator hook, or in a host
program that distributes all device memory at start-up.  Its split-K scratch is a fixed
array inside the library, shared by all calls, so two things are checked here through
the C ABI: the result equals the ordinary entry point's (which uses caller-provided
scratch) and the CPU oracle's within the fp32 tolerance of the kernel tests, and a second
call right after the first — which finds the first call's leftovers in the array — is
just as good.  Oversized
problems must be refused with a clear code instead of overrunning the array.

The file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-4   # same fp32 tolerance as tests/test_kernels_gpu.py


@pytest.fixture(scope="module")
def lib(built):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    L = ctypes.CDLL(built["liborion_kernels.so"])
    vp, i = ctypes.c_void_p, ctypes.c_int
    L.ob200_conv2d_fprop_noalloc.argtypes = [vp] * 6 + [i] * 15 + [i, i, i, vp]
    L.ob200_conv2d_fprop_noalloc.restype = i
    L.ob200_conv2d_fprop_ex.argtypes = [vp] * 6 + [i] * 15 + [i, i, vp, vp, i, vp]
    L.ob200_conv2d_fprop_ex.restype = i
    return L


def _args(x, w, y, shift, relu, stride, pad):
    Nb, H, W, C = x.shape
    K, R, S, _ = w.shape
    return [x.data_ptr(), w.data_ptr(), y.data_ptr(), None, shift.data_ptr(), None, relu, 0, Nb, H, W, C, K, R, S, stride, stride,
            pad, pad, 1, 1]


def _rel(a, b):
    return ((a.double() - b.double()).abs().max() / b.double().abs().max()).item()


@pytest.mark.parametrize("shape,bn,splits", [((4, 7, 7, 512, 512, 3, 1, 1), 64, 8), ((4, 14, 14, 256, 256, 3, 1, 1), 128, 4),
                                             ((2, 7, 7, 2048, 512, 1, 1, 0), 64, 16)])
def test_noalloc_matches_the_ordinary_entry_point_twice_in_a_row(lib, shape, bn, splits):
    Nb, H, W, C, K, R, stride, pad = shape
    torch.manual_seed(99)
    stream = torch.cuda.current_stream().cuda_stream
    P = (H + 2 * pad - R) // stride + 1
    tiles = ((Nb * P * P + 127) // 128) * ((K + bn - 1) // bn)
    for attempt in range(2):
        x = torch.randn(Nb, H, W, C, device="cuda")
        w = torch.randn(K, R, R, C, device="cuda") / (C * R * R) ** 0.5
        shift = torch.randn(K, device="cuda")
        want = torch.empty(Nb, P, P, K, device="cuda")
        got = torch.full_like(want, float("nan"))
        scratch = torch.empty(tiles * splits * 128 * bn, device="cuda")
        counters = torch.zeros(tiles, dtype=torch.int32, device="cuda")
        rc = lib.ob200_conv2d_fprop_ex(*_args(x, w, want, shift, 1, stride, pad), bn, splits, scratch.data_ptr(),
                                       counters.data_ptr(), 148, stream)
        assert rc == 0
        rc = lib.ob200_conv2d_fprop_noalloc(*_args(x, w, got, shift, 1, stride, pad), bn, splits, 148, stream)
        assert rc == 0, "call %d returned %d" % (attempt, rc)
        torch.cuda.synchronize()
        assert not torch.isnan(got).any()
        assert _rel(got, want) < TOL, "call %d differs from ob200_conv2d_fprop_ex" % attempt
        from oracle import numeric_oracle as O
        assert O.rel_err(got, O.conv2d_nhwc(x, w, (stride, stride), (pad, pad), shift=shift, act=1)) < TOL, \
            "call %d differs from the CPU oracle" % attempt
    lib.ob200_conv2d_fprop_noalloc_status.restype = ctypes.c_int
    assert lib.ob200_conv2d_fprop_noalloc_status() == 0, "a kernel wait ran out"


def test_noalloc_without_split_k_is_bit_identical(lib):
    torch.manual_seed(5)
    stream = torch.cuda.current_stream().cuda_stream
    x = torch.randn(2, 14, 14, 64, device="cuda")
    w = torch.randn(96, 3, 3, 64, device="cuda") / 24.0
    shift = torch.randn(96, device="cuda")
    a, b = torch.empty(2, 14, 14, 96, device="cuda"), torch.empty(2, 14, 14, 96, device="cuda")
    assert lib.ob200_conv2d_fprop_ex(*_args(x, w, a, shift, 0, 1, 1), 128, 1, None, None, 148, stream) == 0
    assert lib.ob200_conv2d_fprop_noalloc(*_args(x, w, b, shift, 0, 1, 1), 128, 1, 148, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(a, b)


def test_noalloc_refuses_problems_larger_than_its_array(lib):
    """32*56*56 rows x 256 channels with split-K would need 784*128*128 floats of scratch: far beyond 2 Mi."""
    stream = torch.cuda.current_stream().cuda_stream
    x = torch.zeros(32, 56, 56, 64, device="cuda")
    w = torch.zeros(256, 3, 3, 64, device="cuda")
    y = torch.zeros(32, 56, 56, 256, device="cuda")
    shift = torch.zeros(256, device="cuda")
    assert lib.ob200_conv2d_fprop_noalloc(*_args(x, w, y, shift, 0, 1, 1), 128, 2, 148, stream) == -3
    assert lib.ob200_conv2d_fprop_noalloc(*_args(x, w, y, shift, 0, 1, 1), 128, 1, 148, stream) == 0   # no scratch needed
    torch.cuda.synchronize()
