"""TEST INFRASTRUCTURE — CPU restatement of the workload arithmetic.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg may import this
file; the product never does.

The reference computes nothing itself: it forwards every captured call to cuDNN 7.6 /
cuBLAS 10.2 / PyTorch 1.12 kernels (reference src/scheduler/utils_sched.cpp:291,347,495),
none of which is part of its repository, and it ships no golden vectors.  Parity is
therefore UNPINNED by the reference; the oracle is the published definition of each
op evaluated in float64 on the CPU (torch CPU kernels), against which the tolerance of
the benchmark specification applies: fp32 rel 1e-4, bf16 rel 2e-2.
"""
import torch
import torch.nn.functional as F


def conv2d_nhwc(x, w, stride, padding, dilation=(1, 1), scale=None, shift=None, residual=None, act=0, groups=1):
    """cudnnConvolutionForward as the reference calls it (utils_sched.cpp:284-296), for NHWC x / KRSC w,
    followed by the optional per-channel affine, residual add and activation of the fused epilogue."""
    xd = x.detach().double().cpu().permute(0, 3, 1, 2)
    wd = w.detach().double().cpu().permute(0, 3, 1, 2)
    y = F.conv2d(xd, wd, stride=stride, padding=padding, dilation=dilation, groups=groups).permute(0, 2, 3, 1)
    if scale is not None:
        y = y * scale.detach().double().cpu()
    if shift is not None:
        y = y + shift.detach().double().cpu()
    if residual is not None:
        y = y + residual.detach().double().cpu()
    if act >= 1:
        y = y.clamp_min(0)
    if act == 2:
        y = y.clamp_max(6)
    return y.contiguous()


def linear(x, w, bias=None, relu=False):
    """cublasSgemm as the reference calls it (utils_sched.cpp:490-501): y = x w^T + b."""
    y = x.detach().double().cpu() @ w.detach().double().cpu().t()
    if bias is not None:
        y = y + bias.detach().double().cpu()
    return y.clamp_min(0) if relu else y


def bn_inference(x, gamma, beta, mean, var, eps, relu=False):
    """cudnnBatchNormalizationForwardInference (utils_sched.cpp:340-353), channel = last dim."""
    d = lambda t: t.detach().double().cpu()
    y = (d(x) - d(mean)) / torch.sqrt(d(var) + eps)
    if gamma is not None:
        y = y * d(gamma)
    if beta is not None:
        y = y + d(beta)
    return y.clamp_min(0) if relu else y


def maxpool_nhwc(x, k, stride, pad):
    return F.max_pool2d(x.detach().double().cpu().permute(0, 3, 1, 2), k, stride, pad).permute(0, 2, 3, 1).contiguous()


def avgpool_nhwc(x):
    return x.detach().double().cpu().mean(dim=(1, 2))


def rel_err(got, want):
    want = want.double().cpu()
    got = got.detach().double().cpu()
    return ((got - want).abs().max() / want.abs().max().clamp_min(1e-30)).item()
