"""ctypes binding of liborion_kernels.so (the sm_100a workload kernels).

Tensors are passed as raw device pointers; torch is used only to own memory and
streams.  There is no fallback: if the library is missing or a launch fails the
call raises.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "lib", "liborion_kernels.so")
_lib = None

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError("liborion_kernels.so is not built; run `python -m orion_b200.build`")
        L = ctypes.CDLL(_LIB_PATH)
        L.ob200_conv2d_fprop.argtypes = [c_void_p] * 6 + [c_int] * 15 + [c_int, c_void_p]
        L.ob200_conv2d_fprop_ex.argtypes = [c_void_p] * 6 + [c_int] * 15 + [c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
        L.ob200_linear.argtypes = [c_void_p] * 4 + [c_int] * 5 + [c_int, c_void_p]
        L.ob200_plan_conv.argtypes = [c_int, c_ll, c_int, c_int, c_int, c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int)]
        L.ob200_bn_inference_f32.argtypes = [c_void_p] * 6 + [c_float, c_ll, c_int, c_int, c_int, c_void_p]
        L.ob200_binary_f32.argtypes = [c_void_p] * 3 + [c_ll, c_int, c_int, c_void_p]
        L.ob200_maxpool_nhwc_f32.argtypes = [c_void_p] * 2 + [c_int] * 7 + [c_int, c_void_p]
        L.ob200_avgpool_nhwc_f32.argtypes = [c_void_p] * 2 + [c_int] * 3 + [c_int, c_void_p]
        L.ob200_conv2d_dgrad.argtypes = [c_void_p] * 3 + [c_int] * 14 + [c_int, c_void_p]
        L.ob200_filter_transpose.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        L.ob200_bn_train_forward_f32.argtypes = [c_void_p] * 9 + [c_float, c_float, c_ll, c_int, c_int, c_void_p]
        L.ob200_bn_backward_f32.argtypes = [c_void_p] * 9 + [c_ll, c_int, c_int, c_void_p]
        L.ob200_relu_backward_f32.argtypes = [c_void_p] * 3 + [c_ll, c_int, c_void_p]
        L.ob200_bn_act_train_forward_f32.argtypes = [c_void_p] * 9 + [c_float, c_float, c_ll, c_int, c_int, c_int, c_void_p]
        L.ob200_bn_act_train_forward_f32.restype = c_int
        L.ob200_bn_act_backward_f32.argtypes = [c_void_p] * 11 + [c_ll, c_int, c_int, c_int, c_void_p]
        L.ob200_bn_act_backward_f32.restype = c_int
        L.ob200_sgd_momentum_f32.argtypes = [c_void_p] * 3 + [c_ll, c_float, c_float, c_float, c_int, c_int, c_int, c_void_p]
        L.ob200_conv2d_wgrad.argtypes = [c_void_p] * 3 + [c_int] * 14 + [c_int, c_void_p]
        L.ob200_conv2d_wgrad.restype = c_int
        L.ob200_layernorm.argtypes = [c_void_p] * 6 + [c_ll, c_int, c_float, c_int, c_int, c_void_p]
        L.ob200_softmax.argtypes = [c_void_p] * 2 + [c_ll, c_int, c_float, c_int, c_int, c_void_p]
        L.ob200_softmax_causal.argtypes = [c_void_p] * 2 + [c_ll, c_int, c_float, c_int, c_int, c_int, c_void_p]
        L.ob200_softmax_causal.restype = c_int
        L.ob200_bias_gelu.argtypes = [c_void_p] * 3 + [c_ll, c_int, c_int, c_int, c_void_p]
        L.ob200_adamw_f32.argtypes = [c_void_p] * 4 + [c_ll] + [c_float] * 5 + [c_int, c_int, c_void_p]
        for name in ("ob200_layernorm", "ob200_softmax", "ob200_bias_gelu", "ob200_adamw_f32"):
            getattr(L, name).restype = c_int
        L.ob200_linear_batched.argtypes = [c_void_p] * 3 + [c_int] * 5 + [c_ll] * 3 + [c_int, c_void_p]
        L.ob200_linear_batched.restype = c_int
        L.ob200_gemm_bf16.argtypes = [c_void_p] * 4 + [c_int] * 5 + [c_ll] * 3 + [c_int] * 2 + [c_ll] * 6 + [c_float, c_int, c_int, c_void_p]
        L.ob200_gemm_bf16.restype = c_int
        L.ob200_gemm_bf16_ex.argtypes = [c_void_p] * 6 + [c_int] * 5 + [c_ll] * 3 + [c_int] * 2 + [c_ll] * 6 + [c_float, c_int, c_int, c_int, c_void_p]
        L.ob200_gemm_bf16_ex.restype = c_int
        L.ob200_colsum.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_ll, c_int, c_int, c_void_p]
        L.ob200_colsum.restype = c_int
        L.ob200_softmax_backward.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_float, c_int, c_int, c_int, c_void_p]
        L.ob200_softmax_backward.restype = c_int
        for name in ("ob200_conv2d_dgrad", "ob200_filter_transpose", "ob200_bn_train_forward_f32", "ob200_bn_backward_f32",
                     "ob200_relu_backward_f32", "ob200_sgd_momentum_f32"):
            getattr(L, name).restype = c_int
        for name in ("ob200_conv2d_fprop", "ob200_conv2d_fprop_ex", "ob200_linear", "ob200_plan_conv", "ob200_bn_inference_f32",
                     "ob200_binary_f32", "ob200_maxpool_nhwc_f32", "ob200_avgpool_nhwc_f32", "ob200_read_status",
                     "ob200_sm_count"):
            getattr(L, name).restype = c_int
        L.ob200_depthwise_conv2d_f32.argtypes = [c_void_p] * 5 + [c_int] * 14 + [c_int, c_void_p]
        L.ob200_depthwise_conv2d_f32.restype = c_int
        L.ob200_tma_launch_count.argtypes = []
        L.ob200_tma_launch_count.restype = c_ll
        L.ob200_pad_channels.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_void_p]
        L.ob200_pad_channels.restype = c_int
        _lib = L
    return _lib


def _check(rc, what):
    if rc != 0:
        raise RuntimeError("%s failed with code %d" % (what, rc))


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _dtype_code(t):
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise TypeError("orion_b200 kernels take float32 or bfloat16, got %s" % t.dtype)


def tma_launch_count():
    """Implicit-GEMM launches so far whose operands were fed by TMA."""
    return lib().ob200_tma_launch_count()


def sm_count():
    return lib().ob200_sm_count()


def read_status():
    """Device status word (synchronises): 0 unless a kernel gave up on a bounded wait."""
    return lib().ob200_read_status()


def conv2d_nhwc(x, w, stride=(1, 1), padding=(0, 0), dilation=(1, 1), scale=None, shift=None, residual=None, relu=False,
                num_ctas=None, bn=None, splits=None, out=None, tf32=False):
    """x: [N, H, W, C] contiguous, w: [K, R, S, C] contiguous -> [N, P, Q, K]."""
    assert x.is_cuda and x.is_contiguous() and w.is_contiguous() and x.dtype == w.dtype
    Nb, H, W, C = x.shape
    K, R, S, C2 = w.shape
    assert C == C2
    P = (H + 2 * padding[0] - dilation[0] * (R - 1) - 1) // stride[0] + 1
    Q = (W + 2 * padding[1] - dilation[1] * (S - 1) - 1) // stride[1] + 1
    y = out if out is not None else torch.empty((Nb, P, Q, K), device=x.device, dtype=x.dtype)
    n = num_ctas or sm_count()
    code = 2 if (tf32 and x.dtype == torch.float32) else _dtype_code(x)
    args = [_ptr(x), _ptr(w), _ptr(y), _ptr(scale), _ptr(shift), _ptr(residual), int(relu), code, Nb, H, W, C, K, R, S,
            stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1]]
    if bn is None and splits is None:
        _check(lib().ob200_conv2d_fprop(*args, n, _stream()), "ob200_conv2d_fprop")
    else:
        bn = bn or 128
        splits = splits or 1
        scratch = counters = None
        if splits > 1:
            tiles = ((Nb * P * Q + 127) // 128) * ((K + bn - 1) // bn)
            scratch = torch.empty(tiles * splits * 128 * bn, device=x.device, dtype=torch.float32)
            counters = torch.zeros(tiles, device=x.device, dtype=torch.int32)
        _check(lib().ob200_conv2d_fprop_ex(*args, bn, splits, _ptr(scratch), _ptr(counters), n, _stream()),
               "ob200_conv2d_fprop_ex")
    return y


def depthwise_conv2d_nhwc(x, w, stride=(1, 1), padding=(0, 0), dilation=(1, 1), scale=None, shift=None, relu=0, tap_major=False,
                          num_ctas=None):
    """x: [N, H, W, C] float32, w: [C, R, S] (or [R, S, C] with tap_major) -> [N, P, Q, C]."""
    assert x.is_cuda and x.is_contiguous() and w.is_contiguous() and x.dtype == torch.float32 and w.dtype == torch.float32
    Nb, H, W, C = x.shape
    R, S = (w.shape[0], w.shape[1]) if tap_major else (w.shape[1], w.shape[2])
    P = (H + 2 * padding[0] - dilation[0] * (R - 1) - 1) // stride[0] + 1
    Q = (W + 2 * padding[1] - dilation[1] * (S - 1) - 1) // stride[1] + 1
    y = torch.empty((Nb, P, Q, C), device=x.device, dtype=x.dtype)
    _check(lib().ob200_depthwise_conv2d_f32(_ptr(x), _ptr(w), _ptr(y), _ptr(scale), _ptr(shift), int(relu), Nb, H, W, C, R, S,
                                            stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1], int(tap_major),
                                            num_ctas or sm_count(), _stream()), "ob200_depthwise_conv2d_f32")
    return y


def pad_channels(x, c_pad, num_ctas=None):
    """[..., C] contiguous -> [..., c_pad] with zeros in the added channels."""
    assert x.is_cuda and x.is_contiguous() and c_pad > x.shape[-1]
    y = torch.empty(x.shape[:-1] + (c_pad,), device=x.device, dtype=x.dtype)
    _check(lib().ob200_pad_channels(_ptr(x), _ptr(y), x.numel() // x.shape[-1], x.shape[-1], c_pad, x.element_size(),
                                    num_ctas or sm_count(), _stream()), "ob200_pad_channels")
    return y


def linear(x, w, bias=None, relu=False, num_ctas=None):
    """x: [M, K], w: [N, K] -> [M, N]."""
    assert x.is_cuda and x.is_contiguous() and w.is_contiguous() and x.dtype == w.dtype
    M, K = x.shape
    N = w.shape[0]
    y = torch.empty((M, N), device=x.device, dtype=x.dtype)
    _check(lib().ob200_linear(_ptr(x), _ptr(w), _ptr(y), _ptr(bias), int(relu), _dtype_code(x), M, N, K,
                              num_ctas or sm_count(), _stream()), "ob200_linear")
    return y


def bn_inference(x, gamma, beta, mean, var, eps, relu=False, num_ctas=None, out=None):
    """Channel-last batch-norm inference: x [..., C] float32."""
    assert x.is_contiguous() and x.dtype == torch.float32
    C = x.shape[-1]
    y = out if out is not None else torch.empty_like(x)
    _check(lib().ob200_bn_inference_f32(_ptr(x), _ptr(y), _ptr(gamma), _ptr(beta), _ptr(mean), _ptr(var), float(eps), x.numel(), C,
                                        int(relu), num_ctas or sm_count(), _stream()), "ob200_bn_inference_f32")
    return y


def binary(a, b=None, mode=0, num_ctas=None, out=None):
    """mode 0: relu(a); 1: a + b; 2: relu(a + b)."""
    assert a.is_contiguous() and a.dtype == torch.float32
    y = out if out is not None else torch.empty_like(a)
    _check(lib().ob200_binary_f32(_ptr(a), _ptr(b), _ptr(y), a.numel(), mode, num_ctas or sm_count(), _stream()),
           "ob200_binary_f32")
    return y


def maxpool_nhwc(x, k, stride, pad, num_ctas=None):
    Nb, H, W, C = x.shape
    P = (H + 2 * pad - k) // stride + 1
    Q = (W + 2 * pad - k) // stride + 1
    y = torch.empty((Nb, P, Q, C), device=x.device, dtype=x.dtype)
    _check(lib().ob200_maxpool_nhwc_f32(_ptr(x), _ptr(y), Nb, H, W, C, k, stride, pad, num_ctas or sm_count(), _stream()),
           "ob200_maxpool_nhwc_f32")
    return y


def avgpool_nhwc(x, num_ctas=None):
    Nb, H, W, C = x.shape
    y = torch.empty((Nb, C), device=x.device, dtype=x.dtype)
    _check(lib().ob200_avgpool_nhwc_f32(_ptr(x), _ptr(y), Nb, H * W, C, num_ctas or sm_count(), _stream()),
           "ob200_avgpool_nhwc_f32")
    return y


def filter_transpose(w):
    """w: [K, R, S, C] -> [C, R, S, K] (the layout ob200_conv2d_dgrad reads)."""
    K, R, S, C = w.shape
    wt = torch.empty((C, R, S, K), device=w.device, dtype=w.dtype)
    _check(lib().ob200_filter_transpose(_ptr(w), _ptr(wt), K, R * S, C, w.element_size(), _stream()), "ob200_filter_transpose")
    return wt


def conv2d_dgrad_nhwc(dy, w, input_hw, stride=(1, 1), padding=(0, 0), dilation=(1, 1), num_ctas=None):
    """dy: [N, P, Q, K], w: [K, R, S, C] -> dx [N, H, W, C]."""
    assert dy.is_contiguous() and w.is_contiguous() and dy.dtype == w.dtype
    Nb, P, Q, K = dy.shape
    K2, R, S, C = w.shape
    assert K == K2
    H, W = input_hw
    wt = filter_transpose(w)
    dx = torch.empty((Nb, H, W, C), device=dy.device, dtype=dy.dtype)
    _check(lib().ob200_conv2d_dgrad(_ptr(dy), _ptr(wt), _ptr(dx), _dtype_code(dy), Nb, H, W, C, K, R, S, stride[0], stride[1],
                                    padding[0], padding[1], dilation[0], dilation[1], num_ctas or sm_count(), _stream()),
           "ob200_conv2d_dgrad")
    return dx


def bn_train_forward(x, gamma, beta, running_mean, running_var, eps, momentum, num_ctas=None):
    """x: [..., C] float32 -> (y, save_mean, save_invstd); running stats are updated in place."""
    assert x.is_contiguous() and x.dtype == torch.float32
    C = x.shape[-1]
    rows = x.numel() // C
    y = torch.empty_like(x)
    save_mean = torch.empty(C, device=x.device)
    save_invstd = torch.empty(C, device=x.device)
    sums = torch.zeros(2 * C, device=x.device, dtype=torch.float64)
    _check(lib().ob200_bn_train_forward_f32(_ptr(x), _ptr(y), _ptr(gamma), _ptr(beta), _ptr(running_mean), _ptr(running_var),
                                            _ptr(save_mean), _ptr(save_invstd), _ptr(sums), float(eps), float(momentum), rows, C,
                                            num_ctas or sm_count(), _stream()), "ob200_bn_train_forward_f32")
    return y, save_mean, save_invstd


def bn_backward(dy, x, gamma, save_mean, save_invstd, num_ctas=None):
    assert dy.is_contiguous() and x.is_contiguous()
    C = x.shape[-1]
    rows = x.numel() // C
    dx = torch.empty_like(x)
    dgamma, dbeta = torch.empty(C, device=x.device), torch.empty(C, device=x.device)
    sums = torch.zeros(2 * C, device=x.device, dtype=torch.float64)
    _check(lib().ob200_bn_backward_f32(_ptr(dy), _ptr(x), _ptr(dx), _ptr(gamma), _ptr(save_mean), _ptr(save_invstd), _ptr(dgamma),
                                       _ptr(dbeta), _ptr(sums), rows, C, num_ctas or sm_count(), _stream()), "ob200_bn_backward_f32")
    return dx, dgamma, dbeta


def bn_act_train_forward(x, gamma, beta, running_mean, running_var, eps, momentum, act=0, residual=None, num_ctas=None):
    """y = act(batch_norm_train(x) [+ residual]); x: [..., C] float32 -> (y, save_mean, save_invstd).  Two launches, no
    scratch to clear; running statistics are updated in place.  act: 0 none, 1 ReLU, 2 ReLU6."""
    assert x.is_contiguous() and x.dtype == torch.float32
    C = x.shape[-1]
    y = torch.empty_like(x)
    save_mean, save_invstd = torch.empty(C, device=x.device), torch.empty(C, device=x.device)
    _check(lib().ob200_bn_act_train_forward_f32(_ptr(x), _ptr(residual), _ptr(y), _ptr(gamma), _ptr(beta), _ptr(running_mean),
                                                _ptr(running_var), _ptr(save_mean), _ptr(save_invstd), float(eps), float(momentum),
                                                x.numel() // C, C, int(act), num_ctas or sm_count(), _stream()),
           "ob200_bn_act_train_forward_f32")
    return y, save_mean, save_invstd


def bn_act_backward(dy, x, gamma, beta, save_mean, save_invstd, act=0, yout=None, want_dres=False, num_ctas=None):
    """Backward of bn_act_train_forward -> (dx, dres or None, dgamma, dbeta).  `yout` (the saved forward output) is only
    needed when the forward pass added a residual before an activation."""
    assert dy.is_contiguous() and x.is_contiguous()
    C = x.shape[-1]
    dx = torch.empty_like(x)
    dres = torch.empty_like(x) if want_dres else None
    dgamma, dbeta = torch.empty(C, device=x.device), torch.empty(C, device=x.device)
    _check(lib().ob200_bn_act_backward_f32(_ptr(dy), _ptr(x), _ptr(yout), _ptr(dx), _ptr(dres), _ptr(gamma), _ptr(beta),
                                           _ptr(save_mean), _ptr(save_invstd), _ptr(dgamma), _ptr(dbeta), x.numel() // C, C, int(act),
                                           num_ctas or sm_count(), _stream()), "ob200_bn_act_backward_f32")
    return dx, dres, dgamma, dbeta


def relu_backward(dy, y, num_ctas=None):
    dx = torch.empty_like(dy)
    _check(lib().ob200_relu_backward_f32(_ptr(dy), _ptr(y), _ptr(dx), dy.numel(), num_ctas or sm_count(), _stream()),
           "ob200_relu_backward_f32")
    return dx


def sgd_momentum_(p, g, m, lr, mu, wd=0.0, nesterov=False, first_step=False, num_ctas=None):
    _check(lib().ob200_sgd_momentum_f32(_ptr(p), _ptr(g), _ptr(m), p.numel(), lr, mu, wd, int(nesterov), int(first_step),
                                        num_ctas or sm_count(), _stream()), "ob200_sgd_momentum_f32")


def sgd_momentum_multi_(params, grads, bufs, lr, mu, wd=0.0, nesterov=False, first_step=False, num_ctas=None):
    """SGD with momentum over lists of tensors in ceil(len / 96) launches."""
    n = len(params)
    vp = ctypes.c_void_p * n
    cnt = (c_ll * n)(*[p.numel() for p in params])
    L = lib()
    L.ob200_sgd_momentum_multi_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_float, c_int, c_int,
                                               c_int, c_void_p]
    L.ob200_sgd_momentum_multi_f32.restype = c_int
    _check(L.ob200_sgd_momentum_multi_f32(vp(*[p.data_ptr() for p in params]), vp(*[g.data_ptr() for g in grads]),
                                          vp(*[m.data_ptr() for m in bufs]), cnt, n, lr, mu, wd, int(nesterov), int(first_step),
                                          num_ctas or sm_count(), _stream()), "ob200_sgd_momentum_multi_f32")


def maxpool_backward_nhwc(dy, x, k, stride, pad, num_ctas=None):
    Nb, H, W, C = x.shape
    dx = torch.empty_like(x)
    L = lib()
    L.ob200_maxpool_backward_nhwc_f32.argtypes = [c_void_p] * 3 + [c_int] * 7 + [c_int, c_void_p]
    L.ob200_maxpool_backward_nhwc_f32.restype = c_int
    _check(L.ob200_maxpool_backward_nhwc_f32(_ptr(dy), _ptr(x), _ptr(dx), Nb, H, W, C, k, stride, pad, num_ctas or sm_count(), _stream()),
           "ob200_maxpool_backward_nhwc_f32")
    return dx


def linear_batched(x, w, num_ctas=None, tf32=False):
    """x: [B, M, K], w: [B, N, K] -> [B, M, N] (y_b = x_b . w_b^T)."""
    assert x.is_contiguous() and w.is_contiguous() and x.dtype == w.dtype and x.shape[0] == w.shape[0]
    B, M, K = x.shape
    N = w.shape[1]
    y = torch.empty((B, M, N), device=x.device, dtype=x.dtype)
    code = 2 if (tf32 and x.dtype == torch.float32) else _dtype_code(x)
    _check(lib().ob200_linear_batched(_ptr(x), _ptr(w), _ptr(y), code, B, M, N, K, M * K, N * K, M * N, num_ctas or sm_count(),
                                      _stream()), "ob200_linear_batched")
    return y


def gemm_bf16(a, b, trans_a=False, trans_b=False, bias=None, alpha=1.0, out_dtype=None, num_ctas=None, tri=0):
    """C = alpha * op(A) . op(B)^T (+ bias) for bfloat16 matrices or stacks of matrices [..., rows, cols] (at most two
    leading batch dimensions, any strides that are multiples of 8 elements, innermost dimension contiguous).
    op(A) is [M, K]: `a` itself, or with trans_a `a` is stored [K, M].  op(B) is [N, K]: `b` itself, or with trans_b `b`
    is stored [K, N].  Returns a contiguous [..., M, N] tensor of `out_dtype` (bfloat16 or float32).  `tri`: the causal-attention
    modes of ob200_gemm_bf16_ex (1: output tiles above the diagonal are left unwritten; 2 / 3: A is lower / upper triangular)."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == b.dim() and 2 <= a.dim() <= 4
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and a.shape[:-2] == b.shape[:-2]
    K, M = (a.shape[-2], a.shape[-1]) if trans_a else (a.shape[-1], a.shape[-2])
    Kb, N = (b.shape[-2], b.shape[-1]) if trans_b else (b.shape[-1], b.shape[-2])
    assert K == Kb
    lead = list(a.shape[:-2])
    nbo, nbi = ([1, 1] + lead)[-2:]
    out_dtype = out_dtype or torch.bfloat16
    c = torch.empty(lead + [M, N], device=a.device, dtype=out_dtype)

    def strides(t):
        st = [0, 0] + list(t.stride()[:-2])
        return st[-1], st[-2]
    a_si, a_so = strides(a)
    b_si, b_so = strides(b)
    _check(lib().ob200_gemm_bf16_ex(_ptr(a), _ptr(b), _ptr(c), _ptr(bias) if bias is not None else None, None, None, M, N, K, int(trans_a),
                                    int(trans_b), a.stride(-2), b.stride(-2), N, nbi, nbo, a_si, a_so, b_si, b_so, M * N, nbi * M * N,
                                    float(alpha), int(out_dtype == torch.float32), int(tri), num_ctas or sm_count(), _stream()),
           "ob200_gemm_bf16_ex")
    return c


def colsum(x, num_ctas=None):
    """Column sums of a contiguous [rows, D] float32 / bfloat16 matrix, in x's type (the bias gradient of a linear layer)."""
    assert x.dim() == 2 and x.is_contiguous()
    out = torch.empty(x.shape[1], device=x.device, dtype=x.dtype)
    _check(lib().ob200_colsum(_ptr(x), _ptr(out), x.shape[0], x.shape[1], x.shape[1], _dtype_code(x), num_ctas or sm_count(), _stream()),
           "ob200_colsum")
    return out


def softmax_backward(prob, dprob, scale=1.0, num_ctas=None, causal_period=0):
    """scale * prob * (dprob - rowsum(prob * dprob)) over the last dimension; with `causal_period` = sequence length, row r is
    query position r % causal_period and the columns behind it are skipped (result 0)."""
    assert prob.is_contiguous() and dprob.is_contiguous() and prob.shape == dprob.shape and prob.dtype == dprob.dtype
    D = prob.shape[-1]
    ds = torch.empty_like(prob)
    _check(lib().ob200_softmax_backward(_ptr(prob), _ptr(dprob), _ptr(ds), prob.numel() // D, D, float(scale), int(causal_period),
                                        _dtype_code(prob), num_ctas or sm_count(), _stream()), "ob200_softmax_backward")
    return ds


def layernorm(x, gamma, beta, eps=1e-5, num_ctas=None):
    """LayerNorm over the last dimension; x float32 or bfloat16, gamma/beta float32."""
    assert x.is_contiguous()
    D = x.shape[-1]
    y = torch.empty_like(x)
    _check(lib().ob200_layernorm(_ptr(x), _ptr(y), _ptr(gamma), _ptr(beta), None, None, x.numel() // D, D, float(eps), _dtype_code(x),
                                 num_ctas or sm_count(), _stream()), "ob200_layernorm")
    return y


def softmax(x, scale=1.0, num_ctas=None, causal_period=0):
    """softmax(x * scale) over the last dimension; with `causal_period` = sequence length, row r is query position
    r % causal_period and later keys are masked out."""
    assert x.is_contiguous()
    D = x.shape[-1]
    y = torch.empty_like(x)
    _check(lib().ob200_softmax_causal(_ptr(x), _ptr(y), x.numel() // D, D, float(scale), int(causal_period), _dtype_code(x),
                                      num_ctas or sm_count(), _stream()), "ob200_softmax_causal")
    return y


def bias_gelu(x, bias=None, num_ctas=None):
    assert x.is_contiguous()
    D = x.shape[-1]
    y = torch.empty_like(x)
    _check(lib().ob200_bias_gelu(_ptr(x), _ptr(y), _ptr(bias), x.numel() // D, D, _dtype_code(x), num_ctas or sm_count(), _stream()),
           "ob200_bias_gelu")
    return y


def adamw_(p, g, m, v, step, lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, num_ctas=None):
    _check(lib().ob200_adamw_f32(_ptr(p), _ptr(g), _ptr(m), _ptr(v), p.numel(), lr, betas[0], betas[1], eps, weight_decay, step,
                                 num_ctas or sm_count(), _stream()), "ob200_adamw_f32")


def conv2d_wgrad_nhwc(x, dy, filter_rs, stride=(1, 1), padding=(0, 0), dilation=(1, 1), num_ctas=None, tf32=False):
    """x: [N, H, W, C], dy: [N, P, Q, K] (float32) -> dw [K, R, S, C]."""
    assert x.is_contiguous() and dy.is_contiguous() and x.dtype == torch.float32 and dy.dtype == torch.float32
    Nb, H, W, C = x.shape
    K = dy.shape[3]
    R, S = filter_rs
    dw = torch.empty((K, R, S, C), device=x.device, dtype=torch.float32)
    _check(lib().ob200_conv2d_wgrad(_ptr(x), _ptr(dy), _ptr(dw), 2 if tf32 else 0, Nb, H, W, C, K, R, S, stride[0], stride[1],
                                    padding[0], padding[1], dilation[0], dilation[1], num_ctas or sm_count(), _stream()),
           "ob200_conv2d_wgrad")
    return dw
