"""Parity of the training-side kernels (data-gradient convolution, batch-norm training forward
and backward, ReLU backward, SGD update) against float64 CPU references, through the C ABI.
Tolerance: float32 relative 1e-4 of the largest expected magnitude (benchmark specification)."""
import pytest
import torch
import torch.nn.functional as F

from oracle import numeric_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-4


@pytest.fixture(scope="module")
def K(built):
    from orion_b200 import kernels
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; the kernels have no CPU fallback")
    torch.manual_seed(4321)
    return kernels


def _dgrad_ref(dy, w, hw, stride, pad, dil):
    """cudnnConvolutionBackwardData by definition: the gradient of conv2d with respect to its input."""
    dyd = dy.detach().double().cpu().permute(0, 3, 1, 2)
    wd = w.detach().double().cpu().permute(0, 3, 1, 2)
    n, c = dy.shape[0], w.shape[3]
    dx = torch.nn.grad.conv2d_input((n, c, hw[0], hw[1]), wd, dyd, stride=stride, padding=pad, dilation=dil)
    return dx.permute(0, 2, 3, 1).contiguous()


@pytest.mark.parametrize("shape", [
    (4, 56, 56, 64, 64, 3, 1, 1), (4, 56, 56, 64, 256, 1, 1, 0), (4, 56, 56, 128, 128, 3, 2, 1), (4, 56, 56, 256, 512, 1, 2, 0),
    (4, 14, 14, 256, 256, 3, 1, 1), (4, 7, 7, 512, 512, 3, 1, 1), (2, 11, 9, 24, 40, 3, 2, 1), (2, 12, 12, 16, 20, 5, 1, 2),
    (1, 224, 224, 3, 64, 7, 2, 3), (2, 16, 16, 32, 32, 3, 1, 2),
    # strided gradients split by parity class: odd image sizes, stride 3, 5x5 taps, 2x2 filter with stride 2, 1x1 with pad
    (2, 15, 13, 32, 64, 3, 2, 1), (2, 14, 14, 32, 32, 3, 3, 1), (2, 12, 12, 16, 64, 5, 2, 2), (2, 8, 8, 48, 32, 2, 2, 0),
    (2, 9, 9, 40, 96, 1, 2, 1), (3, 7, 7, 64, 32, 3, 2, 0),
])
def test_conv_dgrad_fp32(K, shape):
    Nb, H, W, C, Ko, R, stride, pad = shape
    dil = 2 if shape == (2, 16, 16, 32, 32, 3, 1, 2) else 1
    P = (H + 2 * pad - dil * (R - 1) - 1) // stride + 1
    Q = (W + 2 * pad - dil * (R - 1) - 1) // stride + 1
    dy = torch.randn(Nb, P, Q, Ko, device="cuda")
    w = torch.randn(Ko, R, R, C, device="cuda") / (Ko * R * R) ** 0.5
    dx = K.conv2d_dgrad_nhwc(dy, w, (H, W), (stride, stride), (pad, pad), (dil, dil))
    assert K.read_status() == 0
    assert O.rel_err(dx, _dgrad_ref(dy, w, (H, W), stride, pad, dil)) < TOL


def test_strided_dgrad_runs_one_tma_launch_per_parity_class(K):
    dy = torch.randn(2, 14, 14, 64, device="cuda")
    w = torch.randn(64, 3, 3, 32, device="cuda") / 24.0
    n0 = K.tma_launch_count()
    dx = K.conv2d_dgrad_nhwc(dy, w, (28, 28), (2, 2), (1, 1))
    assert K.tma_launch_count() - n0 == 4
    assert O.rel_err(dx, _dgrad_ref(dy, w, (28, 28), 2, 1, 1)) < TOL
    dyb, wb = dy.bfloat16(), w.bfloat16()
    dxb = K.conv2d_dgrad_nhwc(dyb, wb, (28, 28), (2, 2), (1, 1))
    assert O.rel_err(dxb, _dgrad_ref(dyb, wb, (28, 28), 2, 1, 1)) < 2e-2
    assert K.read_status() == 0


def test_conv_dgrad_bf16_and_filter_transpose(K):
    w = torch.randn(40, 3, 3, 24, device="cuda")
    assert torch.equal(K.filter_transpose(w), w.permute(3, 1, 2, 0).contiguous())
    dy = torch.randn(2, 14, 14, 64, device="cuda", dtype=torch.bfloat16)
    wb = (torch.randn(64, 3, 3, 64, device="cuda") / 24.0).to(torch.bfloat16)
    dx = K.conv2d_dgrad_nhwc(dy, wb, (14, 14), (1, 1), (1, 1))
    assert O.rel_err(dx, _dgrad_ref(dy, wb, (14, 14), 1, 1, 1)) < 2e-2


@pytest.mark.parametrize("shape", [(32, 56, 56, 64), (4, 7, 7, 2048), (3, 5, 5, 24), (2, 3, 2, 8)])
def test_bn_training_forward_and_backward(K, shape):
    C = shape[-1]
    x = (torch.randn(*shape, device="cuda") * 2.0 + 0.7)
    g, b = torch.rand(C, device="cuda") + 0.5, torch.randn(C, device="cuda")
    rm, rv = torch.randn(C, device="cuda"), torch.rand(C, device="cuda") + 0.5
    rm_ref, rv_ref = rm.double().cpu().clone(), rv.double().cpu().clone()
    xd = x.double().cpu().reshape(-1, C).requires_grad_(True)
    want = F.batch_norm(xd, rm_ref, rv_ref, g.double().cpu(), b.double().cpu(), True, 0.1, 1e-5)
    y, mean, invstd = K.bn_train_forward(x, g, b, rm, rv, 1e-5, 0.1)
    assert O.rel_err(y.reshape(-1, C), want.detach()) < 1e-5
    assert O.rel_err(mean, xd.detach().mean(0)) < 1e-5
    assert O.rel_err(invstd, 1.0 / torch.sqrt(xd.detach().var(0, unbiased=False) + 1e-5)) < 1e-5
    assert O.rel_err(rm, rm_ref) < 1e-5 and O.rel_err(rv, rv_ref) < 1e-5          # running statistics updated in place
    dy = torch.randn(*shape, device="cuda")
    gd, bd = g.double().cpu().requires_grad_(True), b.double().cpu().requires_grad_(True)
    out = F.batch_norm(xd, None, None, gd, bd, True, 0.1, 1e-5)
    out.backward(dy.double().cpu().reshape(-1, C))
    dx, dgamma, dbeta = K.bn_backward(dy, x, g, mean, invstd)
    assert O.rel_err(dx.reshape(-1, C), xd.grad) < 1e-4
    assert O.rel_err(dgamma, gd.grad) < 1e-4 and O.rel_err(dbeta, bd.grad) < 1e-4


@pytest.mark.parametrize("shape", [(32, 14, 14, 256), (8, 7, 7, 2048), (4, 9, 11, 24), (64, 28, 28, 32)])
@pytest.mark.parametrize("act,with_res", [(0, False), (1, False), (2, False), (1, True), (0, True)])
def test_bn_fused_with_residual_and_activation(K, shape, act, with_res):
    """y = act(batch_norm_train(x) + residual) in two launches forward and two backward, twice in a row (the second call
    finds the scratch the first one's finishing CTAs cleaned), against float64 autograd on the CPU."""
    C = shape[-1]
    for attempt in range(2):
        x = (torch.randn(*shape, device="cuda") * 2.0 + 0.7)
        res = torch.randn(*shape, device="cuda") if with_res else None
        g, b = torch.rand(C, device="cuda") + 0.5, torch.randn(C, device="cuda") * 0.5
        rm, rv = torch.randn(C, device="cuda"), torch.rand(C, device="cuda") + 0.5
        rm_ref, rv_ref = rm.double().cpu().clone(), rv.double().cpu().clone()
        xd = x.double().cpu().reshape(-1, C).requires_grad_(True)
        rd = res.double().cpu().reshape(-1, C).requires_grad_(True) if with_res else None
        gd, bd = g.double().cpu().requires_grad_(True), b.double().cpu().requires_grad_(True)
        pre = F.batch_norm(xd, rm_ref, rv_ref, gd, bd, True, 0.1, 1e-5)
        if with_res:
            pre = pre + rd
        want = F.relu(pre) if act == 1 else F.relu6(pre) if act == 2 else pre
        y, mean, invstd = K.bn_act_train_forward(x, g, b, rm, rv, 1e-5, 0.1, act=act, residual=res)
        assert O.rel_err(y.reshape(-1, C), want.detach()) < 1e-5
        assert O.rel_err(rm, rm_ref) < 1e-5 and O.rel_err(rv, rv_ref) < 1e-5
        dy = torch.randn(*shape, device="cuda")
        # The gradient reference uses the activation pattern of the float32 forward pass: an input within rounding
        # distance of the activation's kink may fall on either side, and that is not what this test is about.
        yc = y.double().cpu().reshape(-1, C)
        mask = torch.ones_like(yc) if act == 0 else ((yc > 0) & (yc < 6)).double() if act == 2 else (yc > 0).double()
        (pre * mask).backward(dy.double().cpu().reshape(-1, C))
        dx, dres, dgamma, dbeta = K.bn_act_backward(dy, x, g, b, mean, invstd, act=act, yout=y if (with_res and act) else None,
                                                    want_dres=with_res)
        assert O.rel_err(dx.reshape(-1, C), xd.grad) < 1e-4
        assert O.rel_err(dgamma, gd.grad) < 1e-4 and O.rel_err(dbeta, bd.grad) < 1e-4
        if with_res:
            assert O.rel_err(dres.reshape(-1, C), rd.grad) < 1e-6


def test_relu_backward_and_sgd(K):
    y = torch.randn(4, 28, 28, 130, device="cuda")
    dy = torch.randn_like(y)
    assert torch.equal(K.relu_backward(dy, y), torch.where(y > 0, dy, torch.zeros_like(dy)))
    odd = torch.randn(1001, device="cuda")
    assert torch.equal(K.relu_backward(odd, odd), torch.where(odd > 0, odd, torch.zeros_like(odd)))
    p = torch.randn(100003, device="cuda")
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.SGD([ref_p], lr=0.1, momentum=0.9, weight_decay=1e-4)
    m = torch.zeros_like(p)
    for step in range(3):
        gstep = torch.randn_like(p)
        ref_p.grad = gstep.clone()
        opt.step()
        K.sgd_momentum_(p, gstep, m, 0.1, 0.9, 1e-4, first_step=(step == 0))
    assert (p - ref_p.detach()).abs().max().item() < 1e-5


def test_wgrad_takes_the_tma_path_when_channels_allow(K):
    """Pixel-major operands by TMA (MN-major tensor-core operands); fewer than 32 input channels gather and transpose."""
    x = torch.randn(2, 12, 12, 64, device="cuda")
    dy = torch.randn(2, 12, 12, 96, device="cuda") / 17.0
    n0 = K.tma_launch_count()
    dw = K.conv2d_wgrad_nhwc(x, dy, (3, 3), (1, 1), (1, 1))
    assert K.tma_launch_count() - n0 == 1
    assert O.rel_err(dw, _wgrad_ref(x, dy, (3, 3), 1, 1, 1)) < TOL
    dw = K.conv2d_wgrad_nhwc(x, dy, (3, 3), (1, 1), (1, 1), tf32=True)
    assert O.rel_err(dw, _wgrad_ref(x, dy, (3, 3), 1, 1, 1)) < 5e-3
    x16 = torch.randn(2, 12, 12, 16, device="cuda")
    n0 = K.tma_launch_count()
    dw = K.conv2d_wgrad_nhwc(x16, dy, (3, 3), (1, 1), (1, 1))
    assert K.tma_launch_count() == n0
    assert O.rel_err(dw, _wgrad_ref(x16, dy, (3, 3), 1, 1, 1)) < TOL
    assert K.read_status() == 0


def _wgrad_ref(x, dy, rs, stride, pad, dil):
    """cudnnConvolutionBackwardFilter by definition: the gradient of conv2d with respect to its weight."""
    xd = x.detach().double().cpu().permute(0, 3, 1, 2)
    dyd = dy.detach().double().cpu().permute(0, 3, 1, 2)
    k, c = dy.shape[3], x.shape[3]
    dw = torch.nn.grad.conv2d_weight(xd, (k, c, rs[0], rs[1]), dyd, stride=stride, padding=pad, dilation=dil)
    return dw.permute(0, 2, 3, 1).contiguous()


@pytest.mark.parametrize("shape", [
    (2, 8, 8, 32, 128, 1, 1, 0), (4, 56, 56, 64, 64, 3, 1, 1), (4, 56, 56, 64, 256, 1, 1, 0), (4, 28, 28, 128, 128, 3, 2, 1),
    (4, 14, 14, 256, 1024, 1, 1, 0), (4, 7, 7, 512, 512, 3, 1, 1), (2, 11, 9, 24, 40, 3, 2, 1), (3, 10, 10, 200, 136, 3, 1, 1),
    # few input channels: one tile covers several taps (4 taps of 32 channels, 2 taps of 48 -> 64, 5x5 = 25 taps, stride 2)
    (3, 12, 12, 32, 96, 3, 1, 1), (2, 13, 13, 48, 200, 5, 1, 2), (2, 16, 16, 64, 64, 3, 2, 1), (2, 9, 9, 36, 20, 2, 1, 0),
])
def test_conv_wgrad_fp32(K, shape):
    Nb, H, W, C, Ko, R, stride, pad = shape
    P = (H + 2 * pad - R) // stride + 1
    Q = (W + 2 * pad - R) // stride + 1
    x = torch.randn(Nb, H, W, C, device="cuda")
    dy = torch.randn(Nb, P, Q, Ko, device="cuda") / (Nb * P * Q) ** 0.5
    dw = K.conv2d_wgrad_nhwc(x, dy, (R, R), (stride, stride), (pad, pad))
    assert K.read_status() == 0
    assert O.rel_err(dw, _wgrad_ref(x, dy, (R, R), stride, pad, 1)) < TOL


@pytest.mark.parametrize("shape,k,stride,pad", [((32, 112, 112, 64), 3, 2, 1), ((2, 9, 11, 8), 3, 2, 1), ((3, 8, 8, 12), 2, 2, 0)])
def test_maxpool_backward_routes_like_torch_including_ties(K, shape, k, stride, pad):
    """Behind a ReLU whole windows are zero: the gradient must go to the first element of the window, as torch's does."""
    import torch.nn.functional as F
    from orion_b200 import torch_ops
    torch_ops.load()
    x = torch.relu(torch.randn(*shape, device="cuda")).permute(0, 3, 1, 2).contiguous(memory_format=torch.channels_last)
    x1 = x.clone().requires_grad_(True)
    x2 = x.clone().requires_grad_(True)
    y1 = torch.ops.orion.maxpool_train(x1, k, stride, pad)
    y2 = F.max_pool2d(x2, k, stride, pad)
    assert torch.equal(y1, y2)
    dy = torch.randn_like(y2)
    y1.backward(dy)
    y2.backward(dy)
    assert (x1.grad - x2.grad).abs().max().item() <= 1e-6 * x2.grad.abs().max().item()


def test_multi_tensor_sgd_matches_torch(K):
    from orion_b200.optim import SGD
    torch.manual_seed(3)
    shapes = [(64, 3, 7, 7), (64,), (1000, 2048), (1001,), (3, 5, 7), (512, 512, 3, 3)] + [(17,)] * 120
    ours = [torch.nn.Parameter(torch.randn(*s, device="cuda")) for s in shapes]
    ref = [torch.nn.Parameter(p.detach().clone()) for p in ours]
    o1 = SGD(ours, lr=0.1, momentum=0.9, weight_decay=1e-4)
    o2 = torch.optim.SGD(ref, lr=0.1, momentum=0.9, weight_decay=1e-4)
    for step in range(3):
        for a, b in zip(ours, ref):
            g = torch.randn_like(a)
            a.grad, b.grad = g.clone(), g.clone()
        o1.step()
        o2.step()
        for a, b in zip(ours, ref):
            assert (a - b).abs().max().item() <= 2e-6 * max(1.0, b.abs().max().item()), step


@pytest.mark.parametrize("shape,stride", [((64, 56, 56, 144), 1), ((64, 112, 112, 96), 2), ((3, 9, 11, 8), 2), ((2, 7, 7, 960), 1),
                                          ((5, 10, 6, 32), 1)])
def test_depthwise_backward_through_the_overrides(K, shape, stride):
    """MobileNetV2's depthwise 3x3 layers: data and filter gradient of the convolution override against float64 on the CPU,
    with no fallback to the stock kernels."""
    import torch.nn.functional as F
    from orion_b200 import torch_ops
    torch_ops.load()
    Nb, H, W, C = shape
    torch.manual_seed(12)
    x = torch.randn(Nb, C, H, W, device="cuda").contiguous(memory_format=torch.channels_last).requires_grad_(True)
    w = (torch.randn(C, 1, 3, 3, device="cuda") / 3.0).requires_grad_(True)
    fb0 = int(torch.ops.orion.fallbacks())
    y = F.conv2d(x, w, None, stride, 1, 1, C)
    dy = torch.randn_like(y)
    y.backward(dy)
    assert int(torch.ops.orion.fallbacks()) == fb0
    xd = x.detach().double().cpu().requires_grad_(True)
    wd = w.detach().double().cpu().requires_grad_(True)
    yd = F.conv2d(xd, wd, None, stride, 1, 1, C)
    yd.backward(dy.double().cpu())
    assert O.rel_err(y.detach(), yd.detach()) < 1e-5
    assert O.rel_err(x.grad, xd.grad) < 1e-5
    assert O.rel_err(w.grad, wd.grad) < 1e-4
