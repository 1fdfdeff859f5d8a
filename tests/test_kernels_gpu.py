"""Parity of the sm_100a kernels against the CPU oracle, through the C ABI.

Tolerances are the benchmark specification's: float32 relative 1e-4, bfloat16 relative 2e-2
(relative to the largest magnitude of the expected tensor)."""
import pytest
import torch

from oracle import numeric_oracle as O

pytestmark = pytest.mark.gpu
FP32_TOL, BF16_TOL = 1e-4, 2e-2


@pytest.fixture(scope="module")
def K(built):
    from orion_b200 import kernels
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; the kernels have no CPU fallback")
    torch.manual_seed(1234)
    return kernels


def _conv(K, Nb, H, W, C, Ko, R, stride, pad, dtype=torch.float32, dil=1, **kw):
    x = torch.randn(Nb, H, W, C, device="cuda", dtype=dtype)
    w = (torch.randn(Ko, R, R, C, device="cuda") / (C * R * R) ** 0.5).to(dtype)
    y = K.conv2d_nhwc(x, w, (stride, stride), (pad, pad), (dil, dil), **kw)
    assert K.read_status() == 0
    want = O.conv2d_nhwc(x, w, (stride, stride), (pad, pad), (dil, dil),
                         scale=kw.get("scale"), shift=kw.get("shift"), residual=kw.get("residual"),
                         act=2 if kw.get("relu") == 2 else int(bool(kw.get("relu"))))
    return O.rel_err(y, want)


RESNET_SHAPES = [
    (4, 224, 224, 3, 64, 7, 2, 3),      # stem: C=3 takes the scalar gather path
    (4, 56, 56, 64, 64, 1, 1, 0), (4, 56, 56, 64, 64, 3, 1, 1), (4, 56, 56, 64, 256, 1, 1, 0),
    (4, 56, 56, 256, 128, 1, 1, 0), (4, 56, 56, 128, 128, 3, 2, 1), (4, 56, 56, 256, 512, 1, 2, 0),
    (4, 28, 28, 512, 256, 1, 1, 0), (4, 28, 28, 256, 256, 3, 2, 1), (4, 14, 14, 256, 1024, 1, 1, 0),
    (4, 14, 14, 1024, 512, 1, 1, 0), (4, 14, 14, 512, 512, 3, 2, 1), (4, 7, 7, 512, 2048, 1, 1, 0),
    (4, 7, 7, 2048, 512, 1, 1, 0), (4, 7, 7, 512, 512, 3, 1, 1),
]


@pytest.mark.parametrize("shape", RESNET_SHAPES)
def test_conv_fp32_resnet50_shapes(K, shape):
    assert _conv(K, *shape) < FP32_TOL


@pytest.mark.parametrize("shape", [(2, 9, 11, 24, 40, 3, 1, 1), (1, 5, 5, 16, 8, 1, 1, 0), (3, 17, 13, 36, 100, 3, 2, 1),
                                   (2, 12, 12, 20, 72, 5, 1, 2), (1, 1, 1, 8, 8, 1, 1, 0), (2, 10, 10, 7, 19, 3, 1, 1)])
def test_conv_fp32_ragged_shapes(K, shape):
    """Row, column and channel tails; channel counts that are not a multiple of 4 (scalar loads and stores)."""
    assert _conv(K, *shape) < FP32_TOL


@pytest.mark.parametrize("dtype,c,cp", [(torch.float32, 3, 4), (torch.float32, 5, 8), (torch.bfloat16, 3, 8)])
def test_pad_channels_and_padded_stem_convolution(K, dtype, c, cp):
    """Zero channels change nothing: the padded stem equals the oracle's convolution of the unpadded one."""
    x = torch.randn(2, 30, 30, c, device="cuda", dtype=dtype)
    xp = K.pad_channels(x, cp)
    assert xp.shape == (2, 30, 30, cp)
    assert torch.equal(xp[..., :c], x) and torch.count_nonzero(xp[..., c:]) == 0
    w = (torch.randn(64, 7, 7, c, device="cuda") / (c * 49) ** 0.5).to(dtype)
    wp = K.pad_channels(w, cp)
    y = K.conv2d_nhwc(xp, wp, (2, 2), (3, 3))
    assert K.read_status() == 0
    want = O.conv2d_nhwc(x, w, (2, 2), (3, 3), (1, 1))
    assert O.rel_err(y, want) < (FP32_TOL if dtype == torch.float32 else BF16_TOL)


def test_tma_feeds_the_eligible_shapes(K):
    """Forward convolutions with whole k-blocks per tap and GEMMs take the TMA path; small channel counts gather."""
    n0 = K.tma_launch_count()
    assert _conv(K, 2, 14, 14, 64, 96, 3, 1, 1) < FP32_TOL          # 3x3, C multiple of 32
    assert _conv(K, 2, 15, 13, 96, 40, 3, 2, 1) < FP32_TOL          # strided, ragged image
    assert _conv(K, 3, 9, 9, 44, 24, 1, 2, 0) < FP32_TOL            # 1x1 strided, channel tail inside a k-block
    assert _conv(K, 2, 12, 12, 32, 32, 3, 1, 2, dil=2) < FP32_TOL   # dilated
    assert _conv(K, 2, 8, 8, 128, 64, 3, 1, 1, dtype=torch.bfloat16) < BF16_TOL
    assert K.tma_launch_count() - n0 == 5
    assert _conv(K, 2, 10, 10, 16, 32, 3, 1, 1) < FP32_TOL          # C below one k-block: gathered
    assert _conv(K, 2, 10, 10, 48, 32, 3, 1, 1) < FP32_TOL          # k-blocks straddle taps: gathered
    assert K.tma_launch_count() - n0 == 5


@pytest.mark.parametrize("shape", [(4, 112, 112, 32, 3, 1, 1), (4, 112, 112, 96, 3, 2, 1), (2, 14, 14, 576, 3, 1, 1),
                                   (2, 7, 7, 960, 3, 1, 1), (3, 9, 11, 24, 5, 2, 2), (1, 6, 6, 8, 3, 1, 0)])
@pytest.mark.parametrize("tap_major", [False, True])
def test_depthwise_convolution(K, shape, tap_major):
    """MobileNetV2's depthwise layers (groups = C): both filter layouts, fused scale/shift and ReLU6."""
    Nb, H, W, C, R, stride, pad = shape
    x = torch.randn(Nb, H, W, C, device="cuda")
    w = torch.randn(C, R, R, device="cuda") / R
    scale, shift = torch.rand(C, device="cuda") + 0.5, torch.randn(C, device="cuda")
    wk = w.permute(1, 2, 0).contiguous() if tap_major else w
    y = K.depthwise_conv2d_nhwc(x, wk, (stride, stride), (pad, pad), scale=scale, shift=shift, relu=2, tap_major=tap_major)
    want = O.conv2d_nhwc(x, w.unsqueeze(-1), (stride, stride), (pad, pad), scale=scale, shift=shift, act=2, groups=C)
    assert O.rel_err(y, want) < FP32_TOL


def test_wide_tiles_in_single_pass_modes(K):
    """128 x 256 tiles (bf16 and single-pass TF32 only): explicit, and picked by the planner for wide outputs."""
    x = torch.randn(8, 28, 28, 128, device="cuda")
    w = torch.randn(512, 3, 3, 128, device="cuda") / 34.0
    shift = torch.randn(512, device="cuda")
    want = O.conv2d_nhwc(x, w, (1, 1), (1, 1), shift=shift, act=1)
    assert O.rel_err(K.conv2d_nhwc(x, w, (1, 1), (1, 1), shift=shift, relu=True, tf32=True, bn=256, splits=1), want) < 5e-3
    assert O.rel_err(K.conv2d_nhwc(x, w, (1, 1), (1, 1), shift=shift, relu=True, tf32=True), want) < 5e-3
    xb, wb = x.bfloat16(), w.bfloat16()
    wantb = O.conv2d_nhwc(xb, wb, (1, 1), (1, 1), shift=shift, act=1)
    assert O.rel_err(K.conv2d_nhwc(xb, wb, (1, 1), (1, 1), shift=shift, relu=True, bn=256, splits=1), wantb) < BF16_TOL
    assert O.rel_err(K.conv2d_nhwc(xb, wb, (1, 1), (1, 1), shift=shift, relu=True), wantb) < BF16_TOL
    # ragged: 300 output channels (256 + 44) and an M tail
    w2 = torch.randn(300, 1, 1, 128, device="cuda").bfloat16()
    x2 = torch.randn(3, 13, 11, 128, device="cuda").bfloat16()
    assert O.rel_err(K.conv2d_nhwc(x2, w2, bn=256, splits=1), O.conv2d_nhwc(x2, w2, (1, 1), (0, 0))) < BF16_TOL
    a, b = torch.randn(4096, 1024, device="cuda").bfloat16(), torch.randn(2048, 1024, device="cuda").bfloat16()
    assert O.rel_err(K.linear(a, b), O.linear(a, b)) < BF16_TOL      # planner takes the wide tile here
    with pytest.raises(RuntimeError):
        K.conv2d_nhwc(x, w, (1, 1), (1, 1), bn=256, splits=1)          # 3xTF32 has no room for it in tensor memory
    assert K.read_status() == 0


def test_conv_dilation_and_empty_batch(K):
    assert _conv(K, 2, 16, 16, 32, 32, 3, 1, 2, dil=2) < FP32_TOL
    x = torch.empty(0, 8, 8, 16, device="cuda")
    w = torch.randn(8, 3, 3, 16, device="cuda")
    assert K.conv2d_nhwc(x, w, (1, 1), (1, 1)).shape == (0, 8, 8, 8)


def test_conv_fused_epilogue(K):
    Ko = 96
    scale, shift = torch.rand(Ko, device="cuda") + 0.5, torch.randn(Ko, device="cuda")
    res = torch.randn(2, 14, 14, Ko, device="cuda")
    for relu in (0, 1, 2):
        assert _conv(K, 2, 14, 14, 64, Ko, 3, 1, 1, scale=scale, shift=shift, residual=res, relu=relu) < FP32_TOL


@pytest.mark.parametrize("bn,splits", [(128, 1), (64, 1), (128, 4), (64, 3), (64, 16)])
def test_conv_tile_width_and_split_k(K, bn, splits):
    """Split-K through caller-provided scratch (one partial tile per split, summed in split order)."""
    x = torch.randn(4, 7, 7, 512, device="cuda")
    w = torch.randn(512, 3, 3, 512, device="cuda") / 68.0
    shift = torch.randn(512, device="cuda")
    want = O.conv2d_nhwc(x, w, (1, 1), (1, 1), shift=shift, act=1)
    y = K.conv2d_nhwc(x, w, (1, 1), (1, 1), shift=shift, relu=True, bn=bn, splits=splits)
    assert K.read_status() == 0
    assert O.rel_err(y, want) < FP32_TOL


@pytest.mark.parametrize("shape", [(4, 7, 7, 512, 512, 3, 1, 1), (4, 14, 14, 256, 256, 3, 1, 1), (4, 7, 7, 2048, 512, 1, 1, 0),
                                   (4, 14, 14, 1024, 256, 1, 1, 0), (4, 56, 56, 64, 64, 3, 1, 1)])
def test_planned_schedule_is_bit_reproducible_for_every_sm_quota(K, shape):
    """Inference batch (4): the entry point picks tile width and split-K factor from the problem and the device alone;
    the SM quota only sets how many CTAs walk the planned units, and partial tiles are added in split order.  So the
    output is the same bit for bit for any quota, and from launch to launch."""
    Nb, H, W, C, Ko, R, stride, pad = shape
    x = torch.randn(Nb, H, W, C, device="cuda")
    w = torch.randn(Ko, R, R, C, device="cuda") / (C * R * R) ** 0.5
    shift = torch.randn(Ko, device="cuda")
    ref = K.conv2d_nhwc(x, w, (stride, stride), (pad, pad), shift=shift, relu=True, num_ctas=148)
    assert O.rel_err(ref, O.conv2d_nhwc(x, w, (stride, stride), (pad, pad), shift=shift, act=1)) < FP32_TOL
    for q in (148, 1, 5, 37, 64, 100, 147):
        y = K.conv2d_nhwc(x, w, (stride, stride), (pad, pad), shift=shift, relu=True, num_ctas=q)
        assert torch.equal(y, ref), q
    assert K.read_status() == 0


def test_split_k_sums_in_split_order_whatever_unit_finishes_first(K):
    """Explicit split-K factor, repeated launches and different quotas (which change which CTA computes which split and
    in what order they finish): identical bits."""
    x = torch.randn(4, 7, 7, 512, device="cuda")
    w = torch.randn(512, 3, 3, 512, device="cuda") / 68.0
    ref = K.conv2d_nhwc(x, w, (1, 1), (1, 1), bn=64, splits=8, num_ctas=148)
    for q in (148, 148, 3, 29, 128):
        assert torch.equal(K.conv2d_nhwc(x, w, (1, 1), (1, 1), bn=64, splits=8, num_ctas=q), ref), q
    assert K.read_status() == 0


def test_long_reductions_keep_their_magnitude(K):
    """A 3x3 512->512 layer on positive data (the worst case for an accumulator that truncates): with the cross terms of
    the 3xTF32 product in an accumulator of their own the result stays within 1e-5 of float64 (it was 6e-5 low)."""
    x = torch.rand(4, 7, 7, 512, device="cuda") + 0.5
    w = (torch.rand(512, 3, 3, 512, device="cuda") + 0.5) / 4608.0
    y = K.conv2d_nhwc(x, w, (1, 1), (1, 1))
    want = O.conv2d_nhwc(x, w, (1, 1), (1, 1))
    assert K.read_status() == 0
    assert O.rel_err(y, want) < 1e-5
    mean_ratio = (y.double().cpu() / want.double().cpu()).mean().item()
    assert abs(mean_ratio - 1.0) < 1e-5


def test_conv_result_does_not_depend_on_the_sm_quota(K):
    """A persistent grid of any size walks the same tiles: without split-K the output is bit-identical."""
    x = torch.randn(4, 28, 28, 128, device="cuda")
    w = torch.randn(128, 3, 3, 128, device="cuda") / 34.0
    ref = K.conv2d_nhwc(x, w, (1, 1), (1, 1), bn=128, splits=1, num_ctas=148)
    for q in (1, 8, 37, 64):
        assert torch.equal(K.conv2d_nhwc(x, w, (1, 1), (1, 1), bn=128, splits=1, num_ctas=q), ref)
    assert K.read_status() == 0


@pytest.mark.parametrize("shape", [(4, 28, 28, 128, 128, 3, 1, 1), (4, 7, 7, 512, 512, 3, 1, 1), (8, 14, 14, 256, 1024, 1, 1, 0),
                                   (2, 9, 11, 24, 40, 3, 1, 1), (4, 56, 56, 64, 64, 1, 1, 0)])
def test_stream_k_schedule_for_any_sm_quota(K, shape):
    """The default schedule cuts the k-blocks of all tiles into one equal range per CTA; tiles that straddle two
    CTAs are summed in scratch.  Any quota gives the oracle's result, launch after launch (scratch is left zero)."""
    Nb, H, W, C, Ko, R, stride, pad = shape
    x = torch.randn(Nb, H, W, C, device="cuda")
    w = torch.randn(Ko, R, R, C, device="cuda") / (C * R * R) ** 0.5
    shift = torch.randn(Ko, device="cuda")
    want = O.conv2d_nhwc(x, w, (stride, stride), (pad, pad), shift=shift, act=1)
    for q in (148, 1, 8, 37, 64, 100, 148):
        y = K.conv2d_nhwc(x, w, (stride, stride), (pad, pad), shift=shift, relu=True, num_ctas=q)
        assert O.rel_err(y, want) < FP32_TOL, q
    assert K.read_status() == 0


def test_conv_is_linear_at_training_batch_size(K):
    """Size-independent property at the BE batch size (32): conv(a*x1 + x2) = a*conv(x1) + conv(x2)."""
    x1 = torch.randn(32, 56, 56, 64, device="cuda")
    x2 = torch.randn(32, 56, 56, 64, device="cuda")
    w = torch.randn(64, 3, 3, 64, device="cuda") / 24.0
    f = lambda x: K.conv2d_nhwc(x, w, (1, 1), (1, 1))
    lhs = f(2.5 * x1 + x2)
    rhs = 2.5 * f(x1) + f(x2)
    assert ((lhs - rhs).abs().max() / rhs.abs().max()).item() < 2e-5
    assert K.read_status() == 0


@pytest.mark.parametrize("shape", [(2, 14, 14, 64, 64, 3, 1, 1), (4, 28, 28, 128, 256, 1, 1, 0), (1, 9, 9, 24, 40, 3, 2, 1)])
def test_conv_bf16(K, shape):
    assert _conv(K, *shape, dtype=torch.bfloat16) < BF16_TOL


@pytest.mark.parametrize("M,N,Kd", [(4, 1000, 2048), (128, 128, 32), (300, 200, 136), (3072, 768, 768), (1, 10, 5)])
def test_linear_fp32(K, M, N, Kd):
    x, w, b = torch.randn(M, Kd, device="cuda"), torch.randn(N, Kd, device="cuda") / Kd ** 0.5, torch.randn(N, device="cuda")
    y = K.linear(x, w, bias=b)
    assert K.read_status() == 0
    assert O.rel_err(y, O.linear(x, w, b)) < FP32_TOL


@pytest.mark.parametrize("M,N,Kd", [(3072, 3072, 768), (257, 130, 72)])
def test_linear_bf16(K, M, N, Kd):
    x = torch.randn(M, Kd, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, Kd, device="cuda") / Kd ** 0.5).to(torch.bfloat16)
    y = K.linear(x, w, relu=True)
    assert K.read_status() == 0
    assert O.rel_err(y, O.linear(x, w, relu=True)) < BF16_TOL


@pytest.mark.parametrize("shape", [(4, 56, 56, 64), (2, 7, 7, 2048), (3, 5, 5, 6), (1, 1, 1, 4)])
def test_bn_inference(K, shape):
    C = shape[-1]
    x = torch.randn(*shape, device="cuda")
    g, b, m = torch.rand(C, device="cuda") + 0.5, torch.randn(C, device="cuda"), torch.randn(C, device="cuda")
    v = torch.rand(C, device="cuda") + 0.1
    for relu in (False, True):
        y = K.bn_inference(x, g, b, m, v, 1e-5, relu=relu)
        assert O.rel_err(y, O.bn_inference(x, g, b, m, v, 1e-5, relu)) < 1e-5


def test_elementwise_and_pooling(K):
    a, b = torch.randn(4, 56, 56, 256, device="cuda"), torch.randn(4, 56, 56, 256, device="cuda")
    assert torch.equal(K.binary(a, mode=0), torch.relu(a))
    assert torch.equal(K.binary(a, b, mode=1), a + b)
    assert torch.equal(K.binary(a, b, mode=2), torch.relu(a + b))
    odd = torch.randn(1031, device="cuda")
    assert torch.equal(K.binary(odd, odd, mode=2), torch.relu(odd + odd))          # tail that is not a multiple of 4
    x = torch.randn(4, 112, 112, 64, device="cuda")
    assert torch.equal(K.maxpool_nhwc(x, 3, 2, 1).double().cpu(), O.maxpool_nhwc(x, 3, 2, 1))
    for shp, (k, st, pd) in (((2, 15, 13, 8), (3, 2, 1)), ((3, 9, 10, 12), (3, 2, 0)), ((2, 11, 11, 16), (2, 2, 0)), ((1, 8, 8, 4), (3, 1, 1))):
        xr = torch.randn(*shp, device="cuda")      # ragged widths (output tails of the four-pixel groups) and the generic kernel
        assert torch.equal(K.maxpool_nhwc(xr, k, st, pd).double().cpu(), O.maxpool_nhwc(xr, k, st, pd))
    z = torch.randn(4, 7, 7, 2048, device="cuda")
    assert O.rel_err(K.avgpool_nhwc(z), O.avgpool_nhwc(z)) < 1e-6


@pytest.mark.parametrize("shape", [(4, 28, 28, 128, 128, 3, 1, 1), (4, 56, 56, 64, 256, 1, 1, 0)])
def test_conv_single_pass_tf32_mode(K, shape):
    """dtype 2: float32 data, products in one TF32 pass (10-bit mantissa).  Expected error ~1e-3, far
    above the fp32 tolerance — which is why it is opt-in — and far below a wrong result."""
    Nb, H, W, C, Ko, R, stride, pad = shape
    x = torch.randn(Nb, H, W, C, device="cuda")
    w = torch.randn(Ko, R, R, C, device="cuda") / (C * R * R) ** 0.5
    y = K.conv2d_nhwc(x, w, (stride, stride), (pad, pad), tf32=True)
    assert K.read_status() == 0
    err = O.rel_err(y, O.conv2d_nhwc(x, w, (stride, stride), (pad, pad)))
    assert 1e-5 < err < 5e-3
