"""ob200_gemm_bf16 through the C ABI against float64 products of the same bfloat16 inputs: all four operand orders,
ragged sizes, strided and batched operands (the attention layouts), split-K, float32 output, bias and alpha."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, trans_a, trans_b, bias, alpha):
    A = a.double().transpose(-1, -2) if trans_a else a.double()
    B = b.double() if trans_b else b.double().transpose(-1, -2)
    c = alpha * (A @ B)
    return c + bias.double() if bias is not None else c


def _check(c, ref, K):
    # bfloat16 inputs are exact in the float64 product; what is left is float32 accumulation and the output rounding
    scale = ref.abs().max().item() + 1e-30
    tol = 2e-2 if c.dtype == torch.bfloat16 else 1e-5
    err = (c.double() - ref).abs().max().item() / scale
    assert err < tol, (err, tuple(c.shape), K)


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 384, 256), (200, 136, 72), (3072, 768, 768), (64, 64, 1024), (1, 8, 8),
                                   (130, 520, 1000)])
def test_operand_orders_and_ragged_sizes(built, trans_a, trans_b, M, N, K):
    from orion_b200 import kernels as K_
    torch.manual_seed(M * 7 + N * 3 + K)
    # leading dimensions must be multiples of 8 elements: allocate padded and slice
    def mat(rows, cols):
        ld = (cols + 7) // 8 * 8
        return torch.randn(rows, ld, device="cuda").to(torch.bfloat16)[:, :cols]
    a = mat(K, M) if trans_a else mat(M, K)
    b = mat(K, N) if trans_b else mat(N, K)
    for out_dtype in (torch.bfloat16, torch.float32):
        c = K_.gemm_bf16(a, b, trans_a, trans_b, out_dtype=out_dtype)
        _check(c, _ref(a, b, trans_a, trans_b, None, 1.0), K)
    assert K_.read_status() == 0


def test_bias_and_alpha(built):
    from orion_b200 import kernels as K_
    torch.manual_seed(3)
    a = torch.randn(300, 256, device="cuda").to(torch.bfloat16)
    b = torch.randn(200, 256, device="cuda").to(torch.bfloat16)
    bias = torch.randn(200, device="cuda")
    c = K_.gemm_bf16(a, b, bias=bias, alpha=0.125, out_dtype=torch.float32)
    _check(c, _ref(a, b, False, False, bias, 0.125), 256)


@pytest.mark.parametrize("M,N,K", [(768, 768, 3072), (2304, 768, 3072), (1024, 1024, 8192), (768, 136, 2000)])
def test_weight_gradient_shapes_take_split_k_and_do_not_depend_on_the_cta_count(built, M, N, K):
    """dW = dY^T . X: both operands [tokens, features]; few output tiles and a long reduction."""
    from orion_b200 import kernels as K_
    torch.manual_seed(K)
    dy = torch.randn(K, M, device="cuda").to(torch.bfloat16)
    x = torch.randn(K, (N + 7) // 8 * 8, device="cuda").to(torch.bfloat16)[:, :N]
    ref = _ref(dy, x, True, True, None, 1.0)
    outs = [K_.gemm_bf16(dy, x, True, True, out_dtype=torch.float32, num_ctas=n) for n in (148, 64, 7)]
    _check(outs[0], ref, K)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    _check(K_.gemm_bf16(dy, x, True, True), ref, K)
    assert K_.read_status() == 0


@pytest.mark.parametrize("B,S,H", [(2, 384, 12), (1, 512, 16), (2, 200, 4)])
def test_attention_products_on_the_fused_projection_layout(built, B, S, H):
    """Q, K, V as strided views of qkv [B, S, 3, H, 64]; P as [B, H, S, S]: the five products of attention and its
    gradient, none with a re-laid-out copy of an operand."""
    from orion_b200 import kernels as K_
    torch.manual_seed(S)
    d = 64
    qkv = (torch.randn(B, S, 3, H, d, device="cuda") * 0.5).to(torch.bfloat16)
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))       # [B, H, S, d] views, row stride 3*H*d
    s = K_.gemm_bf16(q, k, alpha=0.125)                                    # scores = Q . K^T
    _check(s, _ref(q, k, False, False, None, 0.125), d)
    p = torch.softmax(s.float(), -1).to(torch.bfloat16)
    o = K_.gemm_bf16(p, v, trans_b=True)                                   # P . V: V is [keys, d]
    _check(o, _ref(p, v, False, True, None, 1.0), S)
    do = torch.randn(B, H, S, d, device="cuda").to(torch.bfloat16)
    dv = K_.gemm_bf16(p, do, trans_a=True, trans_b=True)                   # dV = P^T . dO
    _check(dv, _ref(p, do, True, True, None, 1.0), S)
    dp = K_.gemm_bf16(do, v)                                               # dP = dO . V^T
    _check(dp, _ref(do, v, False, False, None, 1.0), d)
    ds = (torch.randn(B, H, S, S, device="cuda") * 0.1).to(torch.bfloat16)
    dq = K_.gemm_bf16(ds, k, trans_b=True)                                 # dQ = dS . K
    _check(dq, _ref(ds, k, False, True, None, 1.0), S)
    dk = K_.gemm_bf16(ds, q, trans_a=True, trans_b=True)                   # dK = dS^T . Q
    _check(dk, _ref(ds, q, True, True, None, 1.0), S)
    assert K_.read_status() == 0


@pytest.mark.parametrize("S", [512, 384, 200])
def test_causal_modes_skip_only_what_is_zero_or_unused(built, S):
    """tri = 1 leaves tiles strictly above the diagonal unwritten and computes the rest; tri = 2 / 3 give the full product when
    A is lower / upper triangular (the probabilities of causal attention and their transpose)."""
    from orion_b200 import kernels as K_
    torch.manual_seed(S)
    B, H, d = 2, 3, 64
    q = torch.randn(B, H, S, d, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, H, S, d, device="cuda").to(torch.bfloat16)
    s = K_.gemm_bf16(q, k, tri=1)
    ref = _ref(q, k, False, False, None, 1.0)
    mask = torch.tril(torch.ones(S, S, dtype=torch.bool, device="cuda"))
    err = torch.where(mask, (s.double() - ref).abs(), torch.zeros_like(ref)).max().item() / ref.abs().max().item()
    assert err < 2e-2
    p = (torch.softmax(torch.randn(B, H, S, S, device="cuda"), -1) * mask).to(torch.bfloat16)     # lower triangular
    v = torch.randn(B, H, S, d, device="cuda").to(torch.bfloat16)
    _check(K_.gemm_bf16(p, v, trans_b=True, tri=2), _ref(p, v, False, True, None, 1.0), S)                   # P . V
    _check(K_.gemm_bf16(p, v, trans_a=True, trans_b=True, tri=3), _ref(p, v, True, True, None, 1.0), S)      # P^T . dO
    assert K_.read_status() == 0
