"""Transformer-side kernels (LayerNorm, softmax, bias+GELU, AdamW, batched GEMM) against float64 CPU
references.  Tolerances: float32 relative 1e-4, bfloat16 relative 2e-2 (benchmark specification)."""
import pytest
import torch
import torch.nn.functional as F

from oracle import numeric_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K(built):
    from orion_b200 import kernels
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; the kernels have no CPU fallback")
    torch.manual_seed(777)
    return kernels


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("rows,D", [(3072, 768), (8192, 1024), (5, 64), (1, 8)])
def test_layernorm(K, rows, D, dtype, tol):
    x = (torch.randn(rows, D, device="cuda") * 3 + 1).to(dtype)
    g, b = torch.rand(D, device="cuda") + 0.5, torch.randn(D, device="cuda")
    want = F.layer_norm(x.double().cpu(), (D,), g.double().cpu(), b.double().cpu(), 1e-5)
    assert O.rel_err(K.layernorm(x, g, b, 1e-5), want) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("rows,D", [(96 * 384, 384), (1000, 512), (3, 8)])
def test_softmax(K, rows, D, dtype, tol):
    x = (torch.randn(rows, D, device="cuda") * 4).to(dtype)
    want = F.softmax(x.double().cpu() * 0.125, dim=-1)
    got = K.softmax(x, 0.125)
    assert O.rel_err(got, want) < tol
    assert (got.float().sum(-1) - 1).abs().max().item() < (1e-4 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_bias_gelu(K, dtype, tol):
    x = torch.randn(3072, 3072, device="cuda").to(dtype)
    bias = torch.randn(3072, device="cuda")
    want = F.gelu(x.double().cpu() + bias.double().cpu())
    assert O.rel_err(K.bias_gelu(x, bias), want) < tol


def test_adamw_matches_torch(K):
    p = torch.randn(50001, device="cuda")
    ref = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref], lr=3e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    for step in range(1, 4):
        g = torch.randn_like(p)
        ref.grad = g.clone()
        opt.step()
        K.adamw_(p, g, m, v, step, 3e-4)
    assert (p - ref.detach()).abs().max().item() < 1e-6


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_batched_gemm_attention_shapes(K, dtype, tol):
    """Q.K^T of BERT-base at batch 8: 96 problems of 384 x 384 x 64, and P.V with V transposed: 384 x 64 x 384."""
    q = torch.randn(96, 384, 64, device="cuda").to(dtype)
    k = torch.randn(96, 384, 64, device="cuda").to(dtype)
    scores = K.linear_batched(q, k)
    assert K.read_status() == 0
    assert O.rel_err(scores, torch.bmm(q.double().cpu(), k.double().cpu().transpose(1, 2))) < tol
    pr = torch.softmax(torch.randn(96, 384, 384, device="cuda"), -1).to(dtype)
    vt = torch.randn(96, 64, 384, device="cuda").to(dtype)
    ctx = K.linear_batched(pr, vt)
    assert O.rel_err(ctx, torch.bmm(pr.double().cpu(), vt.double().cpu().transpose(1, 2))) < tol
    odd = K.linear_batched(torch.randn(3, 130, 72, device="cuda"), torch.randn(3, 50, 72, device="cuda"))
    assert odd.shape == (3, 130, 50) and K.read_status() == 0


# ---------------------------------------------------------------------------------------------- training side
@pytest.fixture(scope="module")
def tops(built):
    from orion_b200 import torch_ops
    torch_ops.load()
    return torch.ops.orion


@pytest.mark.parametrize("rows,D,dtype", [(3072, 768, torch.bfloat16), (8192, 1024, torch.bfloat16), (37, 256, torch.float32),
                                          (1000, 512, torch.float32), (5, 8, torch.bfloat16)])
def test_layernorm_training_forward_and_backward(tops, rows, D, dtype):
    """y = LayerNorm(x) and its three gradients through the autograd op, against float64 on the CPU (bfloat16: inputs and
    parameters rounded to bfloat16 first, tolerance 2e-2 of the tensor's largest entry; float32: 1e-4)."""
    torch.manual_seed(5)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    x = (torch.randn(rows, D, device="cuda") * 1.5 + 0.3).to(dtype).requires_grad_(True)
    g = (torch.rand(D, device="cuda") + 0.5).to(dtype).requires_grad_(True)
    b = torch.randn(D, device="cuda").to(dtype).requires_grad_(True)
    dy = torch.randn(rows, D, device="cuda").to(dtype)
    y = tops.layernorm_train(x, g, b, 1e-5)
    y.backward(dy)
    xd, gd, bd = (t.detach().double().cpu().requires_grad_(True) for t in (x, g, b))
    want = F.layer_norm(xd, (D,), gd, bd, 1e-5)
    want.backward(dy.double().cpu())
    assert O.rel_err(y.detach(), want.detach()) < tol
    assert O.rel_err(x.grad, xd.grad) < tol
    assert O.rel_err(g.grad, gd.grad) < tol and O.rel_err(b.grad, bd.grad) < tol


@pytest.mark.parametrize("rows,D,dtype", [(3072, 3072, torch.bfloat16), (8192, 4096, torch.bfloat16), (33, 64, torch.float32),
                                          (700, 96, torch.bfloat16)])
def test_bias_gelu_training_forward_and_backward(tops, rows, D, dtype):
    torch.manual_seed(6)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    x = torch.randn(rows, D, device="cuda").to(dtype).requires_grad_(True)
    b = (torch.randn(D, device="cuda") * 0.5).to(dtype).requires_grad_(True)
    dy = torch.randn(rows, D, device="cuda").to(dtype)
    y = tops.bias_gelu_train(x, b)
    y.backward(dy)
    xd, bd = (t.detach().double().cpu().requires_grad_(True) for t in (x, b))
    want = F.gelu(xd + bd)
    want.backward(dy.double().cpu())
    assert O.rel_err(y.detach(), want.detach()) < tol
    assert O.rel_err(x.grad, xd.grad) < tol
    assert O.rel_err(b.grad, bd.grad) < tol


@pytest.mark.parametrize("rows,V,dtype", [(1024, 32000, torch.bfloat16), (64, 1000, torch.float32), (7, 8, torch.bfloat16)])
def test_cross_entropy_forward_and_backward_from_the_logits_own_type(tops, rows, V, dtype):
    """Mean cross-entropy over a vocabulary-sized row and its gradient (written in the logits' type) against float64."""
    torch.manual_seed(7)
    logits = (torch.randn(rows, V, device="cuda") * 2.0).to(dtype).requires_grad_(True)
    target = torch.randint(0, V, (rows,), device="cuda")
    loss = tops.cross_entropy(logits, target)
    (loss * 3.0).backward()
    ld = logits.detach().double().cpu().requires_grad_(True)
    want = F.cross_entropy(ld, target.cpu())
    (want * 3.0).backward()
    assert abs(loss.item() - want.item()) / want.item() < 1e-5
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert O.rel_err(logits.grad, ld.grad) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_multi_tensor_adamw_matches_torch(tops, dtype):
    from orion_b200.optim import AdamW
    torch.manual_seed(8)
    shapes = [(768, 768), (768,), (3072, 768), (30528, 64), (2,), (5, 7)] + [(33,)] * 150
    ours = [torch.nn.Parameter(torch.randn(*s, device="cuda").to(dtype)) for s in shapes]
    ref = [torch.nn.Parameter(p.detach().clone().float()) for p in ours]     # float32 reference of the same arithmetic
    o1 = AdamW(ours, lr=1e-2, weight_decay=0.01)
    o2 = torch.optim.AdamW(ref, lr=1e-2, weight_decay=0.01)
    for step in range(3):
        for a, b in zip(ours, ref):
            g = torch.randn_like(b).to(dtype)
            a.grad, b.grad = g.clone(), g.float()
        o1.step()
        o2.step()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    for a, b in zip(ours, ref):
        assert (a.float() - b).abs().max().item() <= tol * max(1.0, b.abs().max().item())


@pytest.mark.parametrize("B,S,H,causal", [(8, 384, 12, False), (2, 384, 12, True), (3, 200, 4, False), (1, 128, 2, True), (2, 37, 3, False),
                                          (1, 300, 1, True)])
def test_fused_attention_matches_float64(tops, B, S, H, causal):
    """softmax(Q K^T / 8 [+ causal mask]) V from the fused projection output [B, S, 3, H, 64], against float64 on the CPU
    (bfloat16 inputs, tolerance 2e-2 of the largest output); ragged sequence lengths use zero-filled key tiles and masks."""
    from orion_b200 import kernels
    torch.manual_seed(40 + S)
    qkv = torch.randn(B, S, 3 * H * 64, device="cuda").to(torch.bfloat16)
    ctx = tops.attention(qkv, H, 0.125, causal).view(B, S, H, 64)
    assert kernels.read_status() == 0
    q, k, v = qkv.double().cpu().view(B, S, 3, H, 64).permute(2, 0, 3, 1, 4)
    want = F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=0.125).permute(0, 2, 1, 3)
    assert O.rel_err(ctx, want) < 2e-2


# ---------------------------------------------------------------------------------------------- training on the own GEMM
@pytest.mark.parametrize("rows,K,N,bias,res", [(3072, 768, 2304, True, False), (3072, 768, 768, True, True), (520, 256, 136, False, True),
                                               (64, 3072, 768, True, True), (8192, 1024, 1024, False, False)])
def test_linear_training_forward_and_three_gradients(tops, rows, K, N, bias, res):
    """y = x w^T + b + residual and dx, dw, db, dresidual through the autograd op, against float64 on the CPU from the same
    bfloat16 values (tolerance 2e-2 of each tensor's largest entry)."""
    from orion_b200 import kernels
    torch.manual_seed(rows + N)
    bf = torch.bfloat16
    x = torch.randn(rows, K, device="cuda").to(bf).requires_grad_(True)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(bf).requires_grad_(True)
    b = torch.randn(N, device="cuda").to(bf).requires_grad_(True) if bias else None
    r = torch.randn(rows, N, device="cuda").to(bf).requires_grad_(True) if res else None
    dy = torch.randn(rows, N, device="cuda").to(bf)
    y = tops.linear_train(x, w, b, r)
    y.backward(dy)
    assert kernels.read_status() == 0
    xd, wd = (t.detach().double().cpu().requires_grad_(True) for t in (x, w))
    bd = b.detach().double().cpu().requires_grad_(True) if bias else None
    rd = r.detach().double().cpu().requires_grad_(True) if res else None
    want = F.linear(xd, wd, bd) + (rd if res else 0)
    want.backward(dy.double().cpu())
    assert O.rel_err(y.detach(), want.detach()) < 2e-2
    assert O.rel_err(x.grad, xd.grad) < 2e-2 and O.rel_err(w.grad, wd.grad) < 2e-2
    if bias:
        assert O.rel_err(b.grad, bd.grad) < 2e-2
    if res:
        assert O.rel_err(r.grad, rd.grad) < 2e-2


@pytest.mark.parametrize("B,S,H,d,causal", [(2, 384, 12, 64, False), (1, 512, 16, 64, True), (2, 200, 3, 64, True), (1, 64, 2, 32, False)])
def test_attention_training_forward_and_gradient(tops, B, S, H, d, causal):
    """Context and d(qkv) of softmax(Q K^T scale [+ causal mask]) V on the fused projection layout, against float64 autograd on
    the CPU from the same bfloat16 qkv (2e-2 of the largest entry)."""
    from orion_b200 import kernels
    torch.manual_seed(S + H)
    scale = 1.0 / d ** 0.5
    qkv = (torch.randn(B, S, 3 * H * d, device="cuda") * 0.7).to(torch.bfloat16).requires_grad_(True)
    dout = torch.randn(B, S, H * d, device="cuda").to(torch.bfloat16)
    out = tops.attention_train(qkv, H, scale, causal)
    out.backward(dout)
    assert kernels.read_status() == 0
    qd = qkv.detach().double().cpu().requires_grad_(True)
    q, k, v = qd.view(B, S, 3, H, d).permute(2, 0, 3, 1, 4)
    want = F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale).permute(0, 2, 1, 3).reshape(B, S, H * d)
    want.backward(dout.double().cpu())
    assert O.rel_err(out.detach(), want.detach()) < 2e-2
    assert O.rel_err(qkv.grad, qd.grad) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_embedding_sum_and_table_gradients(tops, dtype):
    torch.manual_seed(9)
    B, S, D, V = 4, 96, 256, 1000
    ids = torch.randint(0, V, (B, S), device="cuda")
    ids[0, :10] = 7   # repeated rows: their gradients add up
    word, pos, typ = (torch.randn(n, D, device="cuda").to(dtype).requires_grad_(True) for n in (V, 128, 2))
    dy = torch.randn(B, S, D, device="cuda").to(dtype)
    out = tops.embedding_train(ids, word, pos, typ)
    out.backward(dy)
    wd, pd, td = (t.detach().double().cpu().requires_grad_(True) for t in (word, pos, typ))
    want = wd[ids.cpu()] + pd[torch.arange(S)][None] + td[0]
    want.backward(dy.double().cpu())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert O.rel_err(out.detach(), want.detach()) < tol
    assert O.rel_err(word.grad, wd.grad) < tol and O.rel_err(pos.grad, pd.grad) < tol and O.rel_err(typ.grad, td.grad) < tol
    out2 = tops.embedding_train(ids, word, pos, None)
    assert O.rel_err(out2.detach(), (wd[ids.cpu()] + pd[torch.arange(S)][None]).detach()) < tol


def test_transformer_layer_trains_on_own_kernels_only(tops):
    """One encoder layer of the training clients (causal and not): output and every parameter gradient of the orion path against
    the stock-module path in float64 on the CPU; no stock GEMM, attention, softmax or LayerNorm kernel may be needed
    (torch.ops.orion.fallbacks() stays put)."""
    import importlib
    tt = importlib.import_module("benchmarking.benchmark_suite.transformer_trainer")
    assert tt.ORION_TRAIN_KERNELS and tt.OWN_GEMM_TRAINING
    torch.manual_seed(21)
    h, heads, ffn, b, s = 256, 4, 512, 2, 128
    for causal in (False, True):
        layer = tt.BertLayer(h, heads, ffn).cuda().to(torch.bfloat16).train()
        ref = tt.BertLayer(h, heads, ffn).double().train()
        ref.load_state_dict({k: v.double().cpu() for k, v in layer.state_dict().items()})
        x = torch.randn(b, s, h, device="cuda").to(torch.bfloat16).requires_grad_(True)
        dy = torch.randn(b, s, h, device="cuda").to(torch.bfloat16)
        before = tops.fallbacks()
        y = layer(x, causal=causal)
        y.backward(dy)
        assert tops.fallbacks() == before
        xd = x.detach().double().cpu().requires_grad_(True)
        want = ref(xd, causal=causal)
        want.backward(dy.double().cpu())
        assert O.rel_err(y.detach(), want.detach()) < 2e-2
        assert O.rel_err(x.grad, xd.grad) < 3e-2
        for (name, p), (_, pr) in zip(layer.named_parameters(), ref.named_parameters()):
            assert O.rel_err(p.grad, pr.grad) < 3e-2, name


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_column_sums_and_softmax_backward_through_the_c_abi(K, dtype, tol):
    torch.manual_seed(12)
    x = torch.randn(3000, 768, device="cuda").to(dtype)
    assert O.rel_err(K.colsum(x), x.double().cpu().sum(0)) < tol
    s = torch.randn(640, 384, device="cuda", dtype=torch.float64)
    p = torch.softmax(s * 0.125, -1).to(dtype)
    dp = torch.randn(640, 384, device="cuda").to(dtype)
    pd, dpd = p.double().cpu(), dp.double().cpu()
    want = 0.125 * pd * (dpd - (pd * dpd).sum(-1, keepdim=True))
    assert O.rel_err(K.softmax_backward(p, dp, 0.125), want) < tol
    # causal rows: columns behind the query position are not read (NaN there must not matter) and come out as zero
    S = 128
    mask = torch.tril(torch.ones(S, S, dtype=torch.bool, device="cuda")).repeat(5, 1)
    pc = (torch.softmax(torch.randn(5 * S, S, device="cuda"), -1) * mask).to(dtype)
    dpc = torch.randn(5 * S, S, device="cuda").to(dtype)
    pcd, dpcd = pc.double().cpu(), (dpc.double() * mask).cpu()
    wantc = 0.5 * pcd * (dpcd - (pcd * dpcd).sum(-1, keepdim=True))
    dpc = torch.where(mask, dpc, torch.full_like(dpc, float("nan")))
    got = K.softmax_backward(pc, dpc, 0.5, causal_period=S)
    assert torch.isfinite(got).all() and O.rel_err(got, wantc) < tol
