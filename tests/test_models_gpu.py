"""Whole-model parity: torchvision models running on the orion kernels (through the dispatcher
overrides, and as prepared models with fused epilogues) against eager PyTorch in float32 on the
CPU — the reference's numeric path.  Tolerance: fp32 relative 1e-4 (benchmark specification)."""
import pytest
import torch
import torchvision

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built):
    from orion_b200 import torch_ops
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    torch_ops.load()
    return torch_ops


def _rel(a, b):
    return ((a.double().cpu() - b.double().cpu()).abs().max() / b.double().abs().max()).item()


@pytest.mark.parametrize("name", ["resnet50", "mobilenet_v2", "resnet101"])
def test_inference_matches_cpu_fp32(ops, name):
    torch.manual_seed(42)
    model = torchvision.models.__dict__[name](num_classes=1000).eval()
    x = torch.randn(4, 3, 224, 224)
    with torch.no_grad():
        want = model(x)
        cuda_model = model.cuda().to(memory_format=torch.channels_last)
        xc = x.cuda().contiguous(memory_format=torch.channels_last)
        before = int(torch.ops.orion.own_launches())
        via_overrides = cuda_model(xc)
        mid = int(torch.ops.orion.own_launches())
        prepared = ops.prepare_inference(cuda_model)
        via_prepared = prepared(xc)
        after = int(torch.ops.orion.own_launches())
    from orion_b200 import kernels
    assert kernels.read_status() == 0
    assert mid > before and after > mid, "the orion kernels did not run"
    # The tensor core adds into its fp32 accumulator by truncation, which shrinks a long reduction slightly; with the
    # cross terms of the 3xTF32 product kept in an accumulator of their own the 104 convolutions of ResNet-101 stay
    # well inside the tolerance.
    tol = 1e-4
    e1, e2 = _rel(via_overrides, want), _rel(via_prepared, want)
    print("%s: relative error %.2e through the overrides, %.2e prepared" % (name, e1, e2))
    assert e1 < tol
    assert e2 < tol
    if name == "resnet50":
        # 53 fused convolutions, max-pool, average pool, classifier: one launch each; one zero-padding of the image to 4 channels
        assert after - mid == 53 + 3 + 1


def test_training_step_runs_on_overridden_forward_convolutions(ops):
    """BE-style training: forward convolutions on the orion kernel, backward on the stock ops;
    the loss must follow the stock path closely for a few SGD steps."""
    def run(override):
        torch.manual_seed(7)
        ops.set_overrides(override)
        m = torchvision.models.resnet18(num_classes=10).cuda().to(memory_format=torch.channels_last).train()
        opt = torch.optim.SGD(m.parameters(), lr=0.01, momentum=0.9)
        x = torch.randn(8, 3, 64, 64, device="cuda").contiguous(memory_format=torch.channels_last)
        y = torch.randint(0, 10, (8,), device="cuda")
        losses = []
        for _ in range(3):
            opt.zero_grad()
            loss = torch.nn.functional.cross_entropy(m(x), y)
            loss.backward()
            opt.step()
            losses.append(loss.item())
        return losses
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ours, stock = run(True), run(False)
    finally:
        ops.set_overrides(True)
    assert abs(ours[0] - stock[0]) / abs(stock[0]) < 1e-4          # same weights, same data: forward parity
    for a, b in zip(ours[1:], stock[1:]):
        assert abs(a - b) / abs(b) < 5e-2                           # later steps only have to stay close


def test_bert_layer_stack_on_orion_kernels_matches_cpu_fp32(ops):
    """BERT-base layers (hidden 768, 12 heads, FFN 3072, sequence 384) on the tcgen05 GEMM / batched GEMM, LayerNorm,
    softmax and GELU kernels against float32 CPU math on the same bfloat16 weights; tolerance bf16 relative 2e-2."""
    from benchmarking.benchmark_suite.transformer_trainer import BertQA
    torch.manual_seed(11)
    cfg = dict(layers=3, hidden=768, heads=12, ffn=3072, vocab=30528, max_pos=512, seq=384)
    model = BertQA(cfg).to(torch.bfloat16).eval()
    ids = torch.randint(0, 30522, (2, 384))
    with torch.no_grad():
        want = model.float()(ids)                      # float32 math on bf16-rounded weights
        model = model.to(torch.bfloat16).cuda()
        before = int(torch.ops.orion.own_launches())
        got = model(ids.cuda(), orion=True)
        after = int(torch.ops.orion.own_launches())
    from orion_b200 import kernels
    assert kernels.read_status() == 0
    assert after - before == 3 * 8 + 2                 # per layer: 4 GEMMs, fused attention, GELU, 2 LayerNorms; + embedding sum and its LayerNorm
    assert _rel(got.float(), want) < 2e-2
