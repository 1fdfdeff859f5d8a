"""Host-side checks of the transformer client definitions (no GPU): the float32 parameter cache of the inference path, the
span-logit layout of the BERT training loss, and that the CPU never takes an orion path."""
import torch

from benchmarking.benchmark_suite import transformer_trainer as tt


def test_float32_copies_are_made_once_per_parameter_version():
    layer = tt.BertLayer(64, 2, 128).to(torch.bfloat16)
    a = tt._f32(layer, layer.qkv.bias)
    assert a.dtype == torch.float32 and torch.equal(a, layer.qkv.bias.detach().float())
    assert tt._f32(layer, layer.qkv.bias) is a                      # same version: the cached tensor
    assert tt._f32(layer, layer.out.bias) is not a
    with torch.no_grad():
        layer.qkv.bias.add_(1.0)                                    # an optimizer step bumps the version
    b = tt._f32(layer, layer.qkv.bias)
    assert b is not a and torch.equal(b, layer.qkv.bias.detach().float())
    layer.qkv.bias.data = torch.zeros_like(layer.qkv.bias)          # .to() / .cuda() swap the storage without a version bump
    assert torch.equal(tt._f32(layer, layer.qkv.bias), torch.zeros(192))
    assert "_f32_cache" not in layer.state_dict()


def test_cpu_models_use_the_stock_modules_and_the_span_loss_layout_matches():
    """On the CPU both models run the stock path whatever the switches say; the two-span loss computed from [2, B, S] logits
    (the layout the orion cross-entropy reads) equals the sum of the two per-span losses of the reference client."""
    import torch.nn.functional as F
    torch.manual_seed(0)
    cfg = dict(tt.BERT, layers=1, hidden=64, heads=2, ffn=128, vocab=128, max_pos=32, seq=16)
    model = tt.BertQA(cfg).train()
    ids = torch.randint(0, 128, (3, 16))
    lab = torch.randint(0, 16, (2, 3))
    assert not model._own_training(ids)
    logits = model(ids)                                             # [B, S, 2]
    want = F.cross_entropy(logits[:, :, 0], lab[0]) + F.cross_entropy(logits[:, :, 1], lab[1])
    lt = logits.permute(2, 0, 1).reshape(2 * 3, 16)                 # rows (span, batch), positions contiguous
    got = 2.0 * F.cross_entropy(lt, lab.reshape(-1))
    assert torch.allclose(got, want, rtol=1e-6, atol=1e-6)
    # the head's bias moves every position of a row alike: no effect on the loss
    with torch.no_grad():
        model.qa.bias.add_(torch.tensor([3.0, -2.0]))
    logits2 = model(ids)
    want2 = F.cross_entropy(logits2[:, :, 0], lab[0]) + F.cross_entropy(logits2[:, :, 1], lab[1])
    assert torch.allclose(want2, want, rtol=1e-5, atol=1e-5)
    lm = tt.DecoderLM(dict(tt.LM, layers=1, hidden=64, heads=2, ffn=128, vocab=96, seq=16)).train()
    out = lm(torch.randint(0, 96, (2, 16)))
    assert out.shape == (2, 16, 96)
