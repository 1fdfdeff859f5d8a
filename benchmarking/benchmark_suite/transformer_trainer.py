"""Language-model clients: `bert_loop` (BERT-base question answering, reference
benchmarking/benchmark_suite/bert_trainer_mock.py:49-234) and `transformer_loop` (language-model
training, reference benchmarking/benchmark_suite/transformer_trainer.py:43-200), with the
reference's argument lists.  The request loop is `run_client` of train_imagenet.py.

Models are defined here (the reference imports NVIDIA's example repositories, which are not part
of it): BERT-base = 12 layers, hidden 768, 12 heads, FFN 3072, vocabulary 30522 padded to 30528,
sequence 384; the training "transformer" client is the benchmark configuration's decoder-only LM
(16 layers, d_model 1024, 16 heads, FFN 4096, vocabulary 32000, sequence 512) — the reference's
Transformer-XL is not reproduced.  Everything is bfloat16 with synthetic token ids.

Inference runs on the orion kernels (tcgen05 GEMM and fused attention, LayerNorm, softmax, GELU), and so does
training (ORION_PREPARE=1, the default): linear layers and attention with all their gradient products on the
bfloat16 GEMM, LayerNorm / GELU / softmax / embedding / cross-entropy forward and backward, one-launch AdamW.
With ORION_PREPARE=0 training uses stock PyTorch modules, whose cuBLASLt / flash-attention / elementwise
launches are captured and scheduled like any other op.
"""
import math
import os

import torch
import torch.nn as nn
import torch.nn.functional as F

from .train_imagenet import run_client

# Training clients use the orion LayerNorm / GELU / cross-entropy / AdamW kernels unless ORION_PREPARE=0 or the overrides are off.
ORION_TRAIN_KERNELS = os.environ.get("ORION_PREPARE", "1") == "1" and os.environ.get("ORION_DISABLE_OVERRIDES", "0") != "1"

FUSED_ATTENTION = os.environ.get("ORION_FUSED_ATTENTION", "1") == "1"
# ORION_OWN_GEMM_TRAINING=0 leaves the GEMMs, the attention and the embeddings of the training clients on the stock kernels
OWN_GEMM_TRAINING = os.environ.get("ORION_OWN_GEMM_TRAINING", "1") == "1"

BERT = dict(layers=12, hidden=768, heads=12, ffn=3072, vocab=30528, max_pos=512, seq=384)
LM = dict(layers=16, hidden=1024, heads=16, ffn=4096, vocab=32000, seq=512)


def _f32(module, p):
    """float32 copy of a parameter for the kernels that take their bias / scale in float32, made once per parameter version
    (an inference model never changes it) instead of one cast kernel per use."""
    cache = module.__dict__.setdefault("_f32_cache", {})
    hit = cache.get(id(p))
    if hit is None or hit[0] != p._version or hit[2] != p.data_ptr():
        hit = (p._version, p.detach().float(), p.data_ptr())
        cache[id(p)] = hit
    return hit[1]


class BertLayer(nn.Module):
    def __init__(self, h, heads, ffn):
        super().__init__()
        self.heads = heads
        self.qkv = nn.Linear(h, 3 * h)
        self.out = nn.Linear(h, h)
        self.ln1 = nn.LayerNorm(h, eps=1e-12)
        self.fc1 = nn.Linear(h, ffn)
        self.fc2 = nn.Linear(ffn, h)
        self.ln2 = nn.LayerNorm(h, eps=1e-12)

    def forward(self, x, causal=False):
        b, s, h = x.shape
        if ORION_TRAIN_KERNELS and OWN_GEMM_TRAINING and x.is_cuda and self.training and x.dtype == torch.bfloat16:
            # every op of the layer, forward and backward, on the orion kernels; residual adds ride in the GEMM epilogues
            ops = torch.ops.orion
            qkv = ops.linear_train(x, self.qkv.weight, self.qkv.bias)
            ctx = ops.attention_train(qkv, self.heads, 1.0 / math.sqrt(h // self.heads), causal)
            x = ops.layernorm_train(ops.linear_train(ctx, self.out.weight, self.out.bias, x), self.ln1.weight, self.ln1.bias, self.ln1.eps)
            hid = ops.bias_gelu_train(ops.linear_train(x, self.fc1.weight, None), self.fc1.bias)
            return ops.layernorm_train(ops.linear_train(hid, self.fc2.weight, self.fc2.bias, x), self.ln2.weight, self.ln2.bias,
                                       self.ln2.eps)
        q, k, v = self.qkv(x).view(b, s, 3, self.heads, h // self.heads).permute(2, 0, 3, 1, 4)
        ctx = F.scaled_dot_product_attention(q, k, v, is_causal=causal).transpose(1, 2).reshape(b, s, h)
        if ORION_TRAIN_KERNELS and x.is_cuda and self.training:
            # LayerNorm and bias + GELU, forward and backward, on the orion kernels (the GEMMs and the attention stay stock)
            ops = torch.ops.orion
            x = ops.layernorm_train((x + self.out(ctx)).contiguous(), self.ln1.weight, self.ln1.bias, self.ln1.eps)
            hid = ops.bias_gelu_train(F.linear(x, self.fc1.weight), self.fc1.bias)
            return ops.layernorm_train((x + self.fc2(hid)).contiguous(), self.ln2.weight, self.ln2.bias, self.ln2.eps)
        x = self.ln1(x + self.out(ctx))
        return self.ln2(x + self.fc2(F.gelu(self.fc1(x))))

    def forward_orion(self, x, causal=False):
        """Same math on the orion kernels (inference): x [B, S, H] bfloat16."""
        ops = torch.ops.orion
        b, s, h = x.shape
        d = h // self.heads
        flat = x.reshape(b * s, h)
        qkv = ops.linear(flat, self.qkv.weight, _f32(self, self.qkv.bias), False)
        if d == 64 and s <= 384 and x.dtype == torch.bfloat16 and FUSED_ATTENTION:
            # scores, softmax and the context product in one kernel, read straight from the projection's output
            ctx = ops.attention(qkv.view(b, s, 3 * h), self.heads, 1.0 / math.sqrt(d), causal)
        else:
            qkv = qkv.view(b, s, 3, self.heads, d)
            q = qkv[:, :, 0].permute(0, 2, 1, 3).reshape(b * self.heads, s, d).contiguous()
            k = qkv[:, :, 1].permute(0, 2, 1, 3).reshape(b * self.heads, s, d).contiguous()
            vt = qkv[:, :, 2].permute(0, 2, 3, 1).reshape(b * self.heads, d, s).contiguous()
            probs = ops.softmax(ops.linear_batched(q, k), 1.0 / math.sqrt(d), s if causal else 0)
            ctx = ops.linear_batched(probs, vt).view(b, self.heads, s, d).permute(0, 2, 1, 3).reshape(b * s, h).contiguous()
        # the residual stream is added in the GEMM epilogue, in float32, before the sum is rounded to bfloat16
        attn = ops.linear(ctx, self.out.weight, _f32(self, self.out.bias), False, flat)
        y = ops.layernorm(attn, _f32(self, self.ln1.weight), _f32(self, self.ln1.bias), self.ln1.eps)
        hid = ops.bias_gelu(ops.linear(y, self.fc1.weight, None, False), _f32(self, self.fc1.bias))
        out = ops.linear(hid, self.fc2.weight, _f32(self, self.fc2.bias), False, y)
        return ops.layernorm(out, _f32(self, self.ln2.weight), _f32(self, self.ln2.bias), self.ln2.eps).view(b, s, h)


class BertQA(nn.Module):
    def __init__(self, cfg=BERT):
        super().__init__()
        h = cfg["hidden"]
        self.word = nn.Embedding(cfg["vocab"], h)
        self.pos = nn.Embedding(cfg["max_pos"], h)
        self.typ = nn.Embedding(2, h)
        self.ln = nn.LayerNorm(h, eps=1e-12)
        self.layers = nn.ModuleList([BertLayer(h, cfg["heads"], cfg["ffn"]) for _ in range(cfg["layers"])])
        self.qa = nn.Linear(h, 2)

    def _own_training(self, ids):
        return ORION_TRAIN_KERNELS and OWN_GEMM_TRAINING and ids.is_cuda and self.training and self.word.weight.dtype == torch.bfloat16

    def embed(self, ids):
        if self._own_training(ids):
            ops = torch.ops.orion
            return ops.layernorm_train(ops.embedding_train(ids, self.word.weight, self.pos.weight, self.typ.weight), self.ln.weight,
                                       self.ln.bias, self.ln.eps)
        pos = torch.arange(ids.shape[1], device=ids.device)
        return self.ln(self.word(ids) + self.pos(pos)[None] + self.typ.weight[0])

    def forward(self, ids, orion=False):
        if orion and ids.is_cuda and self.word.weight.dtype == torch.bfloat16:
            ops = torch.ops.orion   # the three lookups and their sum in one kernel, then the orion LayerNorm
            b, s = ids.shape
            emb = ops.embedding_train(ids.contiguous(), self.word.weight, self.pos.weight, self.typ.weight)
            x = ops.layernorm(emb.view(b * s, -1), _f32(self, self.ln.weight), _f32(self, self.ln.bias), self.ln.eps).view(b, s, -1)
        else:
            x = self.embed(ids)
        for layer in self.layers:
            x = layer.forward_orion(x) if orion else layer(x)
        return self.qa(x)   # [B, S, 2]: start / end logits

    def span_logits(self, ids):
        """Training on the orion kernels: the start / end logits as [2, B, S] (positions contiguous, the layout the
        loss reads), computed as qa.weight . x^T.  The head's bias is left out: it shifts all positions of a row alike,
        so the position softmax, the loss and every gradient are the same without it (its own gradient is zero)."""
        b, s = ids.shape
        x = self.embed(ids)
        for layer in self.layers:
            x = layer(x)
        return torch.ops.orion.linear_train(self.qa.weight, x.view(b * s, -1), None).view(2, b, s)


class DecoderLM(nn.Module):
    def __init__(self, cfg=LM):
        super().__init__()
        h = cfg["hidden"]
        self.word = nn.Embedding(cfg["vocab"], h)
        self.pos = nn.Embedding(cfg["seq"], h)
        self.layers = nn.ModuleList([BertLayer(h, cfg["heads"], cfg["ffn"]) for _ in range(cfg["layers"])])
        self.ln = nn.LayerNorm(h)
        self.head = nn.Linear(h, cfg["vocab"], bias=False)

    def forward(self, ids, orion=False):
        if (not orion and ORION_TRAIN_KERNELS and OWN_GEMM_TRAINING and ids.is_cuda and self.training
                and self.word.weight.dtype == torch.bfloat16):
            ops = torch.ops.orion
            x = ops.embedding_train(ids.contiguous(), self.word.weight, self.pos.weight)
            for layer in self.layers:
                x = layer(x, causal=True)
            return ops.linear_train(ops.layernorm_train(x, self.ln.weight, self.ln.bias, self.ln.eps), self.head.weight, None)
        if orion and ids.is_cuda and self.word.weight.dtype == torch.bfloat16:
            x = torch.ops.orion.embedding_train(ids.contiguous(), self.word.weight, self.pos.weight)
        else:
            pos = torch.arange(ids.shape[1], device=ids.device)
            x = self.word(ids) + self.pos(pos)[None]
        if not orion:
            for layer in self.layers:
                x = layer(x, causal=True)
            return self.head(self.ln(x))
        # inference on the orion kernels: causal softmax, final LayerNorm and the vocabulary projection included
        ops = torch.ops.orion
        for layer in self.layers:
            x = layer.forward_orion(x, causal=True)
        b, s, h = x.shape
        y = ops.layernorm(x.reshape(b * s, h), _f32(self, self.ln.weight), _f32(self, self.ln.bias), self.ln.eps)
        return ops.linear(y, self.head.weight, None, False).view(b, s, -1)


def _adamw(params, lr):
    if ORION_TRAIN_KERNELS and torch.cuda.is_available():
        from orion_b200.optim import AdamW
        return AdamW(params, lr=lr)
    return torch.optim.AdamW(params, lr=lr)


def _pinned(t):
    return t.pin_memory() if torch.cuda.is_available() else t


def bert_loop(batchsize, train, num_iters, rps, uniform, dummy_data, local_rank, barriers, client_barrier, tid, input_file=""):
    seq, vocab = BERT["seq"], 30522
    resident = os.environ.get("ORION_RESIDENT_INPUTS", "0") == "1"

    def build(device):
        model = BertQA().to(device).to(torch.bfloat16)
        ids = _pinned(torch.randint(0, vocab, (batchsize, seq)))
        labels = _pinned(torch.randint(0, seq, (2, batchsize)))
        state = {"ids": ids.to(device, non_blocking=True), "lab": labels.to(device, non_blocking=True)}
        if train:
            model.train()
            opt = _adamw(model.parameters(), lr=3e-5)

            def step(batch_idx):
                if not resident:
                    state["ids"] = ids.to(device, non_blocking=True)
                    state["lab"] = labels.to(device, non_blocking=True)
                opt.zero_grad()
                if ORION_TRAIN_KERNELS and OWN_GEMM_TRAINING:
                    # both span losses in one pass over the [2 * B, S] logits: mean over 2B rows = half the sum of the two means
                    lt = model.span_logits(state["ids"])
                    loss = 2.0 * torch.ops.orion.cross_entropy(lt.view(-1, seq), state["lab"].view(-1))
                else:
                    logits = model(state["ids"]).float()
                    loss = F.cross_entropy(logits[:, :, 0], state["lab"][0]) + F.cross_entropy(logits[:, :, 1], state["lab"][1])
                loss.backward()
                opt.step()
                return loss
            return step
        model.eval()
        use_orion = os.environ.get("ORION_PREPARE", "1") == "1"

        def step(batch_idx):
            if not resident:
                state["ids"] = ids.to(device, non_blocking=True)
            return model(state["ids"], orion=use_orion)
        return step

    run_client(tid, train, num_iters, rps, uniform, barriers, input_file, batchsize, build)


def transformer_loop(batchsize, train, num_iters, rps, uniform, dummy_data, local_rank, barriers, client_barrier, tid, input_file=""):
    seq, vocab = LM["seq"], LM["vocab"]
    resident = os.environ.get("ORION_RESIDENT_INPUTS", "0") == "1"

    def build(device):
        model = DecoderLM().to(device).to(torch.bfloat16)
        tokens = _pinned(torch.randint(0, vocab, (batchsize, seq + 1)))
        state = {"tok": tokens.to(device, non_blocking=True)}
        if train:
            model.train()
            opt = _adamw(model.parameters(), lr=3e-4)

            def step(batch_idx):
                if not resident:
                    state["tok"] = tokens.to(device, non_blocking=True)
                opt.zero_grad()
                logits = model(state["tok"][:, :-1])
                if ORION_TRAIN_KERNELS:   # loss and its gradient straight from the bfloat16 logits, one pass each
                    loss = torch.ops.orion.cross_entropy(logits.reshape(-1, vocab), state["tok"][:, 1:].reshape(-1))
                else:
                    loss = F.cross_entropy(logits.float().view(-1, vocab), state["tok"][:, 1:].reshape(-1))
                loss.backward()
                opt.step()
                return loss
            return step
        model.eval()
        use_orion = os.environ.get("ORION_PREPARE", "1") == "1"

        def step(batch_idx):
            if not resident:
                state["tok"] = tokens.to(device, non_blocking=True)
            return model(state["tok"][:, :-1], orion=use_orion)[:, -1]
        return step

    run_client(tid, train, num_iters, rps, uniform, barriers, input_file, batchsize, build)
