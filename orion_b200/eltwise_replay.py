"""Times the HBM-bound kernels (batch norm, elementwise, pooling, depthwise convolution, LayerNorm,
softmax, GELU, optimizer steps) at the sizes the benchmark configurations use, one launch each per
iteration, with CUDA events on the launching stream and the L2 flushed before every launch.

    python -m orion_b200.eltwise_replay [--iters 5] [--warm 2]

Prints one JSON line per kernel: algorithmic bytes (what the op has to read and write once),
microseconds per launch and achieved GB/s.  The algorithmic byte counts are the ones the kernels are
measured against: 8 B per element for an in/out elementwise op, 12 B for training batch norm forward
(read for the statistics, read and write for the normalisation), 20 B for its backward, and so on.
"""
import argparse
import json

import torch

from orion_b200 import kernels as K


def cases():
    dev = torch.device("cuda", torch.cuda.current_device())
    f32 = dict(device=dev, dtype=torch.float32)
    out = []

    def add(name, nbytes, fn):
        out.append((name, nbytes, fn))

    # ResNet-50 training, batch 32: the 56x56x256 activation (102.8 MB) and the 28x28x512 one (51.4 MB)
    for (n, h, c) in ((32, 56, 256), (32, 28, 512)):
        x = torch.randn(n, h, h, c, **f32)
        dy = torch.randn_like(x)
        g, b = torch.rand(c, **f32) + 0.5, torch.randn(c, **f32)
        rm, rv = torch.zeros(c, **f32), torch.ones(c, **f32)
        _, sm, si = K.bn_train_forward(x, g, b, rm, rv, 1e-5, 0.1)
        e = x.numel()
        tag = "%dx%dx%dx%d" % (n, h, h, c)
        # the fused entry points the training clients use: statistics + finish in one launch, activation and residual in the other
        y_res, _, _ = K.bn_act_train_forward(x, g, b, rm, rv, 1e-5, 0.1, act=1, residual=dy)
        add("bn_act_forward+relu " + tag, 12 * e, lambda x=x, g=g, b=b, rm=rm, rv=rv: K.bn_act_train_forward(x, g, b, rm, rv, 1e-5, 0.1, act=1))
        add("bn_act_forward+add+relu " + tag, 16 * e,
            lambda x=x, g=g, b=b, rm=rm, rv=rv, dy=dy: K.bn_act_train_forward(x, g, b, rm, rv, 1e-5, 0.1, act=1, residual=dy))
        add("bn_act_backward+relu " + tag, 20 * e, lambda dy=dy, x=x, g=g, b=b, sm=sm, si=si: K.bn_act_backward(dy, x, g, b, sm, si, act=1))
        add("bn_act_backward+add+relu " + tag, 28 * e,
            lambda dy=dy, x=x, g=g, b=b, sm=sm, si=si, y=y_res: K.bn_act_backward(dy, x, g, b, sm, si, act=1, yout=y, want_dres=True))
        add("bn_train_forward " + tag, 12 * e, lambda x=x, g=g, b=b, rm=rm, rv=rv: K.bn_train_forward(x, g, b, rm, rv, 1e-5, 0.1))
        add("bn_backward " + tag, 20 * e, lambda dy=dy, x=x, g=g, sm=sm, si=si: K.bn_backward(dy, x, g, sm, si))
        add("bn_inference+relu " + tag, 8 * e, lambda x=x, g=g, b=b, rm=rm, rv=rv: K.bn_inference(x, g, b, rm, rv, 1e-5, relu=True))
        add("add+relu " + tag, 12 * e, lambda x=x, dy=dy: K.binary(x, dy, 2))
        add("relu_backward " + tag, 12 * e, lambda x=x, dy=dy: K.relu_backward(dy, x))
    x = torch.randn(32, 112, 112, 64, **f32)
    add("maxpool 3x3/2 32x112x112x64", 4 * (x.numel() + x.numel() // 4), lambda x=x: K.maxpool_nhwc(x, 3, 2, 1))
    dyp = torch.randn(32, 56, 56, 64, **f32)
    add("maxpool_backward 3x3/2 32x112x112x64", 4 * (2 * x.numel() + 2 * dyp.numel()), lambda x=x, dyp=dyp: K.maxpool_backward_nhwc(dyp, x, 3, 2, 1))
    x = torch.randn(256, 7, 7, 2048, **f32)
    add("avgpool 256x7x7x2048", 4 * (x.numel() + 256 * 2048), lambda x=x: K.avgpool_nhwc(x))
    # MobileNetV2 batch 64: depthwise 3x3 on 112x112x96 (stride 2) and 56x56x144 (stride 1), fused scale/shift/ReLU6
    for (n, h, c, s) in ((64, 112, 96, 2), (64, 56, 144, 1)):
        x = torch.randn(n, h, h, c, **f32)
        w = torch.randn(3, 3, c, **f32)
        sc, sh = torch.rand(c, **f32) + 0.5, torch.randn(c, **f32)
        ho = (h + 2 - 3) // s + 1
        add("depthwise 3x3/%d %dx%dx%dx%d" % (s, n, h, h, c), 4 * (x.numel() + n * ho * ho * c),
            lambda x=x, w=w, sc=sc, sh=sh, s=s: K.depthwise_conv2d_nhwc(x, w, (s, s), (1, 1), scale=sc, shift=sh, relu=2, tap_major=True))
    # BERT-base batch 8 x 384 (bf16) and the decoder LM batch 16 x 512
    x = torch.randn(64 * 384, 768, device=dev).bfloat16()
    g, b = torch.ones(768, **f32), torch.zeros(768, **f32)
    add("layernorm bf16 24576x768", 4 * x.numel(), lambda x=x, g=g, b=b: K.layernorm(x, g, b))
    x = torch.randn(8 * 12 * 8 * 384, 384, device=dev).bfloat16()
    add("softmax bf16 294912x384", 4 * x.numel(), lambda x=x: K.softmax(x, 0.125))
    x = torch.randn(32 * 384, 3072, device=dev).bfloat16()
    bias = torch.randn(3072, **f32)
    add("bias+gelu bf16 12288x3072", 4 * x.numel(), lambda x=x, bias=bias: K.bias_gelu(x, bias))
    # gradient side of the transformer clients: softmax backward on the LM's probabilities, a bias gradient
    pr = torch.softmax(torch.randn(16 * 16 * 512, 512, device=dev), -1).bfloat16()
    dp = torch.randn(16 * 16 * 512, 512, device=dev).bfloat16()
    add("softmax_backward bf16 131072x512", 6 * pr.numel(), lambda pr=pr, dp=dp: K.softmax_backward(pr, dp, 0.125))
    dyl = torch.randn(8192, 4096, device=dev).bfloat16()
    add("colsum bf16 8192x4096", 2 * dyl.numel(), lambda dyl=dyl: K.colsum(dyl))
    # optimizer steps over 25.6 M parameters (ResNet-50)
    p_, g_, m_, v_ = (torch.randn(25_600_000, **f32) for _ in range(4))
    v_.abs_()
    add("sgd_momentum 25.6M", 20 * p_.numel(), lambda: K.sgd_momentum_(p_, g_, m_, 0.1, 0.9))
    add("adamw 25.6M", 28 * p_.numel(), lambda: K.adamw_(p_, g_, m_, v_, 10, 1e-3))
    # the same 25.6 M parameters as 161 tensors of ResNet-50's sizes in two launches
    chunks = torch.split(p_, [150_000] * 160 + [25_600_000 - 160 * 150_000])
    gch = torch.split(g_, [150_000] * 160 + [25_600_000 - 160 * 150_000])
    mch = torch.split(m_, [150_000] * 160 + [25_600_000 - 160 * 150_000])
    add("sgd_momentum_multi 25.6M in 161 tensors", 20 * p_.numel(), lambda: K.sgd_momentum_multi_(list(chunks), list(gch), list(mch), 0.1, 0.9))
    return out


def replay(iters=5, warm=2, only=None):
    """Times every case (or those whose name starts with one of `only`); returns a list of
    {"kernel", "algorithmic_bytes", "us", "GBps"}."""
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    out = []
    for name, nbytes, fn in cases():
        if only is not None and not any(name.startswith(o) for o in only):
            continue
        total = 0.0
        for it in range(warm + iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            if it >= warm:
                total += e0.elapsed_time(e1)
        us = total * 1e3 / iters
        out.append({"kernel": name, "algorithmic_bytes": nbytes, "us": us, "GBps": nbytes / us / 1e3})
    if K.read_status() != 0:
        raise RuntimeError("a kernel reported a timed-out wait")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warm", type=int, default=2)
    a = ap.parse_args()
    for r in replay(a.iters, a.warm):
        print(json.dumps({"kernel": r["kernel"], "algorithmic_MB": round(r["algorithmic_bytes"] / 1e6, 1), "us": round(r["us"], 1),
                          "GBps": round(r["GBps"], 1)}), flush=True)


if __name__ == "__main__":
    main()
