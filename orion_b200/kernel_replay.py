"""Replay the convolution launches of a model through the C ABI, for timing and for profiler
captures.

    python -m orion_b200.kernel_replay --model resnet50 --batch 32 --iters 5 --warm 3
    python -m orion_b200.kernel_replay --case 32,56,56,64,64,3,1,1 --iters 3 --warm 1     # one layer

Prints one JSON line: algorithmic FLOP per launch, average launch time measured with CUDA
events on the launching stream, achieved TFLOP/s.  Between iterations a buffer larger than L2
is rewritten so that no iteration finds its operands cached.
"""
import argparse
import json


def conv_layers_resnet50():
    """(C, K, R, stride, pad, H) of every convolution of torchvision's ResNet-50 (input size H=W)."""
    layers = [(3, 64, 7, 2, 3, 224)]
    h, cin = 56, 64
    for width, blocks, stride in ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)):
        for b in range(blocks):
            s = stride if b == 0 else 1
            layers.append((cin, width, 1, 1, 0, h))
            layers.append((width, width, 3, s, 1, h))
            hout = h // s
            layers.append((width, width * 4, 1, 1, 0, hout))
            if b == 0:
                layers.append((cin, width * 4, 1, s, 0, h))
            cin, h = width * 4, hout
    return layers


def replay(layers, batch, iters, warm, dtype="float32", flush_mb=160):
    import torch
    from orion_b200 import kernels as K
    dev = torch.device("cuda", torch.cuda.current_device())
    tf32 = dtype == "tf32"
    tdtype = torch.float32 if tf32 else getattr(torch, dtype)
    flops, work = 0.0, []
    for (c, k, r, s, p, h) in layers:
        x = torch.randn(batch, h, h, c, device=dev).to(tdtype)
        w = (torch.randn(k, r, r, c, device=dev) * (1.0 / (c * r * r) ** 0.5)).to(tdtype)
        ho = (h + 2 * p - r) // s + 1
        flops += 2.0 * batch * ho * ho * k * c * r * r
        epc = 16 // x.element_size()
        if c % epc:                              # filters are padded once, ahead of time
            w = torch.nn.functional.pad(w, (0, epc - c % epc)).contiguous()
        work.append((x, w, (s, s), (p, p)))
    flush = torch.empty(flush_mb * 1024 * 1024, dtype=torch.uint8, device=dev) if flush_mb else None
    stream = torch.cuda.current_stream()
    total_ms, launches = 0.0, 0
    for it in range(warm + iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for (x, w, s, p) in work:
            if x.shape[-1] != w.shape[-1]:      # 3-channel stem: the image is padded per call, as the torch op does
                x = K.pad_channels(x, w.shape[-1])
            K.conv2d_nhwc(x, w, s, p, tf32=tf32)
        e1.record(stream)
        e1.synchronize()
        if it >= warm:
            total_ms += e0.elapsed_time(e1)
            launches += len(work)
    status = K.read_status()
    if status != 0:
        raise RuntimeError("a kernel reported a timed-out wait (status %d)" % status)
    per_launch_flop = flops / len(work)
    avg_launch_s = total_ms * 1e-3 / max(1, launches)
    return {"achieved_tflops": per_launch_flop / avg_launch_s / 1e12, "launches": launches, "avg_launch_us": avg_launch_s * 1e6,
            "flop_per_launch": per_launch_flop, "batch": batch, "dtype": dtype, "layers": len(work)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--case", default="", help="Nb,H,W,C,K,R,stride,pad of a single layer")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warm", type=int, default=3)
    ap.add_argument("--dtype", default="float32", help="float32 (3xTF32), tf32 (float32 data, one TF32 pass) or bfloat16")
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args()
    if a.case:
        nb, h, w, c, k, r, s, p = [int(v) for v in a.case.split(",")]
        layers, batch = [(c, k, r, s, p, h)], nb
    else:
        layers, batch = conv_layers_resnet50(), a.batch
    print(json.dumps(replay(layers, batch, a.iters, a.warm, a.dtype, 0 if a.no_flush else 160)))


if __name__ == "__main__":
    main()
