"""Baseline without a scheduler: the high-priority inference client and the best-effort training client
as two threads of one process, each on its own CUDA stream (priority -1 for the inference stream, 0 for
the training stream), every kernel launched the moment its client issues it.  This is the reference's
"native streams" comparison point (related/baselines/vision/train_imagenet.py:19-22, where
`torch.cuda.Stream(priority=-1 / 0)` pick the streams and nothing intercepts the launches).

    python benchmarking/native_streams.py --model resnet50 --hp-batch 4 --be-batch 32 --rps 80 --requests 600 \
        [--solo hp|be] [--out result.json]

Same models, kernels, data and request process as the scheduled clients (benchmark_suite/train_imagenet.py):
prepared inference model on the orion kernels, training client through the dispatcher overrides, N(0,1)
images from pinned host memory copied per request, Poisson arrivals, latency counted from the scheduled
arrival.  Prints one JSON line.
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np
import torch
from torchvision import models

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--hp-batch", type=int, default=4)
    ap.add_argument("--be-batch", type=int, default=32)
    ap.add_argument("--rps", type=float, default=80.0, help="0 = closed loop")
    ap.add_argument("--requests", type=int, default=600)
    ap.add_argument("--solo", default="", help="hp or be: run only that client")
    ap.add_argument("--be-seconds", type=float, default=8.0, help="length of a solo training run")
    ap.add_argument("--out", default="")
    a = ap.parse_args()

    from orion_b200 import torch_ops
    torch_ops.load()
    torch.manual_seed(42)
    np.random.seed(42)
    dev = torch.device("cuda", 0)
    hp_stream, be_stream = torch.cuda.Stream(priority=-1), torch.cuda.Stream(priority=0)
    done = threading.Event()
    ready = threading.Barrier(1 if a.solo else 2)
    res = {}
    lr = 0.05 if a.model == "mobilenet_v2" else 0.1

    def hp_client():
        with torch.cuda.stream(hp_stream), torch.no_grad():
            with torch_ops.TRACE_LOCK:
                model = models.__dict__[a.model](num_classes=1000).to(dev).to(memory_format=torch.channels_last).eval()
                model = torch_ops.prepare_inference(model)
                x_host = torch.randn(a.hp_batch, 3, 224, 224).contiguous(memory_format=torch.channels_last).pin_memory()
                for _ in range(10):
                    model(x_host.to(dev, non_blocking=True)).cpu()
            ready.wait()
            gaps = np.random.exponential(1.0 / a.rps, a.requests) if a.rps > 0 else np.zeros(a.requests)
            lat, t0 = [], time.time()
            next_start = time.time()
            for i in range(a.requests):
                # open loop: request i may start no earlier than the previous scheduled start plus its gap, and its
                # latency counts from that scheduled start (queueing behind a late predecessor included)
                while a.rps > 0 and time.time() < next_start:
                    time.sleep(min(1e-4, max(0.0, next_start - time.time())))
                scheduled = next_start if a.rps > 0 else time.time()
                model(x_host.to(dev, non_blocking=True)).cpu()
                lat.append(time.time() - scheduled)
                next_start = scheduled + gaps[i]
            lat = np.array(lat) * 1e3
            res["hp"] = {"p50_ms": float(np.percentile(lat, 50)), "p99_ms": float(np.percentile(lat, 99)),
                         "requests": a.requests, "seconds": time.time() - t0}
        done.set()

    def be_client():
        with torch.cuda.stream(be_stream):
            with torch_ops.TRACE_LOCK:
                model = models.__dict__[a.model](num_classes=1000).to(dev).to(memory_format=torch.channels_last).train()
            opt = torch.optim.SGD(model.parameters(), lr=lr, momentum=0.9)
            crit = torch.nn.CrossEntropyLoss().to(dev)
            x_host = torch.randn(a.be_batch, 3, 224, 224).contiguous(memory_format=torch.channels_last).pin_memory()
            t_host = torch.randint(0, 1000, (a.be_batch,)).pin_memory()

            def step():
                opt.zero_grad()
                loss = crit(model(x_host.to(dev, non_blocking=True)), t_host.to(dev, non_blocking=True))
                loss.backward()
                opt.step()
                return float(loss.detach())

            with torch_ops.TRACE_LOCK:
                step()
            for _ in range(9):
                step()
            ready.wait()
            n, t0 = 0, time.time()
            while not done.is_set():
                step()
                n += 1
                if a.solo == "be" and time.time() - t0 > a.be_seconds:
                    done.set()
            res["be"] = {"samples_per_s": n * a.be_batch / (time.time() - t0), "iterations": n}

    threads = []
    if a.solo != "be":
        threads.append(threading.Thread(target=hp_client))
    if a.solo != "hp":
        threads.append(threading.Thread(target=be_client))
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    res["config"] = {"model": a.model, "hp_batch": a.hp_batch, "be_batch": a.be_batch, "rps": a.rps, "solo": a.solo or None,
                     "streams": "torch.cuda.Stream(priority=-1) / (priority=0), no interception, no scheduler"}
    line = json.dumps(res)
    print(line)
    if a.out:
        with open(a.out, "w") as f:
            f.write(line + "\n")


if __name__ == "__main__":
    main()
