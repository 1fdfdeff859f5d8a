"""Runs a few training steps of a shortened BERT client (BERT-base width, `--layers` encoder layers, batch 8 x 384 tokens,
bfloat16, AdamW) on the orion kernels, outside the scheduler: the launch sequence of one step is what a profiler lists.

    python -m orion_b200.transformer_step_replay [--layers 2] [--steps 3]

Prints one JSON line: milliseconds per step (CUDA events on the launching stream) and the number of launches of this
repository's kernels per step.
"""
import argparse
import json
import sys
import os

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    a = ap.parse_args()
    from orion_b200 import torch_ops
    from orion_b200.optim import AdamW
    from benchmarking.benchmark_suite import transformer_trainer as tt
    torch_ops.load()
    torch.manual_seed(1)
    model = tt.BertQA(dict(tt.BERT, layers=a.layers)).cuda().to(torch.bfloat16).train()
    opt = AdamW(model.parameters(), lr=3e-5)
    ids = torch.randint(0, 30522, (8, 384), device="cuda")
    lab = torch.randint(0, 384, (2, 8), device="cuda")
    times, launches = [], []
    for _ in range(a.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = int(torch.ops.orion.own_launches())
        e0.record()
        opt.zero_grad()
        loss = 2.0 * torch.ops.orion.cross_entropy(model.span_logits(ids).view(-1, 384), lab.view(-1))
        loss.backward()
        opt.step()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
        launches.append(int(torch.ops.orion.own_launches()) - before)
    print(json.dumps({"layers": a.layers, "ms_per_step": times[-1], "own_launches_per_step": launches[-1], "loss": float(loss)}))


if __name__ == "__main__":
    main()
