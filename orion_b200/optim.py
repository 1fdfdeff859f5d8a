"""Optimizers of the training clients on the orion kernels.

`AdamW` has torch.optim.AdamW's constructor and semantics (decoupled weight decay, bias correction, state in the
parameters' type) and performs the step in a few launches over all parameters (ob200_adamw_multi).

`SGD` has torch.optim.SGD's constructor and semantics (momentum, weight decay, Nesterov; dampening 0) and performs the
whole step in one or two kernel launches over all parameters (ob200_sgd_momentum_multi_f32) — the role the multi-tensor
("foreach") kernels play in the reference's training profiles (reference benchmarking/model_kernels/resnet50_32_fb1)."""
import torch

from . import torch_ops


class SGD(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False):
        if dampening != 0.0:
            raise ValueError("orion_b200.optim.SGD supports dampening 0 only")
        if nesterov and momentum <= 0:
            raise ValueError("Nesterov momentum requires a momentum")
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay, nesterov=nesterov))
        torch_ops.load()

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            params = [p for p in group["params"] if p.grad is not None]
            if not params:
                continue
            fresh = [p for p in params if "momentum_buffer" not in self.state[p]]
            if fresh and len(fresh) != len(params):
                # mixed: parameters that got their first gradient later than the others take a step of their own
                self._launch(group, fresh, True)
                params = [p for p in params if p not in set(fresh)]
                fresh = []
            self._launch(group, params, bool(fresh))
        return loss

    def _launch(self, group, params, first):
        if not params:
            return
        if any(not (p.is_cuda and p.dtype == torch.float32 and p.grad.dtype == torch.float32 and not p.grad.is_sparse and
                    p.grad.stride() == p.stride()) for p in params):
            raise RuntimeError("orion_b200.optim.SGD needs dense float32 CUDA parameters whose gradients share their layout")
        if first:
            for p in params:
                self.state[p]["momentum_buffer"] = torch.empty_like(p, memory_format=torch.preserve_format)
        bufs = [self.state[p]["momentum_buffer"] for p in params]
        torch.ops.orion.sgd_step(params, [p.grad for p in params], bufs, group["lr"], group["momentum"], group["weight_decay"],
                                 group["nesterov"], first)


class AdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        torch_ops.load()

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            by_step = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["step"] += 1
                by_step.setdefault((st["step"], p.dtype), []).append(p)
            for (step, _), params in by_step.items():
                torch.ops.orion.adamw_step(params, [p.grad for p in params], [self.state[p]["exp_avg"] for p in params],
                                           [self.state[p]["exp_avg_sq"] for p in params], group["lr"], group["betas"][0],
                                           group["betas"][1], group["eps"], group["weight_decay"], step)
        return loss
