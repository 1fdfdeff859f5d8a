"""PyTorch adapter: loads liborion_torch.so (dispatcher overrides + `torch.ops.orion.*`)
and prepares inference models so that each conv + batch-norm (+ residual add)
(+ ReLU/ReLU6) group runs as ONE launch of the implicit-GEMM kernel.

`prepare_inference(model)` is the only call a client script adds; everything it
builds still goes through the scheduler, because every launch of
liborion_kernels.so passes the cudaLaunchKernel trap of the capture library.
"""
import operator
import os
import threading

import torch
import torch.fx as fx
import torch.nn as nn
import torch.nn.functional as F

_HERE = os.path.dirname(os.path.abspath(__file__))
_GLUE = os.path.join(_HERE, "lib", "liborion_torch.so")
_loaded = False
# torch.fx.symbolic_trace patches nn.Module.__call__ process-wide while it runs.  Client threads
# of one process therefore take this lock around everything that calls a module during their
# first iteration (when models are prepared), and prepare_inference holds it while tracing.
TRACE_LOCK = threading.RLock()


def load():
    """Load the adapter; from then on aten::convolution / cudnn_batch_norm on CUDA
    tensors in channels-last layout run on the orion kernels."""
    global _loaded
    if not _loaded:
        if not os.path.exists(_GLUE):
            raise RuntimeError("liborion_torch.so is not built; run `python -m orion_b200.build`")
        torch.ops.load_library(_GLUE)
        _loaded = True
    return torch.ops.orion


def set_sm_quota(n):
    """CTA count of the persistent kernels launched by the calling thread."""
    return load().set_sm_quota(int(n))


def set_overrides(on):
    return load().set_overrides(1 if on else 0)


class FusedConv(nn.Module):
    """conv -> (folded batch-norm) -> (+ residual) -> activation in one kernel launch."""

    def __init__(self, conv, bn=None, act=0):
        super().__init__()
        assert conv.padding_mode == "zeros"
        w = conv.weight.detach()
        self.depthwise = conv.groups > 1
        if self.depthwise:
            # groups = C, multiplier 1 (MobileNetV2): the filter is kept tap-major, [R, S, C]
            assert conv.groups == conv.in_channels == conv.out_channels and w.dtype == torch.float32 and conv.groups % 4 == 0
            w = w[:, 0].permute(1, 2, 0).contiguous()
        # a channel count that does not fill 16-byte chunks (the 3-channel stem) is zero-padded once here;
        # the op pads the activation to match on every call
        epc = 16 // w.element_size()
        if not self.depthwise and w.shape[1] % epc:
            w = torch.nn.functional.pad(w, (0, 0, 0, 0, 0, epc - w.shape[1] % epc))
        self.register_buffer("weight", w if self.depthwise else w.contiguous(memory_format=torch.channels_last))
        k = conv.out_channels
        if bn is not None:
            inv = torch.rsqrt(bn.running_var.detach().double() + bn.eps)
            g = bn.weight.detach().double() if bn.weight is not None else torch.ones(k, dtype=torch.float64, device=w.device)
            b = bn.bias.detach().double() if bn.bias is not None else torch.zeros(k, dtype=torch.float64, device=w.device)
            scale = g * inv
            shift = b - bn.running_mean.detach().double() * scale
            if conv.bias is not None:
                shift = shift + conv.bias.detach().double() * scale
            self.register_buffer("scale", scale.float().contiguous())
            self.register_buffer("shift", shift.float().contiguous())
        else:
            self.scale = None
            if conv.bias is not None:
                self.register_buffer("shift", conv.bias.detach().float().contiguous())
            else:
                self.shift = None
        self.act = act
        self.stride, self.padding, self.dilation = list(conv.stride), list(conv.padding), list(conv.dilation)

    def forward(self, x, residual=None):
        if self.depthwise:
            assert residual is None
            return torch.ops.orion.depthwise_bn_act(x, self.weight, self.scale, self.shift, self.act, self.stride, self.padding,
                                                    self.dilation)
        return torch.ops.orion.conv_bn_act(x, self.weight, self.scale, self.shift, residual, self.act, self.stride,
                                           self.padding, self.dilation)


class OrionMaxPool(nn.Module):
    def __init__(self, k, stride, pad):
        super().__init__()
        self.k, self.stride, self.pad = k, stride, pad

    def forward(self, x):
        return torch.ops.orion.maxpool(x, self.k, self.stride, self.pad)


class OrionAvgPool(nn.Module):
    def forward(self, x):
        n, c = x.shape[0], x.shape[1]
        return torch.ops.orion.avgpool(x).view(n, c, 1, 1)


class OrionLinear(nn.Module):
    def __init__(self, lin):
        super().__init__()
        self.register_buffer("weight", lin.weight.detach().contiguous())
        if lin.bias is not None:
            self.register_buffer("bias", lin.bias.detach().float().contiguous())
        else:
            self.bias = None

    def forward(self, x):
        return torch.ops.orion.linear(x.contiguous(), self.weight, self.bias, False)


def _one(v):
    return v[0] if isinstance(v, (tuple, list)) else v


def _square(v):
    """True if a kernel-size / stride / padding argument is one number or the same number twice."""
    return not isinstance(v, (tuple, list)) or all(e == v[0] for e in v)


def _act_of(node, mods):
    """0 if `node` is not an activation the epilogue can apply, else 1 (ReLU) / 2 (ReLU6)."""
    if node.op == "call_module":
        m = mods.get(node.target)
        if isinstance(m, nn.ReLU):
            return 1
        if isinstance(m, nn.ReLU6):
            return 2
        if isinstance(m, nn.Hardtanh) and m.min_val == 0 and m.max_val == 6:
            return 2
    if node.op == "call_function" and node.target in (F.relu, torch.relu):
        return 1
    if node.op == "call_function" and node.target is F.relu6:
        return 2
    if node.op == "call_method" and node.target in ("relu", "relu_"):
        return 1
    return 0


class FusedBNAct(nn.Module):
    """BatchNorm2d (training mode) -> (+ residual) -> ReLU / ReLU6 as one differentiable op of two launches forward and
    two backward (`orion::bn_act_train`).  The wrapped BatchNorm2d keeps its parameters and running statistics."""

    def __init__(self, bn, act):
        super().__init__()
        self.bn = bn
        self.act = act
        self._pending_batches = 0   # num_batches_tracked is kept on the host and written back when the state is read
        self.register_state_dict_pre_hook(lambda module, prefix, keep_vars: module.flush_batch_counter())

    def flush_batch_counter(self):
        if self._pending_batches and self.bn.num_batches_tracked is not None:
            self.bn.num_batches_tracked += self._pending_batches
        self._pending_batches = 0

    def forward(self, x, residual=None):
        bn = self.bn
        fused = (bn.training and bn.track_running_stats and bn.momentum is not None and bn.affine and x.is_cuda and
                 x.dtype == torch.float32 and x.dim() == 4 and x.shape[1] % 4 == 0 and x.shape[1] <= 8192 and
                 x.is_contiguous(memory_format=torch.channels_last) and
                 (residual is None or residual.is_contiguous(memory_format=torch.channels_last)))
        if not fused:
            y = bn(x)
            if residual is not None:
                y = y + residual
            return F.relu(y) if self.act == 1 else F.relu6(y) if self.act == 2 else y
        self._pending_batches += 1
        return torch.ops.orion.bn_act_train(x, residual, bn.weight, bn.bias, bn.running_mean, bn.running_var, bn.momentum, bn.eps,
                                            self.act)


class OrionMaxPoolTrain(nn.Module):
    """MaxPool2d with a gradient kernel of its own (no index tensor is stored)."""

    def __init__(self, k, stride, pad):
        super().__init__()
        self.k, self.stride, self.pad = k, stride, pad

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.float32 and x.shape[1] % 4 == 0 and x.is_contiguous(memory_format=torch.channels_last):
            return torch.ops.orion.maxpool_train(x, self.k, self.stride, self.pad)
        return F.max_pool2d(x, self.k, self.stride, self.pad)


def prepare_training(model):
    """Return a training-mode GraphModule of `model` (torchvision-style CNN) in which every BatchNorm2d -> ReLU / ReLU6 and
    BatchNorm2d -> add -> ReLU group is one `FusedBNAct` module and max-pools run on the orion kernels in both directions.
    Parameters are the model's own objects (create the optimizer before or after, as you like); convolutions keep going
    through the dispatcher overrides."""
    load()
    model = model.train()
    with TRACE_LOCK:
        gm = fx.symbolic_trace(model)
    mods = dict(gm.named_modules())
    g = gm.graph
    n_fused = 0
    for node in list(g.nodes):
        m = mods.get(node.target) if node.op == "call_module" else None
        if isinstance(m, nn.MaxPool2d) and not m.ceil_mode and _one(m.dilation) == 1 and not m.return_indices and \
                _square(m.kernel_size) and _square(m.stride or m.kernel_size) and _square(m.padding) and _square(m.dilation):
            name = "orion_pool_%d" % n_fused
            n_fused += 1
            gm.add_module(name, OrionMaxPoolTrain(_one(m.kernel_size), _one(m.stride or m.kernel_size), _one(m.padding)))
            with g.inserting_before(node):
                new = g.call_module(name, node.args)
            node.replace_all_uses_with(new)
            g.erase_node(node)
            continue
        if node.op != "call_module" or not isinstance(mods.get(node.target), nn.BatchNorm2d):
            continue
        bn = mods[node.target]
        users = list(node.users)
        if len(users) != 1:
            continue
        u = users[0]
        act, act_node, add_node, res = _act_of(u, mods), None, None, None
        if act:
            act_node = u
        elif u.op == "call_function" and u.target in (operator.add, operator.iadd, torch.add) and len(u.args) == 2 and not u.kwargs \
                and all(isinstance(a, fx.Node) for a in u.args):
            other = u.args[1] if u.args[0] is node else u.args[0]
            uu = list(u.users)
            if other is not node and len(uu) == 1 and _act_of(uu[0], mods):
                add_node, res, act, act_node = u, other, _act_of(uu[0], mods), uu[0]
        if not act:
            continue
        name = "orion_bn_%d" % n_fused
        n_fused += 1
        gm.add_module(name, FusedBNAct(bn, act))
        with g.inserting_before(act_node):
            new = g.call_module(name, (node.args[0],) if res is None else (node.args[0], res))
        act_node.replace_all_uses_with(new)
        for dead in (act_node, add_node, node):
            if dead is not None and len(dead.users) == 0:
                g.erase_node(dead)
    g.lint()
    gm.delete_all_unused_submodules()
    gm.recompile()
    gm.train()
    return gm


class PlannedModel(nn.Module):
    """A prepared model whose whole forward pass is one call into the adapter (`orion::plan_run`): the layers are
    launched from C++ in order, so the interpreter is entered once per request, not once per layer."""

    def __init__(self, gm, plan_id):
        super().__init__()
        self.gm = gm          # keeps the parameters / buffers of the plan alive; also the per-layer path
        self.plan_id = plan_id

    def forward(self, x):
        return torch.ops.orion.plan_run(self.plan_id, x)


def _build_plan(gm):
    """Flatten a prepared GraphModule into an adapter-side plan; returns the plan id, or None when the graph has a
    node the plan executor does not know (the per-layer GraphModule is used then)."""
    ops = torch.ops.orion
    mods = dict(gm.named_modules())
    nodes = list(gm.graph.nodes)
    placeholders = [n for n in nodes if n.op == "placeholder"]
    outputs = [n for n in nodes if n.op == "output"]
    if len(placeholders) != 1 or len(outputs) != 1 or not isinstance(outputs[0].args[0], fx.Node):
        return None
    slot = {placeholders[0]: 0}
    steps = []

    def new_slot(node):
        slot[node] = len(slot)
        return slot[node]

    for node in nodes:
        if node.op in ("placeholder", "output"):
            continue
        args = [a for a in node.args if isinstance(a, fx.Node)]
        if not args or any(a not in slot for a in args) or node.kwargs and any(isinstance(v, fx.Node) for v in node.kwargs.values()):
            return None
        src = slot[args[0]]
        if node.op == "call_module":
            m = mods.get(node.target)
            if isinstance(m, FusedConv):
                res = slot[args[1]] if len(args) > 1 else -1
                steps.append((1 if m.depthwise else 0, src, res, new_slot(node), m.weight, m.scale, m.shift, m.act, m.stride, m.padding,
                              m.dilation))
            elif isinstance(m, OrionMaxPool):
                steps.append((2, src, -1, new_slot(node), None, None, None, 0, [m.stride], [m.pad], [m.k]))
            elif isinstance(m, OrionAvgPool):
                steps.append((3, src, -1, new_slot(node), None, None, None, 0, [], [], []))
            elif isinstance(m, OrionLinear):
                steps.append((4, src, -1, new_slot(node), m.weight, None, m.bias, 0, [], [], []))
            elif isinstance(m, (nn.Dropout, nn.Identity)):
                steps.append((7, src, -1, new_slot(node), None, None, None, 0, [], [], []))
            else:
                return None
        elif node.op == "call_function" and node.target in (torch.flatten,) and (len(node.args) < 2 or node.args[1] == 1):
            steps.append((6, src, -1, new_slot(node), None, None, None, 0, [], [], []))
        elif node.op == "call_function" and node.target is F.adaptive_avg_pool2d and tuple(
                node.args[1] if isinstance(node.args[1], (tuple, list)) else (node.args[1],) * 2) == (1, 1):
            steps.append((3, src, -1, new_slot(node), None, None, None, 0, [], [], []))
        elif node.op == "call_function" and node.target in (operator.add, operator.iadd, torch.add) and len(args) == 2 and not node.kwargs:
            steps.append((5, src, slot[args[1]], new_slot(node), None, None, None, 0, [], [], []))
        else:
            return None
    plan = ops.plan_create(len(slot), slot[outputs[0].args[0]])
    for (kind, src, res, dst, w, scale, shift, act, stride, pad, dil) in steps:
        ops.plan_add(plan, kind, src, res, dst, w, scale, shift, act, list(stride), list(pad), list(dil))
    return plan


def prepare_inference(model, plan=True):
    """Return an eval-mode copy of `model` (torchvision-style CNN, on its CUDA device,
    float32) whose conv/bn/add/relu groups, pooling layers and classifier run on the
    orion kernels.  With `plan` (default) the result runs its whole forward pass from one adapter call
    where every layer is one the adapter knows; otherwise, and for other graphs, layer by layer."""
    load()
    model = model.eval()
    with TRACE_LOCK:
        gm = fx.symbolic_trace(model)
    mods = dict(gm.named_modules())
    g = gm.graph
    counter = [0]

    def add_module(m):
        name = "orion_%d" % counter[0]
        counter[0] += 1
        gm.add_module(name, m)
        return name

    for node in list(g.nodes):
        if node.op != "call_module":
            continue
        m = mods.get(node.target)
        depthwise = isinstance(m, nn.Conv2d) and m.groups > 1 and m.groups == m.in_channels == m.out_channels and \
            m.groups % 4 == 0 and m.weight.dtype == torch.float32
        if isinstance(m, nn.Conv2d) and (m.groups == 1 or depthwise) and m.padding_mode == "zeros" and isinstance(m.padding, tuple):
            bn_node, bn = None, None
            users = list(node.users)
            if len(users) == 1 and users[0].op == "call_module" and isinstance(mods.get(users[0].target), nn.BatchNorm2d) \
                    and mods[users[0].target].running_mean is not None and mods[users[0].target].running_var is not None:
                bn_node, bn = users[0], mods[users[0].target]   # a batch norm without running statistics stays unfused
            last = bn_node or node
            act, act_node, res, add_node = 0, None, None, None
            users = list(last.users)
            if len(users) == 1:
                u = users[0]
                a = _act_of(u, mods)
                if a:
                    act, act_node = a, u
                elif u.op == "call_function" and u.target in (operator.add, operator.iadd, torch.add) and len(u.args) == 2 \
                        and not u.kwargs and all(isinstance(x, fx.Node) for x in u.args):
                    other = u.args[1] if u.args[0] is last else u.args[0]
                    if other is not last and not depthwise:
                        add_node, res = u, other
                        uu = list(u.users)
                        if len(uu) == 1 and _act_of(uu[0], mods):
                            act, act_node = _act_of(uu[0], mods), uu[0]
            fused = FusedConv(m, bn, act)
            name = add_module(fused)
            anchor = act_node or add_node or last
            with g.inserting_before(anchor):
                new = g.call_module(name, (node.args[0],) if res is None else (node.args[0], res))
            anchor.replace_all_uses_with(new)
            for dead in (act_node, add_node, bn_node, node):
                if dead is not None and len(dead.users) == 0:
                    g.erase_node(dead)
        elif isinstance(m, nn.MaxPool2d) and not m.ceil_mode and _one(m.dilation) == 1 and not m.return_indices and \
                _square(m.kernel_size) and _square(m.stride or m.kernel_size) and _square(m.padding) and _square(m.dilation):
            name = add_module(OrionMaxPool(_one(m.kernel_size), _one(m.stride or m.kernel_size), _one(m.padding)))
            with g.inserting_before(node):
                new = g.call_module(name, node.args)
            node.replace_all_uses_with(new)
            g.erase_node(node)
        elif isinstance(m, nn.AdaptiveAvgPool2d) and _one(m.output_size) == 1:
            name = add_module(OrionAvgPool())
            with g.inserting_before(node):
                new = g.call_module(name, node.args)
            node.replace_all_uses_with(new)
            g.erase_node(node)
        elif isinstance(m, nn.Linear):
            name = add_module(OrionLinear(m))
            with g.inserting_before(node):
                new = g.call_module(name, node.args)
            node.replace_all_uses_with(new)
            g.erase_node(node)
    g.lint()
    gm.delete_all_unused_submodules()
    gm.recompile()
    if plan and os.environ.get("ORION_PLAN", "1") == "1":
        plan_id = _build_plan(gm)
        if plan_id is not None:
            return PlannedModel(gm, plan_id)
    return gm
