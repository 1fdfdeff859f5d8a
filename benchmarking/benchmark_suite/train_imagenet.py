"""Vision client loop: same entry point, arguments and output file as the reference's
benchmarking/benchmark_suite/train_imagenet.py:71-241 (`imagenet_loop`).

Request process (reference :172-204): an inference client is open-loop — request i
may start no earlier than the previous start plus sleep_times[i] (exponential for
Poisson arrivals, constant for `uniform`, or read from `input_file`), the first ten
requests run back to back as warm-up, and a request's latency is counted from its
scheduled start, so queueing delay is included.  `rps == 0` means closed loop.  A
training client runs iterations back to back until the scheduler tells it to stop.
After every request the client calls `block(i)` of the capture library, which
returns when the scheduler has seen the request's last kernel complete.

What differs from the reference script, on purpose:
  * the client runs under the CUDA stream the scheduler created for it (stock torch
    keeps one allocator pool per stream, which replaces the reference's patched
    per-thread allocator);
  * synthetic data follows the benchmark configuration: N(0,1) images, labels
    uniform in [0, 1000), SGD with momentum 0.9 (`ORION_CLIENT_REFERENCE_DATA=1`
    restores the reference's uniform images / all-one labels / plain SGD);
  * inference models are prepared with orion_b200.torch_ops.prepare_inference
    (`ORION_PREPARE=0` leaves the model untouched: its convolutions and batch norms
    still reach the orion kernels through the dispatcher overrides);
  * each request reads its result back to the host (`ORION_READBACK=0` disables).

`run_client` holds the loop; `imagenet_loop` only says how to build the model and what one
request does, and so do the language-model clients in transformer_trainer.py.
"""
import json
import os
import random
import threading
import time
from ctypes import cdll, c_bool, c_void_p

import numpy as np
import torch
from torchvision import models

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def seed_everything(seed):
    random.seed(seed)
    os.environ["PYTHONHASHSEED"] = str(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)


def capture_library():
    path = os.environ.get("ORION_CAPTURE_LIB") or os.path.join(_ROOT, "orion_b200", "lib", "liborion_capture.so")
    lib = cdll.LoadLibrary(path)
    lib.stop.restype = c_bool
    lib.orion_capture_client_stream.restype = c_void_p
    return lib


class DummyDataLoader:
    """Endless stream of one pinned synthetic batch (reference :33-43)."""

    def __init__(self, batchsize, reference_data=False):
        pin = torch.cuda.is_available()
        if reference_data:
            self.data = torch.rand([batchsize, 3, 224, 224])
            self.target = torch.ones([batchsize], dtype=torch.long)
        else:
            self.data = torch.randn([batchsize, 3, 224, 224])
            self.target = torch.randint(0, 1000, [batchsize], dtype=torch.long)
        # channels-last on the host already, so the host-to-device copy lands in the kernels' layout
        self.data = self.data.contiguous(memory_format=torch.channels_last)
        if pin:
            self.data = self.data.pin_memory()
            self.target = self.target.pin_memory()

    def __iter__(self):
        return self

    def __next__(self):
        return self.data, self.target


def _sleep_times(rps, uniform, num_iters, input_file):
    if rps > 0 and input_file == "":
        return [1.0 / rps] * num_iters if uniform else list(np.random.exponential(scale=1.0 / rps, size=num_iters))
    if input_file != "":
        with open(input_file) as f:
            return json.load(f)
    return [0.0] * num_iters


def run_client(tid, train, num_iters, rps, uniform, barriers, input_file, batchsize, build):
    """The request loop shared by every client kind.  `build(device)` creates the model on the
    current CUDA stream and returns `step(batch_idx)`, which issues one request / training
    iteration (including the host-to-device copy of its inputs) and returns a device tensor
    that is read back to the host after the request completed."""
    import contextlib
    seed_everything(42)
    backend_lib = capture_library()
    sleep_times = _sleep_times(rps, uniform, num_iters, input_file)
    readback = os.environ.get("ORION_READBACK", "1") == "1"
    out_dir = os.environ.get("ORION_OUT_DIR", ".")
    # Requests left out of the latency statistics: the protocol's ten warm-up requests plus any further
    # untimed ones the experiment asks for (ORION_EXTRA_WARMUP_REQUESTS).
    skip = 10 + max(0, int(os.environ.get("ORION_EXTRA_WARMUP_REQUESTS", "0")))

    barriers[0].wait()   # the scheduler has run setup(): streams exist, this thread is registered

    stream_ptr = backend_lib.orion_capture_client_stream(tid)
    stream = torch.cuda.ExternalStream(stream_ptr) if stream_ptr else torch.cuda.current_stream()
    timings = []
    end_times = []   # wall-clock time at which each request / iteration completed
    start = time.time()
    batch_idx = 0
    with torch.cuda.stream(stream):
        from orion_b200 import torch_ops
        torch_ops.load()
        quota = int(os.environ.get("ORION_BE_SM_QUOTA", "0")) if train else 0
        if quota > 0:
            torch_ops.set_sm_quota(quota)
        if train and os.environ.get("ORION_DISABLE_OVERRIDES", "0") == "1":
            torch_ops.set_overrides(False)   # training client on the stock cuDNN / ATen kernels (still captured and scheduled)
        if train and os.environ.get("ORION_TRAIN_TF32", "0") == "1":
            torch.ops.orion.set_tf32(1)   # training convolutions in one TF32 pass, like stock cuDNN's default
        with torch_ops.TRACE_LOCK:
            step = build(torch.device("cuda", torch.cuda.current_device()))
        result = None
        next_startup = time.time()
        open_loop = rps > 0 or input_file != ""
        while batch_idx < num_iters:
            if train:
                start_iter = time.time()
                # iteration 0 overlaps with other clients preparing their models (see TRACE_LOCK)
                with (torch_ops.TRACE_LOCK if batch_idx == 0 else contextlib.nullcontext()):
                    result = step(batch_idx)
                backend_lib.block(batch_idx)
                if readback and result is not None:
                    result = float(result.detach())
                end_times.append(time.time())
                timings.append(end_times[-1] - start_iter)
                batch_idx += 1
                if batch_idx == 1 or batch_idx == 10:
                    barriers[0].wait()
                    if batch_idx == 10:
                        start = time.time()
                if backend_lib.stop():
                    break
            else:
                with torch.no_grad():
                    if open_loop and time.time() < next_startup:
                        wait = next_startup - time.time()
                        if wait > 2e-4:
                            time.sleep(wait - 1e-4)
                        continue
                    with (torch_ops.TRACE_LOCK if batch_idx == 0 else contextlib.nullcontext()):
                        result = step(batch_idx)
                    backend_lib.block(batch_idx)
                    if readback and result is not None:
                        result = result.cpu()   # a plain device-to-host copy: no extra kernel in the op stream
                    end_times.append(time.time())
                    timings.append(end_times[-1] - next_startup)
                    if batch_idx >= 10 and open_loop:
                        next_startup += sleep_times[batch_idx]
                    else:
                        next_startup = time.time()
                    batch_idx += 1
                    if batch_idx == 1 or batch_idx == 10:
                        barriers[0].wait()
                        if batch_idx == 10:
                            next_startup = time.time()
                            start = time.time()
                    if backend_lib.stop():
                        break

    barriers[0].wait()
    total_time = time.time() - start
    measured = sorted(timings[skip:])
    data_out = {"throughput": (batch_idx - 10) / total_time if total_time > 0 else 0.0, "iterations": batch_idx,
                "batchsize": batchsize, "total_time": total_time}
    if not train and measured:
        # the measured window opens when the last untimed request completed
        data_out.update({"measured_requests": len(measured), "measure_start_time": end_times[skip - 1],
                         "measure_end_time": end_times[-1],
                         "latencies_ms": [round(t * 1000, 4) for t in timings[skip:]],
                         "p50_latency": float(np.percentile(measured, 50)) * 1000,
                         "p95_latency": float(np.percentile(measured, 95)) * 1000,
                         "p99_latency": float(np.percentile(measured, 99)) * 1000,
                         "mean_latency": float(np.mean(measured)) * 1000})
    elif train and timings[10:]:
        data_out["samples_per_s"] = data_out["throughput"] * batchsize
        data_out["iteration_end_times"] = end_times
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "client_%d.json" % tid), "w") as f:
        json.dump(data_out, f)


def imagenet_loop(model_name, batchsize, train, num_iters, rps, uniform, dummy_data, local_rank, barriers, client_barrier, tid,
                  input_file=""):
    if not dummy_data:
        raise NotImplementedError("only synthetic data is available (dummy_data=true)")
    reference_data = os.environ.get("ORION_CLIENT_REFERENCE_DATA", "0") == "1"
    resident = os.environ.get("ORION_RESIDENT_INPUTS", "0") == "1"

    def build(device):
        from orion_b200 import torch_ops
        model = models.__dict__[model_name](num_classes=1000)
        model = model.to(device).to(memory_format=torch.channels_last)
        loader = DummyDataLoader(batchsize, reference_data)
        data, target = next(loader)
        state = {"x": data.to(device, non_blocking=True), "t": target.to(device, non_blocking=True)}
        if train:
            model.train()
            if os.environ.get("ORION_PREPARE", "1") == "1" and os.environ.get("ORION_DISABLE_OVERRIDES", "0") != "1":
                model = torch_ops.prepare_training(model)   # batch norm + residual + ReLU groups as one op each
            momentum = 0.0 if reference_data else 0.9
            lr = 0.05 if (model_name == "mobilenet_v2" and not reference_data) else 0.1
            if os.environ.get("ORION_PREPARE", "1") == "1" and os.environ.get("ORION_DISABLE_OVERRIDES", "0") != "1":
                from orion_b200.optim import SGD   # the whole update in one or two launches
                optimizer = SGD(model.parameters(), lr=lr, momentum=momentum)
            else:
                optimizer = torch.optim.SGD(model.parameters(), lr=lr, momentum=momentum)
            criterion = torch.nn.CrossEntropyLoss().to(device)

            def step(batch_idx):
                if not resident:
                    state["x"] = data.to(device, non_blocking=True)
                    state["t"] = target.to(device, non_blocking=True)
                optimizer.zero_grad()
                loss = criterion(model(state["x"]), state["t"])
                loss.backward()
                optimizer.step()
                return loss
            return step
        model.eval()
        if os.environ.get("ORION_PREPARE", "1") == "1":
            model = torch_ops.prepare_inference(model)

        def step(batch_idx):
            if not resident:
                state["x"] = data.to(device, non_blocking=True)
            return model(state["x"])
        return step

    run_client(tid, train, num_iters, rps, uniform, barriers, input_file, batchsize, build)
