"""Launcher: same command line and JSON client list as the reference's
benchmarking/launch_jobs.py:44-148.

    LD_PRELOAD=orion_b200/lib/liborion_capture.so \
    python benchmarking/launch_jobs.py --algo orion --config_file cfg.json --orion_max_be_duration 160000

JSON: a list of client dicts {arch, kernel_file, [additional_kernel_file], num_kernels,
[additional_num_kernels], num_iters, args{model_name, batchsize, rps, uniform, dummy_data,
train, [input_file]}}; the high-priority client is the last entry (reference
src/scheduler/scheduler_eval.cpp:256).  One Python thread per client plus one
scheduler thread, all in this process.  Kernel-file paths may be relative to the
config file.  The libraries are found inside this repository unless ORION_HOME
points elsewhere.
"""
import argparse
import json
import os
import sys
import threading
from ctypes import cdll

_ROOT = os.environ.get("ORION_HOME") or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

import torch  # noqa: E402

from benchmarking.benchmark_suite.train_imagenet import imagenet_loop, seed_everything  # noqa: E402
from src.scheduler_frontend import PyScheduler  # noqa: E402

function_dict = {
    "resnet50": imagenet_loop,
    "resnet101": imagenet_loop,
    "mobilenet_v2": imagenet_loop,
}


def _register_optional_clients():
    # Language-model clients are optional: they are added when their module is present.
    try:
        from benchmarking.benchmark_suite.transformer_trainer import bert_loop, transformer_loop
        function_dict["bert"] = bert_loop
        function_dict["transformer"] = transformer_loop
    except ImportError:
        pass


def scheduler_library():
    path = os.environ.get("ORION_SCHED_LIB") or os.path.join(_ROOT, "orion_b200", "lib", "liborion_sched.so")
    if not os.path.exists(path):
        raise RuntimeError("%s is not built; run `python -m orion_b200.build`" % path)
    return cdll.LoadLibrary(path)


def launch_jobs(config_dict_list, input_args, run_eval, config_dir="."):
    seed_everything(42)
    _register_optional_clients()
    num_clients = len(config_dict_list)
    barriers = [threading.Barrier(num_clients + 1) for _ in range(num_clients)]
    client_barrier = threading.Barrier(num_clients)
    py_scheduler = PyScheduler(scheduler_library(), num_clients)

    def path_of(p):
        return p if p is None or os.path.isabs(p) else os.path.join(config_dir, p)

    model_names = [c["arch"] for c in config_dict_list]
    model_files = [path_of(c["kernel_file"]) for c in config_dict_list]
    additional_model_files = [path_of(c.get("additional_kernel_file")) for c in config_dict_list]
    num_kernels = [c["num_kernels"] for c in config_dict_list]
    additional_num_kernels = [c.get("additional_num_kernels") for c in config_dict_list]
    num_iters = [c["num_iters"] for c in config_dict_list]
    train_list = [c["args"]["train"] for c in config_dict_list]

    def guarded(fn, kwargs):
        # A client that dies would leave the others waiting at a barrier for ever: end the run instead.
        try:
            fn(**kwargs)
        except BaseException:
            import traceback
            traceback.print_exc()
            sys.stderr.write("orion: a client thread failed; aborting the run\n")
            sys.stderr.flush()
            py_scheduler.shutdown()
            os._exit(3)

    threads, tids = [], []
    for i, c in enumerate(config_dict_list):
        if c["arch"] not in function_dict:
            raise ValueError("unknown client arch %r (have %s)" % (c["arch"], sorted(function_dict)))
        kwargs = dict(c["args"])
        kwargs.update({"num_iters": num_iters[i], "local_rank": 0, "barriers": barriers, "client_barrier": client_barrier,
                       "tid": i})
        t = threading.Thread(target=guarded, args=(function_dict[c["arch"]], kwargs))
        t.start()
        tids.append(t.native_id)
        threads.append(t)

    reef = input_args.algo == "reef"
    sched_thread = threading.Thread(target=py_scheduler.run_scheduler, args=(
        barriers, tids, model_names, model_files, additional_model_files, num_kernels, additional_num_kernels, num_iters,
        True, run_eval, reef, input_args.algo == "sequential",
        input_args.reef_depth if reef else input_args.orion_max_be_duration, input_args.orion_hp_limit,
        input_args.orion_start_update, train_list))
    sched_thread.start()
    for t in threads:
        t.join()
    sched_thread.join()
    out_dir = os.environ.get("ORION_OUT_DIR", ".")
    info = {"stats": py_scheduler.stats(), "total_time": py_scheduler.total_time,
            "hp_latency_ms_scheduler_side": py_scheduler.durations_ms(num_clients - 1)[-5000:]}
    try:   # launches of the orion kernels made through the PyTorch adapter in this process
        info["own_launches"] = int(torch.ops.orion.own_launches())
        info["fallbacks"] = int(torch.ops.orion.fallbacks())
    except (AttributeError, RuntimeError):
        pass
    with open(os.path.join(out_dir, "scheduler.json"), "w") as f:
        json.dump(info, f)
    return py_scheduler


def main(argv=None):
    parser = argparse.ArgumentParser()
    parser.add_argument("--algo", type=str, required=True, help="choose one of orion | reef | sequential")
    parser.add_argument("--config_file", type=str, required=True, help="path to the experiment configuration file")
    parser.add_argument("--reef_depth", type=int, default=1, help="If reef is used, this stands for the queue depth")
    parser.add_argument("--orion_max_be_duration", type=int, default=1,
                        help="If orion is used, the maximum aggregate duration of on-the-fly best-effort kernels")
    parser.add_argument("--orion_start_update", type=int, default=1,
                        help="If orion is used, and the high priority job is training, this is the kernel id after which the update phase starts")
    parser.add_argument("--orion_hp_limit", type=int, default=1,
                        help="If orion is used, and the high priority job is training, this shows the maximum tolerated training iteration time")
    args = parser.parse_args(argv)
    if args.algo not in ("orion", "reef", "sequential"):
        parser.error("--algo must be orion, reef or sequential")
    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get("ORION_DEVICE", "0")))
    with open(args.config_file) as f:
        config = json.load(f)
    launch_jobs(config, args, True, os.path.dirname(os.path.abspath(args.config_file)))


if __name__ == "__main__":
    main()
