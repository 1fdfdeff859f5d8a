"""Experiment helpers: profile a client, build launch_jobs configurations and run
solo / co-located experiments as child processes under the capture library.

A run is always a child process because the capture library must be preloaded
(LD_PRELOAD) before torch loads the CUDA runtime.
"""
import json
import os
import subprocess
import sys
import threading

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CAPTURE_LIB = os.path.join(ROOT, "orion_b200", "lib", "liborion_capture.so")

# batch size and mode of the clients in the benchmark configurations
CLIENTS = {
    "resnet50_hp": dict(arch="resnet50", batchsize=4, train=False),
    "resnet50_be": dict(arch="resnet50", batchsize=32, train=True),
    "resnet101_hp": dict(arch="resnet101", batchsize=4, train=False),
    "mobilenet_v2_hp": dict(arch="mobilenet_v2", batchsize=4, train=False),
    "mobilenet_v2_be": dict(arch="mobilenet_v2", batchsize=64, train=True),
    "bert_hp": dict(arch="bert", batchsize=8, train=False),
    "bert_be": dict(arch="bert", batchsize=8, train=True),
    "transformer_be": dict(arch="transformer", batchsize=16, train=True),
}


def _child_env(extra=None, preload=True):
    env = dict(os.environ)
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    if preload:
        env["LD_PRELOAD"] = CAPTURE_LIB + ((" " + env["LD_PRELOAD"]) if env.get("LD_PRELOAD") else "")
    if extra:
        env.update({k: str(v) for k, v in extra.items()})
    return env


def client_args(arch, batchsize, train, rps=0, uniform=False):
    args = {"batchsize": batchsize, "rps": rps, "uniform": uniform, "dummy_data": True, "train": train}
    if arch not in ("bert", "transformer"):
        args["model_name"] = arch
    return args


def run_unscheduled(arch, batchsize, train, iters):
    """Body of a profiling child: one client loop without a scheduler."""
    from benchmarking.benchmark_suite.train_imagenet import imagenet_loop
    from benchmarking.benchmark_suite.transformer_trainer import bert_loop, transformer_loop
    loop = {"bert": bert_loop, "transformer": transformer_loop}.get(arch, imagenet_loop)
    barrier = threading.Barrier(1)
    loop(num_iters=iters, local_rank=0, barriers=[barrier], client_barrier=barrier, tid=0, **client_args(arch, batchsize, train))


def profile_client(name, out_dir, iters=12, device=0, timeout=600, extra_env=None):
    """Record `<name>_fb0` (first iteration) and `<name>_fb1` (steady state) profile files
    for one client; returns (path0, rows0, path1, rows1)."""
    c = CLIENTS[name]
    out_dir = os.path.abspath(out_dir)
    os.makedirs(out_dir, exist_ok=True)
    p0 = os.path.join(out_dir, name + "_fb0")
    p1 = os.path.join(out_dir, name + "_fb1")
    env = {"ORION_PROFILE_OUT0": p0, "ORION_PROFILE_OUT": p1, "ORION_PROFILE_ITER": 5, "ORION_OUT_DIR": out_dir,
           "CUDA_VISIBLE_DEVICES": os.environ.get("CUDA_VISIBLE_DEVICES", str(device))}
    env.update(extra_env or {})
    code = "from orion_b200.experiments import run_unscheduled; run_unscheduled(%r, %d, %r, %d)" % (
        c["arch"], c["batchsize"], c["train"], iters)
    res = subprocess.run([sys.executable, "-c", code], env=_child_env(env), capture_output=True, text=True, timeout=timeout,
                         cwd=ROOT)
    if res.returncode != 0 or not os.path.exists(p1):
        raise RuntimeError("profiling %s failed (rc %d):\n%s\n%s" % (name, res.returncode, res.stdout[-3000:], res.stderr[-3000:]))
    return p0, _rows(p0), p1, _rows(p1)


def _rows(path):
    with open(path) as f:
        return max(0, sum(1 for _ in f) - 1)


def client_entry(name, profiles, num_iters, rps=0, uniform=False):
    c = CLIENTS[name]
    p0, n0, p1, n1 = profiles
    return {"arch": c["arch"], "kernel_file": p0, "num_kernels": n0, "additional_kernel_file": p1,
            "additional_num_kernels": n1, "num_iters": num_iters,
            "args": client_args(c["arch"], c["batchsize"], c["train"], rps, uniform)}


def run_launch_jobs(config, out_dir, algo="orion", depth=160000, extra_env=None, timeout=600, reef_depth=12):
    """Run benchmarking/launch_jobs.py on `config` (a list of client entries) in a child
    process; returns {"clients": [client_i.json...], "scheduler": {...}}."""
    out_dir = os.path.abspath(out_dir)
    os.makedirs(out_dir, exist_ok=True)
    cfg_path = os.path.join(out_dir, "config.json")
    with open(cfg_path, "w") as f:
        json.dump(config, f, indent=1)
    for i in range(len(config)):
        p = os.path.join(out_dir, "client_%d.json" % i)
        if os.path.exists(p):
            os.remove(p)
    env = {"ORION_OUT_DIR": out_dir}
    env.update(extra_env or {})
    cmd = [sys.executable, os.path.join(ROOT, "benchmarking", "launch_jobs.py"), "--algo", algo, "--config_file", cfg_path,
           "--orion_max_be_duration", str(int(depth)), "--reef_depth", str(int(reef_depth))]
    log_path = os.path.join(out_dir, "launch.log")
    with open(log_path, "w") as log:
        try:
            rc = subprocess.run(cmd, env=_child_env(env), stdout=log, stderr=subprocess.STDOUT, timeout=timeout, cwd=ROOT).returncode
        except subprocess.TimeoutExpired:
            rc = -999
    if rc != 0:
        with open(log_path) as f:
            tail = f.read()[-3000:]
        raise RuntimeError("launch_jobs failed (rc %d); see %s\n%s" % (rc, log_path, tail))
    out = {"clients": [], "scheduler": None}
    for i in range(len(config)):
        with open(os.path.join(out_dir, "client_%d.json" % i)) as f:
            out["clients"].append(json.load(f))
    sp = os.path.join(out_dir, "scheduler.json")
    if os.path.exists(sp):
        with open(sp) as f:
            out["scheduler"] = json.load(f)
    return out
