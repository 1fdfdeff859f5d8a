"""In-tree build of the native parts: the sm_100a kernel library, the scheduler and
capture libraries, and the trace-replay tool.

    python -m orion_b200.build            # build what is stale
    python -m orion_b200.build --force

Outputs (git-ignored): orion_b200/lib/*.so and orion_b200/bin/*.  nvcc
cross-compiles sm_100a without a GPU, so this also runs on a CPU-only machine.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
BIN = os.path.join(HERE, "bin")
ROOT = os.path.dirname(HERE)

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--cudart", "shared"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _site_include(pkg):
    try:
        mod = __import__("nvidia." + pkg, fromlist=["__path__"])
        return os.path.join(list(mod.__path__)[0], "include")
    except Exception:
        return None


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("build step failed: %s\n%s\n%s" % (" ".join(cmd), res.stdout[-4000:], res.stderr[-4000:]))


def _glob(sub, exts):
    d = os.path.join(CSRC, sub)
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(exts))


def build_kernels(force=False):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    srcs = _glob("kernels", (".cu",))
    deps = srcs + _glob("kernels", (".h", ".cuh"))
    out = os.path.join(LIB, "liborion_kernels.so")
    if force or _stale(out, deps):
        os.makedirs(LIB, exist_ok=True)
        _run([nvcc] + NVCC_FLAGS + ["-shared", "-o", out] + srcs)
    return out


def build_host(force=False):
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(BIN, exist_ok=True)
    outs = []
    policy_hdrs = _glob("policy", (".h", ".hpp"))
    replay = os.path.join(BIN, "orion_replay")
    src = os.path.join(CSRC, "sched", "replay_main.cpp")
    if force or _stale(replay, [src] + policy_hdrs):
        _run(["g++"] + CXX_FLAGS + [src, "-o", replay])
    outs.append(replay)
    cuda_inc = "/usr/local/cuda/include"
    incs = ["-I" + cuda_inc]
    for pkg in ("cudnn", "cublas"):
        inc = _site_include(pkg)
        if inc:
            incs.append("-I" + inc)
    capture_src = _glob("capture", (".cpp",))
    capture_hdr = _glob("capture", (".h", ".hpp"))
    if capture_src:
        out = os.path.join(LIB, "liborion_capture.so")
        if force or _stale(out, capture_src + capture_hdr + policy_hdrs):
            _run(["g++"] + CXX_FLAGS + ["-shared", "-o", out] + capture_src + incs + ["-ldl"])
        outs.append(out)
    sched_src = [s for s in _glob("sched", (".cpp",)) if not s.endswith("replay_main.cpp")]
    if sched_src:
        out = os.path.join(LIB, "liborion_sched.so")
        if force or _stale(out, sched_src + _glob("sched", (".h", ".hpp")) + capture_hdr + policy_hdrs):
            _run(["g++"] + CXX_FLAGS + ["-shared", "-o", out] + sched_src + incs + ["-ldl"])
        outs.append(out)
    return outs


def build_glue(force=False):
    """The PyTorch adapter (dispatcher overrides + orion:: ops); links liborion_kernels.so."""
    import torch
    from torch.utils import cpp_extension
    src = os.path.join(CSRC, "torch_glue", "glue.cpp")
    out = os.path.join(LIB, "liborion_torch.so")
    if force or _stale(out, [src]):
        os.makedirs(LIB, exist_ok=True)
        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-w", src, "-o", out,
               "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI), "-I/usr/local/cuda/include"]
        cmd += ["-I" + p for p in cpp_extension.include_paths()]
        cmd += ["-L" + tlib, "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
                "-L" + LIB, "-lorion_kernels", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib]
        _run(cmd)
    return out


def build_all(force=False):
    return [build_kernels(force)] + build_host(force) + [build_glue(force)]


if __name__ == "__main__":
    for path in build_all("--force" in sys.argv):
        print(path)
