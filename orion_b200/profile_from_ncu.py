"""Per-kernel profile file from Nsight Compute exports, by the reference's rules.

The recorder inside the capture library writes the profile files the scheduler reads from a live run.  This module is the other
route the reference offers (reference PROFILE.md:27-54): post-process two ncu exports of one request / iteration —
`output_ncu.csv` (`ncu --csv`, one row per kernel and metric) and `raw_ncu.csv` (the raw page, one row per kernel) — into the
five-column file `Name,Profile,Memory_footprint,SM_usage,Duration`.  It restates the four scripts of the reference:

  * process_ncu.py:14-37        one record per kernel from the long export (a kernel starts at its `DRAM Frequency` row)
  * get_num_blocks.py:27-50     SM need = ceil(grid / blocks per SM), blocks per SM = min over the thread, shared-memory and
                                register limits
  * roofline_analysis.py:36-68  class: with scalar float32 arithmetic, arithmetic intensity against `ai_threshold`; without,
                                1 if compute throughput >= 60 %, else 0 if DRAM throughput >= 60 %, else -1 (unknown)
  * generate_file.py:6-17,41-176  rows: memset / memcpy dropped, cuDNN helper kernels folded into the `Conv` row they precede
                                (largest SM need, summed duration, merged class), `BatchNorm` rows, names cut at the template
                                bracket, `Memory_footprint` always 0

including their quirks (the register limit is always 65 536 whatever is passed; for model type `transformer` every kernel that
reaches the name rules takes the split-K pairing branch and keeps its full name).  Device limits default to a B200's; with the
reference's defaults (`V100`) the output equals the reference scripts' byte for byte (tests/test_profile_csv.py against
tests/golden/ncu_pipeline/).

    python -m orion_b200.profile_from_ncu --results_dir <dir with output_ncu.csv and raw_ncu.csv> --output <file> \\
        [--model_type vision|bert|transformer] [--device b200|v100] [--ai_threshold X]
"""
import argparse
import csv
from math import ceil, floor

DEVICES = {
    # max threads, max blocks (unused by the rule, as in the reference), shared memory bytes per SM
    "v100": dict(max_threads_sm=2048, max_blocks_sm=80, max_shmem_sm=65536, ai_threshold=9.72),    # the reference's defaults
    # B200: 148 SMs x 128 lanes x 2 FLOP x 1.9 GHz = 72 TFLOP/s of scalar float32 (what the rule's instruction counts measure)
    # over the measured 6.54 TB/s copy bandwidth
    "b200": dict(max_threads_sm=2048, max_blocks_sm=32, max_shmem_sm=233472, ai_threshold=11.0),
}

METRICS = ["Duration", "Block Size", "Grid Size", "Compute (SM) [%]", "DRAM Throughput", "Registers Per Thread",
           "Static Shared Memory Per Block"]
FADD = "smsp__sass_thread_inst_executed_op_fadd_pred_on.sum.per_cycle_elapsed [inst/cycle]"
FMUL = "smsp__sass_thread_inst_executed_op_fmul_pred_on.sum.per_cycle_elapsed [inst/cycle]"
FFMA = "smsp__sass_thread_inst_executed_op_ffma_pred_on.sum.per_cycle_elapsed [inst/cycle]"
CYCLES = "smsp__cycles_elapsed.avg.per_second [cycle/nsecond]"
BYTES = "dram__bytes.sum.per_second [Gbyte/second]"


def _num(v):
    return float(str(v).replace(",", "").replace("'", ""))


def process_ncu(long_csv):
    """[{name, dram, duration, compute, block, grid, regs, shmem}] in launch order (process_ncu.py: metrics are taken in the
    order ncu lists them: DRAM Throughput, Duration, Compute (SM) [%], Block Size, Grid Size, Registers Per Thread, Static
    Shared Memory Per Block)."""
    kernels = []
    with open(long_csv, newline="") as f:
        for row in csv.DictReader(f):
            metric = row["Metric Name"]
            if metric == "DRAM Frequency":
                kernels.append([row["Kernel Name"]])
            elif metric in METRICS and kernels:
                kernels[-1].append(_num(row["Metric Value"]))
    out = []
    for k in kernels:
        if len(k) != 8:
            raise ValueError("kernel %r: expected 7 metrics after 'DRAM Frequency', found %d" % (k[0][:60], len(k) - 1))
        out.append(dict(name=k[0], dram=k[1], duration=k[2], compute=k[3], block=k[4], grid=k[5], regs=k[6], shmem=k[7]))
    return out


def sm_needed(k, max_threads_sm, max_shmem_sm):
    """get_num_blocks.py:27-50."""
    by_threads = ceil(max_threads_sm / k["block"])
    by_shmem = ceil(max_shmem_sm / k["shmem"]) if k["shmem"] > 0 else by_threads
    regs_per_warp = ceil(32 * k["regs"] / 256) * 256
    warps_per_sm = floor((65536 / regs_per_warp) / 4) * 4
    by_regs = int(warps_per_sm / ceil(k["block"] / 32))
    return ceil(k["grid"] / min(by_threads, by_shmem, by_regs))


def roofline_class(k, raw, ai_threshold):
    """roofline_analysis.py:36-68; `raw` is the kernel's row of the raw export."""
    add, mul, fma = _num(raw[FADD]), _num(raw[FMUL]), _num(raw[FFMA])
    if add or mul or fma:
        ai = (add + mul + fma * 2) * _num(raw[CYCLES]) / _num(raw[BYTES])
        return 1 if ai > ai_threshold else 0
    if k["compute"] >= 60.0:
        return 1
    if k["dram"] >= 60.0:
        return 0
    return -1


def _merge(classes, main):
    """generate_file.py:6-17."""
    s = set(classes)
    s.discard(-1)
    if not s:
        return -1
    if s == {0}:
        return 0
    if s == {1}:
        return 1
    return main


CONV_KERNELS = ("scudnn", "implicit_convolve_sgemm", "explicit_convolve_sgemm", "dgrad_engine", "wgrad_alg0_engine",
                "wgrad_alg1_engine_NHWC", "dgrad2d_alg1_1", "wgrad2d_grouped_direct_kernel", "dgrad2d_grouped_direct_kernel",
                "conv2d_grouped_direct_kernel", "convolve_common_engine_float_NHWC", "cutlass_cudnn::Kernel",
                "xmma_cudnn::gemm::kernel")
CONV_HELPERS = ("cudnn::winograd", "cudnn::gemm", "computeOffsetsKernel", "scalePackedTensor_kernel", "fft", "nchwToNhwcKernel",
                "nhwcToNchwKernel", "nhwcToFoldedNhwcKernel", "foldedNhwcToNhwcKernel", "nhwcAddPaddingKernel", "im2col4d_kernel")


def generate_rows(kernels, model_type):
    """generate_file.py:41-176.  `kernels`: dicts with name, cls, sm, duration."""
    rows, pending = [], []

    def close_conv(k):
        pending.append((k["sm"], k["duration"], k["cls"]))
        rows.append(["Conv", _merge([p[2] for p in pending], k["cls"]), 0, max(p[0] for p in pending), sum(p[1] for p in pending)])
        pending.clear()

    for i, k in enumerate(kernels):
        x = k["name"]
        if "memset" in x or "memcpy" in x:
            continue
        x = x.replace("<unnamed>", "(anonymous namespace)")
        if "cudnn" in x and "LSTM" not in x:
            if "bn_fw" in x or "bn_bw" in x:
                rows.append(["BatchNorm", k["cls"], 0, k["sm"], k["duration"]])
            elif any(s in x for s in CONV_KERNELS):
                close_conv(k)
            elif any(s in x for s in CONV_HELPERS):
                pending.append((k["sm"], k["duration"], k["cls"]))
            else:
                rows.append([x, k["cls"], 0, k["sm"], k["duration"]])
        elif "sm80_xmma" in x or "implicit_convolve_sgemm" in x:
            close_conv(k)
        elif model_type == "vision" and ("volta_sgemm_128x64_nn" in x or "volta_sgemm_128x64_nt" in x):
            rows.append(["Conv", k["cls"], 0, k["sm"], k["duration"]])
        elif "volta_gcgemm_32x32_nt" in x:
            raise NotImplementedError("volta_gcgemm_32x32_nt rows need the nsys grid columns the reference reads for them")
        elif "splitKreduce_kernel" in x:
            continue   # part of a cuBLAS product
        elif model_type == "transformer":
            # the reference's test `'volta_sgemm_32x128_tn' in x or 'ampere_sgemm_32x128_tn'` is always true: every remaining
            # kernel is paired with a split-K reduce kernel that follows it and keeps its full name
            sm, dur, cls = k["sm"], k["duration"], k["cls"]
            if i < len(kernels) - 1 and "splitKreduce_kernel" in kernels[i + 1]["name"]:
                nxt = kernels[i + 1]
                sm = max(sm, nxt["sm"])
                dur += nxt["duration"]
                cls = _merge([cls, nxt["cls"]], cls)
            rows.append([x, cls, 0, sm, dur])
        else:
            rows.append([x.split("<")[0], k["cls"], 0, k["sm"], k["duration"]])
    return rows


def convert(results_dir, output, model_type="vision", device="b200", ai_threshold=None, max_threads_sm=None, max_shmem_sm=None):
    lim = dict(DEVICES[device])
    if ai_threshold is not None:
        lim["ai_threshold"] = ai_threshold
    if max_threads_sm is not None:
        lim["max_threads_sm"] = max_threads_sm
    if max_shmem_sm is not None:
        lim["max_shmem_sm"] = max_shmem_sm
    kernels = process_ncu(results_dir + "/output_ncu.csv")
    with open(results_dir + "/raw_ncu.csv", newline="") as f:
        raw = list(csv.DictReader(f))
    if len(raw) != len(kernels):
        raise ValueError("output_ncu.csv holds %d kernels, raw_ncu.csv %d" % (len(kernels), len(raw)))
    for k, r in zip(kernels, raw):
        k["sm"] = sm_needed(k, lim["max_threads_sm"], lim["max_shmem_sm"])
        k["cls"] = roofline_class(k, r, lim["ai_threshold"])
    rows = generate_rows(kernels, model_type)
    with open(output, "w") as f:
        f.write("Name,Profile,Memory_footprint,SM_usage,Duration\n")
        for r in rows:
            f.write(",".join(str(v) for v in r) + "\n")
    return len(rows)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--results_dir", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--model_type", default="vision", choices=["vision", "bert", "transformer"])
    ap.add_argument("--device", default="b200", choices=sorted(DEVICES))
    ap.add_argument("--ai_threshold", type=float, default=None)
    a = ap.parse_args()
    n = convert(a.results_dir, a.output, a.model_type, a.device, a.ai_threshold)
    print("%d rows -> %s (num_kernels of the client entry = the row count)" % (n, a.output))


if __name__ == "__main__":
    main()
