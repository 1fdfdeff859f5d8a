"""Pins the reference's profile post-processing (ncu output -> benchmarking/model_kernels file) on synthetic inputs.

The reference turns Nsight Compute output into a per-kernel profile in four scripts (reference PROFILE.md:27-54):
profiling/postprocessing/process_ncu.py, get_num_blocks.py, roofline_analysis.py, generate_file.py.  This script writes two
small synthetic ncu exports (the long `output_ncu.csv` and the wide `raw_ncu.csv`) whose kernels exercise every rule the
scripts have — SM need from threads / shared memory / registers, class from arithmetic intensity or from the 60 % throughput
marks or unknown, grouping of cuDNN helper kernels into one Conv row, BatchNorm rows, names cut at the template bracket, memset /
memcpy / split-K reduce rows dropped — runs the reference's own four scripts on them, for the three model types, and stores
inputs and outputs under tests/golden/ncu_pipeline/.  `tests/test_profile_csv.py` checks that orion_b200/profile_from_ncu.py
produces the same files from the same inputs.

    python tests/golden/make_profile_pipeline_golden.py      # needs the reference checkout (default /root/reference)
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "ncu_pipeline")
REF = os.environ.get("ORION_REFERENCE", "/root/reference")
PP = os.path.join(REF, "profiling", "postprocessing")

FADD = "smsp__sass_thread_inst_executed_op_fadd_pred_on.sum.per_cycle_elapsed [inst/cycle]"
FMUL = "smsp__sass_thread_inst_executed_op_fmul_pred_on.sum.per_cycle_elapsed [inst/cycle]"
FFMA = "smsp__sass_thread_inst_executed_op_ffma_pred_on.sum.per_cycle_elapsed [inst/cycle]"
CYC = "smsp__cycles_elapsed.avg.per_second [cycle/nsecond]"
BYT = "dram__bytes.sum.per_second [Gbyte/second]"

# name, dram %, duration ns, compute %, block, grid, regs/thread, static shmem, fadd, fmul, ffma, cycles/ns, GB/s
KERNELS = [
    ("void at::native::vectorized_elementwise_kernel<4, at::native::CUDAFunctor_add<float>, at::detail::Array<char*, 3> >(int, at::native::CUDAFunctor_add<float>, at::detail::Array<char*, 3>)",
     71.2, 5408, 12.5, 128, 6272, 16, 0, "0.52", "0", "0", 1.38, 612.4),
    ("void cudnn::winograd_nonfused::winogradForwardData4x4<float, float>(cudnn::winograd_nonfused::WinogradDataParams<float, float>)",
     40.1, 9120, 33.0, 256, 1024, 40, 0, "0", "0.1", "3.9", 1.38, 301.0),
    ("void cudnn::winograd_nonfused::winogradForwardFilter4x4<float, float>(cudnn::winograd_nonfused::WinogradFilterParams<float, float>)",
     12.0, 2048, 8.0, 256, 64, 32, 0, "0", "0", "0", 1.38, 40.0),
    ("volta_scudnn_winograd_128x128_ldg1_ldg4_relu_tile148t_nt_v1", 22.5, 48224, 88.4, 256, 196, 126, 49152, "1.1", "0.3", "102.4", 1.38, 150.2),
    ("void cudnn::bn_fw_tr_1C11_kernel_NCHW<float, float, int, 512, true, 1, true>(cudnnTensorStruct, float const*, cudnnTensorStruct, float*, float const*, float const*, float, float, float*, float*, float*, float*, float, float)",
     80.3, 30112, 20.0, 512, 64, 32, 8192, "2.2", "1.0", "1.1", 1.38, 700.0),
    ("[CUDA memset]", 0.0, 1500, 0.0, 1, 1, 16, 0, "0", "0", "0", 1.38, 1.0),
    ("void at::native::(anonymous namespace)::max_pool_forward_nchw<float, float>(int, float const*, int, int, int, int, int, int, int, int, int, int, int, int, int, int, float*, long*)",
     65.0, 20480, 30.0, 256, 3136, 29, 0, "0", "0", "0", 1.38, 560.0),
    ("void at::native::reduce_kernel<512, 1, at::native::ReduceOp<float, at::native::MeanOps<float, float>, unsigned int, float, 4> >(at::native::ReduceOp<float, at::native::MeanOps<float, float>, unsigned int, float, 4>)",
     10.0, 7008, 61.5, 512, 2048, 32, 16, "0", "0", "0", 1.38, 90.0),
    ("void at::native::elementwise_kernel<128, 2, void at::native::gpu_kernel_impl<at::native::direct_copy_kernel_cuda(at::TensorIteratorBase&)::{lambda()#1}>(at::TensorIteratorBase&, const&)::{lambda(int)#1}>(int, {lambda(int)#1})",
     30.0, 3008, 25.0, 128, 98, 18, 0, "0", "0", "0", 1.38, 260.0),
    ("sm80_xmma_fprop_implicit_gemm_tf32f32_tf32f32_f32_nhwckrsc_nchw_tilesize128x128x16_stage4_warpsize2x2x1_g1_tensor16x8x8_execute_kernel_cudnn",
     35.0, 61440, 72.0, 128, 392, 168, 0, "0", "0", "0", 1.38, 310.0),
    ("volta_sgemm_128x64_nn", 18.0, 15360, 90.1, 128, 64, 120, 12288, "0", "0.2", "55.0", 1.38, 120.0),
    ("void splitKreduce_kernel<float, float, float, float>(cublasSplitKParams<float>, float const*, float const*, float*, float const*, float const*, float const*)",
     50.0, 2560, 10.0, 256, 16, 24, 0, "0.4", "0", "0", 1.38, 400.0),
    ("void cudnn::cnn::im2col4d_kernel<float, long>(cudnn::cnn::im2col4d_params, cudnnConvolutionStruct, cudnnTensor4dStruct, float const*, float*)",
     55.0, 11008, 15.0, 256, 512, 36, 0, "0", "0", "0", 1.38, 480.0),
    ("void implicit_convolve_sgemm<float, float, 128, 5, 5, 3, 3, 3, 1, false, false, true>(int, int, int, float const*, int, float*, float const*, kernel_conv_params, unsigned long long, int, float, float, int, float const*, float const*, bool, int, int)",
     25.0, 40960, 75.0, 64, 1568, 96, 9216, "0.8", "0.5", "70.0", 1.38, 210.0),
    ("void at::native::(anonymous namespace)::softmax_warp_forward<float, float, float, 10, true>(float*, float const*, int, int, int)",
     5.0, 2304, 4.0, 128, 1, 20, 0, "0.05", "0.02", "0.01", 1.38, 30.0),
    ("[CUDA memcpy DtoH]", 0.0, 1800, 0.0, 1, 1, 16, 0, "0", "0", "0", 1.38, 1.0),
]


def write_inputs(d):
    with open(os.path.join(d, "output_ncu.csv"), "w") as f:
        f.write('"ID","Process ID","Process Name","Host Name","Kernel Name","Kernel Time","Context","Stream","Section Name",'
                '"Metric Name","Metric Unit","Metric Value"\n')
        for i, k in enumerate(KERNELS):
            name = k[0].replace('"', '""')
            metrics = [("GPU Speed Of Light Throughput", "DRAM Frequency", "cycle/nsecond", "0.88"),
                       ("GPU Speed Of Light Throughput", "SM Frequency", "cycle/nsecond", "1.38"),
                       ("GPU Speed Of Light Throughput", "Memory [%]", "%", "50.0"),
                       ("GPU Speed Of Light Throughput", "DRAM Throughput", "%", str(k[1])),
                       ("GPU Speed Of Light Throughput", "Duration", "nsecond", str(k[2])),
                       ("GPU Speed Of Light Throughput", "Compute (SM) [%]", "%", str(k[3])),
                       ("Launch Statistics", "Block Size", "", str(k[4])),
                       ("Launch Statistics", "Grid Size", "", str(k[5])),
                       ("Launch Statistics", "Registers Per Thread", "register/thread", str(k[6])),
                       ("Launch Statistics", "Static Shared Memory Per Block", "byte/block", str(k[7])),
                       ("Launch Statistics", "Threads", "thread", str(k[4] * k[5]))]
            for sec, m, u, v in metrics:
                f.write('"%d","4242","python3","127.0.0.1","%s","2022-Jan-01 00:00:00","1","7","%s","%s","%s","%s"\n' % (i, name, sec, m, u, v))
    with open(os.path.join(d, "raw_ncu.csv"), "w") as f:
        f.write('"ID","Kernel Name","%s","%s","%s","%s","%s"\n' % (FADD, FMUL, FFMA, CYC, BYT))
        for i, k in enumerate(KERNELS):
            f.write('"%d","%s","%s","%s","%s","%s","%s"\n' % (i, k[0].replace('"', '""'), k[8], k[9], k[10], k[11], k[12]))


def main():
    if not os.path.isdir(PP):
        sys.exit("reference checkout not found at " + REF)
    os.makedirs(OUT, exist_ok=True)
    d = tempfile.mkdtemp(prefix="orion_ncu_")
    write_inputs(d)
    # The reference's roofline script indexes a name-indexed Series with integers (`comp_throughput[index - startp]`), which the
    # pandas of its time (1.x) answered by position; pandas 3 raises KeyError.  The scripts are run unmodified behind a shim that
    # restores that one behaviour.
    shim = ("import pandas as pd, runpy, sys\n"
            "_orig = pd.Series.__getitem__\n"
            "def _getitem(self, key):\n"
            "    try:\n"
            "        return _orig(self, key)\n"
            "    except KeyError:\n"
            "        if isinstance(key, int):\n"
            "            return self.iloc[key]\n"
            "        raise\n"
            "pd.Series.__getitem__ = _getitem\n"
            "script = sys.argv[1]\n"
            "sys.argv = sys.argv[1:]\n"
            "runpy.run_path(script, run_name='__main__')\n")
    run = lambda *a: subprocess.run([sys.executable, "-c", shim] + list(a), check=True, capture_output=True, text=True)
    run(os.path.join(PP, "process_ncu.py"), "--results_dir", d)
    run(os.path.join(PP, "get_num_blocks.py"), "--results_dir", d)
    run(os.path.join(PP, "roofline_analysis.py"), "--results_dir", d)
    for model_type in ("vision", "bert", "transformer"):
        run(os.path.join(PP, "generate_file.py"), "--input_file_name", os.path.join(d, "output_ncu_sms_roofline.csv"),
            "--output_file_name", os.path.join(d, "model_kernels_" + model_type), "--model_type", model_type)
    for f in ("output_ncu.csv", "raw_ncu.csv", "output_ncu_processed.csv", "output_ncu_sms.csv", "output_ncu_sms_roofline.csv",
              "model_kernels_vision", "model_kernels_bert", "model_kernels_transformer"):
        shutil.copy(os.path.join(d, f), os.path.join(OUT, f))
        print(f, os.path.getsize(os.path.join(OUT, f)), "bytes")
    shutil.rmtree(d, ignore_errors=True)


if __name__ == "__main__":
    main()
