// Per-kernel profile recorder: produces files in the benchmarking/model_kernels
// format (`Name,Profile,Memory_footprint,SM_usage,Duration`, one row per scheduled
// compute op in launch order) from an *unscheduled* run of one client under the
// capture library.
//
// It takes the place of the reference's offline pipeline (ncu/nsys CSVs post-processed
// by profiling/postprocessing/*.py) and keeps that pipeline's column definitions:
//   * SM_usage  = ceil(grid blocks / resident blocks per SM), the number of SMs needed
//                 to run all blocks at once (get_num_blocks.py:27-50) — here the
//                 residency comes from the occupancy API instead of V100 tables;
//                 library calls whose launch shape is not visible get the device's
//                 SM count;
//   * Duration  = device time of the op in ns, from an event pair recorded around the op on its
//                 stream.  The pairs of one iteration are read when the iteration ends (block(it)),
//                 so the stream is never drained between two ops: while the device has work queued
//                 the pair brackets the kernel alone; when the host is the slower side (small batches)
//                 it also contains the idle gap until the launch arrives, as a timeline view would
//                 show for that op.  The cost of an empty pair, measured once, is subtracted;
//   * Profile   = 1 compute-bound / 0 memory-bound / -1 unknown.  The reference decides this from
//                 ncu counters: arithmetic intensity against `ai_threshold`, else >= 60 % of the
//                 compute or DRAM throughput (roofline_analysis.py:51-71).  The orion kernels
//                 announce their class themselves (orion_capture_annotate): the launcher knows the
//                 algorithmic FLOP and bytes of the problem and compares their ratio with the
//                 device's measured peak FLOP/s over measured HBM bytes/s.  Only foreign kernels
//                 (stock ATen / cuDNN / cuBLAS launches) are classified by what the op is: GEMM /
//                 convolution calls are compute-bound; batch-norm, elementwise, pooling, reduction
//                 and copy kernels are memory-bound;
//   * memory ops are not rows (generate_file.py:50-52); Memory_footprint is 0.
//
// Use: ORION_PROFILE_OUT=<file> [ORION_PROFILE_OUT0=<file for iteration 0>]
//      [ORION_PROFILE_ITER=<n, default 3>] LD_PRELOAD=liborion_capture.so python client.py
// Iterations are delimited by the client's block(it) calls; iteration 0 is written
// to ORION_PROFILE_OUT0, iteration ORION_PROFILE_ITER to ORION_PROFILE_OUT.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <string>
#include <vector>

#include "capture_core.h"

namespace {

struct Row {
    std::string name;
    int profile;
    int sm;
    float ns;
    int pair;       // index of the event pair that brackets the op
};

struct Annotation {
    bool set = false;
    int op_class = -1;
    double flop = 0, bytes = 0;
};
thread_local Annotation tls_note;

struct Recorder {
    bool enabled = false;
    std::string out, out0;
    int steady_iter = 3;
    int cur_iter = 0;
    std::mutex mu;
    std::vector<Row> rows;
    int sm_count = 0;
    // real runtime entry points
    cudaError_t (*event_create)(cudaEvent_t*) = nullptr;
    cudaError_t (*event_record)(cudaEvent_t, cudaStream_t) = nullptr;
    cudaError_t (*event_sync)(cudaEvent_t) = nullptr;
    cudaError_t (*event_elapsed)(float*, cudaEvent_t, cudaEvent_t) = nullptr;
    cudaError_t (*func_name)(const char**, const void*) = nullptr;
    cudaError_t (*occupancy)(int*, const void*, int, size_t, unsigned) = nullptr;
    cudaError_t (*dev_attr)(int*, cudaDeviceAttr, int) = nullptr;
    std::vector<cudaEvent_t> ev_a, ev_b;   // event pairs, reused by every iteration
    int pairs_used = 0;
    float empty_pair_ms = 0.f;
    bool bound = false;
} R;

void* real_sym(const char* name) {
    void* p = dlsym(RTLD_NEXT, name);
    if (p) return p;
    void* h = dlopen("libcudart.so.12", RTLD_NOW | RTLD_NOLOAD);
    return h ? dlsym(h, name) : nullptr;
}

bool bind() {
    if (R.bound) return R.event_create != nullptr;
    R.bound = true;
    R.event_create = (decltype(R.event_create))real_sym("cudaEventCreate");
    R.event_record = (decltype(R.event_record))real_sym("cudaEventRecord");
    R.event_sync = (decltype(R.event_sync))real_sym("cudaEventSynchronize");
    R.event_elapsed = (decltype(R.event_elapsed))real_sym("cudaEventElapsedTime");
    R.func_name = (decltype(R.func_name))real_sym("cudaFuncGetName");
    R.occupancy = (decltype(R.occupancy))real_sym("cudaOccupancyMaxActiveBlocksPerMultiprocessorWithFlags");
    R.dev_attr = (decltype(R.dev_attr))real_sym("cudaDeviceGetAttribute");
    if (!R.event_create || !R.event_record || !R.event_sync || !R.event_elapsed) {
        R.event_create = nullptr;
        return false;
    }
    {   // device time of an empty pair (two events back to back on an idle stream)
        cudaEvent_t a = nullptr, b = nullptr;
        R.event_create(&a);
        R.event_create(&b);
        float best = 1e9f;
        for (int k = 0; k < 8 && a && b; k++) {
            R.event_record(a, nullptr);
            R.event_record(b, nullptr);
            R.event_sync(b);
            float ms = 0.f;
            if (R.event_elapsed(&ms, a, b) == cudaSuccess && ms < best) best = ms;
        }
        R.empty_pair_ms = best < 1e8f ? best : 0.f;
        R.ev_a.push_back(a);
        R.ev_b.push_back(b);
    }
    if (R.dev_attr) R.dev_attr(&R.sm_count, cudaDevAttrMultiProcessorCount, 0);
    if (R.sm_count <= 0) R.sm_count = 148;
    return true;
}

const char* type_name(int t) {
    switch (t) {
        case ORION_CUDNN_CONV_RECORD: case ORION_CUDNN_CONV_DATA_RECORD: case ORION_CUDNN_CONV_FILTER_RECORD:
        case ORION_CUDNN_BACKEND_EXECUTE_RECORD: return "Conv";
        case ORION_CUDNN_BNORM_RECORD: case ORION_CUDNN_BNORM_INF_RECORD: case ORION_CUDNN_BNORM_BACKWARD_RECORD: return "BatchNorm";
        case ORION_CUBLAS_SGEMM_RECORD: case ORION_CUBLAS_SGEMM_STRIDED_RECORD: case ORION_CUBLAS_GEMMEX_RECORD:
        case ORION_CUBLAS_GEMMEX_STRIDED_RECORD: case ORION_CUBLASLT_MATMUL_RECORD: return "Gemm";
        default: return "Kernel";
    }
}

int classify(int type, const std::string& name) {
    if (type != ORION_KERNEL_RECORD && type != ORION_KERNEL_EXC_RECORD)
        return (type == ORION_CUDNN_BNORM_RECORD || type == ORION_CUDNN_BNORM_INF_RECORD || type == ORION_CUDNN_BNORM_BACKWARD_RECORD) ? 0 : 1;
    static const char* compute[] = {"igemm", "gemm", "conv", "cutlass", "xmma", "wgrad", "dgrad"};
    static const char* memory[] = {"elementwise", "reduce", "bn_", "batch_norm", "pool", "binary_", "copy", "Copy", "softmax",
                                   "nll_loss", "fill", "cat", "index", "multi_tensor", "layer_norm", "dropout"};
    for (const char* k : memory)
        if (name.find(k) != std::string::npos) return 0;
    for (const char* k : compute)
        if (name.find(k) != std::string::npos) return 1;
    return -1;
}

void write_rows(const std::string& path) {
    if (path.empty()) return;
    FILE* f = fopen(path.c_str(), "w");
    if (!f) {
        fprintf(stderr, "orion: cannot write profile %s\n", path.c_str());
        return;
    }
    fprintf(f, "Name,Profile,Memory_footprint,SM_usage,Duration\n");
    for (const Row& r : R.rows) fprintf(f, "%s,%d,0,%d,%.0f\n", r.name.c_str(), r.profile, r.sm, r.ns);
    fclose(f);
    fprintf(stderr, "orion: wrote %zu profile rows to %s\n", R.rows.size(), path.c_str());
}

struct Init {
    Init() {
        const char* o = getenv("ORION_PROFILE_OUT");
        if (!o || !*o) return;
        R.enabled = true;
        R.out = o;
        if (const char* o0 = getenv("ORION_PROFILE_OUT0")) R.out0 = o0;
        if (const char* it = getenv("ORION_PROFILE_ITER")) R.steady_iter = atoi(it);
    }
} g_init;

}  // namespace

namespace orion_capture {

bool profile_enabled() { return R.enabled; }

void profile_begin(Gate* g) {
    g->prof_start = nullptr;
    if (orion_is_memop(g->type)) return;
    R.mu.lock();   // held until profile_end: one op is timed at a time
    if (!bind()) {
        R.mu.unlock();
        return;
    }
    if (R.pairs_used == (int)R.ev_a.size()) {
        cudaEvent_t a = nullptr, b = nullptr;
        R.event_create(&a);
        R.event_create(&b);
        R.ev_a.push_back(a);
        R.ev_b.push_back(b);
    }
    g->prof_start = R.ev_a[R.pairs_used];
    R.event_record(R.ev_a[R.pairs_used], (cudaStream_t)g->stream);
}

void profile_end(Gate* g) {
    if (!g->prof_start) return;
    R.event_record(R.ev_b[R.pairs_used], (cudaStream_t)g->stream);
    Row row;
    row.pair = R.pairs_used++;
    row.name = type_name(g->type);
    row.sm = R.sm_count;
    if (g->launch) {
        const char* nm = nullptr;
        if (R.func_name && R.func_name(&nm, g->launch->func) == cudaSuccess && nm) {
            row.name = nm;
            // names are cut at the template bracket, commas would break the CSV (generate_file.py:160-164)
            size_t lt = row.name.find('<');
            if (lt != std::string::npos) row.name.resize(lt);
            for (char& c : row.name)
                if (c == ',') c = ';';
        }
        long long blocks = (long long)g->launch->grid[0] * g->launch->grid[1] * g->launch->grid[2];
        int threads = (int)(g->launch->block[0] * g->launch->block[1] * g->launch->block[2]);
        int per_sm = 0;
        if (R.occupancy && R.occupancy(&per_sm, g->launch->func, threads, g->launch->shared_mem, 0) == cudaSuccess && per_sm > 0)
            row.sm = (int)((blocks + per_sm - 1) / per_sm);
        else
            row.sm = (int)blocks;
    }
    if (tls_note.set) row.profile = tls_note.op_class;   // an orion kernel: its launcher announced the class
    else row.profile = classify(g->type, row.name);
    tls_note.set = false;
    row.ns = 0.f;
    R.rows.push_back(row);
    R.mu.unlock();
}

// Reads the event pairs of the iteration that just ended.
static void resolve_durations() {
    for (Row& r : R.rows) {
        float ms = 0.f;
        if (R.event_sync(R.ev_b[r.pair]) == cudaSuccess && R.event_elapsed(&ms, R.ev_a[r.pair], R.ev_b[r.pair]) == cudaSuccess) {
            ms -= R.empty_pair_ms;
            r.ns = ms > 0.0005f ? ms * 1e6f : 500.f;   // never below half a microsecond
        }
    }
    R.pairs_used = 0;
}

void profile_mark_iteration(int it) {
    if (!R.enabled) return;
    std::lock_guard<std::mutex> lk(R.mu);
    if (R.bound && R.event_create) resolve_durations();
    if (it == 0) write_rows(R.out0);
    if (it == R.steady_iter) write_rows(R.out);
    R.rows.clear();
    R.cur_iter = it + 1;
}

}  // namespace orion_capture

// A kernel library announces the class of the launch it is about to make from the calling thread:
// op_class 1 compute-bound, 0 memory-bound, -1 unknown; flop / bytes are the algorithmic work of the problem.
extern "C" void orion_capture_annotate(int op_class, double flop, double bytes) {
    if (!R.enabled) return;
    tls_note.set = true;
    tls_note.op_class = op_class;
    tls_note.flop = flop;
    tls_note.bytes = bytes;
}
