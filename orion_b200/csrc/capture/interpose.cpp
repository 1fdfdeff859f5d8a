// LD_PRELOAD interposers: every GPU-work entry point an unmodified PyTorch client
// can reach is trapped here, queued for the scheduler, and — once granted — run by
// the calling thread on the granted stream.
//
// Trapped set = the reference's (src/cuda_capture/intercept_temp.cpp:145-458,
// intercept_cudnn.cpp, intercept_cublas.cpp) minus the cuDNN RNN calls (gone from
// cuDNN 9), plus what torch 2.x calls instead of them: cudaLaunchKernelExC,
// cublasGemmEx, cublasGemmStridedBatchedEx, cublasLtMatmul, cudnnBackendExecute.
// A thread that is not a registered client (including the scheduler's own) falls
// through to the real symbol, as in the reference (intercept_temp.cpp:449-456).
//
// Unlike the reference, descriptors are never leaked (its cudnnDestroy* no-ops,
// intercept_cudnn.cpp:643-679, exist because it replays calls after the caller
// returned; here the caller itself performs the call before returning), and the
// real return code reaches the caller.
#include <cublasLt.h>
#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <cudnn.h>
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>

#include "capture_core.h"

using namespace orion_capture;

// The real symbol: next in the global lookup order when the library was loaded at
// start-up, else (torch dlopen()s cuDNN and cuBLAS privately) from the library's own handle.
static void* find_real(const char* name) {
    void* p = dlsym(RTLD_NEXT, name);
    if (p) return p;
    static const char* sonames[] = {"libcudart.so.12", "libcublas.so.12", "libcublasLt.so.12", "libcudnn.so.9",
                                    "libcudnn_graph.so.9", "libcudnn_cnn.so.9", "libcudnn_ops.so.9", "libcudnn_adv.so.9"};
    for (const char* so : sonames) {
        void* h = dlopen(so, RTLD_NOW | RTLD_NOLOAD);
        if (!h) continue;
        p = dlsym(h, name);
        if (p) return p;
    }
    return nullptr;
}

template <typename F>
static inline F resolve(F& slot, const char* name) {
    if (!slot) {
        slot = (F)find_real(name);
        if (!slot) {
            fprintf(stderr, "orion: real symbol %s not found behind the capture library\n", name);
            abort();
        }
    }
    return slot;
}
#define REAL(name) resolve(real_##name, #name)

static cudaError_t (*real_cudaEventRecord)(cudaEvent_t, cudaStream_t);
namespace orion_capture {
void real_event_record(void* event, void* stream) {
    if (!real_cudaEventRecord) {
        real_cudaEventRecord = (decltype(real_cudaEventRecord))find_real("cudaEventRecord");
        if (!real_cudaEventRecord) return;   // host-only process: nothing to record
    }
    real_cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream);
}
}  // namespace orion_capture

extern "C" {

// ------------------------------------------------------------------ CUDA runtime
static cudaError_t (*real_cudaLaunchKernel)(const void*, dim3, dim3, void**, size_t, cudaStream_t);
cudaError_t cudaLaunchKernel(const void* func, dim3 gridDim, dim3 blockDim, void** args, size_t sharedMem, cudaStream_t stream) {
    REAL(cudaLaunchKernel);
    Gate g;
    if (!gate_begin(&g, ORION_KERNEL_RECORD, stream, (uint64_t)(uintptr_t)func))
        return real_cudaLaunchKernel(func, gridDim, blockDim, args, sharedMem, stream);
    gridDim.x = clamp_grid(func, gridDim.x, g.num_ctas);   // persistent kernels take the SM quota of the grant
    LaunchInfo li{func, {gridDim.x, gridDim.y, gridDim.z}, {blockDim.x, blockDim.y, blockDim.z}, sharedMem};
    g.launch = &li;
    cudaError_t e = real_cudaLaunchKernel(func, gridDim, blockDim, args, sharedMem, (cudaStream_t)g.stream);
    gate_end(&g);
    return e;
}

static cudaError_t (*real_cudaLaunchKernelExC)(const cudaLaunchConfig_t*, const void*, void**);
cudaError_t cudaLaunchKernelExC(const cudaLaunchConfig_t* config, const void* func, void** args) {
    REAL(cudaLaunchKernelExC);
    Gate g;
    if (!gate_begin(&g, ORION_KERNEL_EXC_RECORD, config->stream, (uint64_t)(uintptr_t)func))
        return real_cudaLaunchKernelExC(config, func, args);
    cudaLaunchConfig_t cfg = *config;
    cfg.stream = (cudaStream_t)g.stream;
    cfg.gridDim.x = clamp_grid(func, cfg.gridDim.x, g.num_ctas);
    LaunchInfo li{func, {cfg.gridDim.x, cfg.gridDim.y, cfg.gridDim.z}, {cfg.blockDim.x, cfg.blockDim.y, cfg.blockDim.z},
                  cfg.dynamicSmemBytes};
    g.launch = &li;
    cudaError_t e = real_cudaLaunchKernelExC(&cfg, func, args);
    gate_end(&g);
    return e;
}

static cudaError_t (*real_cudaMemcpyAsync)(void*, const void*, size_t, enum cudaMemcpyKind, cudaStream_t);
static cudaError_t (*real_cudaStreamSynchronize)(cudaStream_t);

// Host-to-device copies of a best-effort client larger than this are issued in pieces, each one waited for before the
// next is queued.  The copy engine serves copies in the order they were queued, whatever the priority of their streams: a
// best-effort batch of tens of megabytes queued in one piece would hold a high-priority request's input copy back for its
// whole duration (hundreds of microseconds on PCIe).  In pieces, the high-priority copy waits for one piece at most.  This
// is the copy engine's counterpart of the SM quota; the policy sees one memcpy record either way.  ORION_BE_COPY_CHUNK
// sets the piece size in bytes (0: never split).
static size_t be_copy_chunk() {
    static const size_t v = [] {
        const char* e = getenv("ORION_BE_COPY_CHUNK");
        return e ? (size_t)strtoull(e, nullptr, 10) : (size_t)1 << 20;
    }();
    return v;
}

cudaError_t cudaMemcpyAsync(void* dst, const void* src, size_t count, enum cudaMemcpyKind kind, cudaStream_t stream) {
    REAL(cudaMemcpyAsync);
    Gate g;
    if (!gate_begin(&g, ORION_MEMCPY_RECORD, stream, 0)) return real_cudaMemcpyAsync(dst, src, count, kind, stream);
    cudaError_t e = cudaSuccess;
    const size_t chunk = be_copy_chunk();
    const orion_shared* sh = orion_capture_shared();
    const bool best_effort = g.idx >= 0 && sh->num_clients > 1 && g.idx < sh->num_clients - 1;
    if (best_effort && kind == cudaMemcpyHostToDevice && chunk > 0 && count > chunk) {
        REAL(cudaStreamSynchronize);
        for (size_t off = 0; off < count && e == cudaSuccess; off += chunk) {
            const size_t n = count - off < chunk ? count - off : chunk;
            e = real_cudaMemcpyAsync((char*)dst + off, (const char*)src + off, n, kind, (cudaStream_t)g.stream);
            if (e == cudaSuccess && off + n < count) e = real_cudaStreamSynchronize((cudaStream_t)g.stream);
        }
    } else {
        e = real_cudaMemcpyAsync(dst, src, count, kind, (cudaStream_t)g.stream);
    }
    gate_end(&g);
    return e;
}

static cudaError_t (*real_cudaMemcpy)(void*, const void*, size_t, enum cudaMemcpyKind);
cudaError_t cudaMemcpy(void* dst, const void* src, size_t count, enum cudaMemcpyKind kind) {
    REAL(cudaMemcpy);
    Gate g;
    if (!gate_begin(&g, ORION_MEMCPY_RECORD, nullptr, 0)) return real_cudaMemcpy(dst, src, count, kind);
    // A blocking copy must see the client's earlier work, which runs on a non-blocking
    // stream the legacy default stream does not wait for: copy on that stream and drain it.
    REAL(cudaMemcpyAsync);
    REAL(cudaStreamSynchronize);
    cudaError_t e = real_cudaMemcpyAsync(dst, src, count, kind, (cudaStream_t)g.stream);
    gate_end(&g);
    cudaError_t e2 = real_cudaStreamSynchronize((cudaStream_t)g.stream);
    return e != cudaSuccess ? e : e2;
}

static cudaError_t (*real_cudaMemsetAsync)(void*, int, size_t, cudaStream_t);
cudaError_t cudaMemsetAsync(void* devPtr, int value, size_t count, cudaStream_t stream) {
    REAL(cudaMemsetAsync);
    Gate g;
    if (!gate_begin(&g, ORION_MEMSET_RECORD, stream, 0)) return real_cudaMemsetAsync(devPtr, value, count, stream);
    cudaError_t e = real_cudaMemsetAsync(devPtr, value, count, (cudaStream_t)g.stream);
    gate_end(&g);
    return e;
}

static cudaError_t (*real_cudaMemset)(void*, int, size_t);
cudaError_t cudaMemset(void* devPtr, int value, size_t count) {
    REAL(cudaMemset);
    Gate g;
    if (!gate_begin(&g, ORION_MEMSET_RECORD, nullptr, 0)) return real_cudaMemset(devPtr, value, count);
    REAL(cudaMemsetAsync);
    REAL(cudaStreamSynchronize);
    cudaError_t e = real_cudaMemsetAsync(devPtr, value, count, (cudaStream_t)g.stream);
    gate_end(&g);
    cudaError_t e2 = real_cudaStreamSynchronize((cudaStream_t)g.stream);
    return e != cudaSuccess ? e : e2;
}

static cudaError_t (*real_cudaMalloc)(void**, size_t);
cudaError_t cudaMalloc(void** devPtr, size_t size) {
    REAL(cudaMalloc);
    Gate g;
    if (!gate_begin(&g, ORION_MALLOC_RECORD, nullptr, 0)) return real_cudaMalloc(devPtr, size);
    cudaError_t e = real_cudaMalloc(devPtr, size);
    gate_end(&g);
    return e;
}

static cudaError_t (*real_cudaFree)(void*);
cudaError_t cudaFree(void* devPtr) {
    REAL(cudaFree);
    Gate g;
    if (!gate_begin(&g, ORION_FREE_RECORD, nullptr, 0)) return real_cudaFree(devPtr);
    cudaError_t e = real_cudaFree(devPtr);
    gate_end(&g);
    return e;
}

// Stream-ordered allocation (torch's cudaMallocAsync allocator backend): queued as the MALLOC / FREE records
// the reference uses for cudaMalloc / cudaFree (intercept_temp.cpp:145-192, 368-415) and run on the granted stream.
static cudaError_t (*real_cudaMallocAsync)(void**, size_t, cudaStream_t);
cudaError_t cudaMallocAsync(void** devPtr, size_t size, cudaStream_t stream) {
    REAL(cudaMallocAsync);
    Gate g;
    if (!gate_begin(&g, ORION_MALLOC_RECORD, stream, 0)) return real_cudaMallocAsync(devPtr, size, stream);
    cudaError_t e = real_cudaMallocAsync(devPtr, size, (cudaStream_t)g.stream);
    gate_end(&g);
    return e;
}

static cudaError_t (*real_cudaFreeAsync)(void*, cudaStream_t);
cudaError_t cudaFreeAsync(void* devPtr, cudaStream_t stream) {
    REAL(cudaFreeAsync);
    Gate g;
    if (!gate_begin(&g, ORION_FREE_RECORD, stream, 0)) return real_cudaFreeAsync(devPtr, stream);
    cudaError_t e = real_cudaFreeAsync(devPtr, (cudaStream_t)g.stream);
    gate_end(&g);
    return e;
}

// Managed allocations pass straight through, as in the reference (intercept_temp.cpp:194-206).
static cudaError_t (*real_cudaMallocManaged)(void**, size_t, unsigned int);
cudaError_t cudaMallocManaged(void** devPtr, size_t size, unsigned int flags) {
    return REAL(cudaMallocManaged)(devPtr, size, flags);
}

// A captured CUDA graph would put a whole iteration on the device behind one call, past every admission rule,
// with kernels the profile has no rows for.  A scheduled client that launches one is stopped with a message
// instead of slipping past the scheduler silently; unscheduled threads launch graphs as usual.
static cudaError_t (*real_cudaGraphLaunch)(cudaGraphExec_t, cudaStream_t);
cudaError_t cudaGraphLaunch(cudaGraphExec_t graphExec, cudaStream_t stream) {
    REAL(cudaGraphLaunch);
    int idx = client_index_of_thread();
    if (idx < 0) idx = client_index_of_stream((void*)stream);
    if (idx >= 0) {
        fprintf(stderr, "orion: client %d called cudaGraphLaunch; captured graphs cannot be scheduled op by op "
                        "(run the client without CUDA graphs)\n", idx);
        return cudaErrorNotSupported;
    }
    return real_cudaGraphLaunch(graphExec, stream);
}

// ------------------------------------------------------------------ cuBLAS
static cublasStatus_t (*real_cublasGetStream_v2)(cublasHandle_t, cudaStream_t*);
static cublasStatus_t (*real_cublasSetStream_v2)(cublasHandle_t, cudaStream_t);

static inline void* cublas_stream(cublasHandle_t h) {
    cudaStream_t s = nullptr;
    REAL(cublasGetStream_v2)(h, &s);
    return (void*)s;
}
// If the client runs on a default stream, move the handle to the granted stream for this call.
static inline void cublas_retarget(cublasHandle_t h, void* user, void* granted) {
    if (user != granted) REAL(cublasSetStream_v2)(h, (cudaStream_t)granted);
}

static cublasStatus_t (*real_cublasSgemm_v2)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const float*,
                                            const float*, int, const float*, int, const float*, float*, int);
cublasStatus_t cublasSgemm_v2(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m, int n, int k,
                              const float* alpha, const float* A, int lda, const float* B, int ldb, const float* beta, float* C,
                              int ldc) {
    REAL(cublasSgemm_v2);
    void* us = cublas_stream(handle);
    Gate g;
    if (!gate_begin(&g, ORION_CUBLAS_SGEMM_RECORD, us, (uint64_t)(uintptr_t)handle))
        return real_cublasSgemm_v2(handle, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc);
    cublas_retarget(handle, us, g.stream);
    cublasStatus_t st = real_cublasSgemm_v2(handle, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc);
    gate_end(&g);
    return st;
}

static cublasStatus_t (*real_cublasSgemmStridedBatched)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int,
                                                       const float*, const float*, int, long long, const float*, int, long long,
                                                       const float*, float*, int, long long, int);
cublasStatus_t cublasSgemmStridedBatched(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m, int n,
                                         int k, const float* alpha, const float* A, int lda, long long strideA, const float* B,
                                         int ldb, long long strideB, const float* beta, float* C, int ldc, long long strideC,
                                         int batchCount) {
    REAL(cublasSgemmStridedBatched);
    void* us = cublas_stream(handle);
    Gate g;
    if (!gate_begin(&g, ORION_CUBLAS_SGEMM_STRIDED_RECORD, us, (uint64_t)(uintptr_t)handle))
        return real_cublasSgemmStridedBatched(handle, transa, transb, m, n, k, alpha, A, lda, strideA, B, ldb, strideB, beta, C, ldc,
                                              strideC, batchCount);
    cublas_retarget(handle, us, g.stream);
    cublasStatus_t st = real_cublasSgemmStridedBatched(handle, transa, transb, m, n, k, alpha, A, lda, strideA, B, ldb, strideB, beta,
                                                       C, ldc, strideC, batchCount);
    gate_end(&g);
    return st;
}

static cublasStatus_t (*real_cublasGemmEx)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*,
                                          const void*, cudaDataType, int, const void*, cudaDataType, int, const void*, void*,
                                          cudaDataType, int, cublasComputeType_t, cublasGemmAlgo_t);
cublasStatus_t cublasGemmEx(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m, int n, int k,
                            const void* alpha, const void* A, cudaDataType Atype, int lda, const void* B, cudaDataType Btype, int ldb,
                            const void* beta, void* C, cudaDataType Ctype, int ldc, cublasComputeType_t computeType,
                            cublasGemmAlgo_t algo) {
    REAL(cublasGemmEx);
    void* us = cublas_stream(handle);
    Gate g;
    if (!gate_begin(&g, ORION_CUBLAS_GEMMEX_RECORD, us, (uint64_t)(uintptr_t)handle))
        return real_cublasGemmEx(handle, transa, transb, m, n, k, alpha, A, Atype, lda, B, Btype, ldb, beta, C, Ctype, ldc, computeType,
                                 algo);
    cublas_retarget(handle, us, g.stream);
    cublasStatus_t st = real_cublasGemmEx(handle, transa, transb, m, n, k, alpha, A, Atype, lda, B, Btype, ldb, beta, C, Ctype, ldc,
                                          computeType, algo);
    gate_end(&g);
    return st;
}

static cublasStatus_t (*real_cublasGemmStridedBatchedEx)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int,
                                                        const void*, const void*, cudaDataType, int, long long, const void*,
                                                        cudaDataType, int, long long, const void*, void*, cudaDataType, int,
                                                        long long, int, cublasComputeType_t, cublasGemmAlgo_t);
cublasStatus_t cublasGemmStridedBatchedEx(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m, int n,
                                          int k, const void* alpha, const void* A, cudaDataType Atype, int lda, long long strideA,
                                          const void* B, cudaDataType Btype, int ldb, long long strideB, const void* beta, void* C,
                                          cudaDataType Ctype, int ldc, long long strideC, int batchCount,
                                          cublasComputeType_t computeType, cublasGemmAlgo_t algo) {
    REAL(cublasGemmStridedBatchedEx);
    void* us = cublas_stream(handle);
    Gate g;
    if (!gate_begin(&g, ORION_CUBLAS_GEMMEX_STRIDED_RECORD, us, (uint64_t)(uintptr_t)handle))
        return real_cublasGemmStridedBatchedEx(handle, transa, transb, m, n, k, alpha, A, Atype, lda, strideA, B, Btype, ldb, strideB,
                                               beta, C, Ctype, ldc, strideC, batchCount, computeType, algo);
    cublas_retarget(handle, us, g.stream);
    cublasStatus_t st = real_cublasGemmStridedBatchedEx(handle, transa, transb, m, n, k, alpha, A, Atype, lda, strideA, B, Btype, ldb,
                                                        strideB, beta, C, Ctype, ldc, strideC, batchCount, computeType, algo);
    gate_end(&g);
    return st;
}

static cublasStatus_t (*real_cublasLtMatmul)(cublasLtHandle_t, cublasLtMatmulDesc_t, const void*, const void*, cublasLtMatrixLayout_t,
                                            const void*, cublasLtMatrixLayout_t, const void*, const void*, cublasLtMatrixLayout_t,
                                            void*, cublasLtMatrixLayout_t, const cublasLtMatmulAlgo_t*, void*, size_t, cudaStream_t);
cublasStatus_t cublasLtMatmul(cublasLtHandle_t lightHandle, cublasLtMatmulDesc_t computeDesc, const void* alpha, const void* A,
                              cublasLtMatrixLayout_t Adesc, const void* B, cublasLtMatrixLayout_t Bdesc, const void* beta,
                              const void* C, cublasLtMatrixLayout_t Cdesc, void* D, cublasLtMatrixLayout_t Ddesc,
                              const cublasLtMatmulAlgo_t* algo, void* workspace, size_t workspaceSizeInBytes, cudaStream_t stream) {
    REAL(cublasLtMatmul);
    Gate g;
    if (!gate_begin(&g, ORION_CUBLASLT_MATMUL_RECORD, stream, (uint64_t)(uintptr_t)lightHandle))
        return real_cublasLtMatmul(lightHandle, computeDesc, alpha, A, Adesc, B, Bdesc, beta, C, Cdesc, D, Ddesc, algo, workspace,
                                   workspaceSizeInBytes, stream);
    cublasStatus_t st = real_cublasLtMatmul(lightHandle, computeDesc, alpha, A, Adesc, B, Bdesc, beta, C, Cdesc, D, Ddesc, algo,
                                            workspace, workspaceSizeInBytes, (cudaStream_t)g.stream);
    gate_end(&g);
    return st;
}

// ------------------------------------------------------------------ cuDNN
static cudnnStatus_t (*real_cudnnGetStream)(cudnnHandle_t, cudaStream_t*);
static cudnnStatus_t (*real_cudnnSetStream)(cudnnHandle_t, cudaStream_t);
static inline void* cudnn_stream(cudnnHandle_t h) {
    cudaStream_t s = nullptr;
    REAL(cudnnGetStream)(h, &s);
    return (void*)s;
}
static inline void cudnn_retarget(cudnnHandle_t h, void* user, void* granted) {
    if (user != granted) REAL(cudnnSetStream)(h, (cudaStream_t)granted);
}

#define ORION_CUDNN_TRAP(name, tag, params, args)                                   \
    static cudnnStatus_t(*real_##name) params;                                      \
    cudnnStatus_t name params {                                                     \
        REAL(name);                                                                 \
        void* us = cudnn_stream(handle);                                            \
        Gate g;                                                                     \
        if (!gate_begin(&g, tag, us, (uint64_t)(uintptr_t)handle)) return real_##name args; \
        cudnn_retarget(handle, us, g.stream);                                       \
        cudnnStatus_t st = real_##name args;                                        \
        gate_end(&g);                                                               \
        return st;                                                                  \
    }

ORION_CUDNN_TRAP(cudnnBackendExecute, ORION_CUDNN_BACKEND_EXECUTE_RECORD,
                 (cudnnHandle_t handle, cudnnBackendDescriptor_t executionPlan, cudnnBackendDescriptor_t variantPack),
                 (handle, executionPlan, variantPack))

ORION_CUDNN_TRAP(cudnnConvolutionForward, ORION_CUDNN_CONV_RECORD,
                 (cudnnHandle_t handle, const void* alpha, const cudnnTensorDescriptor_t xDesc, const void* x,
                  const cudnnFilterDescriptor_t wDesc, const void* w, const cudnnConvolutionDescriptor_t convDesc,
                  cudnnConvolutionFwdAlgo_t algo, void* workSpace, size_t workSpaceSizeInBytes, const void* beta,
                  const cudnnTensorDescriptor_t yDesc, void* y),
                 (handle, alpha, xDesc, x, wDesc, w, convDesc, algo, workSpace, workSpaceSizeInBytes, beta, yDesc, y))

ORION_CUDNN_TRAP(cudnnConvolutionBackwardData, ORION_CUDNN_CONV_DATA_RECORD,
                 (cudnnHandle_t handle, const void* alpha, const cudnnFilterDescriptor_t wDesc, const void* w,
                  const cudnnTensorDescriptor_t dyDesc, const void* dy, const cudnnConvolutionDescriptor_t convDesc,
                  cudnnConvolutionBwdDataAlgo_t algo, void* workSpace, size_t workSpaceSizeInBytes, const void* beta,
                  const cudnnTensorDescriptor_t dxDesc, void* dx),
                 (handle, alpha, wDesc, w, dyDesc, dy, convDesc, algo, workSpace, workSpaceSizeInBytes, beta, dxDesc, dx))

ORION_CUDNN_TRAP(cudnnConvolutionBackwardFilter, ORION_CUDNN_CONV_FILTER_RECORD,
                 (cudnnHandle_t handle, const void* alpha, const cudnnTensorDescriptor_t xDesc, const void* x,
                  const cudnnTensorDescriptor_t dyDesc, const void* dy, const cudnnConvolutionDescriptor_t convDesc,
                  cudnnConvolutionBwdFilterAlgo_t algo, void* workSpace, size_t workSpaceSizeInBytes, const void* beta,
                  const cudnnFilterDescriptor_t dwDesc, void* dw),
                 (handle, alpha, xDesc, x, dyDesc, dy, convDesc, algo, workSpace, workSpaceSizeInBytes, beta, dwDesc, dw))

ORION_CUDNN_TRAP(cudnnBatchNormalizationForwardInference, ORION_CUDNN_BNORM_INF_RECORD,
                 (cudnnHandle_t handle, cudnnBatchNormMode_t mode, const void* alpha, const void* beta,
                  const cudnnTensorDescriptor_t xDesc, const void* x, const cudnnTensorDescriptor_t yDesc, void* y,
                  const cudnnTensorDescriptor_t bnScaleBiasMeanVarDesc, const void* bnScale, const void* bnBias,
                  const void* estimatedMean, const void* estimatedVariance, double epsilon),
                 (handle, mode, alpha, beta, xDesc, x, yDesc, y, bnScaleBiasMeanVarDesc, bnScale, bnBias, estimatedMean,
                  estimatedVariance, epsilon))

ORION_CUDNN_TRAP(cudnnBatchNormalizationForwardTrainingEx, ORION_CUDNN_BNORM_RECORD,
                 (cudnnHandle_t handle, cudnnBatchNormMode_t mode, cudnnBatchNormOps_t bnOps, const void* alpha, const void* beta,
                  const cudnnTensorDescriptor_t xDesc, const void* xData, const cudnnTensorDescriptor_t zDesc, const void* zData,
                  const cudnnTensorDescriptor_t yDesc, void* yData, const cudnnTensorDescriptor_t bnScaleBiasMeanVarDesc,
                  const void* bnScale, const void* bnBias, double exponentialAverageFactor, void* resultRunningMean,
                  void* resultRunningVariance, double epsilon, void* resultSaveMean, void* resultSaveInvVariance,
                  cudnnActivationDescriptor_t activationDesc, void* workspace, size_t workSpaceSizeInBytes, void* reserveSpace,
                  size_t reserveSpaceSizeInBytes),
                 (handle, mode, bnOps, alpha, beta, xDesc, xData, zDesc, zData, yDesc, yData, bnScaleBiasMeanVarDesc, bnScale, bnBias,
                  exponentialAverageFactor, resultRunningMean, resultRunningVariance, epsilon, resultSaveMean, resultSaveInvVariance,
                  activationDesc, workspace, workSpaceSizeInBytes, reserveSpace, reserveSpaceSizeInBytes))

ORION_CUDNN_TRAP(cudnnBatchNormalizationBackwardEx, ORION_CUDNN_BNORM_BACKWARD_RECORD,
                 (cudnnHandle_t handle, cudnnBatchNormMode_t mode, cudnnBatchNormOps_t bnOps, const void* alphaDataDiff,
                  const void* betaDataDiff, const void* alphaParamDiff, const void* betaParamDiff, const cudnnTensorDescriptor_t xDesc,
                  const void* xData, const cudnnTensorDescriptor_t yDesc, const void* yData, const cudnnTensorDescriptor_t dyDesc,
                  const void* dyData, const cudnnTensorDescriptor_t dzDesc, void* dzData, const cudnnTensorDescriptor_t dxDesc,
                  void* dxData, const cudnnTensorDescriptor_t dBnScaleBiasDesc, const void* bnScaleData, const void* bnBiasData,
                  void* dBnScaleData, void* dBnBiasData, double epsilon, const void* savedMean, const void* savedInvVariance,
                  cudnnActivationDescriptor_t activationDesc, void* workSpace, size_t workSpaceSizeInBytes, void* reserveSpace,
                  size_t reserveSpaceSizeInBytes),
                 (handle, mode, bnOps, alphaDataDiff, betaDataDiff, alphaParamDiff, betaParamDiff, xDesc, xData, yDesc, yData, dyDesc,
                  dyData, dzDesc, dzData, dxDesc, dxData, dBnScaleBiasDesc, bnScaleData, bnBiasData, dBnScaleData, dBnBiasData,
                  epsilon, savedMean, savedInvVariance, activationDesc, workSpace, workSpaceSizeInBytes, reserveSpace,
                  reserveSpaceSizeInBytes))

}  // extern "C"
