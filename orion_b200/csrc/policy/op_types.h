// Captured-call type tags shared by the capture shim, the scheduler and the
// trace tools.  Values 0..16 are the reference's `enum func_type`
// (src/cuda_capture/intercept_temp.h:642-660) so that a trace recorded against
// either implementation carries the same numbers; values >= 17 are the entry
// points torch 2.x really calls and that the reference does not trap.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum orion_rec_type {
    ORION_KERNEL_RECORD = 0,
    ORION_MEMCPY_RECORD = 1,
    ORION_MALLOC_RECORD = 2,
    ORION_FREE_RECORD = 3,
    ORION_MEMSET_RECORD = 4,
    ORION_CUDNN_CREATE_RECORD = 5,          /* never queued by the reference; unsupported */
    ORION_CUDNN_CONV_RECORD = 6,
    ORION_CUDNN_BNORM_RECORD = 7,
    ORION_CUDNN_BNORM_RESERVE_RECORD = 8,   /* never queued by the reference; unsupported */
    ORION_CUDNN_BNORM_INF_RECORD = 9,
    ORION_CUDNN_RNN_INF_RECORD = 10,
    ORION_CUDNN_RNN_TRAIN_RECORD = 11,
    ORION_CUDNN_CONV_DATA_RECORD = 12,
    ORION_CUDNN_CONV_FILTER_RECORD = 13,
    ORION_CUDNN_BNORM_BACKWARD_RECORD = 14,
    ORION_CUBLAS_SGEMM_RECORD = 15,
    ORION_CUBLAS_SGEMM_STRIDED_RECORD = 16,
    /* extensions */
    ORION_CUBLAS_GEMMEX_RECORD = 17,
    ORION_CUBLAS_GEMMEX_STRIDED_RECORD = 18,
    ORION_CUBLASLT_MATMUL_RECORD = 19,
    ORION_CUDNN_BACKEND_EXECUTE_RECORD = 20,
    ORION_KERNEL_EXC_RECORD = 21,
    ORION_REC_TYPE_COUNT = 22
};

/* MALLOC/MEMCPY/MEMSET/FREE bypass every admission rule and do not advance the
 * per-iteration op counter (scheduler_eval.cpp:333,364; utils_sched.cpp:251-283). */
static inline int orion_is_memop(int type) {
    return type == ORION_MEMCPY_RECORD || type == ORION_MALLOC_RECORD ||
           type == ORION_FREE_RECORD || type == ORION_MEMSET_RECORD;
}

/* The reference's record type for an entry point it does not trap but whose role one of its own records plays
 * (torch 2.x calls cublasGemmEx / cublasLtMatmul where torch 1.12 called cublasSgemm, cudnnBackendExecute where it
 * called cudnnConvolutionForward, cudaLaunchKernelExC where it called cudaLaunchKernel).  Recorded arrival scripts
 * carry these numbers so that the reference scheduler, whose replay switch knows only 0..16, can replay them. */
static inline int orion_reference_type(int type) {
    switch (type) {
        case ORION_CUBLAS_GEMMEX_RECORD: case ORION_CUBLASLT_MATMUL_RECORD: return ORION_CUBLAS_SGEMM_RECORD;
        case ORION_CUBLAS_GEMMEX_STRIDED_RECORD: return ORION_CUBLAS_SGEMM_STRIDED_RECORD;
        case ORION_CUDNN_BACKEND_EXECUTE_RECORD: return ORION_CUDNN_CONV_RECORD;
        case ORION_KERNEL_EXC_RECORD: return ORION_KERNEL_RECORD;
        default: return type;
    }
}

/* Types the reference's replay switch aborts on (utils_sched.cpp:514-516). */
static inline int orion_is_unsupported(int type) {
    return type < 0 || type >= ORION_REC_TYPE_COUNT || type == ORION_CUDNN_CREATE_RECORD ||
           type == ORION_CUDNN_BNORM_RESERVE_RECORD;
}

#ifdef __cplusplus
}
#endif
