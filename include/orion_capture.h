/* liborion_capture.so — C ABI of the capture (interception) library.
 *
 * Loaded with LD_PRELOAD, it interposes the CUDA runtime / cuBLAS / cuDNN entry
 * points listed below with their exact vendor signatures (not re-declared here)
 * and exports the two control calls client scripts bind with ctypes.  It replaces
 * the reference's libinttemp.so (reference src/cuda_capture/intercept_temp.cpp,
 * intercept_cudnn.cpp, intercept_cublas.cpp, utils_interc.cpp).
 *
 * Interposed: cudaLaunchKernel, cudaLaunchKernelExC, cudaMemcpy, cudaMemcpyAsync,
 * cudaMemset, cudaMemsetAsync, cudaMalloc, cudaFree, cudaMallocAsync, cudaFreeAsync,
 * cudaMallocManaged (passed through), cudaGraphLaunch (refused with cudaErrorNotSupported
 * when a scheduled client calls it); cublasSgemm_v2,
 * cublasSgemmStridedBatched, cublasGemmEx, cublasGemmStridedBatchedEx,
 * cublasLtMatmul; cudnnBackendExecute, cudnnConvolutionForward,
 * cudnnConvolutionBackwardData, cudnnConvolutionBackwardFilter,
 * cudnnBatchNormalizationForwardInference, cudnnBatchNormalizationForwardTrainingEx,
 * cudnnBatchNormalizationBackwardEx.
 */
#ifndef ORION_CAPTURE_H
#define ORION_CAPTURE_H
#include <stdbool.h>

#ifdef __cplusplus
extern "C" {
#endif

/* reference intercept_temp.cpp:125-130: returns when request `it` of the calling
 * client has completed on the GPU. */
void block(int it);

/* reference intercept_temp.cpp:132-141: true once the scheduler asked the calling
 * client to stop; acknowledges the request. */
bool stop(void);

/* ---- additions: no counterpart in the reference ---- */
struct orion_shared;
struct orion_shared* orion_capture_shared(void);     /* shared block the scheduler attaches to (replaces the nine globals of
                                                       reference intercept_temp.cpp:8-19) */
int orion_capture_op(int type);                      /* queue one op of a record type with no CUDA call behind it */
int orion_capture_client_index(void);                /* client index of the calling thread, -1 if none */
void* orion_capture_client_stream(int idx);          /* cudaStream_t of client idx, NULL before setup */
int orion_capture_register_thread(int idx);          /* register the calling thread as a helper thread of client idx */
unsigned long long orion_capture_count(int type);    /* scheduled calls of a record type (-1: passed-through calls) */
unsigned long long orion_capture_seen(int type);     /* all intercepted calls of a record type */

/* SM quota of grants.  The reference stores the SM need of the high-priority op it released
 * (reference src/scheduler/scheduler_eval.cpp:317) and never reads it; here a best-effort grant carries
 * "device SMs minus that need" as its quota, and a kernel whose library declared it elastic (any grid
 * width gives the same result) is launched with at most quota x ctas_per_sm blocks. */
int orion_capture_mark_elastic(const void* func, int ctas_per_sm);   /* func: the handle passed to cudaLaunchKernel */
int orion_capture_quota_hint(void);                  /* quota the calling client would be granted now (0: whole device) */
int orion_capture_last_quota(void);                  /* quota carried by the calling thread's latest grant */
unsigned orion_capture_clamp_grid(const void* func, unsigned grid_x, int num_ctas);   /* grid width under a quota */
unsigned long long orion_capture_clamped_launches(void);   /* launches cut to their quota so far */

#ifdef __cplusplus
}
#endif
#endif
