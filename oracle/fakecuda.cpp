// TEST INFRASTRUCTURE — not part of the product.
//
// Stand-ins for the 19 CUDA runtime / cuDNN / cuBLAS entry points that the
// reference scheduler looks up with dlsym(RTLD_DEFAULT, ...) and asserts non-NULL
// (src/scheduler/utils_sched.cpp:159-237).  The scheduler calls them through
// pointers that carry the real signatures; nothing here reads an argument, so each
// stub is variadic and only counts its calls.  No CUDA header is included on
// purpose: the real prototypes would clash with these definitions.
extern "C" {
int oracle_stub_calls[32];
#define ORACLE_STUB(name, tag)   \
    int name(...) {              \
        oracle_stub_calls[tag]++; \
        return 0;                \
    }
ORACLE_STUB(cudaLaunchKernel, 0)
ORACLE_STUB(cudaMemcpy, 1)
ORACLE_STUB(cudaMemcpyAsync, 1)
ORACLE_STUB(cudaMalloc, 2)
ORACLE_STUB(cudaFree, 3)
ORACLE_STUB(cudaMemset, 4)
ORACLE_STUB(cudaMemsetAsync, 4)
ORACLE_STUB(cudnnCreate, 5)
ORACLE_STUB(cudnnGetBatchNormalizationTrainingExReserveSpaceSize, 8)
ORACLE_STUB(cudnnConvolutionForward, 6)
ORACLE_STUB(cudnnBatchNormalizationForwardTrainingEx, 7)
ORACLE_STUB(cudnnBatchNormalizationForwardInference, 9)
ORACLE_STUB(cudnnRNNForwardInference, 10)
ORACLE_STUB(cudnnRNNForwardTraining, 11)
ORACLE_STUB(cudnnBatchNormalizationBackwardEx, 14)
ORACLE_STUB(cudnnConvolutionBackwardData, 12)
ORACLE_STUB(cudnnConvolutionBackwardFilter, 13)
ORACLE_STUB(cublasSgemm_v2, 15)
ORACLE_STUB(cublasSgemmStridedBatched, 16)
}
