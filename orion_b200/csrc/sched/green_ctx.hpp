// Green-context SM partition for the best-effort stream (CUDA driver API >= 12.4,
// bound at run time from libcuda.so.1).
//
// The reference trusts the profiled SM need of each best-effort kernel
// (src/scheduler/scheduler_eval.cpp:340); on Blackwell the budget can be enforced
// by hardware instead: the best-effort client's stream is created inside a green
// context that owns `be_sms` SMs, so whatever the policy admits can never occupy
// more than that, and the remaining SMs are always free for the high-priority
// stream (which stays in the primary context and may use every SM).
#pragma once
#include <cuda.h>
#include <dlfcn.h>

#include <string>

namespace orion {

class GreenCtx {
public:
    int be_sms = 0;          // SMs actually granted to the best-effort partition
    int total_sms = 0;
    std::string error;

    bool create(int want_be_sms) {
        void* h = dlopen("libcuda.so.1", RTLD_NOW);
        if (!h) return fail("libcuda.so.1 not loadable");
        auto p_cuCtxGetDevice = (CUresult(*)(CUdevice*))dlsym(h, "cuCtxGetDevice");
        auto p_getRes = (CUresult(*)(CUdevice, CUdevResource*, CUdevResourceType))dlsym(h, "cuDeviceGetDevResource");
        auto p_split = (CUresult(*)(CUdevResource*, unsigned int*, const CUdevResource*, CUdevResource*, unsigned int,
                                    unsigned int))dlsym(h, "cuDevSmResourceSplitByCount");
        auto p_desc = (CUresult(*)(CUdevResourceDesc*, CUdevResource*, unsigned int))dlsym(h, "cuDevResourceGenerateDesc");
        auto p_create = (CUresult(*)(CUgreenCtx*, CUdevResourceDesc, CUdevice, unsigned int))dlsym(h, "cuGreenCtxCreate");
        stream_create_ = (CUresult(*)(CUstream*, CUgreenCtx, unsigned int, int))dlsym(h, "cuGreenCtxStreamCreate");
        if (!p_cuCtxGetDevice || !p_getRes || !p_split || !p_desc || !p_create || !stream_create_)
            return fail("driver lacks the green-context entry points");
        CUdevice dev;
        if (p_cuCtxGetDevice(&dev) != CUDA_SUCCESS) return fail("no current CUDA context");
        CUdevResource all;
        if (p_getRes(dev, &all, CU_DEV_RESOURCE_TYPE_SM) != CUDA_SUCCESS) return fail("cuDeviceGetDevResource failed");
        total_sms = (int)all.sm.smCount;
        if (want_be_sms <= 0 || want_be_sms >= total_sms) return fail("best-effort SM quota must be in (0, device SMs)");
        CUdevResource part, rest;
        unsigned int groups = 1;
        if (p_split(&part, &groups, &all, &rest, 0, (unsigned int)want_be_sms) != CUDA_SUCCESS || groups < 1)
            return fail("cuDevSmResourceSplitByCount failed");
        CUdevResourceDesc desc;
        if (p_desc(&desc, &part, 1) != CUDA_SUCCESS) return fail("cuDevResourceGenerateDesc failed");
        if (p_create(&ctx_, desc, dev, CU_GREEN_CTX_DEFAULT_STREAM) != CUDA_SUCCESS) return fail("cuGreenCtxCreate failed");
        be_sms = (int)part.sm.smCount;
        return true;
    }

    // which: 0 = best-effort partition; anything else has no partition (primary context).
    void* stream(int which, int priority) {
        if (which != 0 || !ctx_ || !stream_create_) return nullptr;
        CUstream s = nullptr;
        if (stream_create_(&s, ctx_, CU_STREAM_NON_BLOCKING, priority) != CUDA_SUCCESS) return nullptr;
        return (void*)s;
    }

private:
    CUgreenCtx ctx_ = nullptr;
    CUresult (*stream_create_)(CUstream*, CUgreenCtx, unsigned int, int) = nullptr;
    bool fail(const char* why) {
        error = why;
        return false;
    }
};

}  // namespace orion
