// Elastic kernels and the scheduler's SM quota.
//
// A kernel is elastic when its blocks walk the work with a gridDim.x stride (or derive their share of the work
// from gridDim.x in some other way), so that any grid width gives the same result.  When the capture library
// of the scheduler is loaded in front of the CUDA runtime, a launch that the scheduler grants with an SM
// quota q is cut to q x (resident CTAs per SM) blocks at the moment it is granted: the persistent kernel's
// CTA count equals the SM budget the policy accounted for.  Without the capture library this header does
// nothing.
#pragma once
#include <dlfcn.h>
#include <stdlib.h>

namespace ob200 {

inline bool mark_elastic(const void* kernel, int ctas_per_sm) {
    using Fn = int (*)(const void*, int);
    static const Fn fn = reinterpret_cast<Fn>(dlsym(RTLD_DEFAULT, "orion_capture_mark_elastic"));
    if (fn) fn(kernel, ctas_per_sm);
    return true;
}

// Announces the class of the launch the calling thread is about to make to the profile recorder of the
// capture library (a no-op unless a profile is being recorded): 1 compute-bound, 0 memory-bound.  It stands
// in for the roofline rule of the reference's profile pipeline (profiling/postprocessing/roofline_analysis.py:51-71),
// which compares a kernel's measured arithmetic intensity with the device's FLOP/s-to-bytes/s ratio.
inline void annotate_launch(int op_class, double flop, double bytes) {
    using Fn = void (*)(int, double, double);
    static const Fn fn = reinterpret_cast<Fn>(dlsym(RTLD_DEFAULT, "orion_capture_annotate"));
    if (fn) fn(op_class, flop, bytes);
}

// Grid width of a grid-stride (elementwise, normalisation) kernel as a multiple of the resident CTAs: with 1 every CTA
// stays for the whole launch; with k > 1 the work is cut into k times as many CTAs that retire one after the other, so that
// the blocks of a kernel on a higher-priority stream find a free slot after 1/k of the launch's duration instead of at its
// end.  ORION_ELT_OVERSUB overrides the default.  A launch that the scheduler cuts to its SM quota is persistent again.
inline int grid_oversubscription() {
    static const int v = [] {
        const char* e = getenv("ORION_ELT_OVERSUB");
        int k = e ? atoi(e) : 1;
        return k < 1 ? 1 : (k > 16 ? 16 : k);
    }();
    return v;
}

// Arithmetic intensity (FLOP per byte of HBM traffic) above which a tensor-core kernel is compute-bound on
// a B200: peak FLOP/s of the precision mode over the copy bandwidth, both as measured on this hardware
// (bf16 1660 TFLOP/s, one TF32 pass 727, three TF32 passes 242; 6.54 TB/s).
inline double ai_threshold(int dtype) { return dtype == 1 ? 254.0 : dtype == 2 ? 111.0 : 37.0; }

}  // namespace ob200

// A launcher of an HBM-bound kernel (elementwise, normalisation, pooling, optimizer): memory class.
#define OB200_HBM_BOUND() ::ob200::annotate_launch(0, 0.0, 0.0)

// Registers `kernel` once (first time the enclosing launcher runs); the expression must name the same
// function (template arguments included) that is launched.
#define OB200_ELASTIC(kernel, ctas_per_sm)                                                                  \
    do {                                                                                                    \
        static const bool ob200_elastic_once_ = ::ob200::mark_elastic((const void*)(kernel), (ctas_per_sm)); \
        (void)ob200_elastic_once_;                                                                          \
    } while (0)

// The same for an HBM-bound kernel: elastic, and announced as memory class.
#define OB200_ELASTIC_HBM(kernel, ctas_per_sm) \
    do {                                       \
        OB200_ELASTIC(kernel, ctas_per_sm);    \
        OB200_HBM_BOUND();                     \
    } while (0)
