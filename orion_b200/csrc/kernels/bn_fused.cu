// Training batch norm fused with what surrounds it in the clients' networks (NHWC, float32):
//
//   forward   y = act( (x - mean) * invstd * gamma + beta  [+ residual] )        act: none / ReLU / ReLU6
//   backward  g = dy where the activation passed its input, else 0
//             dx = gamma * invstd * (g - mean(g) - xhat * mean(g * xhat)),  dgamma = sum g * xhat,  dbeta = sum g,
//             dresidual = g
//
// Two launches per direction and no scratch to clear:
//   1. a reduction over a persistent grid: every CTA reduces a slab of rows for a group of channels and adds its
//      partial sums to a double-precision scratch with atomicAdd; the CTA that arrives last on the group's counter
//      FINISHES the group — forward: mean, inverse standard deviation, running statistics; backward: the three
//      per-channel coefficients of dx = a*g + b*x + k and the parameter gradients — and puts the scratch and the
//      counter back to zero, so the next call finds them clean;
//   2. an elementwise pass with per-channel coefficients.
// The backward pass needs no stored mask: without a residual the activation's input is recomputed from x with the
// very instructions the forward pass used (same bits, same decision); with a residual it is read from the saved
// output.  Algorithmic bytes per element: forward 12 B (+4 B with a residual), backward 20 B (+4 B to read the saved
// output and +4 B to write dresidual when there is a residual).
//
// They take the place of cudnnBatchNormalizationForwardTrainingEx / cudnnBatchNormalizationBackwardEx
// (reference src/scheduler/utils_sched.cpp:297-339,398-438) and of the ReLU / residual-add / ReLU-backward
// elementwise kernels that reach the reference through its cudaLaunchKernel trap
// (reference src/cuda_capture/intercept_temp.cpp:418-458).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <mutex>
#include <unordered_map>

#include "elastic.h"
#include "pdl.cuh"

namespace ob200 {

constexpr int BF_THREADS = 256;
constexpr int BF_MAX_C = 8192;

// Activation input of one element, exactly as the forward pass computed it.
__device__ __forceinline__ float bn_affine(float x, float a, float b) { return fmaf(x, a, b); }
__device__ __forceinline__ bool act_passes(float pre, int act) { return act == 0 || (pre > 0.f && (act == 1 || pre < 6.f)); }
__device__ __forceinline__ float act_apply(float v, int act) {
    if (act) v = fmaxf(v, 0.f);
    if (act == 2) v = fminf(v, 6.f);
    return v;
}

struct FinishFwd {
    float* save_mean;
    float* save_invstd;
    float* running_mean;
    float* running_var;
    float eps, momentum;
};
struct FinishBwd {
    const float* gamma;
    const float* mean;
    const float* invstd;
    float* coef;      // [3][C]: a, b, k of dx = a*g + b*x + k
    float* dgamma;
    float* dbeta;
};

// MODE 0: sums of x and x^2.  MODE 1: sums of g and g * xhat, g = dy masked by the activation.
// MASK (MODE 1): 0 no activation, 1 recompute the activation input from x, 2 read the saved output.
template <int MODE, int MASK>
__global__ void __launch_bounds__(BF_THREADS) bn_reduce_finish_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                                     const float* __restrict__ yout, const float* __restrict__ beta,
                                                                     int act, double* __restrict__ sums, int* __restrict__ counters,
                                                                     long long rows, int C, FinishFwd ff, FinishBwd fb) {
    extern __shared__ float sh[];   // [blockDim.y][blockDim.x][8]
    __shared__ int s_last;
    const int cq = blockDim.x, ry = blockDim.y;
    const int c_groups = (C / 4 + cq - 1) / cq;
    const int slabs = gridDim.x / c_groups;   // the launcher makes the grid a multiple of c_groups
    const int cg = blockIdx.x % c_groups, slab = blockIdx.x / c_groups;
    const int c = (cg * cq + threadIdx.x) * 4;
    float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
    if (c < C && slab < slabs) {
        float4 mu = s0, is = s0, fa = s0, fbv = s0;
        if (MODE == 1) {
            mu = __ldg(reinterpret_cast<const float4*>(fb.mean + c));
            is = __ldg(reinterpret_cast<const float4*>(fb.invstd + c));
            if (MASK == 1) {   // forward coefficients: a = invstd * gamma, b = beta - mean * a
                const float4 g = fb.gamma ? __ldg(reinterpret_cast<const float4*>(fb.gamma + c)) : make_float4(1.f, 1.f, 1.f, 1.f);
                const float4 be = beta ? __ldg(reinterpret_cast<const float4*>(beta + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
                fa = make_float4(is.x * g.x, is.y * g.y, is.z * g.z, is.w * g.w);
                fbv = make_float4(be.x - mu.x * fa.x, be.y - mu.y * fa.y, be.z - mu.z * fa.z, be.w - mu.w * fa.w);
            }
        }
        const long long per = (rows + slabs - 1) / slabs;
        const long long r0 = slab * per, r1 = r0 + per < rows ? r0 + per : rows;
        constexpr int U = MODE == 0 ? 8 : 4;   // rows per trip, all loads issued before the first use
        auto acc = [&](const float4& v, const float4& x, const float4& yo) {
            if (MODE == 0) {
                s0.x += v.x; s0.y += v.y; s0.z += v.z; s0.w += v.w;
                s1.x += v.x * v.x; s1.y += v.y * v.y; s1.z += v.z * v.z; s1.w += v.w * v.w;
            } else {
                float4 g = v;
                if (MASK == 1) {
                    if (!act_passes(bn_affine(x.x, fa.x, fbv.x), act)) g.x = 0.f;
                    if (!act_passes(bn_affine(x.y, fa.y, fbv.y), act)) g.y = 0.f;
                    if (!act_passes(bn_affine(x.z, fa.z, fbv.z), act)) g.z = 0.f;
                    if (!act_passes(bn_affine(x.w, fa.w, fbv.w), act)) g.w = 0.f;
                } else if (MASK == 2) {   // the saved output is act(pre): it passed iff the output lies strictly inside the range
                    if (!act_passes(yo.x, act)) g.x = 0.f;
                    if (!act_passes(yo.y, act)) g.y = 0.f;
                    if (!act_passes(yo.z, act)) g.z = 0.f;
                    if (!act_passes(yo.w, act)) g.w = 0.f;
                }
                s0.x += g.x; s0.y += g.y; s0.z += g.z; s0.w += g.w;
                s1.x += g.x * (x.x - mu.x) * is.x; s1.y += g.y * (x.y - mu.y) * is.y;
                s1.z += g.z * (x.z - mu.z) * is.z; s1.w += g.w * (x.w - mu.w) * is.w;
            }
        };
        long long r = r0 + threadIdx.y;
        for (; r + (long long)(U - 1) * ry < r1; r += (long long)U * ry) {
            float4 v[U], x[U], yo[U];
#pragma unroll
            for (int u = 0; u < U; u++) v[u] = __ldcs(reinterpret_cast<const float4*>(a + (r + (long long)u * ry) * C + c));
            if (MODE == 1) {
#pragma unroll
                for (int u = 0; u < U; u++) x[u] = __ldcs(reinterpret_cast<const float4*>(b + (r + (long long)u * ry) * C + c));
                if (MASK == 2) {
#pragma unroll
                    for (int u = 0; u < U; u++) yo[u] = __ldcs(reinterpret_cast<const float4*>(yout + (r + (long long)u * ry) * C + c));
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) acc(v[u], x[u], yo[u]);
        }
        for (; r < r1; r += ry) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(a + r * C + c));
            float4 x = v, yo = v;
            if (MODE == 1) {
                x = __ldcs(reinterpret_cast<const float4*>(b + r * C + c));
                if (MASK == 2) yo = __ldcs(reinterpret_cast<const float4*>(yout + r * C + c));
            }
            acc(v, x, yo);
        }
    }
    float* mine = sh + ((size_t)threadIdx.y * cq + threadIdx.x) * 8;
    mine[0] = s0.x; mine[1] = s0.y; mine[2] = s0.z; mine[3] = s0.w;
    mine[4] = s1.x; mine[5] = s1.y; mine[6] = s1.z; mine[7] = s1.w;
    __syncthreads();
    for (int half = ry / 2; half > 0; half >>= 1) {
        if ((int)threadIdx.y < half) {
            const float* other = sh + ((size_t)(threadIdx.y + half) * cq + threadIdx.x) * 8;
#pragma unroll
            for (int k = 0; k < 8; k++) mine[k] += other[k];
        }
        __syncthreads();
    }
    if (threadIdx.y == 0 && c < C) {
#pragma unroll
        for (int k = 0; k < 4; k++) {
            atomicAdd(sums + c + k, (double)mine[k]);
            atomicAdd(sums + C + c + k, (double)mine[4 + k]);
        }
    }
    // The CTA that arrives last on its channel group's counter finishes the group.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0 && threadIdx.y == 0) s_last = atomicAdd(counters + cg, 1) == slabs - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.y == 0 && c < C) {
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const double sa = __ldcg(sums + c + k), sb = __ldcg(sums + C + c + k);
            sums[c + k] = 0.0;
            sums[C + c + k] = 0.0;
            if (MODE == 0) {
                const double m = sa / (double)rows;
                double var = sb / (double)rows - m * m;
                if (var < 0) var = 0;
                ff.save_mean[c + k] = (float)m;
                ff.save_invstd[c + k] = (float)(1.0 / sqrt(var + (double)ff.eps));
                if (ff.running_mean) ff.running_mean[c + k] = (1.f - ff.momentum) * ff.running_mean[c + k] + ff.momentum * (float)m;
                if (ff.running_var) {
                    const double unbiased = rows > 1 ? var * (double)rows / (double)(rows - 1) : var;
                    ff.running_var[c + k] = (1.f - ff.momentum) * ff.running_var[c + k] + ff.momentum * (float)unbiased;
                }
            } else {
                const float g = fb.gamma ? fb.gamma[c + k] : 1.f;
                const float m = fb.mean[c + k], is = fb.invstd[c + k];
                const float sd = (float)sa, sx = (float)sb;
                const float inv_rows = 1.0f / (float)rows;
                const float aa = g * is;
                const float bb = -aa * is * sx * inv_rows;
                fb.coef[c + k] = aa;
                fb.coef[C + c + k] = bb;
                fb.coef[2 * C + c + k] = -aa * sd * inv_rows - bb * m;
                if (fb.dbeta) fb.dbeta[c + k] = sd;
                if (fb.dgamma) fb.dgamma[c + k] = sx;
            }
        }
    }
    if (threadIdx.x == 0 && threadIdx.y == 0) counters[cg] = 0;
}

// y = act(x * a + b [+ residual]) with a = invstd * gamma, b = beta - mean * a.  When the grid stride is a multiple of
// the channel-quad count a thread stays on one channel quad and computes its coefficients once.
template <bool RES>
__global__ void __launch_bounds__(BF_THREADS) bn_act_apply_kernel(const float4* __restrict__ x, const float4* __restrict__ res,
                                                                 float4* __restrict__ y, const float* __restrict__ gamma,
                                                                 const float* __restrict__ beta, const float* __restrict__ mean,
                                                                 const float* __restrict__ invstd, long long n4, int c4, int act) {
    pdl_launch_dependents();   // a convolution behind this kernel may set itself up meanwhile (pdl.cuh)
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    auto coef = [&](int c, float4& a, float4& b) {
        const float4 m = __ldg(reinterpret_cast<const float4*>(mean + c));
        const float4 is = __ldg(reinterpret_cast<const float4*>(invstd + c));
        float4 g = make_float4(1.f, 1.f, 1.f, 1.f), be = make_float4(0.f, 0.f, 0.f, 0.f);
        if (gamma) g = __ldg(reinterpret_cast<const float4*>(gamma + c));
        if (beta) be = __ldg(reinterpret_cast<const float4*>(beta + c));
        a = make_float4(is.x * g.x, is.y * g.y, is.z * g.z, is.w * g.w);
        b = make_float4(be.x - m.x * a.x, be.y - m.y * a.y, be.z - m.z * a.z, be.w - m.w * a.w);
    };
    auto one = [&](const float4& v, const float4& r, const float4& a, const float4& b) {
        float4 o = make_float4(bn_affine(v.x, a.x, b.x), bn_affine(v.y, a.y, b.y), bn_affine(v.z, a.z, b.z), bn_affine(v.w, a.w, b.w));
        if (RES) { o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w; }
        return make_float4(act_apply(o.x, act), act_apply(o.y, act), act_apply(o.z, act), act_apply(o.w, act));
    };
    if (stride % c4 == 0) {
        if (i >= n4) return;
        float4 a, b;
        coef((int)(i % c4) * 4, a, b);
        constexpr int U = RES ? 2 : 4;
        for (; i + (U - 1) * stride < n4; i += U * stride) {
            float4 v[U], r[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                v[u] = __ldcs(x + i + u * stride);
                if (RES) r[u] = __ldcs(res + i + u * stride);
            }
#pragma unroll
            for (int u = 0; u < U; u++) y[i + u * stride] = one(v[u], r[u], a, b);
        }
        for (; i < n4; i += stride) {
            const float4 v = __ldcs(x + i);
            y[i] = one(v, RES ? __ldcs(res + i) : v, a, b);
        }
        return;
    }
    for (; i < n4; i += stride) {
        float4 a, b;
        coef((int)(i % c4) * 4, a, b);
        const float4 v = __ldcs(x + i);
        y[i] = one(v, RES ? __ldcs(res + i) : v, a, b);
    }
}

// dx = a*g + b*x + k with g = dy masked by the activation; dres = g.
template <int MASK, bool DRES>
__global__ void __launch_bounds__(BF_THREADS) bn_act_backward_apply_kernel(const float4* __restrict__ dy, const float4* __restrict__ x,
                                                                          const float4* __restrict__ yout, float4* __restrict__ dx,
                                                                          float4* __restrict__ dres, const float* __restrict__ coefs,
                                                                          const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                          const float* __restrict__ mean,
                                                                          const float* __restrict__ invstd, long long n4, int c4,
                                                                          int act) {
    pdl_launch_dependents();   // a convolution behind this kernel may set itself up meanwhile (pdl.cuh)
    const int C = c4 * 4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    struct Co { float4 a, b, k, fa, fb; };
    auto coef = [&](int c, Co& o) {
        o.a = __ldg(reinterpret_cast<const float4*>(coefs + c));
        o.b = __ldg(reinterpret_cast<const float4*>(coefs + C + c));
        o.k = __ldg(reinterpret_cast<const float4*>(coefs + 2 * C + c));
        if (MASK == 1) {
            const float4 m = __ldg(reinterpret_cast<const float4*>(mean + c));
            const float4 is = __ldg(reinterpret_cast<const float4*>(invstd + c));
            const float4 g = gamma ? __ldg(reinterpret_cast<const float4*>(gamma + c)) : make_float4(1.f, 1.f, 1.f, 1.f);
            const float4 be = beta ? __ldg(reinterpret_cast<const float4*>(beta + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
            o.fa = make_float4(is.x * g.x, is.y * g.y, is.z * g.z, is.w * g.w);
            o.fb = make_float4(be.x - m.x * o.fa.x, be.y - m.y * o.fa.y, be.z - m.z * o.fa.z, be.w - m.w * o.fa.w);
        }
    };
    auto one = [&](long long idx, const float4& d, const float4& v, const float4& yo, const Co& o) {
        float4 g = d;
        if (MASK == 1) {
            if (!act_passes(bn_affine(v.x, o.fa.x, o.fb.x), act)) g.x = 0.f;
            if (!act_passes(bn_affine(v.y, o.fa.y, o.fb.y), act)) g.y = 0.f;
            if (!act_passes(bn_affine(v.z, o.fa.z, o.fb.z), act)) g.z = 0.f;
            if (!act_passes(bn_affine(v.w, o.fa.w, o.fb.w), act)) g.w = 0.f;
        } else if (MASK == 2) {
            if (!act_passes(yo.x, act)) g.x = 0.f;
            if (!act_passes(yo.y, act)) g.y = 0.f;
            if (!act_passes(yo.z, act)) g.z = 0.f;
            if (!act_passes(yo.w, act)) g.w = 0.f;
        }
        if (DRES) dres[idx] = g;
        dx[idx] = make_float4(fmaf(o.a.x, g.x, fmaf(o.b.x, v.x, o.k.x)), fmaf(o.a.y, g.y, fmaf(o.b.y, v.y, o.k.y)),
                              fmaf(o.a.z, g.z, fmaf(o.b.z, v.z, o.k.z)), fmaf(o.a.w, g.w, fmaf(o.b.w, v.w, o.k.w)));
    };
    if (stride % c4 == 0) {
        if (i >= n4) return;
        Co o;
        coef((int)(i % c4) * 4, o);
        for (; i + stride < n4; i += 2 * stride) {
            float4 d[2], v[2], yo[2];
#pragma unroll
            for (int u = 0; u < 2; u++) {
                d[u] = __ldcs(dy + i + u * stride);
                v[u] = __ldcs(x + i + u * stride);
                if (MASK == 2) yo[u] = __ldcs(yout + i + u * stride);
            }
#pragma unroll
            for (int u = 0; u < 2; u++) one(i + u * stride, d[u], v[u], yo[u], o);
        }
        for (; i < n4; i += stride) {
            const float4 v = __ldcs(x + i);
            one(i, __ldcs(dy + i), v, MASK == 2 ? __ldcs(yout + i) : v, o);
        }
        return;
    }
    for (; i < n4; i += stride) {
        Co o;
        coef((int)(i % c4) * 4, o);
        const float4 v = __ldcs(x + i);
        one(i, __ldcs(dy + i), v, MASK == 2 ? __ldcs(yout + i) : v, o);
    }
}

// Per-(device, stream) scratch: double sums and group counters (both zero between calls: the finishing CTA cleans
// up), and the coefficient table of the backward pass (overwritten by every call).  Calls on one stream are ordered,
// which is all the kernels rely on.
struct BnScratch {
    double* sums = nullptr;
    int* counters = nullptr;
    float* coef = nullptr;
};
static std::mutex g_bn_mu;
static std::unordered_map<uint64_t, BnScratch> g_bn_scratch;

static BnScratch* bn_scratch_for(cudaStream_t s) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    const uint64_t key = ((uint64_t)dev << 56) ^ (uint64_t)(uintptr_t)s;
    thread_local uint64_t cached_key = ~0ull;
    thread_local BnScratch* cached = nullptr;
    if (key == cached_key && cached) return cached;
    std::lock_guard<std::mutex> lk(g_bn_mu);
    auto it = g_bn_scratch.find(key);
    if (it == g_bn_scratch.end()) {
        BnScratch sc;
        if (cudaMalloc(&sc.sums, 2 * BF_MAX_C * sizeof(double)) != cudaSuccess) return nullptr;
        if (cudaMalloc(&sc.counters, BF_MAX_C / 4 * sizeof(int)) != cudaSuccess) return nullptr;
        if (cudaMalloc(&sc.coef, 3 * BF_MAX_C * sizeof(float)) != cudaSuccess) return nullptr;
        cudaMemsetAsync(sc.sums, 0, 2 * BF_MAX_C * sizeof(double), s);
        cudaMemsetAsync(sc.counters, 0, BF_MAX_C / 4 * sizeof(int), s);
        it = g_bn_scratch.emplace(key, sc).first;
    }
    cached_key = key;
    cached = &it->second;   // entries are never erased; unordered_map nodes do not move
    return cached;
}

struct ReduceShape {
    int cq, ry, c_groups;
    long long slabs;
};
static ReduceShape reduce_shape(long long rows, int C, int num_ctas) {
    ReduceShape r;
    r.cq = C / 4 < 32 ? C / 4 : 32;   // channel quads per CTA (x); row lanes (y) fill up to 256 threads
    int ry = BF_THREADS / r.cq, pow2 = 1;
    while (pow2 * 2 <= ry) pow2 *= 2;
    r.ry = pow2;
    r.c_groups = (C / 4 + r.cq - 1) / r.cq;
    r.slabs = (long long)num_ctas * 2 / r.c_groups;
    if (r.slabs > (rows + r.ry - 1) / r.ry) r.slabs = (rows + r.ry - 1) / r.ry;
    if (r.slabs < 1) r.slabs = 1;
    return r;
}

static inline int apply_grid(long long items, int num_ctas, int per_sm, int c4) {
    long long want = (items + BF_THREADS - 1) / BF_THREADS, cap = (long long)num_ctas * per_sm * grid_oversubscription();
    if (want < 1) want = 1;
    int g = (int)(want < cap ? want : cap);
    int need = 1;   // smallest grid multiple that makes grid * BF_THREADS divisible by c4
    while (((long long)need * BF_THREADS) % c4 != 0 && need < 4096) need++;
    if (need > 1 && g >= need && need <= 64) g -= g % need;
    return g;
}

}  // namespace ob200

using namespace ob200;

// y = act(batch_norm_train(x) [+ residual]); act 0 none, 1 ReLU, 2 ReLU6.  x, residual, y: [rows, C] float32, C % 4 == 0,
// C <= 8192.  Writes save_mean / save_invstd [C] and updates the running statistics (either may be NULL).
extern "C" int ob200_bn_act_train_forward_f32(const float* x, const float* residual, float* y, const float* gamma, const float* beta,
                                              float* running_mean, float* running_var, float* save_mean, float* save_invstd,
                                              float eps, float momentum, long long rows, int C, int act, int num_ctas, void* stream) {
    if (rows <= 0) return 0;
    if (C <= 0 || (C & 3) || C > BF_MAX_C || num_ctas <= 0 || !save_mean || !save_invstd || act < 0 || act > 2) return -1;
    if (((uintptr_t)x | (uintptr_t)residual | (uintptr_t)y | (uintptr_t)gamma | (uintptr_t)beta | (uintptr_t)save_mean |
         (uintptr_t)save_invstd) % 16)
        return -2;
    cudaStream_t s = (cudaStream_t)stream;
    BnScratch* sc = bn_scratch_for(s);
    if (!sc) return -1;
    const ReduceShape rs = reduce_shape(rows, C, num_ctas);
    FinishFwd ff{save_mean, save_invstd, running_mean, running_var, eps, momentum};
    FinishBwd fb{};
    OB200_HBM_BOUND();
    bn_reduce_finish_kernel<0, 0><<<(unsigned)(rs.slabs * rs.c_groups), dim3(rs.cq, rs.ry), (size_t)rs.cq * rs.ry * 8 * sizeof(float), s>>>(
        x, nullptr, nullptr, nullptr, 0, sc->sums, sc->counters, rows, C, ff, fb);
    const long long n4 = rows * C / 4;
    const int grid = apply_grid(n4, num_ctas, 6, C / 4);
    if (residual) {
        OB200_ELASTIC_HBM(bn_act_apply_kernel<true>, 6);
        bn_act_apply_kernel<true><<<grid, BF_THREADS, 0, s>>>((const float4*)x, (const float4*)residual, (float4*)y, gamma, beta, save_mean,
                                                              save_invstd, n4, C / 4, act);
    } else {
        OB200_ELASTIC_HBM(bn_act_apply_kernel<false>, 6);
        bn_act_apply_kernel<false><<<grid, BF_THREADS, 0, s>>>((const float4*)x, nullptr, (float4*)y, gamma, beta, save_mean, save_invstd, n4,
                                                               C / 4, act);
    }
    return (int)cudaGetLastError();
}

// Backward of the above.  yout: the saved output of the forward pass, needed (and read) only when the forward pass had a
// residual and an activation; otherwise pass NULL and the activation's input is recomputed from x.  dres receives the
// gradient of the residual (NULL when there was none).  dgamma / dbeta may be NULL.
extern "C" int ob200_bn_act_backward_f32(const float* dy, const float* x, const float* yout, float* dx, float* dres, const float* gamma,
                                         const float* beta, const float* save_mean, const float* save_invstd, float* dgamma,
                                         float* dbeta, long long rows, int C, int act, int num_ctas, void* stream) {
    if (rows <= 0) return 0;
    if (C <= 0 || (C & 3) || C > BF_MAX_C || num_ctas <= 0 || act < 0 || act > 2) return -1;
    if (((uintptr_t)dy | (uintptr_t)x | (uintptr_t)yout | (uintptr_t)dx | (uintptr_t)dres | (uintptr_t)gamma | (uintptr_t)beta |
         (uintptr_t)save_mean | (uintptr_t)save_invstd) % 16)
        return -2;
    cudaStream_t s = (cudaStream_t)stream;
    BnScratch* sc = bn_scratch_for(s);
    if (!sc) return -1;
    const int mask = act == 0 ? 0 : (yout ? 2 : 1);
    const ReduceShape rs = reduce_shape(rows, C, num_ctas);
    FinishFwd ff{};
    FinishBwd fb{gamma, save_mean, save_invstd, sc->coef, dgamma, dbeta};
    const unsigned rgrid = (unsigned)(rs.slabs * rs.c_groups);
    const dim3 rblock(rs.cq, rs.ry);
    const size_t rsmem = (size_t)rs.cq * rs.ry * 8 * sizeof(float);
    OB200_HBM_BOUND();
    if (mask == 0)
        bn_reduce_finish_kernel<1, 0><<<rgrid, rblock, rsmem, s>>>(dy, x, nullptr, beta, act, sc->sums, sc->counters, rows, C, ff, fb);
    else if (mask == 1)
        bn_reduce_finish_kernel<1, 1><<<rgrid, rblock, rsmem, s>>>(dy, x, nullptr, beta, act, sc->sums, sc->counters, rows, C, ff, fb);
    else
        bn_reduce_finish_kernel<1, 2><<<rgrid, rblock, rsmem, s>>>(dy, x, yout, beta, act, sc->sums, sc->counters, rows, C, ff, fb);
    const long long n4 = rows * C / 4;
    const int grid = apply_grid(n4, num_ctas, 6, C / 4);
#define OB200_BWD(MASK, DRES)                                                                                                          \
    do {                                                                                                                              \
        OB200_ELASTIC_HBM((bn_act_backward_apply_kernel<MASK, DRES>), 6);                                                              \
        bn_act_backward_apply_kernel<MASK, DRES><<<grid, BF_THREADS, 0, s>>>((const float4*)dy, (const float4*)x, (const float4*)yout, \
                                                                             (float4*)dx, (float4*)dres, sc->coef, gamma, beta,       \
                                                                             save_mean, save_invstd, n4, C / 4, act);                 \
    } while (0)
    if (dres) {
        if (mask == 0) OB200_BWD(0, true);
        else if (mask == 1) OB200_BWD(1, true);
        else OB200_BWD(2, true);
    } else {
        if (mask == 0) OB200_BWD(0, false);
        else if (mask == 1) OB200_BWD(1, false);
        else OB200_BWD(2, false);
    }
#undef OB200_BWD
    return (int)cudaGetLastError();
}
