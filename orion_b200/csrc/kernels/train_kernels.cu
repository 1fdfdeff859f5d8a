// HBM-bound kernels of the training clients (NHWC, float32): batch-norm training forward and
// backward, ReLU backward, the filter re-layout the data-gradient convolution needs, and the
// SGD-with-momentum update.  They stand in for cudnnBatchNormalizationForwardTrainingEx /
// cudnnBatchNormalizationBackwardEx (reference src/scheduler/utils_sched.cpp:297-339,398-438) and
// for the at::native elementwise / foreach kernels that reach the reference through its
// cudaLaunchKernel trap (reference src/cuda_capture/intercept_temp.cpp:418-458).
//
// Batch-norm statistics are reduced in two steps: every CTA of a persistent grid reduces a slab
// of rows per channel (float per thread, shared-memory tree per CTA) and adds its partial sums to
// a double-precision scratch of 2*C entries with atomicAdd; a second kernel normalises.  The
// caller zeroes the scratch (a cudaMemsetAsync on the same stream).
// Algorithmic bytes per element: forward 3x4 B (read for statistics, read + write to normalise),
// backward 5x4 B (dy and x twice, dx once).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include "elastic.h"

namespace ob200 {

constexpr int TR_THREADS = 256;

// ------------------------------------------------------------------ per-channel reductions
// Threads are laid out as (row lane, channel quad): blockDim.x = cq threads cover 4*cq channels,
// blockDim.y row lanes stride over the rows of the CTA's slab.  mode 0: sum x, sum x^2.
// mode 1: sum dy, sum dy * xhat  with xhat = (x - mean) * invstd.
__global__ void __launch_bounds__(TR_THREADS) bn_reduce_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                              const float* __restrict__ mean, const float* __restrict__ invstd,
                                                              double* __restrict__ out, long long rows, int C, int mode) {
    extern __shared__ float sh[];   // [blockDim.y][blockDim.x][8]
    const int cq = blockDim.x, ry = blockDim.y;
    const int c_groups = (C / 4 + cq - 1) / cq;
    const int slabs = gridDim.x / c_groups > 0 ? gridDim.x / c_groups : 1;
    const int cg = blockIdx.x % c_groups, slab = blockIdx.x / c_groups;
    if (slab >= slabs) return;
    const int c = (cg * cq + threadIdx.x) * 4;
    float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
    if (c < C) {
        float4 mu = s0, is = s0;
        if (mode == 1) {
            mu = __ldg(reinterpret_cast<const float4*>(mean + c));
            is = __ldg(reinterpret_cast<const float4*>(invstd + c));
        }
        const long long per = (rows + slabs - 1) / slabs;
        const long long r0 = slab * per, r1 = r0 + per < rows ? r0 + per : rows;
        // Eight rows per trip, all loads issued before the first use: the kernel is bound by bytes in flight.
        constexpr int U = 8;
        long long r = r0 + threadIdx.y;
        for (; r + (long long)(U - 1) * ry < r1; r += (long long)U * ry) {
            float4 v[U], x[U];
#pragma unroll
            for (int u = 0; u < U; u++) v[u] = __ldcs(reinterpret_cast<const float4*>(a + (r + (long long)u * ry) * C + c));
            if (mode == 1) {
#pragma unroll
                for (int u = 0; u < U; u++) x[u] = __ldcs(reinterpret_cast<const float4*>(b + (r + (long long)u * ry) * C + c));
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                s0.x += v[u].x; s0.y += v[u].y; s0.z += v[u].z; s0.w += v[u].w;
                if (mode == 0) {
                    s1.x += v[u].x * v[u].x; s1.y += v[u].y * v[u].y; s1.z += v[u].z * v[u].z; s1.w += v[u].w * v[u].w;
                } else {
                    s1.x += v[u].x * (x[u].x - mu.x) * is.x; s1.y += v[u].y * (x[u].y - mu.y) * is.y;
                    s1.z += v[u].z * (x[u].z - mu.z) * is.z; s1.w += v[u].w * (x[u].w - mu.w) * is.w;
                }
            }
        }
        for (; r < r1; r += ry) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(a + r * C + c));
            s0.x += v.x; s0.y += v.y; s0.z += v.z; s0.w += v.w;
            if (mode == 0) {
                s1.x += v.x * v.x; s1.y += v.y * v.y; s1.z += v.z * v.z; s1.w += v.w * v.w;
            } else {
                const float4 x = __ldcs(reinterpret_cast<const float4*>(b + r * C + c));
                s1.x += v.x * (x.x - mu.x) * is.x; s1.y += v.y * (x.y - mu.y) * is.y;
                s1.z += v.z * (x.z - mu.z) * is.z; s1.w += v.w * (x.w - mu.w) * is.w;
            }
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
            atomicAdd(out + c + k, (double)mine[k]);
            atomicAdd(out + C + c + k, (double)mine[4 + k]);
        }
    }
}

// Finish the statistics (one thread per channel): mean, inverse std, running-stat update.
__global__ void bn_stats_finish_kernel(const double* __restrict__ sums, float* __restrict__ save_mean,
                                       float* __restrict__ save_invstd, float* __restrict__ running_mean,
                                       float* __restrict__ running_var, long long rows, int C, float eps, float momentum) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const double m = sums[c] / (double)rows;
    double var = sums[C + c] / (double)rows - m * m;
    if (var < 0) var = 0;
    save_mean[c] = (float)m;
    save_invstd[c] = (float)(1.0 / sqrt(var + (double)eps));
    if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * (float)m;
    if (running_var) {
        const double unbiased = rows > 1 ? var * (double)rows / (double)(rows - 1) : var;
        running_var[c] = (1.f - momentum) * running_var[c] + momentum * (float)unbiased;
    }
}

// y = (x - mean) * invstd * gamma + beta.
// When the grid stride is a multiple of the channel-quad count every thread stays on one channel quad,
// so the per-channel coefficients are computed once per thread and the loop is loads, FMAs and stores.
__global__ void __launch_bounds__(TR_THREADS) bn_apply_kernel(const float4* __restrict__ x, float4* __restrict__ y,
                                                             const float* __restrict__ gamma, const float* __restrict__ beta,
                                                             const float* __restrict__ mean, const float* __restrict__ invstd,
                                                             long long n4, int c4) {
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
    if (stride % c4 == 0) {
        if (i >= n4) return;
        float4 a, b;
        coef((int)(i % c4) * 4, a, b);
        for (; i + 3 * stride < n4; i += 4 * stride) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u] = __ldcs(x + i + u * stride);
#pragma unroll
            for (int u = 0; u < 4; u++)
                y[i + u * stride] = make_float4(fmaf(v[u].x, a.x, b.x), fmaf(v[u].y, a.y, b.y), fmaf(v[u].z, a.z, b.z), fmaf(v[u].w, a.w, b.w));
        }
        for (; i < n4; i += stride) {
            const float4 v = __ldcs(x + i);
            y[i] = make_float4(fmaf(v.x, a.x, b.x), fmaf(v.y, a.y, b.y), fmaf(v.z, a.z, b.z), fmaf(v.w, a.w, b.w));
        }
        return;
    }
    for (; i < n4; i += stride) {
        float4 a, b;
        coef((int)(i % c4) * 4, a, b);
        const float4 v = __ldcs(x + i);
        y[i] = make_float4(fmaf(v.x, a.x, b.x), fmaf(v.y, a.y, b.y), fmaf(v.z, a.z, b.z), fmaf(v.w, a.w, b.w));
    }
}

// dx = gamma * invstd * (dy - sum_dy/M - xhat * sum_dy_xhat/M) = a*dy + b*x + c per channel;
// dgamma = sum_dy_xhat, dbeta = sum_dy.  Same fixed-channel fast path as bn_apply_kernel.
__global__ void __launch_bounds__(TR_THREADS) bn_backward_apply_kernel(const float4* __restrict__ dy, const float4* __restrict__ x,
                                                                      float4* __restrict__ dx, const float* __restrict__ gamma,
                                                                      const float* __restrict__ mean,
                                                                      const float* __restrict__ invstd,
                                                                      const double* __restrict__ sums, float* __restrict__ dgamma,
                                                                      float* __restrict__ dbeta, long long n4, int c4,
                                                                      long long rows) {
    const int C = c4 * 4;
    const float inv_rows = 1.0f / (float)rows;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    auto coef = [&](int c, bool publish, float4& a, float4& b, float4& k) {
        const float4 g = gamma ? __ldg(reinterpret_cast<const float4*>(gamma + c)) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 m = __ldg(reinterpret_cast<const float4*>(mean + c));
        const float4 is = __ldg(reinterpret_cast<const float4*>(invstd + c));
        const float sd[4] = {(float)sums[c], (float)sums[c + 1], (float)sums[c + 2], (float)sums[c + 3]};
        const float sx[4] = {(float)sums[C + c], (float)sums[C + c + 1], (float)sums[C + c + 2], (float)sums[C + c + 3]};
        const float gg[4] = {g.x, g.y, g.z, g.w}, mm[4] = {m.x, m.y, m.z, m.w}, ii[4] = {is.x, is.y, is.z, is.w};
        float aa[4], bb[4], kk[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            aa[e] = gg[e] * ii[e];
            bb[e] = -aa[e] * ii[e] * sx[e] * inv_rows;
            kk[e] = -aa[e] * sd[e] * inv_rows - bb[e] * mm[e];
        }
        a = make_float4(aa[0], aa[1], aa[2], aa[3]);
        b = make_float4(bb[0], bb[1], bb[2], bb[3]);
        k = make_float4(kk[0], kk[1], kk[2], kk[3]);
        if (publish) {   // the first row's threads also publish the parameter gradients
            if (dbeta) { dbeta[c] = sd[0]; dbeta[c + 1] = sd[1]; dbeta[c + 2] = sd[2]; dbeta[c + 3] = sd[3]; }
            if (dgamma) { dgamma[c] = sx[0]; dgamma[c + 1] = sx[1]; dgamma[c + 2] = sx[2]; dgamma[c + 3] = sx[3]; }
        }
    };
    auto apply = [](const float4& d, const float4& v, const float4& a, const float4& b, const float4& k) {
        return make_float4(fmaf(a.x, d.x, fmaf(b.x, v.x, k.x)), fmaf(a.y, d.y, fmaf(b.y, v.y, k.y)), fmaf(a.z, d.z, fmaf(b.z, v.z, k.z)),
                           fmaf(a.w, d.w, fmaf(b.w, v.w, k.w)));
    };
    if (stride % c4 == 0) {
        if (i >= n4) return;
        float4 a, b, k;
        coef((int)(i % c4) * 4, i < c4, a, b, k);
        for (; i + stride < n4; i += 2 * stride) {
            float4 d[2], v[2];
#pragma unroll
            for (int u = 0; u < 2; u++) { d[u] = __ldcs(dy + i + u * stride); v[u] = __ldcs(x + i + u * stride); }
#pragma unroll
            for (int u = 0; u < 2; u++) dx[i + u * stride] = apply(d[u], v[u], a, b, k);
        }
        for (; i < n4; i += stride) dx[i] = apply(__ldcs(dy + i), __ldcs(x + i), a, b, k);
        return;
    }
    for (; i < n4; i += stride) {
        float4 a, b, k;
        coef((int)(i % c4) * 4, i < c4, a, b, k);
        dx[i] = apply(__ldcs(dy + i), __ldcs(x + i), a, b, k);
    }
}

// dx = dy where y > 0 else 0
__global__ void __launch_bounds__(TR_THREADS) relu_backward_kernel(const float4* __restrict__ dy, const float4* __restrict__ y,
                                                                  float4* __restrict__ dx, long long n4) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        const float4 d = __ldcs(dy + i), v = __ldcs(y + i);
        dx[i] = make_float4(v.x > 0.f ? d.x : 0.f, v.y > 0.f ? d.y : 0.f, v.z > 0.f ? d.z : 0.f, v.w > 0.f ? d.w : 0.f);
    }
}
__global__ void relu_backward_tail_kernel(const float* dy, const float* y, float* dx, long long begin, long long n) {
    for (long long i = begin + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dx[i] = y[i] > 0.f ? dy[i] : 0.f;
}

// Filter re-layout for the data gradient: w[K][RS][C] -> wt[C][RS][K] (element size 4 or 2 bytes).
template <typename E>
__global__ void __launch_bounds__(TR_THREADS) filter_transpose_kernel(const E* __restrict__ w, E* __restrict__ wt, int K, int RS,
                                                                     int C) {
    __shared__ E tile[32][33];
    const int rs = blockIdx.z;
    const int k0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
    for (int j = ty; j < 32; j += 8) {
        const int k = k0 + j, c = c0 + tx;
        if (k < K && c < C) tile[j][tx] = w[((long long)k * RS + rs) * C + c];
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        const int c = c0 + j, k = k0 + tx;
        if (k < K && c < C) wt[((long long)c * RS + rs) * K + k] = tile[tx][j];
    }
}

// SGD with momentum (torch.optim.SGD semantics, dampening 0): g += wd*p; m = mu*m + g (m = g on the
// first step); p -= lr * (nesterov ? g + mu*m : m).  20 B per parameter.
__global__ void __launch_bounds__(TR_THREADS) sgd_momentum_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                                 float* __restrict__ m, long long n, float lr, float mu, float wd,
                                                                 int nesterov, int first_step) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float grad = g[i] + wd * p[i];
        float mom = first_step ? grad : mu * m[i] + grad;
        m[i] = mom;
        p[i] -= lr * (nesterov ? grad + mu * mom : mom);
    }
}

// The same update for a whole list of parameter tensors in one launch.  The pointers travel in the kernel's parameter
// block (no table in device memory to build or copy); the work is cut into chunks of SGD_CHUNK elements and the blocks of
// a persistent grid walk the chunks.
constexpr int SGD_MAX_TENSORS = 96;
constexpr int SGD_CHUNK = 16384;
struct SgdTable {
    float* p[SGD_MAX_TENSORS];
    const float* g[SGD_MAX_TENSORS];
    float* m[SGD_MAX_TENSORS];
    int first_chunk[SGD_MAX_TENSORS + 1];   // prefix sum of ceil(n / SGD_CHUNK)
    long long n[SGD_MAX_TENSORS];
    int count;
};
__global__ void __launch_bounds__(TR_THREADS) sgd_momentum_multi_kernel(const __grid_constant__ SgdTable t, float lr, float mu, float wd,
                                                                       int nesterov, int first_step) {
    const int total_chunks = t.first_chunk[t.count];
    for (int chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
        int lo = 0, hi = t.count - 1;   // last tensor whose first chunk is <= chunk
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (t.first_chunk[mid] <= chunk) lo = mid; else hi = mid - 1;
        }
        const long long begin = (long long)(chunk - t.first_chunk[lo]) * SGD_CHUNK;
        const long long end = begin + SGD_CHUNK < t.n[lo] ? begin + SGD_CHUNK : t.n[lo];
        float* __restrict__ p = t.p[lo];
        const float* __restrict__ g = t.g[lo];
        float* __restrict__ m = t.m[lo];
        if ((((uintptr_t)p | (uintptr_t)g | (uintptr_t)m) & 15) == 0) {
            const long long e4 = begin + ((end - begin) & ~3LL);
            for (long long i = begin + 4LL * threadIdx.x; i < e4; i += 4LL * blockDim.x) {
                float4 pv = *reinterpret_cast<float4*>(p + i);
                const float4 gv = __ldcs(reinterpret_cast<const float4*>(g + i));
                float4 mv = first_step ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<float4*>(m + i);
                float* pe = &pv.x;
                float* me = &mv.x;
                const float* ge = &gv.x;
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float grad = ge[e] + wd * pe[e];
                    const float mom = first_step ? grad : mu * me[e] + grad;
                    me[e] = mom;
                    pe[e] -= lr * (nesterov ? grad + mu * mom : mom);
                }
                *reinterpret_cast<float4*>(m + i) = mv;
                *reinterpret_cast<float4*>(p + i) = pv;
            }
            for (long long i = e4 + threadIdx.x; i < end; i += blockDim.x) {
                const float grad = g[i] + wd * p[i];
                const float mom = first_step ? grad : mu * m[i] + grad;
                m[i] = mom;
                p[i] -= lr * (nesterov ? grad + mu * mom : mom);
            }
        } else {
            for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
                const float grad = g[i] + wd * p[i];
                const float mom = first_step ? grad : mu * m[i] + grad;
                m[i] = mom;
                p[i] -= lr * (nesterov ? grad + mu * mom : mom);
            }
        }
    }
}

// Grid for the per-channel elementwise kernels: like grid_for, rounded down so that the grid stride (grid *
// TR_THREADS float4 elements) is a multiple of the channel-quad count whenever that costs little.
static inline int grid_for_channels(long long items, int num_ctas, int per_sm, int c4);

static inline int grid_for(long long items, int num_ctas, int per_sm) {
    long long want = (items + TR_THREADS - 1) / TR_THREADS;
    long long cap = (long long)num_ctas * per_sm * grid_oversubscription();
    if (want < 1) want = 1;
    return (int)(want < cap ? want : cap);
}

static inline int grid_for_channels(long long items, int num_ctas, int per_sm, int c4) {
    int g = grid_for(items, num_ctas, per_sm);
    int need = 1;   // smallest grid multiple that makes grid * TR_THREADS divisible by c4
    while (((long long)need * TR_THREADS) % c4 != 0 && need < 4096) need++;
    if (need > 1 && g >= need && need <= 64) g -= g % need;
    return g;
}

static cudaError_t launch_reduce(const float* a, const float* b, const float* mean, const float* invstd, double* out, long long rows,
                                 int C, int mode, int num_ctas, cudaStream_t s) {
    int cq = C / 4 < 32 ? C / 4 : 32;   // channel quads per CTA (x); rows lanes (y) fill up to 256 threads
    int ry = TR_THREADS / cq;
    int pow2 = 1;
    while (pow2 * 2 <= ry) pow2 *= 2;
    ry = pow2;
    const int c_groups = (C / 4 + cq - 1) / cq;
    static const int slab_factor = getenv("ORION_BN_SLABS") ? atoi(getenv("ORION_BN_SLABS")) : 2;
    long long slabs = (long long)num_ctas * slab_factor / c_groups;
    if (slabs < 1) slabs = 1;
    if (slabs > (rows + ry - 1) / ry) slabs = (rows + ry - 1) / ry;
    if (slabs < 1) slabs = 1;
    dim3 block(cq, ry);
    OB200_HBM_BOUND();
    bn_reduce_kernel<<<(unsigned)(slabs * c_groups), block, (size_t)cq * ry * 8 * sizeof(float), s>>>(a, b, mean, invstd, out, rows,
                                                                                                        C, mode);
    return cudaGetLastError();
}

}  // namespace ob200

using namespace ob200;

// x, y: [rows, C] float32 with C % 4 == 0; sums: 2*C doubles, zero on entry (scratch).
extern "C" int ob200_bn_train_forward_f32(const float* x, float* y, const float* gamma, const float* beta, float* running_mean,
                                          float* running_var, float* save_mean, float* save_invstd, double* sums, float eps,
                                          float momentum, long long rows, int C, int num_ctas, void* stream) {
    if (rows <= 0) return 0;
    if (C <= 0 || (C & 3) || num_ctas <= 0 || !sums || !save_mean || !save_invstd) return -1;
    if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)gamma | (uintptr_t)beta | (uintptr_t)save_mean | (uintptr_t)save_invstd) % 16) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = launch_reduce(x, nullptr, nullptr, nullptr, sums, rows, C, 0, num_ctas, s);
    if (e != cudaSuccess) return (int)e;
    OB200_HBM_BOUND();
    bn_stats_finish_kernel<<<(C + 127) / 128, 128, 0, s>>>(sums, save_mean, save_invstd, running_mean, running_var, rows, C, eps,
                                                           momentum);
    const long long n4 = rows * C / 4;
    OB200_ELASTIC_HBM(bn_apply_kernel, 6);
    bn_apply_kernel<<<grid_for_channels(n4, num_ctas, 6, C / 4), TR_THREADS, 0, s>>>((const float4*)x, (float4*)y, gamma, beta, save_mean, save_invstd,
                                                                    n4, C / 4);
    return (int)cudaGetLastError();
}

// sums: 2*C doubles, zero on entry (scratch).  dgamma / dbeta may be NULL.
extern "C" int ob200_bn_backward_f32(const float* dy, const float* x, float* dx, const float* gamma, const float* save_mean,
                                     const float* save_invstd, float* dgamma, float* dbeta, double* sums, long long rows, int C,
                                     int num_ctas, void* stream) {
    if (rows <= 0) return 0;
    if (C <= 0 || (C & 3) || num_ctas <= 0 || !sums) return -1;
    if (((uintptr_t)dy | (uintptr_t)x | (uintptr_t)dx | (uintptr_t)gamma | (uintptr_t)save_mean | (uintptr_t)save_invstd) % 16) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = launch_reduce(dy, x, save_mean, save_invstd, sums, rows, C, 1, num_ctas, s);
    if (e != cudaSuccess) return (int)e;
    const long long n4 = rows * C / 4;
    OB200_ELASTIC_HBM(bn_backward_apply_kernel, 6);
    bn_backward_apply_kernel<<<grid_for_channels(n4, num_ctas, 6, C / 4), TR_THREADS, 0, s>>>((const float4*)dy, (const float4*)x, (float4*)dx, gamma,
                                                                             save_mean, save_invstd, sums, dgamma, dbeta, n4, C / 4,
                                                                             rows);
    return (int)cudaGetLastError();
}

extern "C" int ob200_relu_backward_f32(const float* dy, const float* y, float* dx, long long n, int num_ctas, void* stream) {
    if (n <= 0) return 0;
    if (num_ctas <= 0) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const bool aligned = ((uintptr_t)dy | (uintptr_t)y | (uintptr_t)dx) % 16 == 0;
    const long long n4 = aligned ? n / 4 : 0;
    OB200_ELASTIC_HBM(relu_backward_kernel, 4);
    if (n4 > 0) relu_backward_kernel<<<grid_for(n4, num_ctas, 4), TR_THREADS, 0, s>>>((const float4*)dy, (const float4*)y, (float4*)dx, n4);
    if (n4 * 4 < n) relu_backward_tail_kernel<<<grid_for(n - n4 * 4, num_ctas, 4), TR_THREADS, 0, s>>>(dy, y, dx, n4 * 4, n);
    return (int)cudaGetLastError();
}

// w: [K, R*S, C] -> wt: [C, R*S, K]; elem_bytes 4 (float32) or 2 (bfloat16).
extern "C" int ob200_filter_transpose(const void* w, void* wt, int K, int RS, int C, int elem_bytes, void* stream) {
    if (K <= 0 || RS <= 0 || C <= 0) return -1;
    dim3 grid((C + 31) / 32, (K + 31) / 32, RS);
    OB200_HBM_BOUND();
    if (elem_bytes == 4)
        filter_transpose_kernel<float><<<grid, TR_THREADS, 0, (cudaStream_t)stream>>>((const float*)w, (float*)wt, K, RS, C);
    else if (elem_bytes == 2)
        filter_transpose_kernel<uint16_t><<<grid, TR_THREADS, 0, (cudaStream_t)stream>>>((const uint16_t*)w, (uint16_t*)wt, K, RS, C);
    else
        return -1;
    return (int)cudaGetLastError();
}

extern "C" int ob200_sgd_momentum_f32(float* p, const float* g, float* m, long long n, float lr, float mu, float wd, int nesterov,
                                      int first_step, int num_ctas, void* stream) {
    if (n <= 0) return 0;
    if (num_ctas <= 0) return -1;
    OB200_ELASTIC_HBM(sgd_momentum_kernel, 4);
    sgd_momentum_kernel<<<grid_for(n, num_ctas, 4), TR_THREADS, 0, (cudaStream_t)stream>>>(p, g, m, n, lr, mu, wd, nesterov, first_step);
    return (int)cudaGetLastError();
}

// SGD with momentum over `count` parameter tensors (host arrays of device pointers and element counts) in
// ceil(count / 96) launches instead of one per tensor.
extern "C" int ob200_sgd_momentum_multi_f32(float* const* p, const float* const* g, float* const* m, const long long* n, int count,
                                            float lr, float mu, float wd, int nesterov, int first_step, int num_ctas, void* stream) {
    if (count <= 0) return 0;
    if (!p || !g || !m || !n || num_ctas <= 0) return -1;
    for (int base = 0; base < count; base += SGD_MAX_TENSORS) {
        SgdTable t;
        t.count = 0;
        t.first_chunk[0] = 0;
        for (int i = base; i < count && t.count < SGD_MAX_TENSORS; i++) {
            if (n[i] <= 0) continue;
            if (!p[i] || !g[i] || !m[i]) return -1;
            const int k = t.count++;
            t.p[k] = p[i];
            t.g[k] = g[i];
            t.m[k] = m[i];
            t.n[k] = n[i];
            t.first_chunk[k + 1] = t.first_chunk[k] + (int)((n[i] + SGD_CHUNK - 1) / SGD_CHUNK);
        }
        if (t.count == 0) continue;
        const int chunks = t.first_chunk[t.count];
        const long long cap = (long long)num_ctas * 4 * grid_oversubscription();
        OB200_ELASTIC_HBM(sgd_momentum_multi_kernel, 4);
        sgd_momentum_multi_kernel<<<(unsigned)(chunks < cap ? chunks : cap), TR_THREADS, 0, (cudaStream_t)stream>>>(t, lr, mu, wd, nesterov,
                                                                                                              first_step);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}
