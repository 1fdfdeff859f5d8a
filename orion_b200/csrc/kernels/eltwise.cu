// HBM-bound NHWC kernels behind the workloads' non-GEMM ops: batch-norm inference,
// ReLU, residual add (+ReLU), max-pool and global average pool.  They stand in for
// cudnnBatchNormalizationForwardInference (src/scheduler/utils_sched.cpp:340-353)
// and for the at::native elementwise / pooling kernels that reach the scheduler
// through the cudaLaunchKernel trap (src/cuda_capture/intercept_temp.cpp:418-458).
//
// All are persistent grid-stride kernels: the launch grid is the SM quota the
// scheduler granted times a fixed number of CTAs per SM, 128-bit accesses wherever
// the channel count allows.  Algorithmic bytes per element: BN 2x4 B (+4 per-channel
// vectors), ReLU 2x4 B, add 3x4 B.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>
#include "elastic.h"
#include "pdl.cuh"

namespace ob200 {

constexpr int ELT_THREADS = 256;
constexpr int ELT_CTAS_PER_SM = 4;

// y = (x - mean) * rsqrt(var + eps) * gamma + beta, channel = innermost dimension.
__global__ void __launch_bounds__(ELT_THREADS) bn_inference_f32_kernel(const float4* __restrict__ x, float4* __restrict__ y,
                                                                     const float* __restrict__ gamma,
                                                                     const float* __restrict__ beta,
                                                                     const float* __restrict__ mean,
                                                                     const float* __restrict__ var, float eps,
                                                                     long long n4, int c4, int relu) {
    pdl_launch_dependents();   // a convolution behind this kernel may set itself up meanwhile (pdl.cuh)
    // y = a * x + b per channel.  When the grid stride is a multiple of the channel-quad count a thread stays on one
    // channel quad: the coefficients (and their square roots) are computed once, the loop keeps four loads in flight.
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    auto coef = [&](int c, float4& a, float4& b) {
        const float4 m = __ldg(reinterpret_cast<const float4*>(mean + c));
        const float4 s2 = __ldg(reinterpret_cast<const float4*>(var + c));
        float4 g = make_float4(1.f, 1.f, 1.f, 1.f), be = make_float4(0.f, 0.f, 0.f, 0.f);
        if (gamma) g = __ldg(reinterpret_cast<const float4*>(gamma + c));
        if (beta) be = __ldg(reinterpret_cast<const float4*>(beta + c));
        a = make_float4(g.x / sqrtf(s2.x + eps), g.y / sqrtf(s2.y + eps), g.z / sqrtf(s2.z + eps), g.w / sqrtf(s2.w + eps));
        b = make_float4(be.x - m.x * a.x, be.y - m.y * a.y, be.z - m.z * a.z, be.w - m.w * a.w);
    };
    const float lo = relu ? 0.f : -INFINITY;
    auto apply = [&](const float4& v, const float4& a, const float4& b) {
        return make_float4(fmaxf(fmaf(v.x, a.x, b.x), lo), fmaxf(fmaf(v.y, a.y, b.y), lo), fmaxf(fmaf(v.z, a.z, b.z), lo),
                           fmaxf(fmaf(v.w, a.w, b.w), lo));
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
            for (int u = 0; u < 4; u++) y[i + u * stride] = apply(v[u], a, b);
        }
        for (; i < n4; i += stride) y[i] = apply(__ldcs(x + i), a, b);
        return;
    }
    for (; i < n4; i += stride) {
        float4 a, b;
        coef((int)(i % c4) * 4, a, b);
        y[i] = apply(__ldcs(x + i), a, b);
    }
}

// Scalar fallback for channel counts that are not a multiple of 4.
__global__ void __launch_bounds__(ELT_THREADS) bn_inference_f32_scalar_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                                            const float* __restrict__ gamma,
                                                                            const float* __restrict__ beta,
                                                                            const float* __restrict__ mean,
                                                                            const float* __restrict__ var, float eps,
                                                                            long long n, int C, int relu) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        float o = (x[i] - mean[c]) * (1.0f / sqrtf(var[c] + eps)) * (gamma ? gamma[c] : 1.f) + (beta ? beta[c] : 0.f);
        y[i] = relu ? fmaxf(o, 0.f) : o;
    }
}

// mode 0: y = relu(a); 1: y = a + b; 2: y = relu(a + b)
__global__ void __launch_bounds__(ELT_THREADS) binary_f32_kernel(const float4* __restrict__ a, const float4* __restrict__ b,
                                                               float4* __restrict__ y, long long n4, int mode) {
    pdl_launch_dependents();   // a convolution behind this kernel may set itself up meanwhile (pdl.cuh)
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        float4 v = __ldcs(a + i);
        if (mode != 0) {
            const float4 w = __ldcs(b + i);
            v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        }
        if (mode != 1) {
            v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
        }
        y[i] = v;
    }
}
__global__ void __launch_bounds__(ELT_THREADS) binary_f32_tail_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                                    float* __restrict__ y, long long begin, long long n, int mode) {
    for (long long i = begin + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = a[i];
        if (mode != 0) v += b[i];
        if (mode != 1) v = fmaxf(v, 0.f);
        y[i] = v;
    }
}

// Max-pool over NHWC with -inf padding; one thread per 4 channels of one output pixel.
__global__ void __launch_bounds__(ELT_THREADS) maxpool_nhwc_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int Nb,
                                                                     int H, int W, int C, int P, int Q, int k, int stride,
                                                                     int pad) {
    pdl_launch_dependents();   // a convolution behind this kernel may set itself up meanwhile (pdl.cuh)
    const int c4 = C >> 2;
    const long long total = (long long)Nb * P * Q * c4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % c4) * 4;
        long long t = i / c4;
        const int q = (int)(t % Q); t /= Q;
        const int p = (int)(t % P);
        const int n = (int)(t / P);
        float4 m = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
        for (int r = 0; r < k; r++) {
            const int h = p * stride - pad + r;
            if (h < 0 || h >= H) continue;
            for (int s = 0; s < k; s++) {
                const int w = q * stride - pad + s;
                if (w < 0 || w >= W) continue;
                const float4 v = __ldg(reinterpret_cast<const float4*>(x + (((long long)n * H + h) * W + w) * C + c));
                m.x = fmaxf(m.x, v.x); m.y = fmaxf(m.y, v.y); m.z = fmaxf(m.z, v.z); m.w = fmaxf(m.w, v.w);
            }
        }
        *reinterpret_cast<float4*>(y + (((long long)n * P + p) * Q + q) * C + c) = m;
    }
}

// 3x3 / stride 2 max-pool (the ResNet stem): a thread produces four consecutive output pixels of one row for
// its channel quad, sharing the nine input columns they need (27 loads for four outputs instead of 36).
__global__ void __launch_bounds__(ELT_THREADS) maxpool3x3s2_nhwc_f32_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                                          int Nb, int H, int W, int C, int P, int Q, int pad) {
    pdl_launch_dependents();   // a convolution behind this kernel may set itself up meanwhile (pdl.cuh)
    const int c4 = C >> 2, qb_n = (Q + 3) / 4;
    const long long total = (long long)Nb * P * qb_n * c4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % c4) * 4;
        long long t = i / c4;
        const int qb = (int)(t % qb_n); t /= qb_n;
        const int p = (int)(t % P);
        const int n = (int)(t / P);
        const float4 lowest = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
        float4 m[4] = {lowest, lowest, lowest, lowest};
        const int w0 = qb * 8 - pad;
#pragma unroll
        for (int r = 0; r < 3; r++) {
            const int h = p * 2 - pad + r;
            if ((unsigned)h >= (unsigned)H) continue;
            const float* xrow = x + (((long long)n * H + h) * W) * C + c;
            float4 v[9];
#pragma unroll
            for (int j = 0; j < 9; j++) {
                const int w = w0 + j;
                v[j] = (unsigned)w < (unsigned)W ? __ldg(reinterpret_cast<const float4*>(xrow + (long long)w * C)) : lowest;
            }
#pragma unroll
            for (int o = 0; o < 4; o++) {
#pragma unroll
                for (int s2 = 0; s2 < 3; s2++) {
                    const float4 a = v[2 * o + s2];
                    m[o].x = fmaxf(m[o].x, a.x); m[o].y = fmaxf(m[o].y, a.y); m[o].z = fmaxf(m[o].z, a.z); m[o].w = fmaxf(m[o].w, a.w);
                }
            }
        }
#pragma unroll
        for (int o = 0; o < 4; o++)
            if (qb * 4 + o < Q) *reinterpret_cast<float4*>(y + (((long long)n * P + p) * Q + qb * 4 + o) * C + c) = m[o];
    }
}

// Max-pool backward over NHWC: one thread per 4 channels of one output pixel finds, per channel, the FIRST largest element
// of its window in row-major scan order (the element torch's forward kernel records, so ties -- frequent behind a ReLU,
// where whole windows are zero -- are routed the same way) and adds the output gradient there.  Windows overlap, so the
// additions are atomic; dx is zero on entry.
__global__ void __launch_bounds__(ELT_THREADS) maxpool_backward_nhwc_f32_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                                                              float* __restrict__ dx, int Nb, int H, int W, int C,
                                                                              int P, int Q, int k, int stride, int pad) {
    pdl_launch_dependents();   // a convolution behind this kernel may set itself up meanwhile (pdl.cuh)
    const int c4 = C >> 2;
    const long long total = (long long)Nb * P * Q * c4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % c4) * 4;
        long long t = i / c4;
        const int q = (int)(t % Q); t /= Q;
        const int p = (int)(t % P);
        const int n = (int)(t / P);
        float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        long long at[4] = {-1, -1, -1, -1};
        for (int r = 0; r < k; r++) {
            const int h = p * stride - pad + r;
            if (h < 0 || h >= H) continue;
            for (int s = 0; s < k; s++) {
                const int w = q * stride - pad + s;
                if (w < 0 || w >= W) continue;
                const long long off = (((long long)n * H + h) * W + w) * C + c;
                const float4 v = __ldg(reinterpret_cast<const float4*>(x + off));
                const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (e[j] > m[j] || at[j] < 0) { m[j] = e[j]; at[j] = off + j; }
            }
        }
        const float4 g = __ldcs(reinterpret_cast<const float4*>(dy + (((long long)n * P + p) * Q + q) * C + c));
        const float ge[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (at[j] >= 0) atomicAdd(dx + at[j], ge[j]);
    }
}

// Global average pool NHWC [Nb, HW, C] -> [Nb, C]; one thread per (image, channel),
// consecutive threads read consecutive channels so every row read is coalesced.
__global__ void __launch_bounds__(ELT_THREADS) avgpool_nhwc_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int Nb,
                                                                     int HW, int C) {
    const long long total = (long long)Nb * C;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const int n = (int)(i / C);
        const float* p = x + (long long)n * HW * C + c;
        float acc = 0.f;
        for (int j = 0; j < HW; j++) acc += p[(long long)j * C];
        y[i] = acc / (float)HW;
    }
}

// The same for C % 4 == 0: a CTA of 256 threads owns 32 float4 channel chunks (128 channels) of one image and splits the
// HW rows over 8 thread rows (independent 16-byte loads, then a fixed-order sum through shared memory), so that even a
// batch-4 request spreads over Nb * C / 128 CTAs instead of a handful.
__global__ void __launch_bounds__(256) avgpool_nhwc_f32_v4_kernel(const float4* __restrict__ x, float4* __restrict__ y, int Nb, int HW, int C4) {
    __shared__ float4 sh[8][32];
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int groups = (C4 + 31) / 32;
    for (int item = blockIdx.x; item < Nb * groups; item += gridDim.x) {
        const int n = item / groups, c4 = (item - n * groups) * 32 + cx;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c4 < C4) {
            const float4* p = x + (long long)n * HW * C4 + c4;
#pragma unroll 4
            for (int j = ry; j < HW; j += 8) {
                const float4 v = __ldg(p + (long long)j * C4);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
        }
        sh[ry][cx] = acc;
        __syncthreads();
        if (ry == 0 && c4 < C4) {
            float4 t = sh[0][cx];
#pragma unroll
            for (int k = 1; k < 8; k++) {
                const float4 v = sh[k][cx];
                t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
            }
            const float inv = 1.0f / (float)HW;
            y[(long long)n * C4 + c4] = make_float4(t.x * inv, t.y * inv, t.z * inv, t.w * inv);
        }
        __syncthreads();
    }
}

static inline int elt_grid(long long work_items, int num_ctas) {
    long long want = (work_items + ELT_THREADS - 1) / ELT_THREADS;
    long long cap = (long long)num_ctas * ELT_CTAS_PER_SM * grid_oversubscription();
    if (want < 1) want = 1;
    return (int)(want < cap ? want : cap);
}

}  // namespace ob200

using namespace ob200;

extern "C" int ob200_bn_inference_f32(const float* x, float* y, const float* gamma, const float* beta, const float* mean,
                                      const float* var, float eps, long long n_elems, int C, int relu, int num_ctas,
                                      void* stream) {
    if (n_elems <= 0) return 0;
    if (C <= 0 || n_elems % C || num_ctas <= 0) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const bool aligned = ((uintptr_t)x | (uintptr_t)y | (uintptr_t)mean | (uintptr_t)var | (uintptr_t)gamma | (uintptr_t)beta) % 16 == 0;
    if ((C & 3) == 0 && aligned) {
        long long n4 = n_elems / 4;
        int grid = elt_grid(n4, num_ctas);
        int need = 1;   // smallest grid multiple that makes grid * ELT_THREADS a multiple of the channel-quad count
        while (((long long)need * ELT_THREADS) % (C / 4) != 0 && need < 64) need++;
        if (need > 1 && need < 64 && grid >= need) grid -= grid % need;
        OB200_ELASTIC_HBM(bn_inference_f32_kernel, ELT_CTAS_PER_SM);
        bn_inference_f32_kernel<<<grid, ELT_THREADS, 0, s>>>((const float4*)x, (float4*)y, gamma, beta, mean, var,
                                                                              eps, n4, C / 4, relu);
    } else {
        OB200_HBM_BOUND();
        bn_inference_f32_scalar_kernel<<<elt_grid(n_elems, num_ctas), ELT_THREADS, 0, s>>>(x, y, gamma, beta, mean, var, eps,
                                                                                          n_elems, C, relu);
    }
    return (int)cudaGetLastError();
}

extern "C" int ob200_binary_f32(const float* a, const float* b, float* y, long long n_elems, int mode, int num_ctas,
                                void* stream) {
    if (n_elems <= 0) return 0;
    if (mode < 0 || mode > 2 || num_ctas <= 0 || (mode != 0 && !b)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const bool aligned = ((uintptr_t)a | (uintptr_t)b | (uintptr_t)y) % 16 == 0;
    long long n4 = aligned ? n_elems / 4 : 0;
    if (n4 > 0) {
        OB200_ELASTIC_HBM(binary_f32_kernel, ELT_CTAS_PER_SM);
        binary_f32_kernel<<<elt_grid(n4, num_ctas), ELT_THREADS, 0, s>>>((const float4*)a, (const float4*)b, (float4*)y, n4, mode);
    }
    if (n4 * 4 < n_elems) {
        OB200_HBM_BOUND();
        binary_f32_tail_kernel<<<elt_grid(n_elems - n4 * 4, num_ctas), ELT_THREADS, 0, s>>>(a, b, y, n4 * 4, n_elems, mode);
    }
    return (int)cudaGetLastError();
}

extern "C" int ob200_maxpool_nhwc_f32(const float* x, float* y, int Nb, int H, int W, int C, int k, int stride, int pad,
                                      int num_ctas, void* stream) {
    if (Nb <= 0) return 0;
    if ((C & 3) || k <= 0 || stride <= 0 || num_ctas <= 0) return -1;
    const int P = (H + 2 * pad - k) / stride + 1, Q = (W + 2 * pad - k) / stride + 1;
    if (k == 3 && stride == 2) {
        const long long total4 = (long long)Nb * P * ((Q + 3) / 4) * (C / 4);
        OB200_ELASTIC_HBM(maxpool3x3s2_nhwc_f32_kernel, ELT_CTAS_PER_SM);
        maxpool3x3s2_nhwc_f32_kernel<<<elt_grid(total4, num_ctas), ELT_THREADS, 0, (cudaStream_t)stream>>>(x, y, Nb, H, W, C, P, Q, pad);
        return (int)cudaGetLastError();
    }
    long long total = (long long)Nb * P * Q * (C / 4);
    OB200_ELASTIC_HBM(maxpool_nhwc_f32_kernel, ELT_CTAS_PER_SM);
    maxpool_nhwc_f32_kernel<<<elt_grid(total, num_ctas), ELT_THREADS, 0, (cudaStream_t)stream>>>(x, y, Nb, H, W, C, P, Q, k, stride,
                                                                                               pad);
    return (int)cudaGetLastError();
}

// dx = gradient of ob200_maxpool_nhwc_f32 (same arguments); dx is cleared on `stream` first.
extern "C" int ob200_maxpool_backward_nhwc_f32(const float* dy, const float* x, float* dx, int Nb, int H, int W, int C, int k,
                                               int stride, int pad, int num_ctas, void* stream) {
    if (Nb < 0 || H <= 0 || W <= 0 || C <= 0 || (C & 3) || k <= 0 || stride <= 0 || pad < 0 || pad >= k || num_ctas <= 0) return -1;
    if (Nb == 0) return 0;
    const int P = (H + 2 * pad - k) / stride + 1, Q = (W + 2 * pad - k) / stride + 1;
    if (P <= 0 || Q <= 0) return -1;
    if (((uintptr_t)dy | (uintptr_t)x | (uintptr_t)dx) % 16) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(dx, 0, (size_t)Nb * H * W * C * sizeof(float), s);
    if (e != cudaSuccess) return (int)e;
    const long long total = (long long)Nb * P * Q * (C / 4);
    OB200_ELASTIC_HBM(maxpool_backward_nhwc_f32_kernel, ELT_CTAS_PER_SM);
    maxpool_backward_nhwc_f32_kernel<<<elt_grid(total, num_ctas), ELT_THREADS, 0, s>>>(dy, x, dx, Nb, H, W, C, P, Q, k, stride, pad);
    return (int)cudaGetLastError();
}

extern "C" int ob200_avgpool_nhwc_f32(const float* x, float* y, int Nb, int HW, int C, int num_ctas, void* stream) {
    if (Nb <= 0) return 0;
    if (HW <= 0 || C <= 0 || num_ctas <= 0) return -1;
    if ((C & 3) == 0 && ((uintptr_t)x | (uintptr_t)y) % 16 == 0) {
        const long long items = (long long)Nb * ((C / 4 + 31) / 32), cap = (long long)num_ctas * 8;
        OB200_ELASTIC_HBM(avgpool_nhwc_f32_v4_kernel, 8);
        avgpool_nhwc_f32_v4_kernel<<<(int)(items < cap ? items : cap), 256, 0, (cudaStream_t)stream>>>((const float4*)x, (float4*)y, Nb, HW, C / 4);
        return (int)cudaGetLastError();
    }
    OB200_ELASTIC_HBM(avgpool_nhwc_f32_kernel, ELT_CTAS_PER_SM);
    avgpool_nhwc_f32_kernel<<<elt_grid((long long)Nb * C, num_ctas), ELT_THREADS, 0, (cudaStream_t)stream>>>(x, y, Nb, HW, C);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- channel padding
// Copies [pixels, C] to [pixels, Cpad] (Cpad > C), zero in the added channels, so that a
// channel count that is not a multiple of a 16-byte chunk (the 3-channel image of a stem
// convolution) can take the vectorised operand path of the implicit-GEMM kernel.
namespace ob200 {
template <typename T>
__global__ void pad_channels_kernel(const T* __restrict__ src, T* __restrict__ dst, long long pixels, int C, int Cpad) {
    const long long total = pixels * Cpad;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long px = i / Cpad;
        const int c = (int)(i - px * Cpad);
        dst[i] = c < C ? src[px * C + c] : T(0);
    }
}
// float32, 3 -> 4 channels: one 16-byte store per pixel.
__global__ void pad_channels_3to4_f32_kernel(const float* __restrict__ src, float4* __restrict__ dst, long long pixels) {
    for (long long px = (long long)blockIdx.x * blockDim.x + threadIdx.x; px < pixels; px += (long long)gridDim.x * blockDim.x) {
        const float* s = src + px * 3;
        dst[px] = make_float4(__ldg(s), __ldg(s + 1), __ldg(s + 2), 0.f);
    }
}
}  // namespace ob200

extern "C" int ob200_pad_channels(const void* src, void* dst, long long pixels, int C, int Cpad, int elem_bytes, int num_ctas,
                                  void* stream) {
    if (pixels <= 0) return 0;
    if (C <= 0 || Cpad <= C || num_ctas <= 0 || (elem_bytes != 2 && elem_bytes != 4)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    OB200_HBM_BOUND();
    if (elem_bytes == 4 && C == 3 && Cpad == 4 && (uintptr_t)dst % 16 == 0)
        ob200::pad_channels_3to4_f32_kernel<<<elt_grid(pixels, num_ctas), ELT_THREADS, 0, s>>>((const float*)src, (float4*)dst, pixels);
    else if (elem_bytes == 4)
        ob200::pad_channels_kernel<float><<<elt_grid(pixels * Cpad, num_ctas), ELT_THREADS, 0, s>>>((const float*)src, (float*)dst, pixels, C, Cpad);
    else
        ob200::pad_channels_kernel<unsigned short><<<elt_grid(pixels * Cpad, num_ctas), ELT_THREADS, 0, s>>>(
            (const unsigned short*)src, (unsigned short*)dst, pixels, C, Cpad);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- depthwise convolution
// y[n,p,q,c] = act( scale[c] * sum_{r,s} x[n, p*sh - ph + r*dh, q*sw - pw + s*dw, c] * w[c][r][s] + shift[c] ),
// NHWC float32, channel multiplier 1 (groups = C): the depthwise layers of MobileNetV2, which the reference
// hands to cudnnConvolutionForward like any other convolution (src/scheduler/utils_sched.cpp:284-296).
// One thread per output pixel and channel quad; a warp covers 32 consecutive channel quads, so every tap is a
// coalesced 512-byte read and neighbouring pixels re-read it from L1/L2.  HBM-bound: 8 B per element.
// w_tap_major = 1: filter stored [R][S][C] (one float4 per tap), 0: [C][R][S] as torch holds it.
namespace ob200 {
__global__ void __launch_bounds__(ELT_THREADS) depthwise_conv_nhwc_f32_kernel(
    const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, const float* __restrict__ scale,
    const float* __restrict__ shift, int relu, int Nb, int H, int W, int C, int R, int S, int P, int Q, int stride_h, int stride_w,
    int pad_h, int pad_w, int dil_h, int dil_w, int w_tap_major) {
    const int c4 = C / 4;
    const long long total = (long long)Nb * P * Q * c4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int cq = (int)(i % c4);
        long long pix = i / c4;
        const int q = (int)(pix % Q);
        pix /= Q;
        const int p = (int)(pix % P);
        const int n = (int)(pix / P);
        const int c = cq * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const int h0 = p * stride_h - pad_h, w0 = q * stride_w - pad_w;
        for (int r = 0; r < R; r++) {
            const int h = h0 + r * dil_h;
            if ((unsigned)h >= (unsigned)H) continue;
            for (int s = 0; s < S; s++) {
                const int ww = w0 + s * dil_w;
                if ((unsigned)ww >= (unsigned)W) continue;
                const float4 v = __ldg(reinterpret_cast<const float4*>(x + (((long long)n * H + h) * W + ww) * C + c));
                float4 f;
                if (w_tap_major) {
                    f = __ldg(reinterpret_cast<const float4*>(w + ((long long)r * S + s) * C + c));
                } else {
                    const int t = r * S + s, rs = R * S;
                    f = make_float4(__ldg(w + (long long)c * rs + t), __ldg(w + (long long)(c + 1) * rs + t),
                                    __ldg(w + (long long)(c + 2) * rs + t), __ldg(w + (long long)(c + 3) * rs + t));
                }
                acc.x = fmaf(v.x, f.x, acc.x); acc.y = fmaf(v.y, f.y, acc.y);
                acc.z = fmaf(v.z, f.z, acc.z); acc.w = fmaf(v.w, f.w, acc.w);
            }
        }
        if (scale) {
            const float4 g = __ldg(reinterpret_cast<const float4*>(scale + c));
            acc.x *= g.x; acc.y *= g.y; acc.z *= g.z; acc.w *= g.w;
        }
        if (shift) {
            const float4 b = __ldg(reinterpret_cast<const float4*>(shift + c));
            acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
        }
        if (relu) {
            acc.x = fmaxf(acc.x, 0.f); acc.y = fmaxf(acc.y, 0.f); acc.z = fmaxf(acc.z, 0.f); acc.w = fmaxf(acc.w, 0.f);
            if (relu == 2) { acc.x = fminf(acc.x, 6.f); acc.y = fminf(acc.y, 6.f); acc.z = fminf(acc.z, 6.f); acc.w = fminf(acc.w, 6.f); }
        }
        reinterpret_cast<float4*>(y)[i] = acc;
    }
}
}  // namespace ob200

// 3x3 depthwise, stride 1 or 2, dilation 1: each thread produces four consecutive output pixels of one row for
// its channel quad, so the 3 x (3 + 3*STRIDE) input vectors it loads are shared by the four outputs (6.75 loads per
// output at stride 1 against 18 in the generic kernel, filter taps included) and the filter is read once.
namespace ob200 {
template <int STRIDE>
__global__ void __launch_bounds__(ELT_THREADS) depthwise3x3_nhwc_f32_kernel(
    const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, const float* __restrict__ scale,
    const float* __restrict__ shift, int relu, int Nb, int H, int W, int C, int P, int Q, int pad_h, int pad_w, int w_tap_major,
    int flip) {
    // flip = 1 uses the filter rotated by 180 degrees: the data gradient of a stride-1 layer is this same convolution of dy
    constexpr int TW = 4, NCOL = (TW - 1) * STRIDE + 3;
    const int c4 = C / 4, qb_n = (Q + TW - 1) / TW;
    const long long total = (long long)Nb * P * qb_n * c4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int cq = (int)(i % c4);
        long long rest = i / c4;
        const int qb = (int)(rest % qb_n);
        rest /= qb_n;
        const int p = (int)(rest % P);
        const int n = (int)(rest / P);
        const int c = cq * 4;
        float4 f[9];
#pragma unroll
        for (int t = 0; t < 9; t++) {
            const int tw = flip ? 8 - t : t;
            if (w_tap_major) f[t] = __ldg(reinterpret_cast<const float4*>(w + (long long)tw * C + c));
            else f[t] = make_float4(__ldg(w + (long long)c * 9 + tw), __ldg(w + (long long)(c + 1) * 9 + tw), __ldg(w + (long long)(c + 2) * 9 + tw),
                                    __ldg(w + (long long)(c + 3) * 9 + tw));
        }
        float4 acc[TW];
#pragma unroll
        for (int t = 0; t < TW; t++) acc[t] = make_float4(0.f, 0.f, 0.f, 0.f);
        const int q0 = qb * TW;
        const int w0 = q0 * STRIDE - pad_w;
#pragma unroll
        for (int r = 0; r < 3; r++) {
            const int h = p * STRIDE - pad_h + r;
            if ((unsigned)h >= (unsigned)H) continue;
            const float* xrow = x + (((long long)n * H + h) * W) * C + c;
            float4 v[NCOL];
#pragma unroll
            for (int j = 0; j < NCOL; j++) {
                const int ww = w0 + j;
                v[j] = (unsigned)ww < (unsigned)W ? __ldg(reinterpret_cast<const float4*>(xrow + (long long)ww * C)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int t = 0; t < TW; t++) {
#pragma unroll
                for (int s2 = 0; s2 < 3; s2++) {
                    const float4 a = v[t * STRIDE + s2], b = f[r * 3 + s2];
                    acc[t].x = fmaf(a.x, b.x, acc[t].x); acc[t].y = fmaf(a.y, b.y, acc[t].y);
                    acc[t].z = fmaf(a.z, b.z, acc[t].z); acc[t].w = fmaf(a.w, b.w, acc[t].w);
                }
            }
        }
        float4 g = make_float4(1.f, 1.f, 1.f, 1.f), b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (scale) g = __ldg(reinterpret_cast<const float4*>(scale + c));
        if (shift) b = __ldg(reinterpret_cast<const float4*>(shift + c));
        const float lo = relu ? 0.f : -INFINITY, hi = relu == 2 ? 6.f : INFINITY;
#pragma unroll
        for (int t = 0; t < TW; t++) {
            if (q0 + t >= Q) break;
            float4 o = make_float4(fmaf(acc[t].x, g.x, b.x), fmaf(acc[t].y, g.y, b.y), fmaf(acc[t].z, g.z, b.z), fmaf(acc[t].w, g.w, b.w));
            o.x = fminf(fmaxf(o.x, lo), hi); o.y = fminf(fmaxf(o.y, lo), hi); o.z = fminf(fmaxf(o.z, lo), hi); o.w = fminf(fmaxf(o.w, lo), hi);
            *reinterpret_cast<float4*>(y + ((((long long)n * P + p) * Q + q0 + t) * C + c)) = o;
        }
    }
}
}  // namespace ob200

extern "C" int ob200_depthwise_conv2d_f32(const float* x, const float* w, float* y, const float* scale, const float* shift, int relu,
                                          int Nb, int H, int W, int C, int R, int S, int stride_h, int stride_w, int pad_h, int pad_w,
                                          int dil_h, int dil_w, int w_tap_major, int num_ctas, void* stream) {
    if (Nb < 0 || H <= 0 || W <= 0 || C <= 0 || (C & 3) || R <= 0 || S <= 0 || stride_h <= 0 || stride_w <= 0 || dil_h <= 0 ||
        dil_w <= 0 || pad_h < 0 || pad_w < 0 || num_ctas <= 0 || relu < 0 || relu > 2)
        return -1;
    if (Nb == 0) return 0;
    const int P = (H + 2 * pad_h - dil_h * (R - 1) - 1) / stride_h + 1;
    const int Q = (W + 2 * pad_w - dil_w * (S - 1) - 1) / stride_w + 1;
    if (P <= 0 || Q <= 0) return -1;
    if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)scale | (uintptr_t)shift) % 16 || (w_tap_major && (uintptr_t)w % 16)) return -2;
    if (R == 3 && S == 3 && dil_h == 1 && dil_w == 1 && stride_h == stride_w && (stride_h == 1 || stride_h == 2)) {
        const long long total4 = (long long)Nb * P * ((Q + 3) / 4) * (C / 4);
        long long want4 = (total4 + ELT_THREADS - 1) / ELT_THREADS, cap4 = (long long)num_ctas * 4;
        const int grid4 = (int)(want4 < cap4 ? want4 : cap4);
        OB200_ELASTIC_HBM(ob200::depthwise3x3_nhwc_f32_kernel<1>, 4);
        OB200_ELASTIC_HBM(ob200::depthwise3x3_nhwc_f32_kernel<2>, 4);
        if (stride_h == 1)
            ob200::depthwise3x3_nhwc_f32_kernel<1><<<grid4, ELT_THREADS, 0, (cudaStream_t)stream>>>(x, w, y, scale, shift, relu, Nb, H, W, C, P,
                                                                                                Q, pad_h, pad_w, w_tap_major, 0);
        else
            ob200::depthwise3x3_nhwc_f32_kernel<2><<<grid4, ELT_THREADS, 0, (cudaStream_t)stream>>>(x, w, y, scale, shift, relu, Nb, H, W, C, P,
                                                                                                Q, pad_h, pad_w, w_tap_major, 0);
        return (int)cudaGetLastError();
    }
    const long long total = (long long)Nb * P * Q * (C / 4);
    // up to eight CTAs of 256 threads per granted SM: the kernel lives on loads in flight
    long long want = (total + ELT_THREADS - 1) / ELT_THREADS, cap = (long long)num_ctas * 8;
    const int grid = (int)(want < cap ? want : cap);
    OB200_ELASTIC_HBM(ob200::depthwise_conv_nhwc_f32_kernel, 8);
    ob200::depthwise_conv_nhwc_f32_kernel<<<grid, ELT_THREADS, 0, (cudaStream_t)stream>>>(x, w, y, scale, shift, relu, Nb, H, W, C, R, S,
                                                                                         P, Q, stride_h, stride_w, pad_h, pad_w, dil_h,
                                                                                         dil_w, w_tap_major);
    return (int)cudaGetLastError();
}


// ---------------------------------------------------------------- depthwise convolution, backward
// Gradients of ob200_depthwise_conv2d_f32 (filter [C][R][S] as torch holds it, dilation 1).  They take the place of the
// conv_depthwise2d_backward_kernel / conv_depthwise2d_grad_weight_kernel launches of the reference's MobileNetV2 training
// profile (reference benchmarking/model_kernels/mobilenetv2_64_fb1), which reach it through the cudaLaunchKernel trap
// (reference src/cuda_capture/intercept_temp.cpp:418-458).
namespace ob200 {

// dx[n,h,w,c] = sum over taps (r,s) with (h + pad - r) and (w + pad - s) divisible by the stride of
//               dy[n, (h + pad - r) / stride, (w + pad - s) / stride, c] * w[c][r][s].
__global__ void __launch_bounds__(ELT_THREADS) depthwise_dgrad_nhwc_f32_kernel(const float* __restrict__ dy, const float* __restrict__ w,
                                                                             float* __restrict__ dx, int Nb, int H, int W, int C, int R,
                                                                             int S, int P, int Q, int stride_h, int stride_w, int pad_h,
                                                                             int pad_w) {
    const int c4 = C / 4;
    const long long total = (long long)Nb * H * W * c4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % c4) * 4;
        long long t = i / c4;
        const int wi = (int)(t % W); t /= W;
        const int hi = (int)(t % H);
        const int n = (int)(t / H);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        // only taps r = (h + pad) mod stride, + stride, ... reach an output row: walk those
        for (int r = (hi + pad_h) % stride_h; r < R; r += stride_h) {
            const int hn = hi + pad_h - r;
            if (hn < 0) break;
            const int p = hn / stride_h;
            if (p >= P) continue;
            for (int sx = (wi + pad_w) % stride_w; sx < S; sx += stride_w) {
                const int wn = wi + pad_w - sx;
                if (wn < 0) break;
                const int q = wn / stride_w;
                if (q >= Q) continue;
                const float4 g = __ldg(reinterpret_cast<const float4*>(dy + (((long long)n * P + p) * Q + q) * C + c));
                const int tap = r * S + sx, RS = R * S;
                acc.x = fmaf(g.x, __ldg(w + (long long)(c + 0) * RS + tap), acc.x);
                acc.y = fmaf(g.y, __ldg(w + (long long)(c + 1) * RS + tap), acc.y);
                acc.z = fmaf(g.z, __ldg(w + (long long)(c + 2) * RS + tap), acc.z);
                acc.w = fmaf(g.w, __ldg(w + (long long)(c + 3) * RS + tap), acc.w);
            }
        }
        *reinterpret_cast<float4*>(dx + i * 4) = acc;
    }
}

// dw[c][r][s] = sum over output pixels of dy[n,p,q,c] * x[n, p*stride - pad + r, q*stride - pad + s, c]  (3x3 filters).
// Threads are (channel quad, pixel lane); every thread keeps the 9 x 4 sums of its channel quad over the pixels it walks, a
// shared-memory tree adds the lanes of a CTA and one atomicAdd per entry adds the CTAs (dw is cleared first).
__global__ void __launch_bounds__(ELT_THREADS) depthwise_wgrad3x3_nhwc_f32_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                                                                float* __restrict__ dw, int Nb, int H, int W, int C, int P,
                                                                                int Q, int stride, int pad, int slabs) {
    extern __shared__ float sh[];   // [blockDim.y][blockDim.x][36]
    const int cq = blockDim.x, ry = blockDim.y;
    const int c_groups = (C / 4 + cq - 1) / cq;
    const int cg = blockIdx.x % c_groups, slab = blockIdx.x / c_groups;
    const int c = (cg * cq + threadIdx.x) * 4;
    float acc[9][4];
#pragma unroll
    for (int t = 0; t < 9; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[t][e] = 0.f;
    if (c < C && slab < slabs) {
        // work items are (image, output row, block of four output columns); a thread loads the 3 x NCOL input window of its
        // block once (NCOL = 6 for stride 1, 9 for stride 2) instead of 9 values per output pixel
        const int qb_n = (Q + 3) / 4;
        const long long items = (long long)Nb * P * qb_n;
        const long long per = (items + slabs - 1) / slabs;
        const long long m0 = slab * per, m1 = m0 + per < items ? m0 + per : items;
        for (long long m = m0 + threadIdx.y; m < m1; m += ry) {
            const int qb = (int)(m % qb_n);
            const long long t2 = m / qb_n;
            const int p = (int)(t2 % P);
            const int n = (int)(t2 / P);
            const int q0 = qb * 4;
            float4 g[4];
#pragma unroll
            for (int t = 0; t < 4; t++)
                g[t] = q0 + t < Q ? __ldcs(reinterpret_cast<const float4*>(dy + ((((long long)n * P + p) * Q + q0 + t) * C + c)))
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
            const int w0 = q0 * stride - pad;
#pragma unroll
            for (int r = 0; r < 3; r++) {
                const int h = p * stride - pad + r;
                if ((unsigned)h >= (unsigned)H) continue;
                const float* xrow = x + (((long long)n * H + h) * W) * C + c;
                if (stride == 1) {
                    float4 v[6];
#pragma unroll
                    for (int j = 0; j < 6; j++)
                        v[j] = (unsigned)(w0 + j) < (unsigned)W ? __ldg(reinterpret_cast<const float4*>(xrow + (long long)(w0 + j) * C))
                                                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int t = 0; t < 4; t++)
#pragma unroll
                        for (int sx = 0; sx < 3; sx++) {
                            const float4 a = v[t + sx];
                            acc[r * 3 + sx][0] = fmaf(g[t].x, a.x, acc[r * 3 + sx][0]);
                            acc[r * 3 + sx][1] = fmaf(g[t].y, a.y, acc[r * 3 + sx][1]);
                            acc[r * 3 + sx][2] = fmaf(g[t].z, a.z, acc[r * 3 + sx][2]);
                            acc[r * 3 + sx][3] = fmaf(g[t].w, a.w, acc[r * 3 + sx][3]);
                        }
                } else {
#pragma unroll
                    for (int t = 0; t < 4; t++)
#pragma unroll
                        for (int sx = 0; sx < 3; sx++) {
                            const int wv = w0 + t * stride + sx;
                            if ((unsigned)wv >= (unsigned)W) continue;
                            const float4 a = __ldg(reinterpret_cast<const float4*>(xrow + (long long)wv * C));
                            acc[r * 3 + sx][0] = fmaf(g[t].x, a.x, acc[r * 3 + sx][0]);
                            acc[r * 3 + sx][1] = fmaf(g[t].y, a.y, acc[r * 3 + sx][1]);
                            acc[r * 3 + sx][2] = fmaf(g[t].z, a.z, acc[r * 3 + sx][2]);
                            acc[r * 3 + sx][3] = fmaf(g[t].w, a.w, acc[r * 3 + sx][3]);
                        }
                }
            }
        }
    }
    float* mine = sh + ((size_t)threadIdx.y * cq + threadIdx.x) * 36;
#pragma unroll
    for (int t = 0; t < 9; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) mine[t * 4 + e] = acc[t][e];
    __syncthreads();
    for (int half = ry / 2; half > 0; half >>= 1) {
        if ((int)threadIdx.y < half) {
            const float* other = sh + ((size_t)(threadIdx.y + half) * cq + threadIdx.x) * 36;
#pragma unroll
            for (int k = 0; k < 36; k++) mine[k] += other[k];
        }
        __syncthreads();
    }
    if (threadIdx.y == 0 && c < C && slab < slabs) {
#pragma unroll
        for (int t = 0; t < 9; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) atomicAdd(dw + (long long)(c + e) * 9 + t, mine[t * 4 + e]);
    }
}

}  // namespace ob200

extern "C" int ob200_depthwise_conv2d_dgrad_f32(const float* dy, const float* w, float* dx, int Nb, int H, int W, int C, int R, int S,
                                                int stride_h, int stride_w, int pad_h, int pad_w, int num_ctas, void* stream) {
    if (Nb < 0 || H <= 0 || W <= 0 || C <= 0 || (C & 3) || R <= 0 || S <= 0 || stride_h <= 0 || stride_w <= 0 || pad_h < 0 || pad_w < 0 ||
        num_ctas <= 0)
        return -1;
    if (Nb == 0) return 0;
    const int P = (H + 2 * pad_h - R) / stride_h + 1, Q = (W + 2 * pad_w - S) / stride_w + 1;
    if (P <= 0 || Q <= 0) return -1;
    if (((uintptr_t)dy | (uintptr_t)dx) % 16) return -2;
    if (R == 3 && S == 3 && stride_h == 1 && stride_w == 1 && pad_h <= 2 && pad_w <= 2) {
        // dx = dy convolved with the filter rotated by 180 degrees, padding 2 - pad: the forward kernel itself
        const long long total4 = (long long)Nb * H * ((W + 3) / 4) * (C / 4);
        long long want4 = (total4 + ELT_THREADS - 1) / ELT_THREADS, cap4 = (long long)num_ctas * 4;
        OB200_ELASTIC_HBM(ob200::depthwise3x3_nhwc_f32_kernel<1>, 4);
        ob200::depthwise3x3_nhwc_f32_kernel<1><<<(int)(want4 < cap4 ? want4 : cap4), ELT_THREADS, 0, (cudaStream_t)stream>>>(
            dy, w, dx, nullptr, nullptr, 0, Nb, P, Q, C, H, W, 2 - pad_h, 2 - pad_w, 0, 1);
        return (int)cudaGetLastError();
    }
    const long long total = (long long)Nb * H * W * (C / 4);
    long long want = (total + ELT_THREADS - 1) / ELT_THREADS, cap = (long long)num_ctas * 8;
    OB200_ELASTIC_HBM(ob200::depthwise_dgrad_nhwc_f32_kernel, 8);
    ob200::depthwise_dgrad_nhwc_f32_kernel<<<(int)(want < cap ? want : cap), ELT_THREADS, 0, (cudaStream_t)stream>>>(
        dy, w, dx, Nb, H, W, C, R, S, P, Q, stride_h, stride_w, pad_h, pad_w);
    return (int)cudaGetLastError();
}

// 3x3 filters, equal strides and paddings in both directions; dw [C][3][3] is cleared on `stream` first.
extern "C" int ob200_depthwise_conv2d_wgrad3x3_f32(const float* dy, const float* x, float* dw, int Nb, int H, int W, int C, int stride,
                                                   int pad, int num_ctas, void* stream) {
    if (Nb < 0 || H <= 0 || W <= 0 || C <= 0 || (C & 3) || stride <= 0 || pad < 0 || num_ctas <= 0) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(dw, 0, (size_t)C * 9 * sizeof(float), s);
    if (e != cudaSuccess) return (int)e;
    if (Nb == 0) return 0;
    const int P = (H + 2 * pad - 3) / stride + 1, Q = (W + 2 * pad - 3) / stride + 1;
    if (P <= 0 || Q <= 0) return -1;
    if (((uintptr_t)dy | (uintptr_t)x) % 16) return -2;
    int cq = C / 4 < 32 ? C / 4 : 32;
    int ry = ELT_THREADS / cq, pow2 = 1;
    while (pow2 * 2 <= ry) pow2 *= 2;
    ry = pow2;
    const int c_groups = (C / 4 + cq - 1) / cq;
    const long long items = (long long)Nb * P * ((Q + 3) / 4);   // blocks of four output columns
    long long slabs = (long long)num_ctas * 4 / c_groups;
    if (slabs > (items + ry - 1) / ry) slabs = (items + ry - 1) / ry;
    if (slabs < 1) slabs = 1;
    const size_t smem = (size_t)cq * ry * 36 * sizeof(float);   // <= 256 * 144 B = 36 KB
    OB200_HBM_BOUND();
    ob200::depthwise_wgrad3x3_nhwc_f32_kernel<<<(unsigned)(slabs * c_groups), dim3(cq, ry), smem, s>>>(dy, x, dw, Nb, H, W, C, P, Q, stride, pad,
                                                                                                   (int)slabs);
    return (int)cudaGetLastError();
}
