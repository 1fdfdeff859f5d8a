// Warp-shuffle row kernels of the transformer clients (float32 or bfloat16 data, float32 math):
// LayerNorm, softmax, bias + GELU, and the AdamW update.  They stand in for the at::native kernels
// that dominate the reference's BERT / Transformer profiles behind its cudaLaunchKernel trap
// (vectorized_layer_norm_kernel, softmax_warp_forward, vectorized_elementwise_kernel;
// reference src/cuda_capture/intercept_temp.cpp:418-458).
//
// All are HBM-bound: one warp owns one row, lanes read 16-byte vectors, reductions use
// __shfl_xor_sync; the grid is persistent (SM quota x warps per CTA) and strides over the rows.
// Algorithmic bytes per element: LayerNorm and softmax read once and write once when a row fits
// the L1/L2 re-read (rows of 384..4096 elements do), GELU 2 accesses, AdamW 7 float accesses.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "elastic.h"
#include "pdl.cuh"
#include "fast_gelu.cuh"

namespace ob200 {

constexpr int ROW_THREADS = 256;   // 8 warps = 8 rows per CTA pass

template <typename T>
struct VecIO;
template <>
struct VecIO<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float (&v)[8]) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    __device__ static void store(float* p, const float (&v)[8]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <>
struct VecIO<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 q = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    __device__ static void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint4 q;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = q;
    }
};

// N (4 or 8) consecutive per-column coefficients as 16-byte loads; `fill` where the vector is absent.
template <int N>
__device__ __forceinline__ void load_cols(const float* __restrict__ p, int i, float fill, float (&o)[8]) {
    if (!p) {
#pragma unroll
        for (int e = 0; e < N; e++) o[e] = fill;
        return;
    }
#pragma unroll
    for (int e = 0; e < N; e += 4) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(p + i + e));
        o[e] = q.x; o[e + 1] = q.y; o[e + 2] = q.z; o[e + 3] = q.w;
    }
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}

// Rows that fit a warp's registers (D <= 32 lanes x CH chunks of 16 bytes) are read once: every lane issues all
// its 16-byte loads up front, the statistics and the result come from registers.  One global read and one write
// per element, and CH independent loads in flight per lane.
template <typename T, int CH>
__global__ void __launch_bounds__(ROW_THREADS) layernorm_regs_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                    const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                    float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                    long long rows, int D, float eps) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    constexpr int N = VecIO<T>::N;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    for (long long row = (long long)blockIdx.x * wpb + wid; row < rows; row += (long long)gridDim.x * wpb) {
        const T* xr = x + row * D;
        float v[CH][8];
#pragma unroll
        for (int c = 0; c < CH; c++) {
            const int i = (c * 32 + lane) * N;
            if (i < D) VecIO<T>::load(xr + i, v[c]);
        }
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < CH; c++)
            if ((c * 32 + lane) * N < D) {
#pragma unroll
                for (int e = 0; e < N; e++) s += v[c][e];
            }
        const float mean = warp_sum(s) / (float)D;
        float q = 0.f;
#pragma unroll
        for (int c = 0; c < CH; c++)
            if ((c * 32 + lane) * N < D) {
#pragma unroll
                for (int e = 0; e < N; e++) q += (v[c][e] - mean) * (v[c][e] - mean);
            }
        const float rstd = rsqrtf(warp_sum(q) / (float)D + eps);
        T* yr = y + row * D;
#pragma unroll
        for (int c = 0; c < CH; c++) {
            const int i = (c * 32 + lane) * N;
            if (i < D) {
                float g[8], b[8];
                load_cols<N>(gamma, i, 1.f, g);
                load_cols<N>(beta, i, 0.f, b);
#pragma unroll
                for (int e = 0; e < N; e++) v[c][e] = fmaf((v[c][e] - mean) * rstd, g[e], b[e]);
                VecIO<T>::store(yr + i, v[c]);
            }
        }
        if (lane == 0) {
            if (mean_out) mean_out[row] = mean;
            if (rstd_out) rstd_out[row] = rstd;
        }
    }
}

template <typename T, int CH>
__global__ void __launch_bounds__(ROW_THREADS) softmax_regs_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int D,
                                                                  float scale, int causal_period) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    constexpr int N = VecIO<T>::N;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    for (long long row = (long long)blockIdx.x * wpb + wid; row < rows; row += (long long)gridDim.x * wpb) {
        const T* xr = x + row * D;
        // causal attention: row r holds the scores of query position r % period; later keys are masked out
        const int last = causal_period > 0 ? (int)(row % causal_period) : D;
        float v[CH][8];
#pragma unroll
        for (int c = 0; c < CH; c++) {
            const int i = (c * 32 + lane) * N;
            if (i < D) VecIO<T>::load(xr + i, v[c]);
        }
        float m = -INFINITY;
#pragma unroll
        for (int c = 0; c < CH; c++)
            if ((c * 32 + lane) * N < D) {
#pragma unroll
                for (int e = 0; e < N; e++) {
                    v[c][e] = ((c * 32 + lane) * N + e > last) ? -INFINITY : v[c][e] * scale;
                    m = fmaxf(m, v[c][e]);
                }
            }
        m = warp_max(m);
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < CH; c++)
            if ((c * 32 + lane) * N < D) {
#pragma unroll
                for (int e = 0; e < N; e++) {
                    v[c][e] = __expf(v[c][e] - m);
                    s += v[c][e];
                }
            }
        const float inv = 1.0f / warp_sum(s);
        T* yr = y + row * D;
#pragma unroll
        for (int c = 0; c < CH; c++) {
            const int i = (c * 32 + lane) * N;
            if (i < D) {
#pragma unroll
                for (int e = 0; e < N; e++) v[c][e] *= inv;
                VecIO<T>::store(yr + i, v[c]);
            }
        }
    }
}

// y = (x - mean) / sqrt(var + eps) * gamma + beta over the last dimension D (D % VecIO<T>::N == 0).
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) layernorm_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ gamma,
                                                               const float* __restrict__ beta, float* __restrict__ mean_out,
                                                               float* __restrict__ rstd_out, long long rows, int D, float eps) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    constexpr int N = VecIO<T>::N;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    for (long long row = (long long)blockIdx.x * wpb + wid; row < rows; row += (long long)gridDim.x * wpb) {
        const T* xr = x + row * D;
        float v[8];
        float s = 0.f;
        for (int i = lane * N; i < D; i += 32 * N) {
            VecIO<T>::load(xr + i, v);
#pragma unroll
            for (int e = 0; e < N; e++) s += v[e];
        }
        const float mean = warp_sum(s) / (float)D;
        float q = 0.f;
        for (int i = lane * N; i < D; i += 32 * N) {
            VecIO<T>::load(xr + i, v);
#pragma unroll
            for (int e = 0; e < N; e++) q += (v[e] - mean) * (v[e] - mean);
        }
        const float rstd = rsqrtf(warp_sum(q) / (float)D + eps);
        T* yr = y + row * D;
        for (int i = lane * N; i < D; i += 32 * N) {
            VecIO<T>::load(xr + i, v);
#pragma unroll
            for (int e = 0; e < N; e++) {
                float o = (v[e] - mean) * rstd;
                if (gamma) o *= __ldg(gamma + i + e);
                if (beta) o += __ldg(beta + i + e);
                v[e] = o;
            }
            VecIO<T>::store(yr + i, v);
        }
        if (lane == 0) {
            if (mean_out) mean_out[row] = mean;
            if (rstd_out) rstd_out[row] = rstd;
        }
    }
}

// y = softmax(x * scale) over the last dimension D.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) softmax_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int D,
                                                             float scale, int causal_period) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    constexpr int N = VecIO<T>::N;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    for (long long row = (long long)blockIdx.x * wpb + wid; row < rows; row += (long long)gridDim.x * wpb) {
        const T* xr = x + row * D;
        const int last = causal_period > 0 ? (int)(row % causal_period) : D;
        float v[8];
        float m = -INFINITY;
        for (int i = lane * N; i < D; i += 32 * N) {
            VecIO<T>::load(xr + i, v);
#pragma unroll
            for (int e = 0; e < N; e++)
                if (i + e <= last) m = fmaxf(m, v[e] * scale);
        }
        m = warp_max(m);
        float s = 0.f;
        for (int i = lane * N; i < D; i += 32 * N) {
            VecIO<T>::load(xr + i, v);
#pragma unroll
            for (int e = 0; e < N; e++)
                if (i + e <= last) s += __expf(v[e] * scale - m);
        }
        const float inv = 1.0f / warp_sum(s);
        T* yr = y + row * D;
        for (int i = lane * N; i < D; i += 32 * N) {
            VecIO<T>::load(xr + i, v);
#pragma unroll
            for (int e = 0; e < N; e++) v[e] = (i + e <= last) ? __expf(v[e] * scale - m) * inv : 0.f;
            VecIO<T>::store(yr + i, v);
        }
    }
}

// y = gelu(x + bias[col]) with the exact (erf) GELU; bias may be NULL.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) bias_gelu_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ bias,
                                                               long long n_vec, int D) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    constexpr int N = VecIO<T>::N;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    // the column of a vector is carried along with 32-bit adds: one 64-bit remainder per thread, not one per vector
    const int step = (int)((stride * N) % D);
    int col = (int)((i * N) % D);
    for (; i + 3 * stride < n_vec; i += 4 * stride) {   // four independent 16-byte loads in flight per thread
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 4; u++) VecIO<T>::load(x + (i + u * stride) * N, v[u]);
#pragma unroll
        for (int u = 0; u < 4; u++) {
            float b[8];
            load_cols<N>(bias, col, 0.f, b);
#pragma unroll
            for (int e = 0; e < N; e++) {
                const float a = v[u][e] + b[e];
                v[u][e] = a * gauss_cdf(a);
            }
            VecIO<T>::store(y + (i + u * stride) * N, v[u]);
            col += step;
            if (col >= D) col -= D;
        }
    }
    for (; i < n_vec; i += stride) {
        float v[8];
        VecIO<T>::load(x + i * N, v);
#pragma unroll
        for (int e = 0; e < N; e++) {
            const float a = v[e] + (bias ? __ldg(bias + col + e) : 0.f);
            v[e] = a * gauss_cdf(a);
        }
        VecIO<T>::store(y + i * N, v);
        col += step;
        if (col >= D) col -= D;
    }
}

// torch.optim.AdamW step on one tensor: p *= 1 - lr*wd; m = b1*m + (1-b1)*g; v = b2*v + (1-b2)*g^2;
// p -= lr/bc1 * m / (sqrt(v)/sqrt(bc2) + eps), with bc = 1 - beta^step computed by the caller.
__global__ void __launch_bounds__(ROW_THREADS) adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                                           float* __restrict__ v, long long n, float lr, float b1, float b2, float eps,
                                                           float wd, float bc1, float bc2_sqrt) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float grad = g[i];
        float param = p[i] * (1.0f - lr * wd);
        const float mi = b1 * m[i] + (1.0f - b1) * grad;
        const float vi = b2 * v[i] + (1.0f - b2) * grad * grad;
        m[i] = mi;
        v[i] = vi;
        param -= (lr / bc1) * mi / (sqrtf(vi) / bc2_sqrt + eps);
        p[i] = param;
    }
}

static inline int row_grid(long long rows, int num_ctas) {
    long long want = (rows + 7) / 8;
    long long cap = (long long)num_ctas * 8;   // eight CTAs of eight warps per granted SM: rows in flight hide the latency
    if (want < 1) want = 1;
    return (int)(want < cap ? want : cap);
}

}  // namespace ob200

using namespace ob200;

static bool vec_ok(const void* a, const void* b, int D, int dtype) {
    const int n = dtype == 1 ? 8 : 4;
    return D > 0 && D % n == 0 && (((uintptr_t)a | (uintptr_t)b) % 16) == 0;
}

extern "C" int ob200_layernorm(const void* x, void* y, const float* gamma, const float* beta, float* mean_out, float* rstd_out,
                               long long rows, int D, float eps, int dtype, int num_ctas, void* stream) {
    if (rows <= 0) return 0;
    if ((dtype != 0 && dtype != 1) || num_ctas <= 0) return -1;
    if (!vec_ok(x, y, D, dtype) || (((uintptr_t)gamma | (uintptr_t)beta) % 16) != 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = row_grid(rows, num_ctas);
    const int chunks = (D / (dtype == 1 ? 8 : 4) + 31) / 32;   // 16-byte chunks per lane
#define OB200_LN(T, CH)                                                                                                             \
    do {                                                                                                                           \
        OB200_ELASTIC_HBM((layernorm_regs_kernel<T, CH>), 8);                                                                          \
        layernorm_regs_kernel<T, CH><<<grid, ROW_THREADS, 0, s>>>((const T*)x, (T*)y, gamma, beta, mean_out, rstd_out, rows, D, eps); \
    } while (0)
    if (dtype == 0) {
        if (chunks <= 2) OB200_LN(float, 2);
        else if (chunks <= 4) OB200_LN(float, 4);
        else if (chunks <= 8) OB200_LN(float, 8);
        else layernorm_kernel<float><<<grid, ROW_THREADS, 0, s>>>((const float*)x, (float*)y, gamma, beta, mean_out, rstd_out, rows, D, eps);
    } else {
        if (chunks <= 2) OB200_LN(__nv_bfloat16, 2);
        else if (chunks <= 4) OB200_LN(__nv_bfloat16, 4);
        else if (chunks <= 8) OB200_LN(__nv_bfloat16, 8);
        else layernorm_kernel<__nv_bfloat16><<<grid, ROW_THREADS, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, gamma, beta, mean_out,
                                                                        rstd_out, rows, D, eps);
    }
#undef OB200_LN
    return (int)cudaGetLastError();
}

extern "C" int ob200_softmax_causal(const void* x, void* y, long long rows, int D, float scale, int causal_period, int dtype,
                                    int num_ctas, void* stream) {
    if (rows <= 0) return 0;
    if ((dtype != 0 && dtype != 1) || num_ctas <= 0 || causal_period < 0) return -1;
    if (!vec_ok(x, y, D, dtype)) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = row_grid(rows, num_ctas);
    const int chunks = (D / (dtype == 1 ? 8 : 4) + 31) / 32;
#define OB200_SM(T, CH)                                                                        \
    do {                                                                                       \
        OB200_ELASTIC_HBM((softmax_regs_kernel<T, CH>), 8);                                        \
        softmax_regs_kernel<T, CH><<<grid, ROW_THREADS, 0, s>>>((const T*)x, (T*)y, rows, D, scale, causal_period); \
    } while (0)
    if (dtype == 0) {
        if (chunks <= 2) OB200_SM(float, 2);
        else if (chunks <= 4) OB200_SM(float, 4);
        else if (chunks <= 8) OB200_SM(float, 8);
        else softmax_kernel<float><<<grid, ROW_THREADS, 0, s>>>((const float*)x, (float*)y, rows, D, scale, causal_period);
    } else {
        if (chunks <= 2) OB200_SM(__nv_bfloat16, 2);
        else if (chunks <= 4) OB200_SM(__nv_bfloat16, 4);
        else if (chunks <= 8) OB200_SM(__nv_bfloat16, 8);
        else softmax_kernel<__nv_bfloat16><<<grid, ROW_THREADS, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, D, scale, causal_period);
    }
#undef OB200_SM
    return (int)cudaGetLastError();
}

extern "C" int ob200_softmax(const void* x, void* y, long long rows, int D, float scale, int dtype, int num_ctas, void* stream) {
    return ob200_softmax_causal(x, y, rows, D, scale, 0, dtype, num_ctas, stream);
}

extern "C" int ob200_bias_gelu(const void* x, void* y, const float* bias, long long rows, int D, int dtype, int num_ctas, void* stream) {
    if (rows <= 0) return 0;
    if ((dtype != 0 && dtype != 1) || num_ctas <= 0) return -1;
    if (!vec_ok(x, y, D, dtype) || ((uintptr_t)bias % 16) != 0) return -2;
    const int n = dtype == 1 ? 8 : 4;
    const long long n_vec = rows * D / n;
    long long want = (n_vec + ROW_THREADS - 1) / ROW_THREADS, cap = (long long)num_ctas * 6;
    const int grid = (int)(want < cap ? want : cap);
    cudaStream_t s = (cudaStream_t)stream;
    OB200_ELASTIC_HBM(bias_gelu_kernel<float>, 6);
    OB200_ELASTIC_HBM(bias_gelu_kernel<__nv_bfloat16>, 6);
    if (dtype == 0)
        bias_gelu_kernel<float><<<grid, ROW_THREADS, 0, s>>>((const float*)x, (float*)y, bias, n_vec, D);
    else
        bias_gelu_kernel<__nv_bfloat16><<<grid, ROW_THREADS, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, bias, n_vec, D);
    return (int)cudaGetLastError();
}

extern "C" int ob200_adamw_f32(float* p, const float* g, float* m, float* v, long long n, float lr, float beta1, float beta2, float eps,
                               float weight_decay, int step, int num_ctas, void* stream) {
    if (n <= 0) return 0;
    if (num_ctas <= 0 || step < 1) return -1;
    const float bc1 = 1.0f - powf(beta1, (float)step);
    const float bc2_sqrt = sqrtf(1.0f - powf(beta2, (float)step));
    long long want = (n + ROW_THREADS - 1) / ROW_THREADS, cap = (long long)num_ctas * 4;
    OB200_ELASTIC_HBM(adamw_kernel, 4);
    adamw_kernel<<<(int)(want < cap ? want : cap), ROW_THREADS, 0, (cudaStream_t)stream>>>(p, g, m, v, n, lr, beta1, beta2, eps,
                                                                                          weight_decay, bc1, bc2_sqrt);
    return (int)cudaGetLastError();
}
