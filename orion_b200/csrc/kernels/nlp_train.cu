// Training-side row kernels of the transformer clients (BERT fine-tuning, decoder-LM training): LayerNorm forward with
// saved statistics and its backward, the backward of bias + GELU, cross-entropy over a large vocabulary (forward and
// backward, straight from bfloat16 logits), and AdamW over a whole parameter list per launch.  float32 math throughout;
// activations float32 or bfloat16, parameters in the activations' type (the clients hold bfloat16 models).
//
// They take the place of the at::native kernels that reach the reference through its cudaLaunchKernel trap
// (reference src/cuda_capture/intercept_temp.cpp:418-458) and that its BERT training profile lists
// (reference benchmarking/model_kernels/bert_8_fb1): layer_norm_grad_input_kernel, GammaBetaBackwardCUDAKernel, the GELU
// backward elementwise kernel, softmax / nll_loss forward and backward, and the multi-tensor optimizer kernels.
//
// Per-column parameter gradients (dgamma, dbeta, dbias) are reduced in two stages with a fixed order: every CTA of the
// row pass writes its column sums to its own slice of a partial buffer, a second kernel adds the slices in CTA order.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

#include "elastic.h"
#include "pdl.cuh"
#include "fast_gelu.cuh"

namespace ob200 {

constexpr int NT_THREADS = 256;     // 8 warps
constexpr int NT_MAX_D = 8192;
constexpr int NT_MAX_PARTS = 600;   // row-pass CTAs whose column sums the second stage adds

template <typename T>
struct Vec8;
template <>
struct Vec8<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float (&v)[8]) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    __device__ static void store(float* p, const float (&v)[8]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <>
struct Vec8<__nv_bfloat16> {
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

__device__ __forceinline__ float nt_warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}
__device__ __forceinline__ float nt_warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}

// ------------------------------------------------------------------ LayerNorm
// One warp per row; a lane owns the 16-byte chunks (c*32 + lane) of the row, CH of them (D <= 32 * CH * N).
template <typename T, int CH>
__global__ void __launch_bounds__(NT_THREADS) ln_train_forward_kernel(const T* __restrict__ x, T* __restrict__ y, const T* __restrict__ gamma,
                                                                     const T* __restrict__ beta, float* __restrict__ mean_out,
                                                                     float* __restrict__ rstd_out, long long rows, int D, float eps) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    constexpr int N = Vec8<T>::N;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    for (long long row = (long long)blockIdx.x * wpb + wid; row < rows; row += (long long)gridDim.x * wpb) {
        const T* xr = x + row * D;
        float v[CH][8];
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < CH; c++) {
            const int i = (c * 32 + lane) * N;
            if (i < D) {
                Vec8<T>::load(xr + i, v[c]);
#pragma unroll
                for (int e = 0; e < N; e++) s += v[c][e];
            }
        }
        const float mean = nt_warp_sum(s) / (float)D;
        float q = 0.f;
#pragma unroll
        for (int c = 0; c < CH; c++)
            if ((c * 32 + lane) * N < D) {
#pragma unroll
                for (int e = 0; e < N; e++) q += (v[c][e] - mean) * (v[c][e] - mean);
            }
        const float rstd = rsqrtf(nt_warp_sum(q) / (float)D + eps);
        T* yr = y + row * D;
#pragma unroll
        for (int c = 0; c < CH; c++) {
            const int i = (c * 32 + lane) * N;
            if (i < D) {
                float g[8], b[8];
                Vec8<T>::load(gamma + i, g);
                Vec8<T>::load(beta + i, b);
#pragma unroll
                for (int e = 0; e < N; e++) v[c][e] = fmaf((v[c][e] - mean) * rstd, g[e], b[e]);
                Vec8<T>::store(yr + i, v[c]);
            }
        }
        if (lane == 0) {
            mean_out[row] = mean;
            rstd_out[row] = rstd;
        }
    }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) with g = dy * gamma; column sums of dy * xhat and dy per CTA.
// The column sums of a warp live in shared memory (each lane adds to its own columns, 16-byte accesses), not in registers:
// with the row's dy and xhat that keeps a thread near 100 registers, so two CTAs share an SM and the whole grid is resident.
template <typename T, int CH>
__global__ void __launch_bounds__(NT_THREADS, 2) ln_backward_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                                                                   const float* __restrict__ mean, const float* __restrict__ rstd,
                                                                   T* __restrict__ dx, float* __restrict__ partial, long long rows, int D) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    constexpr int N = Vec8<T>::N;
    extern __shared__ float sh[];   // [warps][2][D]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    float* acc_g = sh + (size_t)(wid * 2 + 0) * D;   // this warp's column sums of dy * xhat
    float* acc_b = sh + (size_t)(wid * 2 + 1) * D;   // and of dy
#pragma unroll
    for (int c = 0; c < CH; c++) {
        const int i = (c * 32 + lane) * N;
        if (i < D) {
#pragma unroll
            for (int e = 0; e < N; e += 4) {
                *reinterpret_cast<float4*>(acc_g + i + e) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4*>(acc_b + i + e) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }
    for (long long row = (long long)blockIdx.x * wpb + wid; row < rows; row += (long long)gridDim.x * wpb) {
        const float mu = mean[row], rs = rstd[row];
        float d[CH][8], xh[CH][8];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int c = 0; c < CH; c++) {
            const int i = (c * 32 + lane) * N;
            if (i < D) {
                float gm[8];
                Vec8<T>::load(dy + row * D + i, d[c]);
                Vec8<T>::load(x + row * D + i, xh[c]);
                Vec8<T>::load(gamma + i, gm);            // L1-resident after the first row
#pragma unroll
                for (int e = 0; e < N; e += 4) {
                    float4 ag = *reinterpret_cast<float4*>(acc_g + i + e), ab = *reinterpret_cast<float4*>(acc_b + i + e);
                    float* pg = &ag.x;
                    float* pb = &ab.x;
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        xh[c][e + k] = (xh[c][e + k] - mu) * rs;
                        pg[k] += d[c][e + k] * xh[c][e + k];
                        pb[k] += d[c][e + k];
                        d[c][e + k] *= gm[e + k];
                        s1 += d[c][e + k];
                        s2 += d[c][e + k] * xh[c][e + k];
                    }
                    *reinterpret_cast<float4*>(acc_g + i + e) = ag;
                    *reinterpret_cast<float4*>(acc_b + i + e) = ab;
                }
            }
        }
        s1 = nt_warp_sum(s1) / (float)D;
        s2 = nt_warp_sum(s2) / (float)D;
#pragma unroll
        for (int c = 0; c < CH; c++) {
            const int i = (c * 32 + lane) * N;
            if (i < D) {
#pragma unroll
                for (int e = 0; e < N; e++) d[c][e] = rs * (d[c][e] - s1 - xh[c][e] * s2);
                Vec8<T>::store(dx + row * D + i, d[c]);
            }
        }
    }
    // warps -> CTA (fixed order), CTA slice of the partial buffer
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) {
        const int which = i / D, col = i - which * D;
        float s = 0.f;
        for (int w = 0; w < wpb; w++) s += sh[(w * 2 + which) * D + col];
        partial[((long long)blockIdx.x * 2 + which) * D + col] = s;
    }
}

// out[which][col] = sum over parts of partial[part][which][col]; written as T.  A CTA of 1024 threads owns 32 consecutive
// (which, col) entries: thread (g, c) adds parts g, g + 32, ... of entry c (one coalesced 128-byte read per part and group),
// then the 32 group sums are added in group order, so the order of the additions is fixed.
template <typename T>
__global__ void __launch_bounds__(1024) colsum_finish_kernel(const float* __restrict__ partial, int parts, int D, int n_which,
                                                            T* __restrict__ out0, T* __restrict__ out1) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    __shared__ float sh[32][33];
    const int c = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int i = blockIdx.x * 32 + c;
    const int total = n_which * D;
    float s = 0.f;
    if (i < total) {
        const int which = i / D, col = i - which * D;
        const float* src = partial + (long long)which * D + col;
        const long long step = (long long)n_which * D;
#pragma unroll 4
        for (int p = g; p < parts; p += 32) s += src[p * step];
    }
    sh[g][c] = s;
    __syncthreads();
    if (g == 0 && i < total) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 32; k++) t += sh[k][c];
        const int which = i / D, col = i - which * D;
        T* out = which == 0 ? out0 : out1;
        if (out) out[col] = (T)t;
    }
}

// ------------------------------------------------------------------ bias + GELU (bias in the activations' type)
template <typename T>
__global__ void __launch_bounds__(NT_THREADS) bias_gelu_forward_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ y,
                                                                      long long n_vec, int D) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    constexpr int N = Vec8<T>::N;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    const int step = (int)((stride * N) % D);   // the column is carried along with 32-bit adds
    int col = (int)((i * N) % D);
    for (; i + stride < n_vec; i += 2 * stride) {   // two independent 16-byte loads in flight per thread
        float v0[8], v1[8], b[8];
        Vec8<T>::load(x + i * N, v0);
        Vec8<T>::load(x + (i + stride) * N, v1);
#pragma unroll
        for (int e = 0; e < 8; e++) b[e] = 0.f;
        if (bias) Vec8<T>::load(bias + col, b);
#pragma unroll
        for (int e = 0; e < N; e++) {
            const float a = v0[e] + b[e];
            v0[e] = a * gauss_cdf(a);
        }
        Vec8<T>::store(y + i * N, v0);
        col += step;
        if (col >= D) col -= D;
        if (bias) Vec8<T>::load(bias + col, b);
#pragma unroll
        for (int e = 0; e < N; e++) {
            const float a = v1[e] + b[e];
            v1[e] = a * gauss_cdf(a);
        }
        Vec8<T>::store(y + (i + stride) * N, v1);
        col += step;
        if (col >= D) col -= D;
    }
    for (; i < n_vec; i += stride) {
        float v[8], b[8];
        Vec8<T>::load(x + i * N, v);
#pragma unroll
        for (int e = 0; e < 8; e++) b[e] = 0.f;
        if (bias) Vec8<T>::load(bias + col, b);
#pragma unroll
        for (int e = 0; e < N; e++) {
            const float a = v[e] + b[e];
            v[e] = a * gauss_cdf(a);
        }
        Vec8<T>::store(y + i * N, v);
        col += step;
        if (col >= D) col -= D;
    }
}

// ------------------------------------------------------------------ bias + GELU backward
// dx = dy * gelu'(x + bias); column sums of dx (= dbias) per CTA.  A thread keeps one 16-byte column chunk and walks rows.
template <typename T>
__global__ void __launch_bounds__(NT_THREADS) bias_gelu_backward_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                                       const T* __restrict__ bias, T* __restrict__ dx,
                                                                       float* __restrict__ partial, long long rows, int D) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    constexpr int N = Vec8<T>::N;
    const int chunks = D / N;                       // 16-byte chunks per row
    const int lanes_x = chunks < NT_THREADS ? chunks : NT_THREADS;   // threads across a row
    const int rows_per_pass = NT_THREADS / lanes_x; // rows a CTA covers per pass (>= 1)
    const int tx = threadIdx.x % lanes_x, ty = threadIdx.x / lanes_x;
    extern __shared__ float sh[];                   // [rows_per_pass][D] for the final reduction
    for (int c0 = tx; c0 < chunks; c0 += lanes_x) {
        const int col = c0 * N;
        float b[8], acc[8];
#pragma unroll
        for (int e = 0; e < 8; e++) b[e] = acc[e] = 0.f;
        if (bias) Vec8<T>::load(bias + col, b);
        if (ty < rows_per_pass) {
            for (long long row = (long long)blockIdx.x * rows_per_pass + ty; row < rows; row += (long long)gridDim.x * rows_per_pass) {
                float d[8], v[8];
                Vec8<T>::load(dy + row * D + col, d);
                Vec8<T>::load(x + row * D + col, v);
#pragma unroll
                for (int e = 0; e < N; e++) {
                    const float a = v[e] + b[e];
                    const float ex = __expf(-0.5f * a * a);
                    const float cdf = gauss_cdf_with_exp(a, ex);
                    const float pdf = 0.3989422804014327f * ex;
                    d[e] *= cdf + a * pdf;
                    acc[e] += d[e];
                }
                Vec8<T>::store(dx + row * D + col, d);
            }
#pragma unroll
            for (int e = 0; e < N; e++) sh[ty * D + col + e] = acc[e];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float s = 0.f;
        for (int r = 0; r < rows_per_pass; r++) s += sh[r * D + i];
        partial[(long long)blockIdx.x * D + i] = s;
    }
}

// ------------------------------------------------------------------ cross-entropy over a large vocabulary
// One CTA per row.  Forward: loss[row] = logsumexp(x) - x[target], lse[row] kept for the backward pass.
template <typename T>
__global__ void __launch_bounds__(NT_THREADS) cross_entropy_forward_kernel(const T* __restrict__ logits, const long long* __restrict__ target,
                                                                          float* __restrict__ loss, float* __restrict__ lse, int V) {
    constexpr int N = Vec8<T>::N;
    __shared__ float red[NT_THREADS / 32];
    __shared__ float s_val;
    const long long row = blockIdx.x;
    const T* xr = logits + row * (long long)V;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    float m = -INFINITY;
    for (int i = threadIdx.x * N; i < V; i += NT_THREADS * N) {
        float v[8];
        Vec8<T>::load(xr + i, v);
#pragma unroll
        for (int e = 0; e < N; e++) m = fmaxf(m, v[e]);
    }
    m = nt_warp_max(m);
    if (lane == 0) red[wid] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = red[0];
        for (int w = 1; w < NT_THREADS / 32; w++) t = fmaxf(t, red[w]);
        s_val = t;
    }
    __syncthreads();
    m = s_val;
    float s = 0.f;
    for (int i = threadIdx.x * N; i < V; i += NT_THREADS * N) {
        float v[8];
        Vec8<T>::load(xr + i, v);
#pragma unroll
        for (int e = 0; e < N; e++) s += __expf(v[e] - m);
    }
    s = nt_warp_sum(s);
    __syncthreads();
    if (lane == 0) red[wid] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < NT_THREADS / 32; w++) t += red[w];
        const float l = m + logf(t);
        lse[row] = l;
        loss[row] = l - (float)xr[target[row]];
    }
}

// dlogits = (exp(x - lse) - onehot(target)) * scale, scale = upstream gradient / rows (read from device memory).
template <typename T>
__global__ void __launch_bounds__(NT_THREADS) cross_entropy_backward_kernel(const T* __restrict__ logits, const long long* __restrict__ target,
                                                                           const float* __restrict__ lse, const float* __restrict__ grad,
                                                                           T* __restrict__ dlogits, int V, float inv_rows) {
    constexpr int N = Vec8<T>::N;
    const long long row = blockIdx.x;
    const T* xr = logits + row * (long long)V;
    T* dr = dlogits + row * (long long)V;
    const float l = lse[row], scale = grad[0] * inv_rows;
    const int t = (int)target[row];
    for (int i = threadIdx.x * N; i < V; i += NT_THREADS * N) {
        float v[8];
        Vec8<T>::load(xr + i, v);
#pragma unroll
        for (int e = 0; e < N; e++) v[e] = (__expf(v[e] - l) - (i + e == t ? 1.f : 0.f)) * scale;
        Vec8<T>::store(dr + i, v);
    }
}

// ------------------------------------------------------------------ AdamW over a parameter list
constexpr int ADAM_MAX_TENSORS = 72;
constexpr int ADAM_CHUNK = 16384;
struct AdamTable {
    void* p[ADAM_MAX_TENSORS];
    const void* g[ADAM_MAX_TENSORS];
    void* m[ADAM_MAX_TENSORS];
    void* v[ADAM_MAX_TENSORS];
    long long n[ADAM_MAX_TENSORS];
    int first_chunk[ADAM_MAX_TENSORS + 1];
    int count;
};
__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T>
__device__ __forceinline__ T from_f(float x);
template <>
__device__ __forceinline__ float from_f<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16(x); }

// torch.optim.AdamW: p *= 1 - lr*wd; m = b1*m + (1-b1)*g; v = b2*v + (1-b2)*g^2; p -= lr/bc1 * m / (sqrt(v)/sqrt(bc2) + eps).
// State tensors have the parameter's type, as torch keeps them; the arithmetic is float32.
template <typename T>
__global__ void __launch_bounds__(NT_THREADS) adamw_multi_kernel(const __grid_constant__ AdamTable t, float lr, float b1, float b2, float eps,
                                                                float wd, float bc1, float bc2_sqrt) {
    const int total_chunks = t.first_chunk[t.count];
    for (int chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
        int lo = 0, hi = t.count - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (t.first_chunk[mid] <= chunk) lo = mid; else hi = mid - 1;
        }
        const long long begin = (long long)(chunk - t.first_chunk[lo]) * ADAM_CHUNK;
        const long long end = begin + ADAM_CHUNK < t.n[lo] ? begin + ADAM_CHUNK : t.n[lo];
        T* __restrict__ p = (T*)t.p[lo];
        const T* __restrict__ g = (const T*)t.g[lo];
        T* __restrict__ m = (T*)t.m[lo];
        T* __restrict__ v = (T*)t.v[lo];
        const float decay = 1.0f - lr * wd, step_size = lr / bc1, inv_bc2 = 1.0f / bc2_sqrt;
        constexpr int N = Vec8<T>::N;
        // 16-byte accesses where the four tensors are 16-byte aligned (chunks start at multiples of 16384 elements)
        const bool vec = ((((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15) == 0);
        const long long vec_end = vec ? begin + (end - begin) / N * N : begin;
        for (long long i = begin + (long long)threadIdx.x * N; i < vec_end; i += (long long)blockDim.x * N) {
            float gv[8], pv[8], mv[8], vv[8];
            Vec8<T>::load(g + i, gv);
            Vec8<T>::load(p + i, pv);
            Vec8<T>::load(m + i, mv);
            Vec8<T>::load(v + i, vv);
#pragma unroll
            for (int e = 0; e < N; e++) {
                mv[e] = b1 * mv[e] + (1.0f - b1) * gv[e];
                vv[e] = b2 * vv[e] + (1.0f - b2) * gv[e] * gv[e];
                pv[e] = pv[e] * decay - step_size * mv[e] / (sqrtf(vv[e]) * inv_bc2 + eps);
            }
            Vec8<T>::store(m + i, mv);
            Vec8<T>::store(v + i, vv);
            Vec8<T>::store(p + i, pv);
        }
        for (long long i = vec_end + threadIdx.x; i < end; i += blockDim.x) {
            const float grad = to_f(g[i]);
            float param = to_f(p[i]) * decay;
            const float mi = b1 * to_f(m[i]) + (1.0f - b1) * grad;
            const float vi = b2 * to_f(v[i]) + (1.0f - b2) * grad * grad;
            m[i] = from_f<T>(mi);
            v[i] = from_f<T>(vi);
            param -= step_size * mi / (sqrtf(vi) * inv_bc2 + eps);
            p[i] = from_f<T>(param);
        }
    }
}

// Per-(device, stream) buffer for the column-sum partials (overwritten by every call; calls on one stream are ordered).
static std::mutex g_nt_mu;
static std::unordered_map<uint64_t, float*> g_nt_partial;
static float* nt_partial_for(cudaStream_t s) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    const uint64_t key = ((uint64_t)dev << 56) ^ (uint64_t)(uintptr_t)s;
    std::lock_guard<std::mutex> lk(g_nt_mu);
    auto it = g_nt_partial.find(key);
    if (it != g_nt_partial.end()) return it->second;
    float* p = nullptr;
    if (cudaMalloc(&p, (size_t)NT_MAX_PARTS * 2 * NT_MAX_D * sizeof(float)) != cudaSuccess) return nullptr;
    g_nt_partial[key] = p;
    return p;
}

static inline bool nt_aligned(const void* a, const void* b = nullptr, const void* c = nullptr, const void* d = nullptr) {
    return (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d) % 16) == 0;
}

}  // namespace ob200

using namespace ob200;

// y = LayerNorm(x) * gamma + beta over the last dimension; mean / rstd [rows] are kept for the backward pass.
// dtype 0 float32, 1 bfloat16 (x, y, gamma, beta all of that type); D a multiple of 4 / 8, D <= 256 * N.
extern "C" int ob200_layernorm_train_forward(const void* x, void* y, const void* gamma, const void* beta, float* mean, float* rstd,
                                             long long rows, int D, float eps, int dtype, int num_ctas, void* stream) {
    if (rows <= 0) return 0;
    const int n = dtype == 1 ? 8 : 4;
    if ((dtype != 0 && dtype != 1) || num_ctas <= 0 || D <= 0 || D % n || D > 8 * 32 * n || !gamma || !beta || !mean || !rstd) return -1;
    if (!nt_aligned(x, y, gamma, beta)) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    long long want = (rows + 7) / 8, cap = (long long)num_ctas * 8;
    const int grid = (int)(want < cap ? want : cap);
    const int chunks = (D / n + 31) / 32;
#define OB200_LNF(T, CH)                                                                                                        \
    do {                                                                                                                       \
        OB200_ELASTIC_HBM((ln_train_forward_kernel<T, CH>), 8);                                                                 \
        ln_train_forward_kernel<T, CH><<<grid, NT_THREADS, 0, s>>>((const T*)x, (T*)y, (const T*)gamma, (const T*)beta, mean, rstd, \
                                                                   rows, D, eps);                                              \
    } while (0)
    if (dtype == 0) {
        if (chunks <= 2) OB200_LNF(float, 2); else if (chunks <= 4) OB200_LNF(float, 4); else OB200_LNF(float, 8);
    } else {
        if (chunks <= 2) OB200_LNF(__nv_bfloat16, 2); else if (chunks <= 4) OB200_LNF(__nv_bfloat16, 4); else OB200_LNF(__nv_bfloat16, 8);
    }
#undef OB200_LNF
    return (int)cudaGetLastError();
}

// dx, dgamma, dbeta of the above (dgamma / dbeta in the activations' type; either may be NULL).
extern "C" int ob200_layernorm_backward(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                                        void* dgamma, void* dbeta, long long rows, int D, int dtype, int num_ctas, void* stream) {
    if (rows <= 0) return 0;
    const int n = dtype == 1 ? 8 : 4;
    if ((dtype != 0 && dtype != 1) || num_ctas <= 0 || D <= 0 || D % n || D > 4 * 32 * n || D > NT_MAX_D || !gamma || !mean || !rstd) return -1;
    if (!nt_aligned(dy, x, gamma, dx)) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    float* partial = nt_partial_for(s);
    if (!partial) return -1;
    long long want = (rows + 7) / 8, cap = (long long)num_ctas * 2;
    if (cap > NT_MAX_PARTS) cap = NT_MAX_PARTS;
    const int grid = (int)(want < cap ? want : cap);
    const size_t smem = (size_t)(NT_THREADS / 32) * 2 * D * sizeof(float);
    const int chunks = (D / n + 31) / 32;
#define OB200_LNB(T, CH)                                                                                                              \
    do {                                                                                                                             \
        static bool attr = false;                                                                                                    \
        if (!attr && smem > 48 * 1024) {                                                                                             \
            cudaFuncSetAttribute(ln_backward_kernel<T, CH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 2 * 1024 * 4);           \
            attr = true;                                                                                                             \
        }                                                                                                                            \
        OB200_HBM_BOUND();                                                                                                           \
        ln_backward_kernel<T, CH><<<grid, NT_THREADS, smem, s>>>((const T*)dy, (const T*)x, (const T*)gamma, mean, rstd, (T*)dx, partial, \
                                                                 rows, D);                                                           \
        OB200_HBM_BOUND();                                                                                                           \
        colsum_finish_kernel<T><<<(2 * D + 31) / 32, 1024, 0, s>>>(partial, grid, D, 2, (T*)dgamma, (T*)dbeta);                      \
    } while (0)
    if (dtype == 0) {
        if (chunks <= 2) OB200_LNB(float, 2); else OB200_LNB(float, 4);
    } else {
        if (chunks <= 2) OB200_LNB(__nv_bfloat16, 2); else OB200_LNB(__nv_bfloat16, 4);
    }
#undef OB200_LNB
    return (int)cudaGetLastError();
}

// y = gelu(x + bias) with the exact (erf) GELU; bias [D] in the activations' type (or NULL).
extern "C" int ob200_bias_gelu_train_forward(const void* x, const void* bias, void* y, long long rows, int D, int dtype, int num_ctas,
                                             void* stream) {
    if (rows <= 0) return 0;
    const int n = dtype == 1 ? 8 : 4;
    if ((dtype != 0 && dtype != 1) || num_ctas <= 0 || D <= 0 || D % n) return -1;
    if (!nt_aligned(x, bias, y)) return -2;
    const long long n_vec = rows * D / n;
    long long want = (n_vec + NT_THREADS - 1) / NT_THREADS, cap = (long long)num_ctas * 6;
    const int grid = (int)(want < cap ? want : cap);
    if (dtype == 0) {
        OB200_ELASTIC_HBM(bias_gelu_forward_kernel<float>, 6);
        bias_gelu_forward_kernel<float><<<grid, NT_THREADS, 0, (cudaStream_t)stream>>>((const float*)x, (const float*)bias, (float*)y, n_vec, D);
    } else {
        OB200_ELASTIC_HBM(bias_gelu_forward_kernel<__nv_bfloat16>, 6);
        bias_gelu_forward_kernel<__nv_bfloat16><<<grid, NT_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)bias,
                                                                                             (__nv_bfloat16*)y, n_vec, D);
    }
    return (int)cudaGetLastError();
}

// dx = dy * gelu'(x + bias), dbias = column sums of dx (NULL: not wanted).  x is the pre-activation without the bias.
extern "C" int ob200_bias_gelu_backward(const void* dy, const void* x, const void* bias, void* dx, void* dbias, long long rows, int D,
                                        int dtype, int num_ctas, void* stream) {
    if (rows <= 0) return 0;
    const int n = dtype == 1 ? 8 : 4;
    if ((dtype != 0 && dtype != 1) || num_ctas <= 0 || D <= 0 || D % n || D > NT_MAX_D) return -1;
    if (!nt_aligned(dy, x, bias, dx)) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    float* partial = nt_partial_for(s);
    if (!partial) return -1;
    const int chunks = D / n;
    const int lanes_x = chunks < NT_THREADS ? chunks : NT_THREADS;
    const int rows_per_pass = NT_THREADS / lanes_x;
    long long want = (rows + rows_per_pass - 1) / rows_per_pass, cap = (long long)num_ctas * 4;
    if (cap > NT_MAX_PARTS) cap = NT_MAX_PARTS;
    const int grid = (int)(want < cap ? want : cap);
    const size_t smem = (size_t)rows_per_pass * D * sizeof(float);
    OB200_HBM_BOUND();
    if (dtype == 0)
        bias_gelu_backward_kernel<float><<<grid, NT_THREADS, smem, s>>>((const float*)dy, (const float*)x, (const float*)bias, (float*)dx,
                                                                       partial, rows, D);
    else
        bias_gelu_backward_kernel<__nv_bfloat16><<<grid, NT_THREADS, smem, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                                               (const __nv_bfloat16*)bias, (__nv_bfloat16*)dx, partial, rows, D);
    if (dbias) {
        OB200_HBM_BOUND();
        if (dtype == 0) colsum_finish_kernel<float><<<(D + 31) / 32, 1024, 0, s>>>(partial, grid, D, 1, (float*)dbias, (float*)nullptr);
        else colsum_finish_kernel<__nv_bfloat16><<<(D + 31) / 32, 1024, 0, s>>>(partial, grid, D, 1, (__nv_bfloat16*)dbias, (__nv_bfloat16*)nullptr);
    }
    return (int)cudaGetLastError();
}

// loss[row] = -log softmax(logits[row])[target[row]] and lse[row] = logsumexp(logits[row]); logits [rows, V], V % 4 / 8 == 0.
extern "C" int ob200_cross_entropy_forward(const void* logits, const long long* target, float* loss, float* lse, long long rows, int V,
                                           int dtype, void* stream) {
    if (rows <= 0) return 0;
    const int n = dtype == 1 ? 8 : 4;
    if ((dtype != 0 && dtype != 1) || V <= 0 || V % n || rows > 0x7fffffffLL || !target || !loss || !lse) return -1;
    if (!nt_aligned(logits)) return -2;
    OB200_HBM_BOUND();
    if (dtype == 0) cross_entropy_forward_kernel<float><<<(unsigned)rows, NT_THREADS, 0, (cudaStream_t)stream>>>((const float*)logits, target, loss, lse, V);
    else cross_entropy_forward_kernel<__nv_bfloat16><<<(unsigned)rows, NT_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, target, loss, lse, V);
    return (int)cudaGetLastError();
}

// dlogits = (softmax(logits) - onehot(target)) * grad[0] / rows: the gradient of the mean loss times the upstream scalar.
extern "C" int ob200_cross_entropy_backward(const void* logits, const long long* target, const float* lse, const float* grad,
                                            void* dlogits, long long rows, int V, int dtype, void* stream) {
    if (rows <= 0) return 0;
    const int n = dtype == 1 ? 8 : 4;
    if ((dtype != 0 && dtype != 1) || V <= 0 || V % n || rows > 0x7fffffffLL || !target || !lse || !grad) return -1;
    if (!nt_aligned(logits, dlogits)) return -2;
    OB200_HBM_BOUND();
    if (dtype == 0)
        cross_entropy_backward_kernel<float><<<(unsigned)rows, NT_THREADS, 0, (cudaStream_t)stream>>>((const float*)logits, target, lse, grad,
                                                                                                   (float*)dlogits, V, 1.0f / (float)rows);
    else
        cross_entropy_backward_kernel<__nv_bfloat16><<<(unsigned)rows, NT_THREADS, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)logits, target, lse, grad, (__nv_bfloat16*)dlogits, V, 1.0f / (float)rows);
    return (int)cudaGetLastError();
}

// One AdamW step (torch.optim.AdamW semantics, step counted from 1) over `count` tensors of one type (dtype 0 float32,
// 1 bfloat16; optimizer state in the same type) in ceil(count / 72) launches.
extern "C" int ob200_adamw_multi(void* const* p, const void* const* g, void* const* m, void* const* v, const long long* n, int count,
                                 float lr, float beta1, float beta2, float eps, float weight_decay, int step, int dtype, int num_ctas,
                                 void* stream) {
    if (count <= 0) return 0;
    if (!p || !g || !m || !v || !n || num_ctas <= 0 || step < 1 || (dtype != 0 && dtype != 1)) return -1;
    const float bc1 = 1.0f - powf(beta1, (float)step);
    const float bc2_sqrt = sqrtf(1.0f - powf(beta2, (float)step));
    for (int base = 0; base < count; base += ADAM_MAX_TENSORS) {
        AdamTable t;
        t.count = 0;
        t.first_chunk[0] = 0;
        for (int i = base; i < count && t.count < ADAM_MAX_TENSORS; i++) {
            if (n[i] <= 0) continue;
            if (!p[i] || !g[i] || !m[i] || !v[i]) return -1;
            const int k = t.count++;
            t.p[k] = p[i]; t.g[k] = g[i]; t.m[k] = m[i]; t.v[k] = v[i];
            t.n[k] = n[i];
            t.first_chunk[k + 1] = t.first_chunk[k] + (int)((n[i] + ADAM_CHUNK - 1) / ADAM_CHUNK);
        }
        if (t.count == 0) continue;
        const int chunks = t.first_chunk[t.count];
        const long long cap = (long long)num_ctas * 4;
        const unsigned grid = (unsigned)(chunks < cap ? chunks : cap);
        if (dtype == 0) {
            OB200_ELASTIC_HBM(adamw_multi_kernel<float>, 4);
            adamw_multi_kernel<float><<<grid, NT_THREADS, 0, (cudaStream_t)stream>>>(t, lr, beta1, beta2, eps, weight_decay, bc1, bc2_sqrt);
        } else {
            OB200_ELASTIC_HBM(adamw_multi_kernel<__nv_bfloat16>, 4);
            adamw_multi_kernel<__nv_bfloat16><<<grid, NT_THREADS, 0, (cudaStream_t)stream>>>(t, lr, beta1, beta2, eps, weight_decay, bc1, bc2_sqrt);
        }
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}
