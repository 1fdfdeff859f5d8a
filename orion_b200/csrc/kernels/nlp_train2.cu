// More gradient-side kernels of the transformer training clients (bfloat16 / float32, HBM-bound):
//   * column sums of a [rows, D] matrix: the bias gradient of a linear layer (the reduce_kernel rows of the reference's
//     benchmarking/model_kernels/bert_8_fb1);
//   * softmax backward: dS = scale * P * (dP - sum_j P_j dP_j) per row (softmax_warp_backward in the same profile);
//   * embedding lookup and its gradient (vectorized_gather_kernel / embedding_backward_feature_kernel there).
// They reach the scheduler through the reference's cudaLaunchKernel trap (src/cuda_capture/intercept_temp.cpp:418-458).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

#include "elastic.h"
#include "pdl.cuh"

namespace ob200 {

constexpr int N2_THREADS = 256;
constexpr int N2_MAX_D = 8192;
constexpr int N2_MAX_PARTS = 592;

template <typename T>
struct Ld8;
template <>
struct Ld8<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float (&v)[8]) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    __device__ static void store(float* p, const float (&v)[8]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <>
struct Ld8<__nv_bfloat16> {
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

// ------------------------------------------------------------------ column sums, two stages, fixed order
// A thread keeps one 16-byte column chunk and walks rows; the CTA's rows are summed through shared memory.
template <typename T>
__global__ void __launch_bounds__(N2_THREADS) colsum_rows_kernel(const T* __restrict__ x, float* __restrict__ partial, long long rows, int D,
                                                                long long ld) {
    constexpr int N = Ld8<T>::N;
    const int chunks = D / N;
    const int lanes_x = chunks < N2_THREADS ? chunks : N2_THREADS;
    const int rows_per_pass = N2_THREADS / lanes_x;
    const int tx = threadIdx.x % lanes_x, ty = threadIdx.x / lanes_x;
    extern __shared__ float sh[];   // [rows_per_pass][D]
    for (int c0 = tx; c0 < chunks; c0 += lanes_x) {
        const int col = c0 * N;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] = 0.f;
        if (ty < rows_per_pass) {
            const long long step = (long long)gridDim.x * rows_per_pass;
            long long row = (long long)blockIdx.x * rows_per_pass + ty;
            for (; row + 3 * step < rows; row += 4 * step) {   // four independent 16-byte loads in flight
                float v[4][8];
#pragma unroll
                for (int u = 0; u < 4; u++) Ld8<T>::load(x + (row + u * step) * ld + col, v[u]);
#pragma unroll
                for (int u = 0; u < 4; u++)
#pragma unroll
                    for (int e = 0; e < N; e++) acc[e] += v[u][e];
            }
            for (; row < rows; row += step) {
                float v[8];
                Ld8<T>::load(x + row * ld + col, v);
#pragma unroll
                for (int e = 0; e < N; e++) acc[e] += v[e];
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

// out[col] = sum of the CTAs' partial sums.  Thread (g, c) of a 1024-thread CTA adds parts g, g + 32, ... of column c (coalesced
// 128-byte reads), then the 32 group sums are added in group order: a fixed order of additions.
template <typename T>
__global__ void __launch_bounds__(1024) colsum_parts_kernel(const float* __restrict__ partial, int parts, int D, T* __restrict__ out) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    __shared__ float sh[32][33];
    const int c = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + c;
    float s = 0.f;
    if (col < D) {
#pragma unroll 4
        for (int p = g; p < parts; p += 32) s += partial[(long long)p * D + col];
    }
    sh[g][c] = s;
    __syncthreads();
    if (g == 0 && col < D) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 32; k++) t += sh[k][c];
        out[col] = (T)t;
    }
}

// ------------------------------------------------------------------ softmax backward, one warp per row
template <typename T>
__global__ void __launch_bounds__(N2_THREADS) softmax_backward_kernel(const T* __restrict__ prob, const T* __restrict__ dprob, T* __restrict__ ds,
                                                                     long long rows, int D, float scale, int causal_period) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    constexpr int N = Ld8<T>::N;
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const int chunks = D / N;
    for (long long row = warp; row < rows; row += nwarps) {
        const T* p = prob + row * D;
        const T* g = dprob + row * D;
        // causal: columns behind the query's own position hold prob = 0 and possibly unwritten dprob
        const int last = causal_period > 0 ? (int)(row % causal_period) : D;
        float dot = 0.f;
        for (int c = lane; c < chunks && c * N <= last; c += 32) {
            float a[8], b[8];
            Ld8<T>::load(p + c * N, a);
            Ld8<T>::load(g + c * N, b);
#pragma unroll
            for (int e = 0; e < N; e++)
                if (c * N + e <= last) dot = fmaf(a[e], b[e], dot);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        T* out = ds + row * D;
        for (int c = lane; c < chunks; c += 32) {   // second read of the row comes from L1 / L2
            float a[8], b[8];
            if (c * N <= last) {
                Ld8<T>::load(p + c * N, a);
                Ld8<T>::load(g + c * N, b);
#pragma unroll
                for (int e = 0; e < N; e++) a[e] = (c * N + e <= last) ? scale * a[e] * (b[e] - dot) : 0.f;
            } else {
#pragma unroll
                for (int e = 0; e < 8; e++) a[e] = 0.f;
            }
            Ld8<T>::store(out + c * N, a);
        }
    }
}

// ------------------------------------------------------------------ embedding lookup and gradient (bfloat16 / float32 rows)
// out[t, :] = sum over tables k of table_k[ids_k[t], :]: up to three tables (word, position, segment) in one pass.
struct EmbTables {
    const void* table[3];
    const long long* ids[3];    // null: the row index is t % period[k]
    long long period[3];
    int count;
};

template <typename T>
__global__ void __launch_bounds__(N2_THREADS) embedding_sum_kernel(const EmbTables tb, T* __restrict__ out, long long tokens, int D) {
    pdl_launch_dependents();   // a GEMM behind this kernel may set itself up meanwhile (pdl.cuh)
    constexpr int N = Ld8<T>::N;
    const int chunks = D / N;
    const long long total = tokens * chunks;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / chunks;
        const int col = (int)(i - t * chunks) * N;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] = 0.f;
        for (int k = 0; k < tb.count; k++) {
            const long long r = tb.ids[k] ? tb.ids[k][t] : t % tb.period[k];
            float v[8];
            Ld8<T>::load(reinterpret_cast<const T*>(tb.table[k]) + r * D + col, v);
#pragma unroll
            for (int e = 0; e < N; e++) acc[e] += v[e];
        }
        Ld8<T>::store(out + t * D + col, acc);
    }
}

__device__ __forceinline__ void emb_atomic_add(float* p, float a, float b) {
    atomicAdd(p, a);
    atomicAdd(p + 1, b);
}
__device__ __forceinline__ void emb_atomic_add(__nv_bfloat16* p, float a, float b) {
    atomicAdd(reinterpret_cast<__nv_bfloat162*>(p), __floats2bfloat162_rn(a, b));
}

// dtable[ids[t], :] += dy[t, :] (ids null: row t % period).  dtable is cleared by the caller's launch before.
template <typename T>
__global__ void __launch_bounds__(N2_THREADS) embedding_backward_kernel(const T* __restrict__ dy, const long long* __restrict__ ids,
                                                                       long long period, T* __restrict__ dtable, long long tokens, int D) {
    constexpr int N = Ld8<T>::N;
    const int chunks = D / N;
    const long long total = tokens * chunks;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / chunks;
        const int col = (int)(i - t * chunks) * N;
        const long long r = ids ? ids[t] : t % period;
        float v[8];
        Ld8<T>::load(dy + t * D + col, v);
        T* dst = dtable + r * D + col;
#pragma unroll
        for (int e = 0; e < N; e += 2) emb_atomic_add(dst + e, v[e], v[e + 1]);
    }
}

static std::mutex g_n2_mu;
static std::unordered_map<uint64_t, float*> g_n2_partial;
static float* n2_partial_for(cudaStream_t s) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    const uint64_t key = ((uint64_t)dev << 56) ^ (uint64_t)(uintptr_t)s;
    std::lock_guard<std::mutex> lk(g_n2_mu);
    auto it = g_n2_partial.find(key);
    if (it != g_n2_partial.end()) return it->second;
    float* p = nullptr;
    if (cudaMalloc(&p, (size_t)N2_MAX_PARTS * N2_MAX_D * sizeof(float)) != cudaSuccess) return nullptr;
    g_n2_partial[key] = p;
    return p;
}

}  // namespace ob200

using namespace ob200;

// out[col] = sum over rows of x[row, col]; x rows `ld` elements apart (ld >= D, a multiple of 4 / 8); out in x's type.
extern "C" int ob200_colsum(const void* x, void* out, long long rows, int D, long long ld, int dtype, int num_ctas, void* stream) {
    const int n = dtype == 1 ? 8 : 4;
    if ((dtype != 0 && dtype != 1) || num_ctas <= 0 || D <= 0 || D % n || D > N2_MAX_D || ld < D || ld % n || rows < 0) return -1;
    if (((uintptr_t)x | (uintptr_t)out) % 16) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    if (rows == 0) return (int)cudaMemsetAsync(out, 0, (size_t)D * (dtype == 1 ? 2 : 4), s);
    float* partial = n2_partial_for(s);
    if (!partial) return -1;
    const int chunks = D / n;
    const int lanes_x = chunks < N2_THREADS ? chunks : N2_THREADS;
    const int rows_per_pass = N2_THREADS / lanes_x;
    long long want = (rows + rows_per_pass - 1) / rows_per_pass, cap = (long long)num_ctas * 2;
    if (cap > N2_MAX_PARTS) cap = N2_MAX_PARTS;
    const int grid = (int)(want < cap ? want : cap);
    const size_t smem = (size_t)rows_per_pass * D * sizeof(float);
    OB200_HBM_BOUND();
    if (dtype == 0) colsum_rows_kernel<float><<<grid, N2_THREADS, smem, s>>>((const float*)x, partial, rows, D, ld);
    else colsum_rows_kernel<__nv_bfloat16><<<grid, N2_THREADS, smem, s>>>((const __nv_bfloat16*)x, partial, rows, D, ld);
    OB200_HBM_BOUND();
    if (dtype == 0) colsum_parts_kernel<float><<<(D + 31) / 32, 1024, 0, s>>>(partial, grid, D, (float*)out);
    else colsum_parts_kernel<__nv_bfloat16><<<(D + 31) / 32, 1024, 0, s>>>(partial, grid, D, (__nv_bfloat16*)out);
    return (int)cudaGetLastError();
}

// ds[row, :] = scale * prob[row, :] * (dprob[row, :] - sum_j prob[row, j] dprob[row, j]); ds may alias dprob.
// causal_period > 0: columns behind position row % causal_period are skipped (ds = 0 there).
extern "C" int ob200_softmax_backward(const void* prob, const void* dprob, void* ds, long long rows, int D, float scale, int causal_period,
                                      int dtype, int num_ctas, void* stream) {
    const int n = dtype == 1 ? 8 : 4;
    if ((dtype != 0 && dtype != 1) || num_ctas <= 0 || D <= 0 || D % n || rows < 0) return -1;
    if (rows == 0) return 0;
    if (((uintptr_t)prob | (uintptr_t)dprob | (uintptr_t)ds) % 16) return -2;
    long long want = (rows + 7) / 8, cap = (long long)num_ctas * 8;
    const int grid = (int)(want < cap ? want : cap);
    OB200_ELASTIC_HBM(softmax_backward_kernel<float>, 8);
    OB200_ELASTIC(softmax_backward_kernel<__nv_bfloat16>, 8);
    if (dtype == 0)
        softmax_backward_kernel<float><<<grid, N2_THREADS, 0, (cudaStream_t)stream>>>((const float*)prob, (const float*)dprob, (float*)ds, rows, D, scale, causal_period);
    else
        softmax_backward_kernel<__nv_bfloat16><<<grid, N2_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)prob, (const __nv_bfloat16*)dprob,
                                                                                         (__nv_bfloat16*)ds, rows, D, scale, causal_period);
    return (int)cudaGetLastError();
}

// out[t, :] = sum_k table_k[row_k(t), :], row_k(t) = ids_k[t], or t % period_k where ids_k is NULL (a position table).
extern "C" int ob200_embedding_sum(const void* const* tables, const long long* const* ids, const long long* periods, int count, void* out,
                                   long long tokens, int D, int dtype, int num_ctas, void* stream) {
    const int n = dtype == 1 ? 8 : 4;
    if ((dtype != 0 && dtype != 1) || count < 1 || count > 3 || num_ctas <= 0 || D <= 0 || D % n || tokens < 0) return -1;
    if (tokens == 0) return 0;
    EmbTables tb;
    tb.count = count;
    for (int k = 0; k < 3; k++) {
        tb.table[k] = k < count ? tables[k] : nullptr;
        tb.ids[k] = k < count ? ids[k] : nullptr;
        tb.period[k] = k < count ? periods[k] : 1;
        if (k < count && (((uintptr_t)tables[k]) % 16 || (!ids[k] && periods[k] <= 0))) return -2;
    }
    if ((uintptr_t)out % 16) return -2;
    const long long total = tokens * (D / n);
    long long want = (total + N2_THREADS - 1) / N2_THREADS, cap = (long long)num_ctas * 8;
    const int grid = (int)(want < cap ? want : cap);
    OB200_ELASTIC_HBM(embedding_sum_kernel<float>, 8);
    OB200_ELASTIC(embedding_sum_kernel<__nv_bfloat16>, 8);
    if (dtype == 0) embedding_sum_kernel<float><<<grid, N2_THREADS, 0, (cudaStream_t)stream>>>(tb, (float*)out, tokens, D);
    else embedding_sum_kernel<__nv_bfloat16><<<grid, N2_THREADS, 0, (cudaStream_t)stream>>>(tb, (__nv_bfloat16*)out, tokens, D);
    return (int)cudaGetLastError();
}

// dtable = 0, then dtable[row(t), :] += dy[t, :] with atomic adds (the order of the adds is not fixed, as in the stock kernel).
extern "C" int ob200_embedding_backward(const void* dy, const long long* ids, long long period, void* dtable, long long table_rows,
                                        long long tokens, int D, int dtype, int num_ctas, void* stream) {
    const int n = dtype == 1 ? 8 : 4;
    if ((dtype != 0 && dtype != 1) || num_ctas <= 0 || D <= 0 || D % n || tokens < 0 || table_rows <= 0 || (!ids && period <= 0)) return -1;
    if (((uintptr_t)dy | (uintptr_t)dtable) % 16) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(dtable, 0, (size_t)table_rows * D * (dtype == 1 ? 2 : 4), s);
    if (e != cudaSuccess) return (int)e;
    if (tokens == 0) return 0;
    const long long total = tokens * (D / n);
    long long want = (total + N2_THREADS - 1) / N2_THREADS, cap = (long long)num_ctas * 8;
    const int grid = (int)(want < cap ? want : cap);
    OB200_ELASTIC_HBM(embedding_backward_kernel<float>, 8);
    OB200_ELASTIC(embedding_backward_kernel<__nv_bfloat16>, 8);
    if (dtype == 0)
        embedding_backward_kernel<float><<<grid, N2_THREADS, 0, s>>>((const float*)dy, ids, period, (float*)dtable, tokens, D);
    else
        embedding_backward_kernel<__nv_bfloat16><<<grid, N2_THREADS, 0, s>>>((const __nv_bfloat16*)dy, ids, period, (__nv_bfloat16*)dtable, tokens, D);
    return (int)cudaGetLastError();
}
