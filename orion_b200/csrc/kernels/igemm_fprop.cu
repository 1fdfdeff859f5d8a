// Implicit-GEMM forward convolution and linear layer on the 5th-generation tensor
// cores (tcgen05.mma, accumulators in TMEM), for NHWC activations and KRSC weights.
//
//   Y[m, k] = epilogue( sum_{r,s,c} X[n, p*sh - ph + r*dh, q*sw - pw + s*dw, c] * Wt[k, r, s, c] )
//   m = (n*P + p)*Q + q;   GEMM view: M = N*P*Q rows, N = K_out columns, K = R*S*C.
//
// It stands in for the cudnnConvolutionForward and cublasSgemm calls the reference
// replays (src/scheduler/utils_sched.cpp:284-296,490-501).
//
// One persistent CTA per granted SM (grid = the SM quota), each walking output
// tiles of 128 x BN.  Warp roles:
//   warps 0-3   epilogue: tcgen05.ld the fp32 accumulator, apply scale/shift,
//               residual and ReLU, store NHWC rows
//   warp  4     allocates TMEM, one lane issues tcgen05.mma and tcgen05.commit
//   warps 5-12  two producer groups of 128 threads that alternate over k-blocks:
//               gather one 128-byte row slice of the im2col matrix (zero-filled at
//               the image border) and of the filter per thread, and write them
//               into shared memory in the 128-byte-swizzled K-major layout
// fp32 inputs run as 3xTF32: each value is split into a TF32-rounded high part and
// the exact remainder, and lo*hi + hi*lo + hi*hi accumulate in fp32, which keeps
// the result within ~1e-6 relative of an fp32 reference.  bf16 inputs use one
// kind::f16 MMA per k-step.
//
// Split-K: when `splits > 1` each work unit covers a contiguous range of k-blocks of
// one tile and adds its partial tile into a zero-initialised fp32 scratch buffer
// with red.global.add; the unit that arrives last on the tile's counter applies the
// epilogue from the scratch sums.  (Accumulation order across splits is not fixed;
// `splits = 1` is bit-reproducible.)
//
// Every mbarrier wait is bounded; on expiry the kernel records a code in the status
// word, releases TMEM and returns.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "igemm_params.h"
#include "sm100_primitives.cuh"

namespace ob200 {

constexpr int BM = 128;
constexpr int EPI_WARPS = 4;
constexpr int MMA_WARP = 4;
constexpr int PROD_GROUPS = 2;
constexpr int NTHREADS = (EPI_WARPS + 1 + 4 * PROD_GROUPS) * 32;   // 416

template <typename T, int BN>
struct Cfg {
    static constexpr bool kSplit = sizeof(T) == 4;            // 3xTF32
    static constexpr int BK = 128 / sizeof(T);                // elements per 128-byte row
    static constexpr int EPC = 16 / sizeof(T);                // elements per 16-byte chunk
    static constexpr int A_BYTES = BM * 128;
    static constexpr int B_BYTES = BN * 128;
    static constexpr int STAGE_BYTES = (A_BYTES + B_BYTES) * (kSplit ? 2 : 1);
    static constexpr int STAGES = (200 * 1024) / STAGE_BYTES > 8 ? 8 : (200 * 1024) / STAGE_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
    static constexpr int TMEM_COLS = 2 * BN;
};

struct SharedCtl {
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    int last_flag;
};

__device__ __forceinline__ void ld_chunk(const float* p, bool ok, float4& v) {
    v = ok ? __ldg(reinterpret_cast<const float4*>(p)) : make_float4(0.f, 0.f, 0.f, 0.f);
}
__device__ __forceinline__ void ld_chunk(const __nv_bfloat16* p, bool ok, uint4& v) {
    v = ok ? __ldg(reinterpret_cast<const uint4*>(p)) : make_uint4(0u, 0u, 0u, 0u);
}

template <typename T>
struct ChunkOf;
template <>
struct ChunkOf<float> {
    using type = float4;
};
template <>
struct ChunkOf<__nv_bfloat16> {
    using type = uint4;
};

// Store one 16-byte chunk of an operand row; fp32 also stores the low-order remainder.
__device__ __forceinline__ void st_chunk(uint8_t* hi, uint8_t* lo, uint32_t off, const float4& v) {
    float4 h, l;
    h.x = tf32_round(v.x); h.y = tf32_round(v.y); h.z = tf32_round(v.z); h.w = tf32_round(v.w);
    l.x = v.x - h.x; l.y = v.y - h.y; l.z = v.z - h.z; l.w = v.w - h.w;
    *reinterpret_cast<float4*>(hi + off) = h;
    *reinterpret_cast<float4*>(lo + off) = l;
}
__device__ __forceinline__ void st_chunk(uint8_t* hi, uint8_t*, uint32_t off, const uint4& v) {
    *reinterpret_cast<uint4*>(hi + off) = v;
}

__device__ __forceinline__ void set_elem(float4& v, int i, float x) {
    if (i == 0) v.x = x; else if (i == 1) v.y = x; else if (i == 2) v.z = x; else v.w = x;
}
__device__ __forceinline__ void set_elem(uint4& v, int i, __nv_bfloat16 x) {
    uint32_t bits = (uint32_t)__bfloat16_as_ushort(x) << ((i & 1) * 16);
    uint32_t* w = (i < 2) ? &v.x : (i < 4) ? &v.y : (i < 6) ? &v.z : &v.w;
    *w |= bits;
}

template <typename T, int BN>
__global__ void __launch_bounds__(NTHREADS, 1) igemm_fprop_kernel(const IgemmParams p) {
    using C = Cfg<T, BN>;
    using Chunk = typename ChunkOf<T>::type;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem + C::STAGES * C::STAGE_BYTES);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(&ctl->full[s], 4);       // one elected lane per producer warp of the owning group
            mbar_init(&ctl->empty[s], 1);      // tcgen05.commit
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&ctl->tmem_full[b], 1);           // tcgen05.commit
            mbar_init(&ctl->tmem_empty[b], EPI_WARPS);  // one elected lane per epilogue warp
        }
        ctl->abort_flag = 0;
        ctl->last_flag = 0;
        fence_barrier_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(&ctl->tmem_base, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctl->tmem_base;
    volatile int* abort_flag = &ctl->abort_flag;

    const int tiles = p.tiles_m * p.tiles_n;
    const int units = tiles * p.splits;
    const int SC = p.S * p.C;

    if (warp < EPI_WARPS) {
        // ------------------------------------------------------------ epilogue
        int local = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x, local++) {
            const int tile = u / p.splits;
            const int tm = tile / p.tiles_n, tn = tile % p.tiles_n;
            const int ab = local & 1;
            if (!mbar_wait(&ctl->tmem_full[ab], (local >> 1) & 1, abort_flag)) {
                if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_TMEM_FULL); }
                break;
            }
            tc_fence_after_sync();
            const int row = warp * 32 + lane;
            const long long m = (long long)tm * BM + row;
            const bool row_ok = m < p.M;
            bool finalize = true;
            float* part = nullptr;
            if (p.splits > 1) {
                // Add this unit's partial tile into the fp32 scratch; the last unit of the tile finalises.
                part = p.scratch + ((long long)tile * BM + row) * BN;
#pragma unroll 1
                for (int cb = 0; cb < BN / 32; cb++) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + ab * BN + cb * 32, r);
                    tmem_ld_wait();
                    if (row_ok) {
#pragma unroll
                        for (int j = 0; j < 32; j++) atomicAdd(part + cb * 32 + j, __uint_as_float(r[j]));
                    }
                }
                __threadfence();
                __syncwarp();
                // All four epilogue warps must have added their rows before the unit counts as arrived.
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (tid == 0) {
                    int prev = atomicAdd(p.counters + tile, 1);
                    ctl->last_flag = (prev == p.splits - 1);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                finalize = ctl->last_flag != 0;
                __threadfence();
            }
            if (finalize) {
#pragma unroll 1
                for (int cb = 0; cb < BN / 32; cb++) {
                    float v[32];
                    if (p.splits > 1) {
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = row_ok ? __ldcg(part + cb * 32 + j) : 0.f;
                        // leave the scratch zeroed for the next launch
                        if (row_ok) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4*>(part + cb * 32 + j) = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    } else {
                        uint32_t r[32];
                        tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + ab * BN + cb * 32, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
                    }
                    if (row_ok) {
                        const int n0 = tn * BN + cb * 32;
                        const long long base = m * p.Kout + n0;
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const int n = n0 + j;
                            if (n < p.Kout) {
                                float x = v[j];
                                if (p.scale) x *= __ldg(p.scale + n);
                                if (p.shift) x += __ldg(p.shift + n);
                                if (p.residual) {
                                    if (sizeof(T) == 4) x += __ldg(reinterpret_cast<const float*>(p.residual) + base + j);
                                    else x += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[base + j]);
                                }
                                if (p.relu) x = fmaxf(x, 0.f);
                                if (p.relu == 2) x = fminf(x, 6.f);
                                v[j] = x;
                            }
                        }
                        if (sizeof(T) == 4) {
                            float* y = reinterpret_cast<float*>(p.y) + base;
                            if ((p.Kout & 3) == 0) {
#pragma unroll
                                for (int j = 0; j < 32; j += 4)
                                    if (n0 + j < p.Kout)
                                        *reinterpret_cast<float4*>(y + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; j++)
                                    if (n0 + j < p.Kout) y[j] = v[j];
                            }
                        } else {
                            __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(p.y) + base;
                            if ((p.Kout & 7) == 0) {
#pragma unroll
                                for (int j = 0; j < 32; j += 8) {
                                    if (n0 + j < p.Kout) {
                                        uint4 o;
                                        __nv_bfloat162 t0 = __floats2bfloat162_rn(v[j], v[j + 1]);
                                        __nv_bfloat162 t1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                                        __nv_bfloat162 t2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
                                        __nv_bfloat162 t3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                                        o.x = *reinterpret_cast<uint32_t*>(&t0);
                                        o.y = *reinterpret_cast<uint32_t*>(&t1);
                                        o.z = *reinterpret_cast<uint32_t*>(&t2);
                                        o.w = *reinterpret_cast<uint32_t*>(&t3);
                                        *reinterpret_cast<uint4*>(y + j) = o;
                                    }
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; j++)
                                    if (n0 + j < p.Kout) y[j] = __float2bfloat16(v[j]);
                            }
                        }
                    }
                }
                if (p.splits > 1 && tid == 0) p.counters[tile] = 0;   // ready for the next launch
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->tmem_empty[ab]);
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------ MMA issue
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(C::kSplit ? 2 : 1, BM, BN);
            uint32_t it = 0;
            int local = 0;
            bool dead = false;
            for (int u = blockIdx.x; u < units && !dead; u += gridDim.x, local++) {
                const int split = u % p.splits;
                const int kb_begin = (int)((long long)p.num_kblocks * split / p.splits);
                const int kb_end = (int)((long long)p.num_kblocks * (split + 1) / p.splits);
                const int ab = local & 1;
                if (!mbar_wait(&ctl->tmem_empty[ab], ((local >> 1) & 1) ^ 1, abort_flag)) {
                    if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_TMEM_EMPTY); }
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d = tmem_base + ab * BN;
                for (int kb = kb_begin; kb < kb_end; kb++, it++) {
                    const int s = it % C::STAGES;
                    if (!mbar_wait(&ctl->full[s], (it / C::STAGES) & 1, abort_flag)) {
                        if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_FULL); }
                        dead = true;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t base = smem_u32(smem + s * C::STAGE_BYTES);
                    if (C::kSplit) {
                        const uint64_t a_hi = umma_desc_sw128(base);
                        const uint64_t a_lo = umma_desc_sw128(base + C::A_BYTES);
                        const uint64_t b_hi = umma_desc_sw128(base + 2 * C::A_BYTES);
                        const uint64_t b_lo = umma_desc_sw128(base + 2 * C::A_BYTES + C::B_BYTES);
#pragma unroll
                        for (int ks = 0; ks < 4; ks++) {
                            const uint64_t o = (uint64_t)(ks * 2);   // 32 bytes per k-step, in 16-byte units
                            umma_tf32(d, a_lo + o, b_hi + o, idesc, (kb > kb_begin || ks > 0) ? 1u : 0u);
                            umma_tf32(d, a_hi + o, b_lo + o, idesc, 1u);
                            umma_tf32(d, a_hi + o, b_hi + o, idesc, 1u);
                        }
                    } else {
                        const uint64_t a = umma_desc_sw128(base);
                        const uint64_t b = umma_desc_sw128(base + C::A_BYTES);
#pragma unroll
                        for (int ks = 0; ks < 4; ks++) {
                            const uint64_t o = (uint64_t)(ks * 2);
                            umma_f16(d, a + o, b + o, idesc, (kb > kb_begin || ks > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(&ctl->empty[s]);   // frees the stage once these MMAs have read it
                }
                if (!dead) umma_commit(&ctl->tmem_full[ab]);
            }
        }
    } else {
        // ------------------------------------------------------------ producers
        const int pw = warp - (MMA_WARP + 1);       // 0..7
        const int group = pw >> 2;                  // producer group
        const int row = (pw & 3) * 32 + lane;       // 0..127: A row, and B row when < BN
        const T* __restrict__ X = reinterpret_cast<const T*>(p.x);
        const T* __restrict__ Wt = reinterpret_cast<const T*>(p.w);
        const bool vec = (p.C % C::EPC) == 0;
        uint32_t it = 0;
        bool dead = false;
        for (int u = blockIdx.x; u < units && !dead; u += gridDim.x) {
            const int tile = u / p.splits, split = u % p.splits;
            const int tm = tile / p.tiles_n, tn = tile % p.tiles_n;
            const int kb_begin = (int)((long long)p.num_kblocks * split / p.splits);
            const int kb_end = (int)((long long)p.num_kblocks * (split + 1) / p.splits);
            const long long m = (long long)tm * BM + row;
            const bool m_ok = m < p.M;
            int n_img = 0, h_base = 0, w_base = 0;
            if (m_ok) {
                const int pq = p.P * p.Q;
                n_img = (int)(m / pq);
                const int rem = (int)(m - (long long)n_img * pq);
                const int op = rem / p.Q, oq = rem - op * p.Q;
                h_base = op * p.stride_h - p.pad_h;
                w_base = oq * p.stride_w - p.pad_w;
            }
            const int kout = tn * BN + row;
            const bool b_ok = row < BN && kout < p.Kout;
            for (int kb = kb_begin; kb < kb_end; kb++, it++) {
                if ((int)(it % PROD_GROUPS) != group) continue;
                const int s = it % C::STAGES;
                const int r = kb / p.kblocks_per_r;
                const int kk0 = (kb - r * p.kblocks_per_r) * C::BK;
                const int h = h_base + r * p.dil_h;
                const bool h_ok = m_ok && h >= 0 && h < p.H;
                Chunk a[8], b[8];
                const T* xrow = X + ((long long)n_img * p.H + (h_ok ? h : 0)) * p.W * p.C;
                const T* wrow = Wt + ((long long)(b_ok ? kout : 0) * p.R + r) * SC;
                if (vec) {
                    int ts = kk0 / p.C, tc = kk0 - ts * p.C;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int kk = kk0 + j * C::EPC;
                        const int w = w_base + ts * p.dil_w;
                        const bool ok = h_ok && kk < SC && w >= 0 && w < p.W;
                        ld_chunk(xrow + (long long)(ok ? w : 0) * p.C + tc, ok, a[j]);
                        ld_chunk(wrow + kk, b_ok && kk < SC, b[j]);
                        tc += C::EPC;
                        if (tc >= p.C) { tc -= p.C; ts++; }
                    }
                } else {
                    int ts = kk0 / p.C, tc = kk0 - ts * p.C;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        Chunk av, bv;
                        ld_chunk((const T*)nullptr, false, av);
                        ld_chunk((const T*)nullptr, false, bv);
#pragma unroll
                        for (int e = 0; e < C::EPC; e++) {
                            const int kk = kk0 + j * C::EPC + e;
                            const int w = w_base + ts * p.dil_w;
                            if (h_ok && kk < SC && w >= 0 && w < p.W) set_elem(av, e, xrow[(long long)w * p.C + tc]);
                            if (b_ok && kk < SC) set_elem(bv, e, wrow[kk]);
                            tc++;
                            if (tc >= p.C) { tc = 0; ts++; }
                        }
                        a[j] = av;
                        b[j] = bv;
                    }
                }
                if (!mbar_wait(&ctl->empty[s], ((it / C::STAGES) & 1) ^ 1, abort_flag)) {
                    if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_EMPTY); }
                    dead = true;
                    break;
                }
                uint8_t* st = smem + s * C::STAGE_BYTES;
                uint8_t* a_hi = st;
                uint8_t* a_lo = st + C::A_BYTES;
                uint8_t* b_hi = st + (C::kSplit ? 2 : 1) * C::A_BYTES;
                uint8_t* b_lo = b_hi + C::B_BYTES;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint32_t off = sw128_offset((uint32_t)row, (uint32_t)j);
                    st_chunk(a_hi, a_lo, off, a[j]);
                    if (row < BN) st_chunk(b_hi, b_lo, off, b[j]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->full[s]);
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

template <typename T, int BN>
static cudaError_t launch_cfg(const IgemmParams& p, int num_ctas, cudaStream_t stream) {
    using C = Cfg<T, BN>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(igemm_fprop_kernel<T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    igemm_fprop_kernel<T, BN><<<num_ctas, NTHREADS, C::SMEM_BYTES, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace ob200

extern "C" int ob200_igemm_launch(const IgemmParams* params, int bn, int num_ctas, void* stream) {
    using namespace ob200;
    IgemmParams p = *params;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (p.dtype == 0) {
        return (int)(bn == 64 ? launch_cfg<float, 64>(p, num_ctas, s) : launch_cfg<float, 128>(p, num_ctas, s));
    } else if (p.dtype == 1) {
        return (int)(bn == 64 ? launch_cfg<__nv_bfloat16, 64>(p, num_ctas, s) : launch_cfg<__nv_bfloat16, 128>(p, num_ctas, s));
    }
    return -1;
}
