// bfloat16 GEMM with either operand in either memory order, for the gradient side of the transformer clients:
//
//   C[b][m, n] = alpha * sum_k A[b][m, k] * B[b][n, k]  (+ bias[n])          b = batch_outer x batch_inner problems
//
// A lies in memory as [M, K] rows (K-major) or as [K, M] rows (MN-major); B as [N, K] rows or as [K, N] rows; row and
// batch strides are free (multiples of 8 elements).  That covers, without a transposed copy of anything,
//   dX = dY . W          (B = W [out, in]: the reduction index `out` is the slow one  -> B MN-major)
//   dW = dY^T . X        (both operands [tokens, features]: the reduction index is the slow one of both -> A and B MN-major)
//   attention:  P.V, dV = P^T.dO, dP = dO.V^T, dQ = dS.K, dK = dS^T.Q straight on the fused projection's [B, S, 3, H, 64]
// which the reference replays as cublasSgemm / cublasSgemmStridedBatched with transpose flags
// (reference src/scheduler/utils_sched.cpp:490-513; rows of benchmarking/model_kernels/bert_8_fb1).
//
// One CTA = 128 x BN output tile per work unit, persistent over units.  Warp 0 issues TMA copies (4-D tensor maps:
// inner, outer, batch_inner, batch_outer; out-of-range elements read as zero, so ragged M, N, K need no special path),
// warp 1 issues tcgen05.mma kind::f16 into one of two tensor-memory accumulators, warps 2-5 drain the other one:
// tcgen05.ld (one output row per thread), alpha / bias / residual in registers, 32 rows x 128 bytes staged in a swizzled
// shared-memory slab per warp and written by a TMA store (two slabs per warp in flight; the tensor map clips ragged edges;
// outputs whose rows are not 16-byte multiples take per-thread stores).  An MN-major operand is declared as such in the instruction
// descriptor; its stage is filled by boxes of 64 reduction rows x 128 bytes, which is the canonical layout (atoms of
// 8 rows x 128 bytes, 1024 bytes apart along the reduction, 8192 bytes apart along M / N).
// Split-K (few output tiles, long reduction: the weight gradients) writes float32 partial matrices that a second
// kernel sums in split order, so the result does not depend on timing or on the CTA count.  Causal attention: `tri` modes
// skip the score tiles above the diagonal and cut the reductions over keys / queries at it.  The kernel is launched as a
// programmatic dependent: its set-up overlaps the tail of the kernel before it in the stream.
// Every wait is bounded; on expiry the kernel sets the status word, frees tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "elastic.h"
#include "sm100_primitives.cuh"

namespace ob200 {

constexpr int GM_BM = 128;
constexpr int GM_BK = 64;
constexpr int GM_THREADS = 192;          // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue
constexpr int GM_A_BYTES = GM_BM * 128;

template <int BN>
struct GemmCfg {
    static constexpr int STAGE_BYTES = GM_A_BYTES + BN * 128;
    static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int EPI_BYTES = 4 * 2 * 4096;   // per epilogue warp two slabs of 32 rows x 128 bytes for the TMA stores
    static constexpr int SMEM = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
};

struct GemmParams {
    void* c;
    float* slabs;            // split-K partial matrices [splits][batch][M][N], or null
    const float* bias;
    const __nv_bfloat16* bias_bf16;   // the same addend given in bfloat16 (a parameter of a bfloat16 model)
    const __nv_bfloat16* residual;    // optional bfloat16 tensor laid out like C, added in float32 before rounding
    int* status;
    int M, N, K;
    int batch, nb_inner;
    long long ldc, c_si, c_so;
    int out_f32;
    int a_mn, b_mn;
    int tiles_m, tiles_n, kblocks, splits, kb_per_split;
    int vec_ok;              // C rows and batch offsets are 16-byte aligned
    int c_tma;               // C is written by TMA stores from swizzled shared-memory slabs (tmap_c)
    int tri;                 // causal attention: 1 = only output tiles that touch n <= m are computed (the rest is left unwritten),
                             // 2 = A[m, k] is zero for k > m (reduction stops behind the tile's last row),
                             // 3 = A[m, k] is zero for k < m (reduction starts at the tile's first row)
    float alpha;
    alignas(64) unsigned char tmap_a[128];
    alignas(64) unsigned char tmap_b[128];
    alignas(64) unsigned char tmap_c[128];
};

struct GemmCtl {
    uint64_t full[8], empty[8], acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ uint64_t gm_desc_mn(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(8192 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}

// k-blocks [kb0, kb1) of work unit (tile row tm, split sp); at least one block, the same for every warp role.
__device__ __forceinline__ void gm_kb_range(const GemmParams& p, int sp, int tm, int& kb0, int& kb1) {
    kb0 = sp * p.kb_per_split;
    kb1 = kb0 + p.kb_per_split < p.kblocks ? kb0 + p.kb_per_split : p.kblocks;
    if (p.tri == 2) {
        const int lim = (tm * GM_BM + GM_BM + GM_BK - 1) / GM_BK;
        if (lim < kb1) kb1 = lim > kb0 ? lim : kb0 + 1;
    } else if (p.tri == 3) {
        const int lo = (tm * GM_BM) / GM_BK;
        if (lo > kb0) kb0 = lo < kb1 ? lo : kb1 - 1;
    }
}
// With a causal mode the work per tile depends on its row, and a CTA's units (u = blockIdx.x + i * gridDim.x) would keep
// hitting the same rows of every problem.  Rotating the tile index by the problem index gives every CTA a mix of rows.
__device__ __forceinline__ int gm_rotate(const GemmParams& p, int t, int b, int tiles_per_problem) {
    return p.tri ? (t + b) % tiles_per_problem : t;
}
template <int BN>
__device__ __forceinline__ bool gm_tile_skipped(const GemmParams& p, int tm, int tn) {
    return p.tri == 1 && tn * BN > tm * GM_BM + GM_BM - 1;
}

template <int BN>
__global__ void __launch_bounds__(GM_THREADS, 1) gemm_bf16_kernel(const __grid_constant__ GemmParams p) {
    using C = GemmCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* epi_smem = smem + C::STAGES * C::STAGE_BYTES;
    GemmCtl* ctl = reinterpret_cast<GemmCtl*>(epi_smem + C::EPI_BYTES);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&ctl->acc_full[a], 1);
            mbar_init(&ctl->acc_empty[a], 4);
        }
        ctl->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(p.tmap_a);
        prefetch_tensormap(p.tmap_b);
        if (p.c_tma) prefetch_tensormap(p.tmap_c);
    }
    if (warp == 1) {
        tmem_alloc(&ctl->tmem_base, C::TMEM_COLS);
        tmem_relinquish();
        tc_fence_before_sync();
    }
    __syncthreads();
    tc_fence_after_sync();
    pdl_wait();
    if (tid == 0) pdl_launch_dependents();
    const uint32_t tmem_base = ctl->tmem_base;
    volatile int* abort_flag = &ctl->abort_flag;
    const int tiles_per_problem = p.tiles_m * p.tiles_n;
    const long long units = (long long)p.batch * tiles_per_problem * p.splits;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool dead = false;
            for (long long u = blockIdx.x; u < units && !dead; u += gridDim.x) {
                const int sp = (int)(u % p.splits);
                const int tile = (int)(u / p.splits);
                const int b = tile / tiles_per_problem, t = gm_rotate(p, tile - b * tiles_per_problem, b, tiles_per_problem);
                const int tm = t / p.tiles_n, tn = t - tm * p.tiles_n;
                const int bi = b % p.nb_inner, bo = b / p.nb_inner;
                if (gm_tile_skipped<BN>(p, tm, tn)) continue;
                int kb0, kb1;
                gm_kb_range(p, sp, tm, kb0, kb1);
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(&ctl->empty[s], ph ^ 1u, abort_flag)) {
                        if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_EMPTY); }
                        dead = true;
                        break;
                    }
                    const uint32_t a_dst = smem_u32(smem + s * C::STAGE_BYTES);
                    const uint32_t b_dst = a_dst + GM_A_BYTES;
                    mbar_arrive_expect_tx(&ctl->full[s], (uint32_t)C::STAGE_BYTES);
                    if (!p.a_mn) {
                        tma_load_tile_4d(a_dst, p.tmap_a, &ctl->full[s], kb * GM_BK, tm * GM_BM, bi, bo);
                    } else {
#pragma unroll
                        for (int g = 0; g < GM_BM / 64; g++)
                            tma_load_tile_4d(a_dst + g * 8192, p.tmap_a, &ctl->full[s], tm * GM_BM + 64 * g, kb * GM_BK, bi, bo);
                    }
                    if (!p.b_mn) {
                        tma_load_tile_4d(b_dst, p.tmap_b, &ctl->full[s], kb * GM_BK, tn * BN, bi, bo);
                    } else {
#pragma unroll
                        for (int g = 0; g < BN / 64; g++)
                            tma_load_tile_4d(b_dst + g * 8192, p.tmap_b, &ctl->full[s], tn * BN + 64 * g, kb * GM_BK, bi, bo);
                    }
                    if (++s == C::STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(1, GM_BM, BN) | (p.a_mn ? UMMA_IDESC_A_MN : 0u) | (p.b_mn ? UMMA_IDESC_B_MN : 0u);
            int s = 0;
            uint32_t ph = 0;
            uint32_t local = 0;
            bool dead = false;
            for (long long u = blockIdx.x; u < units && !dead; u += gridDim.x) {
                const int sp = (int)(u % p.splits);
                const int tile = (int)(u / p.splits);
                const int t = gm_rotate(p, tile % tiles_per_problem, tile / tiles_per_problem, tiles_per_problem);
                const int tm = t / p.tiles_n, tn = t - tm * p.tiles_n;
                if (gm_tile_skipped<BN>(p, tm, tn)) continue;
                int kb0, kb1;
                gm_kb_range(p, sp, tm, kb0, kb1);
                const uint32_t ab = local & 1u, use = local >> 1;
                local++;
                if (!mbar_wait(&ctl->acc_empty[ab], (use & 1u) ^ 1u, abort_flag)) {
                    if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_TMEM_EMPTY); }
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d = tmem_base + ab * BN;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(&ctl->full[s], ph, abort_flag)) {
                        if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_FULL); }
                        dead = true;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_base = smem_u32(smem + s * C::STAGE_BYTES), b_base = a_base + GM_A_BYTES;
#pragma unroll
                    for (int ks = 0; ks < GM_BK / 16; ks++) {
                        // 16 reduction indices further on: 32 bytes along a K-major row, two 8-row atoms of an MN-major tile
                        const uint64_t ad = p.a_mn ? gm_desc_mn(a_base + ks * 2048) : umma_desc_sw128(a_base) + (uint64_t)ks * 2;
                        const uint64_t bd = p.b_mn ? gm_desc_mn(b_base + ks * 2048) : umma_desc_sw128(b_base) + (uint64_t)ks * 2;
                        umma_f16(d, ad, bd, idesc, (kb > kb0 || ks > 0) ? 1u : 0u);
                    }
                    umma_commit(&ctl->empty[s]);
                    if (++s == C::STAGES) { s = 0; ph ^= 1u; }
                }
                if (!dead) umma_commit(&ctl->acc_full[ab]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue: thread = output row
        const int q = warp & 3;                       // tensor-memory lane group this warp may read
        const int r = q * 32 + lane;
        uint32_t local = 0;
        uint32_t slab_i = 0;
        for (long long u = blockIdx.x; u < units; u += gridDim.x) {
            const int sp = (int)(u % p.splits);
            const int tile = (int)(u / p.splits);
            const int b = tile / tiles_per_problem, t = gm_rotate(p, tile - b * tiles_per_problem, b, tiles_per_problem);
            const int tm = t / p.tiles_n, tn = t - tm * p.tiles_n;
            const int bi = b % p.nb_inner, bo = b / p.nb_inner;
            if (gm_tile_skipped<BN>(p, tm, tn)) continue;
            const uint32_t ab = local & 1u, use = local >> 1;
            local++;
            if (!mbar_wait(&ctl->acc_full[ab], use & 1u, abort_flag)) {
                if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_TMEM_FULL); }
                break;
            }
            tc_fence_after_sync();
            const int m = tm * GM_BM + r;
            const int n0 = tn * BN;
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + ab * BN;
            const bool to_slab = p.splits > 1;
            const bool row_ok = m < p.M;
            float* srow = to_slab ? p.slabs + (((long long)sp * p.batch + b) * p.M + m) * p.N : nullptr;
            const long long c_off = (long long)bo * p.c_so + (long long)bi * p.c_si + (long long)m * p.ldc;
            const bool by_tma = p.c_tma && !to_slab;
            const int m0w = tm * GM_BM + q * 32;      // first row of this warp's 32
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (n0 + c0 >= p.N) break;            // warp-uniform
                uint32_t v[32];
                tmem_ld_32x32(t_row + c0, v);
                tmem_ld_wait();
                const int n = n0 + c0;
                const bool full = n + 32 <= p.N;
                if (to_slab) {
                    if (!row_ok) continue;
                    if (full && (p.N & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4*>(srow + n + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                                   __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (n + j < p.N) srow[n + j] = __uint_as_float(v[j]);
                    }
                    continue;
                }
                if (!row_ok && !by_tma) continue;
                float f[32];
#pragma unroll
                for (int j = 0; j < 32; j++) f[j] = __uint_as_float(v[j]) * p.alpha;
                if (p.bias) {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (full || n + j < p.N) f[j] += __ldg(p.bias + n + j);
                }
                if (p.bias_bf16) {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (full || n + j < p.N) f[j] += __bfloat162float(p.bias_bf16[n + j]);
                }
                if (p.residual && row_ok) {
                    const __nv_bfloat16* res = p.residual + c_off + n;
                    if (full && p.vec_ok) {
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) {
                            const uint4 rv = __ldg(reinterpret_cast<const uint4*>(res + ch * 8));
                            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                f[ch * 8 + e * 2] += __low2float(h2[e]);
                                f[ch * 8 + e * 2 + 1] += __high2float(h2[e]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (n + j < p.N) f[j] += __bfloat162float(res[j]);
                    }
                }
                if (by_tma) {
                    // Stage the warp's 32 rows x 128 bytes in a swizzled slab (16-byte chunk index XOR row % 8: conflict-free
                    // stores), then one TMA store per slab: 64 bfloat16 or 32 float32 columns.  Two slabs alternate; before a
                    // slab is rewritten the store issued from it two slabs ago must have read it.
                    const int half = p.out_f32 ? 0 : ((c0 >> 5) & 1);
                    uint8_t* slab = epi_smem + (warp - 2) * 8192 + (slab_i & 1) * 4096;
                    if (half == 0) {
                        if (lane == 0) bulk_wait_group_read<1>();
                        __syncwarp();
                    }
                    uint8_t* rowp = slab + lane * 128;
                    if (p.out_f32) {
#pragma unroll
                        for (int ch = 0; ch < 8; ch++)
                            *reinterpret_cast<float4*>(rowp + ((ch ^ (lane & 7)) << 4)) = make_float4(f[ch * 4], f[ch * 4 + 1], f[ch * 4 + 2], f[ch * 4 + 3]);
                    } else {
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) {
                            uint4 pk;
                            uint32_t* w = &pk.x;
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const __nv_bfloat162 h2 = __floats2bfloat162_rn(f[ch * 8 + e * 2], f[ch * 8 + e * 2 + 1]);
                                w[e] = *reinterpret_cast<const uint32_t*>(&h2);
                            }
                            *reinterpret_cast<uint4*>(rowp + (((half * 4 + ch) ^ (lane & 7)) << 4)) = pk;
                        }
                    }
                    const bool slab_done = p.out_f32 || half == 1 || c0 + 32 >= BN || n + 32 >= p.N;
                    if (slab_done) {
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && m0w < p.M) {
                            tma_store_tile_4d(p.tmap_c, smem_u32(slab), n - half * 32, m0w, bi, bo);
                            bulk_commit_group();
                        }
                        slab_i++;
                    }
                    continue;
                }
                if (p.out_f32) {
                    float* out = reinterpret_cast<float*>(p.c) + c_off + n;
                    if (full && p.vec_ok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(out + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (n + j < p.N) out[j] = f[j];
                    }
                } else {
                    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.c) + c_off + n;
                    if (full && p.vec_ok) {
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) {
                            uint4 pk;
                            uint32_t* w = &pk.x;
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const __nv_bfloat162 h2 = __floats2bfloat162_rn(f[ch * 8 + e * 2], f[ch * 8 + e * 2 + 1]);
                                w[e] = *reinterpret_cast<const uint32_t*>(&h2);
                            }
                            *reinterpret_cast<uint4*>(out + ch * 8) = pk;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (n + j < p.N) out[j] = __float2bfloat16_rn(f[j]);
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->acc_empty[ab]);
        }
        if (lane == 0) bulk_wait_group<0>();   // the slabs must outlive the stores that read them
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// Sums the split-K partial matrices in split order, applies alpha and the bias, writes C.
__global__ void __launch_bounds__(256) gemm_splitk_finish_kernel(const float* __restrict__ slabs, void* __restrict__ c,
                                                                 const float* __restrict__ bias,
                                                                 const __nv_bfloat16* __restrict__ bias_bf16,
                                                                 const __nv_bfloat16* __restrict__ residual, int splits, int batch, int nb_inner,
                                                                 int M, int N, long long ldc, long long c_si, long long c_so,
                                                                 int out_f32, float alpha) {
    const long long per_split = (long long)batch * M * N;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per_split; i += (long long)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; s++) acc += slabs[(long long)s * per_split + i];
        const int n = (int)(i % N);
        const long long bm = i / N;
        const int m = (int)(bm % M), b = (int)(bm / M);
        acc = acc * alpha + (bias ? bias[n] : 0.f) + (bias_bf16 ? __bfloat162float(bias_bf16[n]) : 0.f);
        const long long off = (long long)(b / nb_inner) * c_so + (long long)(b % nb_inner) * c_si + (long long)m * ldc + n;
        if (residual) acc += __bfloat162float(residual[off]);
        if (out_f32) reinterpret_cast<float*>(c)[off] = acc;
        else reinterpret_cast<__nv_bfloat16*>(c)[off] = __float2bfloat16_rn(acc);
    }
}

using GmEncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static GmEncodeTiledFn gm_encode_fn() {
    static const GmEncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<GmEncodeTiledFn>(f);
    }();
    return fn;
}

// Tensor map of one operand: `inner` contiguous elements per row, `outer` rows `ld` elements apart, two batch levels.
static bool gm_make_map(unsigned char* out, const void* base, long long inner, long long outer, long long ld, int nb_inner,
                        long long s_inner, int nb_outer, long long s_outer, int box_inner, int box_outer) {
    GmEncodeTiledFn enc = gm_encode_fn();
    if (!enc) return false;
    // a batch level of one problem still needs a legal (non-zero, 16-byte multiple) stride
    const long long si = nb_inner > 1 ? s_inner : ld * outer, so = nb_outer > 1 ? s_outer : si * (nb_inner > 1 ? nb_inner : 1);
    cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)nb_inner, (cuuint64_t)nb_outer};
    cuuint64_t strides[3] = {(cuuint64_t)ld * 2, (cuuint64_t)si * 2, (cuuint64_t)so * 2};
    cuuint32_t box[4] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1, 1};
    cuuint32_t steps[4] = {1, 1, 1, 1};
    return enc(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, steps,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN>
static int gm_launch(const GemmParams& p, int grid, cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set[dev] = true;
    }
    OB200_ELASTIC(gemm_bf16_kernel<BN>, 1);
    // Programmatic dependent launch: the kernel's set-up (barriers, tensor memory, descriptor prefetch) may overlap the tail of
    // the kernel before it in the stream; it reads and writes global memory only behind its griddepcontrol.wait.
    static const bool pdl = [] {   // ORION_PDL=0: plain stream order between consecutive kernels
        const char* e = getenv("ORION_PDL");
        return !(e && e[0] == '0');
    }();
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(GM_THREADS);
    cfg.dynamicSmemBytes = GemmCfg<BN>::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<BN>, p);
}

}  // namespace ob200

extern "C" int* ob200_status_word_for_current_device(void);
extern "C" float* ob200_stream_slabs(void* stream, size_t* bytes);
extern "C" int ob200_plan_sm_count(void);

// See include/orion_kernels.h.  Returns 0, -1 (unsupported sizes), -2 (misaligned pointers or strides), -4 (no TMA descriptor).
extern "C" int ob200_gemm_bf16_ex(const void* a, const void* b, void* c, const float* bias, const void* bias_bf16, const void* residual,
                                  int M, int N, int K, int a_mn, int b_mn, long long lda, long long ldb, long long ldc, int batch_inner,
                                  int batch_outer, long long a_si, long long a_so, long long b_si, long long b_so, long long c_si,
                                  long long c_so, float alpha, int out_f32, int tri, int num_ctas, void* stream);

extern "C" int ob200_gemm_bf16(const void* a, const void* b, void* c, const float* bias, int M, int N, int K, int a_mn, int b_mn,
                               long long lda, long long ldb, long long ldc, int batch_inner, int batch_outer, long long a_si,
                               long long a_so, long long b_si, long long b_so, long long c_si, long long c_so, float alpha, int out_f32,
                               int num_ctas, void* stream) {
    return ob200_gemm_bf16_ex(a, b, c, bias, nullptr, nullptr, M, N, K, a_mn, b_mn, lda, ldb, ldc, batch_inner, batch_outer, a_si, a_so,
                              b_si, b_so, c_si, c_so, alpha, out_f32, 0, num_ctas, stream);
}

extern "C" int ob200_gemm_bf16_ex(const void* a, const void* b, void* c, const float* bias, const void* bias_bf16, const void* residual,
                                  int M, int N, int K, int a_mn, int b_mn, long long lda, long long ldb, long long ldc, int batch_inner,
                                  int batch_outer, long long a_si, long long a_so, long long b_si, long long b_so, long long c_si,
                                  long long c_so, float alpha, int out_f32, int tri, int num_ctas, void* stream) {
    using namespace ob200;
    if (tri < 0 || tri > 3) return -1;
    if (M < 0 || N < 0 || K <= 0 || batch_inner < 0 || batch_outer < 0 || num_ctas <= 0 || lda <= 0 || ldb <= 0 || ldc < N) return -1;
    if (M == 0 || N == 0 || batch_inner == 0 || batch_outer == 0) return 0;
    if (((uintptr_t)a | (uintptr_t)b) % 16 || (lda | ldb) % 8) return -2;
    if ((batch_inner > 1 && ((a_si | b_si) % 8)) || (batch_outer > 1 && ((a_so | b_so) % 8))) return -2;
    const long long batch_ll = (long long)batch_inner * batch_outer;
    if (batch_ll > 0x7fffffffLL) return -1;
    GemmParams p;
    memset(&p, 0, sizeof p);
    p.c = c; p.bias = bias;
    p.bias_bf16 = reinterpret_cast<const __nv_bfloat16*>(bias_bf16);
    p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
    p.status = ob200_status_word_for_current_device();
    p.M = M; p.N = N; p.K = K;
    p.batch = (int)batch_ll; p.nb_inner = batch_inner;
    p.ldc = ldc; p.c_si = c_si; p.c_so = c_so;
    p.out_f32 = out_f32 ? 1 : 0;
    p.a_mn = a_mn ? 1 : 0; p.b_mn = b_mn ? 1 : 0;
    p.alpha = alpha;
    p.tri = tri;
    const int cal = out_f32 ? 4 : 8;   // elements per 16 bytes of C
    p.vec_ok = ((uintptr_t)c % 16 == 0) && ((uintptr_t)residual % 16 == 0) && (!residual || !out_f32) && (ldc % cal == 0) && (batch_inner == 1 || c_si % cal == 0) && (batch_outer == 1 || c_so % cal == 0);
    const int plan = ob200_plan_sm_count();
    const int tiles_m = (M + GM_BM - 1) / GM_BM;
    // Tile width: 256 columns halve the re-reads of A where the grid still fills the device; 64 for narrow outputs.
    // A 128 x 128 tile is bound by operand traffic (32 KB per k-block), a 128 x 256 tile takes about 1.5 times as long for
    // twice the work: pick the width whose number of waves times that cost is smaller.
    int bn = N <= 64 ? 64 : 128;
    if (N >= 256) {
        const long long t128 = batch_ll * tiles_m * ((N + 127) / 128), t256 = batch_ll * tiles_m * ((N + 255) / 256);
        const long long w128 = (t128 + plan - 1) / plan, w256 = (t256 + plan - 1) / plan;
        if (w256 * 3 < w128 * 2 + 1 && t256 * 2 > plan) bn = 256;
    }
    p.tiles_m = tiles_m;
    p.tiles_n = (N + bn - 1) / bn;
    p.kblocks = (K + GM_BK - 1) / GM_BK;
    const long long tiles = batch_ll * p.tiles_m * p.tiles_n;
    if (tiles > 0x7fffffffLL) return -1;
    // Split-K: few tiles, long reduction.  Planned for the device's SM count, never for the quota of the call, so the
    // summation order (and the result, bit for bit) is the same for every quota.
    int splits = 1;
    if (tiles * 2 <= plan && p.kblocks >= 8 && tri == 0) {
        splits = (int)(plan / tiles);
        if (splits > p.kblocks / 4) splits = p.kblocks / 4;
        if (splits > 16) splits = 16;
        size_t slab_bytes = 0;
        float* slabs = ob200_stream_slabs(stream, &slab_bytes);
        const size_t per_split = (size_t)batch_ll * M * N * sizeof(float);
        if (!slabs || per_split == 0) splits = 1;
        else if ((size_t)splits * per_split > slab_bytes) splits = (int)(slab_bytes / per_split);
        if (splits < 2) splits = 1;
        p.slabs = splits > 1 ? slabs : nullptr;
    }
    p.kb_per_split = (p.kblocks + splits - 1) / splits;
    p.splits = (p.kblocks + p.kb_per_split - 1) / p.kb_per_split;   // every split owns at least one k-block
    if (p.splits <= 1) { p.splits = 1; p.slabs = nullptr; p.kb_per_split = p.kblocks; }
    const bool ok_a = a_mn ? gm_make_map(p.tmap_a, a, M, K, lda, batch_inner, a_si, batch_outer, a_so, 64, GM_BK)
                           : gm_make_map(p.tmap_a, a, K, M, lda, batch_inner, a_si, batch_outer, a_so, GM_BK, GM_BM);
    const bool ok_b = b_mn ? gm_make_map(p.tmap_b, b, N, K, ldb, batch_inner, b_si, batch_outer, b_so, 64, GM_BK)
                           : gm_make_map(p.tmap_b, b, K, N, ldb, batch_inner, b_si, batch_outer, b_so, GM_BK, bn);
    if (!ok_a || !ok_b) return -4;
    // C by TMA stores when its rows and batch offsets are 16-byte multiples (always true for the layouts of the clients)
    {
        const int es = out_f32 ? 4 : 2;
        const bool aligned = ((uintptr_t)c % 16 == 0) && (ldc * es) % 16 == 0 && (batch_inner == 1 || (c_si * es) % 16 == 0) &&
                             (batch_outer == 1 || (c_so * es) % 16 == 0);
        static const bool tma_off = [] { const char* e = getenv("ORION_GEMM_TMA_STORE"); return e && e[0] == '0'; }();
        if (aligned && !tma_off && p.splits == 1) {
            GmEncodeTiledFn enc = gm_encode_fn();
            const long long si = batch_inner > 1 ? c_si : ldc * M, so = batch_outer > 1 ? c_so : si * (batch_inner > 1 ? batch_inner : 1);
            cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)batch_inner, (cuuint64_t)batch_outer};
            cuuint64_t strides[3] = {(cuuint64_t)ldc * es, (cuuint64_t)si * es, (cuuint64_t)so * es};
            cuuint32_t box[4] = {(cuuint32_t)(128 / es), 32, 1, 1};
            cuuint32_t steps[4] = {1, 1, 1, 1};
            if (enc && enc(reinterpret_cast<CUtensorMap*>(p.tmap_c), out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                           c, dims, strides, box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
                p.c_tma = 1;
        }
    }
    const long long units = tiles * p.splits;
    int grid = units < num_ctas ? (int)units : num_ctas;
    // ORION_GEMM_TILES_PER_CTA=t (t > 0): a CTA retires after about t work units instead of staying for the whole launch, so
    // that the blocks of a higher-priority kernel find a free SM after a few microseconds (the grid is then wider than the
    // quota; the scheduler's cut to the quota, where it applies, still holds).
    static const int tiles_per_cta = [] { const char* e = getenv("ORION_GEMM_TILES_PER_CTA"); return e ? atoi(e) : 0; }();
    if (tiles_per_cta > 0) {
        const long long want = (units + tiles_per_cta - 1) / tiles_per_cta;
        if (want > grid) grid = want > 0x7fffffffLL ? 0x7fffffff : (int)want;
    }
    {
        const double flop = 2.0 * batch_ll * M * (double)N * K;
        const double bytes = 2.0 * batch_ll * ((double)M * K + (double)N * K) + (out_f32 ? 4.0 : 2.0) * batch_ll * (double)M * N;
        annotate_launch(flop / bytes > ai_threshold(1) ? 1 : 0, flop, bytes);
    }
    int rc = bn == 256 ? gm_launch<256>(p, grid, (cudaStream_t)stream)
                       : bn == 128 ? gm_launch<128>(p, grid, (cudaStream_t)stream) : gm_launch<64>(p, grid, (cudaStream_t)stream);
    if (rc != 0 || p.splits == 1) return rc;
    const long long elems = batch_ll * M * N;
    long long blocks = (elems + 255) / 256;
    if (blocks > 4LL * num_ctas) blocks = 4LL * num_ctas;
    OB200_ELASTIC_HBM(gemm_splitk_finish_kernel, 4);
    gemm_splitk_finish_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(p.slabs, c, bias, p.bias_bf16, p.residual, p.splits, p.batch, p.nb_inner, M, N, ldc, c_si,
                                                                            c_so, p.out_f32, alpha);
    return (int)cudaGetLastError();
}
