// Fused self-attention forward for the transformer inference clients (bfloat16, head dimension 64, sequences up to 384):
//
//   ctx[b, q, h*64 + :] = softmax( Q[b,h,q,:] . K[b,h,:,:]^T * scale  (+ causal mask) ) . V[b,h,:,:]
//
// read straight from the fused projection output qkv [B, S, 3, H, 64] and written as [B, S, H*64] — no probability tensor
// and no re-laid-out Q / K / V copies in HBM.  It stands in for the two cublasSgemmStridedBatched calls around a softmax
// kernel that the reference replays for an attention layer (reference src/scheduler/utils_sched.cpp:502-513).
//
// One work item = 128 query rows of one (batch, head); a persistent grid walks the items.  Per item:
//   1. one thread issues TMA copies of the Q tile (128 x 64), the K tiles and the V tiles (up to 384 x 64 each) into
//      128-byte-swizzled shared memory;
//   2. S = Q . K^T on the tensor cores (tcgen05.mma kind::f16, N = 128 per key tile) into tensor memory (one fp32 column
//      per key: up to 384 columns);
//   3. four warps (one thread per query row = tensor-memory lane) read their row twice — maximum, then exp and sum — and
//      write the unnormalised probabilities as bfloat16 into shared memory in the K-major swizzled layout of an A operand;
//   4. O = P . V on the tensor cores; V stays as it lies in memory ([key][64]: the reduction index is the slow one), so it is
//      declared MN-major to the tensor core;
//   5. the same four warps read O (64 columns), divide by the row sum and store 128 bytes per row.
// Every wait is bounded; on expiry the kernel sets the status word, frees tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "elastic.h"
#include "sm100_primitives.cuh"

namespace ob200 {

constexpr int AT_D = 64;            // head dimension
constexpr int AT_QROWS = 128;       // query rows per work item
constexpr int AT_MAX_KEYS = 384;
constexpr int AT_THREADS = 160;     // warps 0-3: softmax / epilogue, warp 4: TMA + MMA issue
constexpr int AT_TILE_BYTES = 128 * 128;   // 128 rows of 64 bfloat16
constexpr int AT_SMEM = AT_TILE_BYTES * (1 + 3 + 3 + 6) + 1024 + 256;   // Q, K x3, V x3, P x6 (64 keys each), align, barriers

struct AttnParams {
    void* ctx;             // [B, S, H*64] bfloat16
    int* status;
    int B, S, H;
    int causal;
    float scale;
    int key_tiles;         // ceil(S / 128)
    int q_tiles;           // ceil(S / 128)
    alignas(64) unsigned char tmap[128];   // qkv as [B][S][3H][64]
};

struct AttnCtl {
    uint64_t loaded, s_done, o_done;
    uint32_t tmem_base;
    int abort_flag;
};

__global__ void __launch_bounds__(AT_THREADS, 1) attention_fwd_kernel(const __grid_constant__ AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;
    uint8_t* k_s = q_s + AT_TILE_BYTES;
    uint8_t* v_s = k_s + 3 * AT_TILE_BYTES;
    uint8_t* p_s = v_s + 3 * AT_TILE_BYTES;
    AttnCtl* ctl = reinterpret_cast<AttnCtl*>(p_s + 6 * AT_TILE_BYTES);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        mbar_init(&ctl->loaded, 1);
        mbar_init(&ctl->s_done, 1);
        mbar_init(&ctl->o_done, 1);
        ctl->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 4) {
        if (lane == 0) prefetch_tensormap(p.tmap);
        tmem_alloc(&ctl->tmem_base, 512);
        tmem_relinquish();
        tc_fence_before_sync();
    }
    __syncthreads();
    tc_fence_after_sync();
    pdl_wait();
    if (tid == 0) pdl_launch_dependents();
    const uint32_t tmem_base = ctl->tmem_base;
    volatile int* abort_flag = &ctl->abort_flag;
    const int items = p.B * p.H * p.q_tiles;
    uint32_t phase = 0;

    for (int item = blockIdx.x; item < items; item += gridDim.x, phase ^= 1u) {
        const int qt = item % p.q_tiles;
        const int bh = item / p.q_tiles;
        const int h = bh % p.H, b = bh / p.H;
        const int q0 = qt * AT_QROWS;
        // causal: keys past the tile's last query row are never needed
        const int kt_used = p.causal ? (q0 + AT_QROWS + 127) / 128 < p.key_tiles ? (q0 + AT_QROWS + 127) / 128 : p.key_tiles : p.key_tiles;
        if (warp == 4) {
            if (lane == 0) {
                // ---- operands
                mbar_arrive_expect_tx(&ctl->loaded, (uint32_t)(AT_TILE_BYTES * (1 + 2 * kt_used)));
                tma_load_tile_4d(smem_u32(q_s), p.tmap, &ctl->loaded, 0, h, q0, b);
                for (int t = 0; t < kt_used; t++) {
                    tma_load_tile_4d(smem_u32(k_s + t * AT_TILE_BYTES), p.tmap, &ctl->loaded, 0, p.H + h, t * 128, b);
                    tma_load_tile_4d(smem_u32(v_s + t * AT_TILE_BYTES), p.tmap, &ctl->loaded, 0, 2 * p.H + h, t * 128, b);
                }
                if (!mbar_wait(&ctl->loaded, phase, abort_flag)) {
                    ctl->abort_flag = 1;
                    if (p.status) atomicExch(p.status, OB200_ERR_WAIT_FULL);
                } else {
                    tc_fence_after_sync();
                    // ---- S = Q . K^T : per key tile one accumulator of 128 columns, four k-steps of 16 over the head dimension
                    const uint32_t idesc_s = umma_idesc(1, 128, 128);
                    const uint64_t qd = umma_desc_sw128(smem_u32(q_s));
                    for (int t = 0; t < kt_used; t++) {
                        const uint64_t kd = umma_desc_sw128(smem_u32(k_s + t * AT_TILE_BYTES));
#pragma unroll
                        for (int ks = 0; ks < 4; ks++) umma_f16(tmem_base + t * 128, qd + (uint64_t)ks * 2, kd + (uint64_t)ks * 2, idesc_s, ks > 0 ? 1u : 0u);
                    }
                    umma_commit(&ctl->s_done);
                }
            }
            __syncwarp();
        }
        // ---- softmax: thread r of warps 0-3 owns query row q0 + r (tensor-memory lane r)
        float row_sum = 1.f;
        if (warp < 4) {
            const int r = warp * 32 + lane;
            const int qpos = q0 + r;
            const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16);
            const int key_end = p.causal ? (qpos + 1 < p.S ? qpos + 1 : p.S) : p.S;   // keys [0, key_end) count
            const int cols = kt_used * 128;
            bool ok = mbar_wait(&ctl->s_done, phase, abort_flag);
            if (!ok && !*abort_flag) {
                ctl->abort_flag = 1;
                if (p.status) atomicExch(p.status, OB200_ERR_WAIT_TMEM_FULL);
            }
            if (ok) {
                tc_fence_after_sync();
                float m = -INFINITY;
                for (int c0 = 0; c0 < cols; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (c0 + j < key_end) m = fmaxf(m, __uint_as_float(v[j]));
                }
                const float ms = m * p.scale;
                float sum = 0.f;
                for (int c0 = 0; c0 < cols; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + c0, v);
                    tmem_ld_wait();
                    // 32 probabilities = four 16-byte chunks of row r in the 64-key block c0 / 64
                    uint8_t* blk = p_s + (c0 >> 6) * AT_TILE_BYTES;
                    const int chunk0 = (c0 & 63) >> 3;
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) {
                        uint4 pk;
                        uint32_t* w = &pk.x;
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int j = ch * 8 + e * 2;
                            const float a = c0 + j < key_end ? __expf(fmaf(__uint_as_float(v[j]), p.scale, -ms)) : 0.f;
                            const float bb = c0 + j + 1 < key_end ? __expf(fmaf(__uint_as_float(v[j + 1]), p.scale, -ms)) : 0.f;
                            const __nv_bfloat162 h2 = __floats2bfloat162_rn(a, bb);
                            // the row sum is taken over the rounded values the tensor core will multiply
                            sum += __low2float(h2) + __high2float(h2);
                            w[e] = *reinterpret_cast<const uint32_t*>(&h2);
                        }
                        *reinterpret_cast<uint4*>(blk + sw128_offset((uint32_t)r, (uint32_t)(chunk0 + ch))) = pk;
                    }
                }
                row_sum = sum;
                fence_proxy_async_smem();   // the tensor core reads P through the async proxy
                tc_fence_before_sync();
            }
        }
        __syncthreads();   // P is complete (or somebody gave up)
        if (*abort_flag) break;
        if (warp == 4 && lane == 0) {
            tc_fence_after_sync();
            // ---- O = P . V : 64 output columns behind the S columns; V is MN-major (rows = keys, 128 bytes of head dimension)
            const uint32_t idesc_o = umma_idesc(1, 128, 64) | UMMA_IDESC_B_MN;
            const uint32_t d_o = tmem_base + AT_MAX_KEYS;
            const int ksteps = kt_used * 8;   // 16 keys each
            for (int ks = 0; ks < ksteps; ks++) {
                const uint32_t p_addr = smem_u32(p_s + (ks >> 2) * AT_TILE_BYTES) + (uint32_t)(ks & 3) * 32u;
                const uint32_t v_addr = smem_u32(v_s) + (uint32_t)ks * 16u * 128u;
                // MN-major operand: atoms of 8 keys x 128 bytes, 1024 bytes apart along the reduction (stride byte offset);
                // the 64 columns are one atom wide, so the leading byte offset is never used
                const uint64_t vd = (uint64_t)((v_addr & 0x3FFFF) >> 4) | ((uint64_t)(8192 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
                                    ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
                umma_f16(d_o, umma_desc_sw128(p_addr), vd, idesc_o, ks > 0 ? 1u : 0u);
            }
            umma_commit(&ctl->o_done);
        }
        if (warp < 4) {
            const int r = warp * 32 + lane;
            const int qpos = q0 + r;
            bool ok = mbar_wait(&ctl->o_done, phase, abort_flag);
            if (!ok && !*abort_flag) {
                ctl->abort_flag = 1;
                if (p.status) atomicExch(p.status, OB200_ERR_WAIT_TMEM_FULL);
            }
            if (ok) {
                tc_fence_after_sync();
                const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16) + AT_MAX_KEYS;
                const float inv = 1.0f / row_sum;
                __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.ctx) + ((long long)b * p.S + qpos) * (p.H * AT_D) + h * AT_D;
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + half * 32, v);
                    tmem_ld_wait();
                    if (qpos < p.S) {
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) {
                            uint4 pk;
                            uint32_t* w = &pk.x;
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[ch * 8 + e * 2]) * inv,
                                                                                __uint_as_float(v[ch * 8 + e * 2 + 1]) * inv);
                                w[e] = *reinterpret_cast<const uint32_t*>(&h2);
                            }
                            *reinterpret_cast<uint4*>(out + half * 32 + ch * 8) = pk;
                        }
                    }
                }
                tc_fence_before_sync();
            }
        }
        __syncthreads();   // tensor memory and shared memory are free for the next item
        if (*abort_flag) break;
    }
    __syncthreads();
    if (warp == 4) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn attn_encode_fn() {
    static const EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

}  // namespace ob200

extern "C" int* ob200_status_word_for_current_device(void);

// qkv: [B, S, 3, H, 64] bfloat16 (the output of the fused Q/K/V projection), ctx: [B, S, H*64] bfloat16; S <= 384.
// causal = 1 masks keys after the query's position.  Returns -1 for unsupported sizes, -2 for misaligned pointers, -4 when
// the TMA descriptor cannot be built.
extern "C" int ob200_attention_fwd_bf16(const void* qkv, void* ctx, int B, int S, int H, int head_dim, float scale, int causal,
                                        int num_ctas, void* stream) {
    using namespace ob200;
    if (B <= 0 || S <= 0) return 0;
    if (head_dim != AT_D || S > AT_MAX_KEYS || H <= 0 || num_ctas <= 0) return -1;
    if (((uintptr_t)qkv | (uintptr_t)ctx) % 16) return -2;
    EncodeTiledFn enc = attn_encode_fn();
    if (!enc) return -4;
    AttnParams p;
    memset(&p, 0, sizeof p);
    p.ctx = ctx;
    p.status = ob200_status_word_for_current_device();
    p.B = B; p.S = S; p.H = H;
    p.causal = causal ? 1 : 0;
    p.scale = scale;
    p.key_tiles = (S + 127) / 128;
    p.q_tiles = (S + 127) / 128;
    cuuint64_t dims[4] = {(cuuint64_t)AT_D, (cuuint64_t)(3 * H), (cuuint64_t)S, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)AT_D * 2, (cuuint64_t)3 * H * AT_D * 2, (cuuint64_t)S * 3 * H * AT_D * 2};
    cuuint32_t box[4] = {AT_D, 1, 128, 1};
    cuuint32_t steps[4] = {1, 1, 1, 1};
    if (enc(reinterpret_cast<CUtensorMap*>(p.tmap), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(qkv), dims, strides, box, steps,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return -4;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set[dev] = true;
    }
    const int items = B * H * p.q_tiles;
    OB200_ELASTIC(attention_fwd_kernel, 1);
    annotate_launch(1, 4.0 * B * H * (double)S * S * AT_D, 2.0 * B * S * H * AT_D * 4.0);
    attention_fwd_kernel<<<items < num_ctas ? items : num_ctas, AT_THREADS, AT_SMEM, (cudaStream_t)stream>>>(p);
    return (int)cudaGetLastError();
}
