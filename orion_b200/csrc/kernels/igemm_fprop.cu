// Implicit-GEMM convolution (forward and data gradient) and linear layer on the
// 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM), for NHWC
// activations and KRSC weights.
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
//   warps 5-8   splitters (fp32 only): split the raw operand rows in shared memory into
//               TF32 high parts (in place) and exact remainders (second buffer)
//   warps 9-16  producers: cp.async 16-byte copies of one
//               128-byte row slice of the im2col matrix (zero-filled at the image
//               border) and of the filter, straight into the 128-byte-swizzled
//               K-major stage buffers, several stages ahead of the MMA
// fp32 inputs run as 3xTF32 (dtype 0; dtype 2 = one TF32 pass, no splitters): each value is split into a TF32-rounded high part and
// the exact remainder, and lo*hi + hi*lo + hi*hi accumulate in fp32, which keeps
// the result within ~1e-6 relative of an fp32 reference.  bf16 inputs use one
// kind::f16 MMA per k-step.
//
// Split-K: when `splits > 1` each work unit covers a contiguous range of k-blocks of
// one tile and writes its partial tile to a slab of its own; the unit that arrives
// last on the tile's counter adds the slabs in split order and applies the epilogue,
// so the result does not depend on which unit finishes first (bit-reproducible for
// a given schedule, like `splits = 1`).
//
// Every mbarrier wait is bounded; on expiry the kernel records a code in the status
// word, releases TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>

#include "igemm_params.h"
#include "elastic.h"
#include "sm100_primitives.cuh"

namespace ob200 {

constexpr int BM = 128;
constexpr int EPI_WARPS = 4;      // warps 0-3; TMA-fed launches add warps 9-12 as a second epilogue group
constexpr int MMA_WARP = 4;
constexpr int SPLIT_WARPS = 4;    // warps 5-8; TMA-fed launches add warps 13-16 as a second splitter group
constexpr int PROD_WARPS = 8;     // warps 9-16 when the operands are gathered with cp.async
constexpr int TMA_WARP = 17;      // one lane issues the TMA copies of TMA-fed launches
constexpr int NTHREADS = 18 * 32;

// ATMEM: 3xTF32 with both parts of the activation tile in tensor memory (forward / data gradient / GEMM).
template <typename T, int BN, int PASSES, bool ATMEM>
struct Cfg {
    static constexpr bool kSplit = sizeof(T) == 4 && PASSES == 3;   // 3xTF32; PASSES == 1 is plain TF32
    static_assert(!ATMEM || kSplit, "tensor-memory activation parts exist only for 3xTF32");
    static constexpr int BK = 128 / sizeof(T);                // elements per 128-byte row
    static constexpr int EPC = 16 / sizeof(T);                // elements per 16-byte chunk
    static constexpr int A_BYTES = BM * 128;
    static constexpr int B_BYTES = BN * 128;
    // Stage: [A raw][A remainder][B raw][B remainder] (3xTF32 from shared memory), [A raw][B raw][B remainder]
    // (activation parts in tensor memory), or [A][B] (one pass).
    static constexpr int STAGE_BYTES = ATMEM ? A_BYTES + 2 * B_BYTES : (A_BYTES + B_BYTES) * (kSplit ? 2 : 1);
    static constexpr int B_OFF = (kSplit && !ATMEM) ? 2 * A_BYTES : A_BYTES;
#ifndef OB200_STAGE_CAP
#define OB200_STAGE_CAP 8
#endif
    static constexpr int BY_SMEM0 = (192 * 1024) / STAGE_BYTES;
    static constexpr int BY_SMEM = BY_SMEM0 > OB200_STAGE_CAP ? OB200_STAGE_CAP : BY_SMEM0;
    static constexpr int BY_TMEM = ATMEM ? (512 - 2 * BN) / 64 : 8;      // 64 tensor-memory columns per stage
    static constexpr int STAGES = BY_SMEM < BY_TMEM ? (BY_SMEM > 8 ? 8 : BY_SMEM) : (BY_TMEM > 8 ? 8 : BY_TMEM);
    static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
    static constexpr int EPI_BYTES = 2 * EPI_WARPS * 32 * 20 * 4;   // per-warp transpose tiles of the epilogue (EPI_LD floats per row)
    static constexpr int SMEM_BYTES = RING_BYTES + EPI_BYTES + 1024 /*align*/ + 512 /*barriers*/;
    // Two accumulators of BN columns; ATMEM adds, per stage, the two parts of the activation tile (32 + 32 columns).
    // Allocations are powers of two.
    static constexpr int A_TMEM_COL0 = 2 * BN;
    static constexpr int TMEM_COLS = ATMEM ? 512 : 2 * BN;
    static_assert(!ATMEM || 2 * BN + STAGES * 64 <= 512, "tensor memory budget");
};

struct SharedCtl {
    uint64_t raw_full[8];
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

// The tensor core reads a float32 operand as TF32 by ignoring the low 13 mantissa bits, so the raw
// value already serves as the high part; only the exact remainder x - trunc(x) is written (second buffer).
// The remainder is rounded to TF32 precision here (to nearest), so the tensor core's truncation of it is exact
// and the split leaves no systematic error: x = trunc_tf32(x) + remainder up to an unbiased 2^-22 relative.
__device__ __forceinline__ float tf32_remainder(float x) {
    return tf32_round(x - __uint_as_float(__float_as_uint(x) & 0xffffe000u));
}
__device__ __forceinline__ void split_chunk(uint8_t* hi, uint8_t* lo) {
    const float4 v = *reinterpret_cast<const float4*>(hi);
    float4 l;
    l.x = tf32_remainder(v.x);
    l.y = tf32_remainder(v.y);
    l.z = tf32_remainder(v.z);
    l.w = tf32_remainder(v.w);
    *reinterpret_cast<float4*>(lo) = l;
}

// 16-byte asynchronous global->shared copy; `ok == false` writes zeros and reads nothing.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool ok) {
    const int bytes = ok ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
// The mbarrier receives one arrival from this thread once all its earlier cp.async copies have landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void set_elem(float4& v, int i, float x) {
    if (i == 0) v.x = x; else if (i == 1) v.y = x; else if (i == 2) v.z = x; else v.w = x;
}
__device__ __forceinline__ void set_elem(uint4& v, int i, __nv_bfloat16 x) {
    uint32_t bits = (uint32_t)__bfloat16_as_ushort(x) << ((i & 1) * 16);
    uint32_t* w = (i < 2) ? &v.x : (i < 4) ? &v.y : (i < 6) ? &v.z : &v.w;
    *w |= bits;
}

constexpr int EPI_LD = 20;   // floats per staged 16-column accumulator row: 16-byte aligned, conflict-free writes

struct EpiCoef {
    float4 scale, shift;
};

// Per-channel multiplier / addend of four consecutive output channels starting at n.
template <typename T>
__device__ __forceinline__ EpiCoef load_coef(const IgemmParams& p, int n) {
    EpiCoef c;
    c.scale = make_float4(1.f, 1.f, 1.f, 1.f);
    c.shift = make_float4(0.f, 0.f, 0.f, 0.f);
    float* sc = &c.scale.x;
    float* sh = &c.shift.x;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        if (n + e < p.Kout) {
            if (p.scale) sc[e] = __ldg(p.scale + n + e);
            if (p.shift) sh[e] = __ldg(p.shift + n + e);
        }
    }
    return c;
}

// Epilogue of four consecutive channels of output row m: affine, residual, activation, store.
template <typename T>
__device__ __forceinline__ void store_out(const IgemmParams& p, const EpiCoef& c, float4 v, long long m, int n, long long y_off) {
    if (n >= p.Kout) return;
    const long long base = y_off + m * p.Kout + n;
    float x[4] = {v.x * c.scale.x + c.shift.x, v.y * c.scale.y + c.shift.y, v.z * c.scale.z + c.shift.z, v.w * c.scale.w + c.shift.w};
    const bool full = (n + 3 < p.Kout) && ((p.Kout & 3) == 0);
    if (p.residual) {
        if (sizeof(T) == 4) {
            const float* res = reinterpret_cast<const float*>(p.residual) + base;
            if (full) {
                const float4 q = __ldg(reinterpret_cast<const float4*>(res));
                x[0] += q.x; x[1] += q.y; x[2] += q.z; x[3] += q.w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (n + e < p.Kout) x[e] += __ldg(res + e);
            }
        } else {
            const __nv_bfloat16* res = reinterpret_cast<const __nv_bfloat16*>(p.residual) + base;
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (n + e < p.Kout) x[e] += __bfloat162float(res[e]);
        }
    }
    if (p.relu) {
#pragma unroll
        for (int e = 0; e < 4; e++) x[e] = fmaxf(x[e], 0.f);
        if (p.relu == 2) {
#pragma unroll
            for (int e = 0; e < 4; e++) x[e] = fminf(x[e], 6.f);
        }
    }
    if (sizeof(T) == 4) {
        float* y = reinterpret_cast<float*>(p.y) + base;
        if (full) {
            *reinterpret_cast<float4*>(y) = make_float4(x[0], x[1], x[2], x[3]);
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (n + e < p.Kout) y[e] = x[e];
        }
    } else {
        __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(p.y) + base;
        if (full) {
            __nv_bfloat162 t0 = __floats2bfloat162_rn(x[0], x[1]);
            __nv_bfloat162 t1 = __floats2bfloat162_rn(x[2], x[3]);
            uint2 o;
            o.x = *reinterpret_cast<uint32_t*>(&t0);
            o.y = *reinterpret_cast<uint32_t*>(&t1);
            *reinterpret_cast<uint2*>(y) = o;
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (n + e < p.Kout) y[e] = __float2bfloat16(x[e]);
        }
    }
}

// Row of y that GEMM row m is stored at.
__device__ __forceinline__ long long out_row(const IgemmParams& p, long long m) {
    if (!p.out_map) return m;
    const int pq = p.OH * p.OW;
    const int n_img = (int)(m / pq);
    const int rem = (int)(m - (long long)n_img * pq);
    const int i = rem / p.OW, j = rem - i * p.OW;
    return ((long long)n_img * p.out_H + i * p.out_mul_h + p.out_add_h) * p.out_W + j * p.out_mul_w + p.out_add_w;
}

// Epilogue of one 32-row x 16-column accumulator chunk held one row per lane in v: the per-warp shared-memory
// tile turns it so that four consecutive lanes own 16 consecutive output channels of one row (full 64-byte
// segments per row, eight rows per warp instruction), then scale/shift, residual, activation and store.
template <typename T>
__device__ __forceinline__ void epilogue_chunk(const IgemmParams& p, float* stage, const float (&v)[16], int lane,
                                               long long tile_row0, int n_chunk, long long y_off) {
    const int sub = lane >> 2, cc = (lane & 3) * 4;
#pragma unroll
    for (int j = 0; j < 16; j += 4)
        *reinterpret_cast<float4*>(stage + lane * EPI_LD + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    __syncwarp();
    const int n = n_chunk + cc;
    const EpiCoef coef = load_coef<T>(p, n);
    if (sizeof(T) == 4 && !p.out_map && (p.Kout & 3) == 0 && n + 3 < p.Kout) {
        // Common case (float32, whole 16-byte groups, rows stored in place): everything that does not depend on the
        // row is decided here, the loop is a shared-memory read, four FMAs, the activation and one 16-byte store.
        float* ycol = reinterpret_cast<float*>(p.y) + y_off + n;
        const float* rcol = p.residual ? reinterpret_cast<const float*>(p.residual) + y_off + n : nullptr;
        const float lo = p.relu ? 0.f : -INFINITY, hi = p.relu == 2 ? 6.f : INFINITY;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int rr = i * 8 + sub;
            const long long m = tile_row0 + rr;
            if (m < p.M) {
                const float4 a = *reinterpret_cast<const float4*>(stage + rr * EPI_LD + cc);
                float4 x = make_float4(fmaf(a.x, coef.scale.x, coef.shift.x), fmaf(a.y, coef.scale.y, coef.shift.y),
                                       fmaf(a.z, coef.scale.z, coef.shift.z), fmaf(a.w, coef.scale.w, coef.shift.w));
                if (rcol) {
                    const float4 q = __ldg(reinterpret_cast<const float4*>(rcol + m * p.Kout));
                    x.x += q.x; x.y += q.y; x.z += q.z; x.w += q.w;
                }
                x.x = fminf(fmaxf(x.x, lo), hi); x.y = fminf(fmaxf(x.y, lo), hi);
                x.z = fminf(fmaxf(x.z, lo), hi); x.w = fminf(fmaxf(x.w, lo), hi);
                *reinterpret_cast<float4*>(ycol + m * p.Kout) = x;
            }
        }
        __syncwarp();
        return;
    }
    // Not unrolled on purpose: the epilogue runs once per tile, and keeping its code small keeps the instruction
    // cache for the roles that loop per k-block.
#pragma unroll 1
    for (int i = 0; i < 4; i++) {
        const int rr = i * 8 + sub;
        const long long m = tile_row0 + rr;
        if (m < p.M) store_out<T>(p, coef, *reinterpret_cast<const float4*>(stage + rr * EPI_LD + cc), out_row(p, m), n, y_off);
    }
    __syncwarp();
}

// mbar_wait that also adds the cycles spent waiting to `acc` (role-level wait breakdown for tuning).
__device__ __forceinline__ bool timed_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, long long& acc) {
    const long long t0 = clock64();   // the first try_wait may already suspend the thread for a while
    const bool ok = mbar_wait(bar, parity, abort_flag);
    acc += clock64() - t0;
    return ok;
}

// Position in the ring of operand stages: stage index and the parity of the number of completed laps.
struct RingPos {
    int s = 0;
    uint32_t ph = 0;
    __device__ __forceinline__ void advance(int stages) {
        if (++s == stages) { s = 0; ph ^= 1u; }
    }
};

// One piece of work of a CTA: k-blocks [kb_begin, kb_end) of output tile `tile`.  nseg is the number of
// pieces the tile is computed in (1: this piece is the whole tile and stores directly); pieces of a cut
// tile accumulate in scratch slot `slot`.
struct Seg {
    int tile, kb_begin, kb_end, nseg, slot;
    int first_cta, my_slab;   // stream-K: first CTA with a piece of this tile; slab this piece is written to
};

// Walks the work of this CTA; every warp role of the CTA runs an identical copy.  Split-K mode hands out
// (tile, split) units round-robin; stream-K mode gives CTA b the range [b*W/G, (b+1)*W/G) of the W = tiles *
// num_kblocks k-blocks laid end to end (position x belongs to CTA ceil((x+1)*G/W) - 1).
struct WorkIter {
    int nk, splits, G, units, u;
    long long W, pos, hi;
    bool sk;
    __device__ __forceinline__ WorkIter(const IgemmParams& p, int tiles) {
        nk = p.num_kblocks;
        splits = p.splits;
        G = gridDim.x;
        sk = p.stream_k != 0;
        units = tiles * p.splits;
        u = blockIdx.x;
        W = (long long)tiles * nk;
        pos = W * blockIdx.x / G;
        hi = W * (blockIdx.x + 1) / G;
    }
    __device__ __forceinline__ int cta_of(long long x) const { return (int)(((x + 1) * G + W - 1) / W) - 1; }
    // Slab holding CTA c's piece of `tile`: the first slab if c's range begins inside the tile, else the second.
    __device__ __forceinline__ int slab_of(int c, int tile) const {
        if (!sk) return tile * splits + c;   // split-K: c is the split index
        return 2 * c + (W * c / G >= (long long)tile * nk ? 0 : 1);
    }
    __device__ __forceinline__ bool next(Seg& s) {
        if (sk) {
            if (pos >= hi) return false;
            s.tile = (int)(pos / nk);
            s.kb_begin = (int)(pos - (long long)s.tile * nk);
            const long long left = hi - pos;
            const int len = left < (long long)(nk - s.kb_begin) ? (int)left : nk - s.kb_begin;
            s.kb_end = s.kb_begin + len;
            const int first = cta_of((long long)s.tile * nk), last = cta_of((long long)s.tile * nk + nk - 1);
            s.nseg = last - first + 1;
            s.slot = first + 1;
            s.first_cta = first;
            s.my_slab = 2 * (int)blockIdx.x + (pos == W * blockIdx.x / G ? 0 : 1);
            pos += len;
            return true;
        }
        if (u >= units) return false;
        s.tile = u / splits;
        const int split = u - s.tile * splits;
        s.kb_begin = (int)((long long)nk * split / splits);
        s.kb_end = (int)((long long)nk * (split + 1) / splits);
        s.nseg = splits;
        s.slot = s.tile;
        s.first_cta = 0;
        s.my_slab = u;          // split-K: slab tile * splits + split
        u += G;
        return true;
    }
};

// Adds four partial sums to scratch with one 16-byte reduction.
__device__ __forceinline__ void red_add_v4(float* dst, const float4& v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

template <typename T, int BN, int PASSES, bool ATMEM>
__global__ void __launch_bounds__(NTHREADS, 1) igemm_fprop_kernel(const __grid_constant__ IgemmParams p) {
    using C = Cfg<T, BN, PASSES, ATMEM>;
    using Chunk = typename ChunkOf<T>::type;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float* epi_stage = reinterpret_cast<float*>(smem + C::RING_BYTES);
    SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem + C::RING_BYTES + C::EPI_BYTES);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    constexpr int stages = C::STAGES;
    constexpr int stage_bytes = C::STAGE_BYTES;
    constexpr int b_off = C::B_OFF;

    if (tid == 0) {
        for (int s = 0; s < stages; s++) {
            // every producer thread, when its copies have landed; or the one TMA-issuing thread plus the byte count
            mbar_init(&ctl->raw_full[s], p.use_tma ? 1 : PROD_WARPS * 32);
            // one elected lane per splitter warp that works on the k-block (one group of four, or both groups)
            mbar_init(&ctl->full[s], (p.use_tma && !ATMEM) ? 2 * SPLIT_WARPS : SPLIT_WARPS);
            mbar_init(&ctl->empty[s], 1);      // tcgen05.commit
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&ctl->tmem_full[b], 1);           // tcgen05.commit
            mbar_init(&ctl->tmem_empty[b], p.use_tma ? 2 * EPI_WARPS : EPI_WARPS);  // one elected lane per epilogue warp
        }
        ctl->abort_flag = 0;
        ctl->last_flag = 0;
        fence_barrier_init();
    }
    if (warp == TMA_WARP && lane == 0 && p.use_tma) {
        prefetch_tensormap(p.tmap_a);   // hide the descriptor fetch behind the rest of the set-up
        prefetch_tensormap(p.tmap_b);
    }
    __syncthreads();   // barriers are initialised: the TMA warp may start copying
    // Everything above touched only this CTA's shared memory and the kernel parameters, so under programmatic
    // dependent launch it overlaps the tail of the previous kernel of the stream.  From here on global memory is
    // read (operands, residual, scratch): wait for that kernel to complete.  The next kernel may start its own
    // set-up as soon as every CTA of this one has got this far.
    pdl_wait();
    if (tid == 0) pdl_launch_dependents();
    uint32_t tmem_base = 0;
    if (warp != TMA_WARP) {
        // Everyone but the TMA warp needs the tensor-memory base; the allocation overlaps the first copies.
        if (warp == MMA_WARP) {
            tmem_alloc(&ctl->tmem_base, C::TMEM_COLS);
            tmem_relinquish();
        }
        tc_fence_before_sync();
        asm volatile("bar.sync 2, %0;" ::"r"(TMA_WARP * 32) : "memory");
        tc_fence_after_sync();
        tmem_base = ctl->tmem_base;
    }
    volatile int* abort_flag = &ctl->abort_flag;

    const int tiles_per_problem = p.tiles_m * p.tiles_n;
    const int tiles = tiles_per_problem * (p.batch > 1 ? p.batch : 1);
    const int SC = p.S * p.C;
    long long waited = 0;
    const long long t_start = clock64();
    // Roles of warps 9-17 depend on how the operands arrive: gathered by eight producer warps, or copied by
    // TMA, which frees those warps for a second epilogue group and a second splitter group.
    const bool tma_roles = p.use_tma != 0;
    const int epi_groups = tma_roles ? 2 : 1;
    const int epi_id = warp < EPI_WARPS ? warp : (tma_roles && warp >= 9 && warp < 13) ? EPI_WARPS + warp - 9 : -1;
    const int split_id = (warp > MMA_WARP && warp <= MMA_WARP + SPLIT_WARPS) ? warp - MMA_WARP - 1
                         : (tma_roles && warp >= 13 && warp < 17)            ? SPLIT_WARPS + warp - 13
                                                                             : -1;

    if (epi_id >= 0) {
        // ------------------------------------------------------------ epilogue
        // Warp (epi_id % 4 == warp % 4) reads TMEM lanes (accumulator rows) 32*(warp % 4) .. +31; with two
        // groups of four warps, group g takes columns [g*BN/2, (g+1)*BN/2).
        const int q = warp & 3;
        const int grp = epi_id >> 2;
        const int col_lo = grp * (BN / epi_groups), col_hi = col_lo + BN / epi_groups;
        const int epi_threads = 128 * epi_groups;
        float* stage = epi_stage + epi_id * (32 * EPI_LD);
        const int sub = lane >> 2;          // row within a group of eight
        const int cc = (lane & 3) * 4;      // first of this lane's four channels within a 16-channel chunk
        const uint32_t tmem_rows = tmem_base + ((uint32_t)(q * 32) << 16);
        const bool cross = ATMEM && p.cross_acc != 0;
        // 32 columns of the finished accumulator, one row per lane (main part plus, if kept apart, the cross terms)
        auto load_acc = [&](uint32_t col, uint32_t (&r)[32]) {
            tmem_ld_32x32(tmem_rows + col, r);
            if (ATMEM && cross) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    uint32_t c[16];
                    tmem_ld_32x16(tmem_rows + BN + col + 16 * h, c);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) r[16 * h + j] = __float_as_uint(__uint_as_float(r[16 * h + j]) + __uint_as_float(c[j]));
                }
            } else {
                tmem_ld_wait();
            }
        };
        int local = 0;
        WorkIter work(p, tiles);
        Seg seg;
        for (; work.next(seg); local++) {
            const int tile = seg.tile;
            const int bidx = tile / tiles_per_problem;
            const int tloc = tile - bidx * tiles_per_problem;
            const int tm = tloc / p.tiles_n, tn = tloc % p.tiles_n;
            const long long y_off = (long long)bidx * p.batch_stride_y;
            // With the cross-term accumulator there is one output buffer (0) and its barriers flip every tile.
            const int ab = cross ? 0 : (local & 1);
            const uint32_t acc_use = cross ? (uint32_t)local : (uint32_t)(local >> 1);
            if (!timed_wait(&ctl->tmem_full[ab], acc_use & 1u, abort_flag, waited)) {
                if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_TMEM_FULL); }
                break;
            }
            tc_fence_after_sync();
            const long long tile_row0 = (long long)tm * BM + q * 32;
            if (p.mode == 1) {
                // Filter gradient: accumulator row = output channel k, columns = channels c of tap (r, s).
                // The result lands in dw[k][r][s][c]; partial sums of different pixel ranges are added atomically.
                const bool multi = p.wg_tpt > 1;
                const int tap0 = multi ? tn * p.wg_tpt : tn / p.ctiles;
                const int cbase = multi ? 0 : (tn - tap0 * p.ctiles) * BN;
                const int taps = p.R * p.S;
                float* dw = reinterpret_cast<float*>(p.y);
#pragma unroll 1
                for (int c32 = col_lo; c32 < col_hi; c32 += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_rows + ab * BN + c32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int h = 0; h < 2; h++) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            *reinterpret_cast<float4*>(stage + lane * EPI_LD + j) = make_float4(
                                __uint_as_float(r[16 * h + j]), __uint_as_float(r[16 * h + j + 1]), __uint_as_float(r[16 * h + j + 2]),
                                __uint_as_float(r[16 * h + j + 3]));
                        __syncwarp();
                        const int ncol = c32 + 16 * h + cc;   // column of the tile -> (tap, channel)
                        const int tap = multi ? tap0 + ncol / p.wg_cr : tap0;
                        const int c = multi ? ncol % p.wg_cr : cbase + ncol;
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int rr = i * 8 + sub;
                            const long long k = tile_row0 + rr;
                            if (k < p.Kout && c < p.C && tap < taps) {
                                const float4 v = *reinterpret_cast<const float4*>(stage + rr * EPI_LD + cc);
                                float* dst = dw + ((long long)k * p.R * p.S + tap) * p.C + c;
                                if (p.splits > 1) red_add_v4(dst, v);
                                else *reinterpret_cast<float4*>(dst) = v;
                            }
                        }
                        __syncwarp();
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->tmem_empty[ab]);
                continue;
            }
            if (seg.nseg > 1) {
                // Piece of a cut tile (stream-K, or one split of split-K).  The partial accumulator goes to this
                // piece's slab, laid out [4-column group][row] so that the lanes (rows) of a warp write consecutive 16 bytes.
                constexpr int SLAB_F4 = BM * BN / 4;
                float4* slabs = reinterpret_cast<float4*>(p.slabs);
                float4* mine = slabs + (long long)seg.my_slab * SLAB_F4;
                const int row = q * 32 + lane;
#pragma unroll 1
                for (int c32 = col_lo; c32 < col_hi; c32 += 32) {
                    uint32_t r[32];
                    load_acc((uint32_t)(ab * BN + c32), r);
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        mine[(c32 / 4 + j) * BM + row] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                                     __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->tmem_empty[ab]);   // the accumulator is out of TMEM
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"r"(epi_threads) : "memory");
                if (tid == 0) {
                    int prev = atomicAdd(p.counters + seg.slot, 1);
                    ctl->last_flag = (prev == seg.nseg - 1);
                }
                asm volatile("bar.sync 1, %0;" ::"r"(epi_threads) : "memory");
                if (ctl->last_flag) {
                    // Last piece to arrive: every slab of the tile is published.  Sum them in CTA (split) order.
                    __threadfence();
#pragma unroll 1
                    for (int c16 = col_lo; c16 < col_hi; c16 += 16) {
                        float acc[16];
#pragma unroll
                        for (int j = 0; j < 16; j++) acc[j] = 0.f;
                        for (int c = seg.first_cta; c < seg.first_cta + seg.nseg; c++) {
                            const float4* src = slabs + (long long)work.slab_of(c, tile) * SLAB_F4;
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                const float4 v = __ldcg(src + (c16 / 4 + j) * BM + row);
                                acc[4 * j] += v.x; acc[4 * j + 1] += v.y; acc[4 * j + 2] += v.z; acc[4 * j + 3] += v.w;
                            }
                        }
                        epilogue_chunk<T>(p, stage, acc, lane, tile_row0, tn * BN + c16, y_off);
                    }
                    if (tid == 0) p.counters[seg.slot] = 0;
                }
                asm volatile("bar.sync 1, %0;" ::"r"(epi_threads) : "memory");   // last_flag is rewritten by the next piece
                continue;
            }
#pragma unroll 1
            for (int c32 = col_lo; c32 < col_hi; c32 += 32) {   // whole tile in one piece: straight to the output
                uint32_t r[32];
                load_acc((uint32_t)(ab * BN + c32), r);
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    float v16[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) v16[j] = __uint_as_float(r[16 * h + j]);
                    epilogue_chunk<T>(p, stage, v16, lane, tile_row0, tn * BN + c32 + 16 * h, y_off);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->tmem_empty[ab]);
        }
        if (p.debug && blockIdx.x == 0 && tid == 0) p.debug[0] = waited;
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------ MMA issue
        if (lane == 0) {
            // A TMA-fed filter gradient keeps both operands the way they lie in memory (pixel-major, i.e.
            // MN-major for this GEMM); everything else stages K-major rows.
            const bool mn_major = p.mode == 1 && p.use_tma;
            const uint32_t idesc = umma_idesc(sizeof(T) == 4 ? 2 : 1, BM, BN) | (mn_major ? (UMMA_IDESC_A_MN | UMMA_IDESC_B_MN) : 0u);
            const uint64_t kstep = mn_major ? (1024 >> 4) : (32 >> 4);   // descriptor address advance per k-step of 8 (16 for bf16)
            RingPos ring;
            int local = 0;
            bool dead = false;
            long long waited2 = 0;
            const bool cross = ATMEM && p.cross_acc != 0;
            WorkIter work(p, tiles);
            Seg seg;
            for (; !dead && work.next(seg); local++) {
                const int kb_begin = seg.kb_begin, kb_end = seg.kb_end;
                const int ab = cross ? 0 : (local & 1);
                const uint32_t acc_use = cross ? (uint32_t)local : (uint32_t)(local >> 1);
                if (!timed_wait(&ctl->tmem_empty[ab], (acc_use & 1u) ^ 1u, abort_flag, waited2)) {
                    if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_TMEM_EMPTY); }
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d = tmem_base + ab * BN;
                for (int kb = kb_begin; kb < kb_end; kb++, ring.advance(stages)) {
                    const int s = ring.s;
                    // fp32: operands are ready when the splitters are done; bf16: when the copies have landed
                    if (!timed_wait(C::kSplit ? &ctl->full[s] : &ctl->raw_full[s], ring.ph, abort_flag, waited)) {
                        if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_FULL); }
                        dead = true;
                        break;
                    }
                    if (!C::kSplit) fence_proxy_async_smem();   // cp.async wrote through the generic proxy
                    tc_fence_after_sync();
                    const uint32_t base = smem_u32(smem + s * stage_bytes);
                    if (C::kSplit) {
                        const uint64_t a_hi = mn_major ? umma_desc_mn(p.mn_desc_bits, base) : umma_desc_sw128(base);
                        const uint64_t a_lo = mn_major ? umma_desc_mn(p.mn_desc_bits, base + C::A_BYTES) : umma_desc_sw128(base + C::A_BYTES);
                        const uint64_t b_hi = mn_major ? umma_desc_mn(p.mn_desc_bits, base + b_off) : umma_desc_sw128(base + b_off);
                        const uint64_t b_lo = mn_major ? umma_desc_mn(p.mn_desc_bits, base + b_off + C::B_BYTES)
                                                       : umma_desc_sw128(base + b_off + C::B_BYTES);
                        if (ATMEM) {
                            const uint32_t ta_hi = tmem_base + C::A_TMEM_COL0 + s * 64, ta_lo = ta_hi + 32;
#pragma unroll
                            for (int ks = 0; ks < 4; ks++) {
                                const uint64_t o = (uint64_t)ks * kstep;
                                const uint32_t first = (kb > kb_begin || ks > 0) ? 1u : 0u;
                                // cross terms: into the main accumulator, or into one of their own (columns BN..2BN)
                                const uint32_t dx = cross ? tmem_base + BN : d;
                                umma_tf32_ts(dx, ta_lo + ks * 8, b_hi + o, idesc, first);
                                umma_tf32_ts(dx, ta_hi + ks * 8, b_lo + o, idesc, 1u);
                                umma_tf32_ts(d, ta_hi + ks * 8, b_hi + o, idesc, cross ? first : 1u);
                            }
                        } else {
#pragma unroll
                            for (int ks = 0; ks < 4; ks++) {
                                const uint64_t o = (uint64_t)ks * kstep;
                                umma_tf32(d, a_lo + o, b_hi + o, idesc, (kb > kb_begin || ks > 0) ? 1u : 0u);
                                umma_tf32(d, a_hi + o, b_lo + o, idesc, 1u);
                                umma_tf32(d, a_hi + o, b_hi + o, idesc, 1u);
                            }
                        }
                    } else {
                        const uint64_t a = mn_major ? umma_desc_mn(p.mn_desc_bits, base) : umma_desc_sw128(base);
                        const uint64_t b = mn_major ? umma_desc_mn(p.mn_desc_bits, base + C::A_BYTES) : umma_desc_sw128(base + C::A_BYTES);
#pragma unroll
                        for (int ks = 0; ks < 4; ks++) {
                            const uint64_t o = (uint64_t)ks * kstep;
                            if (sizeof(T) == 4) umma_tf32(d, a + o, b + o, idesc, (kb > kb_begin || ks > 0) ? 1u : 0u);
                            else umma_f16(d, a + o, b + o, idesc, (kb > kb_begin || ks > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(&ctl->empty[s]);   // frees the stage once these MMAs have read it
                }
                if (!dead) umma_commit(&ctl->tmem_full[ab]);
            }
            if (p.debug && blockIdx.x == 0) { p.debug[1] = waited; p.debug[2] = waited2; }
        }
    } else if (split_id >= 0) {
        // ------------------------------------------------------------ splitters (fp32 only)
        // Write, for every raw fp32 operand value the producers or TMA put into shared memory, the exact
        // remainder x - tf32(x) into the second buffer.  The work is elementwise, so the 16-byte chunks of the
        // two tiles are simply dealt out to the splitter threads in address order.
        if (C::kSplit) {
            // With two splitter groups (TMA-fed launches) the groups take alternate k-blocks: splitting one k-block is
            // a chain of latencies (barrier wake-up, shared-memory reads, tcgen05.st and its wait, fence, arrive), so
            // two k-blocks in flight double the rate where sharing one k-block between the groups did not.
            // (Only where the activation parts go to tensor memory; the shared-memory variant is bound by the traffic
            // itself, there both groups share every k-block.)
            const bool alternate = ATMEM && tma_roles;
            const int st_id = alternate ? (split_id & 3) * 32 + lane : split_id * 32 + lane;
            const int st_threads = (tma_roles && !alternate ? 2 * SPLIT_WARPS : SPLIT_WARPS) * 32;
            const int grp = alternate ? split_id >> 2 : 0, ngrp = alternate ? 2 : 1;
            int turn = 0;
            RingPos ring;
            bool dead = false;
            WorkIter work(p, tiles);
            Seg seg;
            while (!dead && work.next(seg)) {
                const int kb_begin = seg.kb_begin, kb_end = seg.kb_end;
                for (int kb = kb_begin; kb < kb_end; kb++, ring.advance(stages)) {
                    const int s = ring.s;
                    const bool mine = turn == grp;
                    if (++turn == ngrp) turn = 0;
                    if (!mine) continue;
                    if (!timed_wait(&ctl->raw_full[s], ring.ph, abort_flag, waited)) {
                        if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_FULL); }
                        dead = true;
                        break;
                    }
                    uint8_t* st = smem + s * stage_bytes;
                    uint8_t* a_hi = st;
                    uint8_t* a_lo = st + C::A_BYTES;
                    uint8_t* b_hi = st + b_off;
                    uint8_t* b_lo = b_hi + C::B_BYTES;
                    if (ATMEM) {
                        // Activation tile: this thread owns row (32*(warp%4) + lane) = its tensor-memory lane.  Both
                        // parts of the row's 32 values go to tensor memory, where the MMA reads its A operand without
                        // touching shared memory again.
                        const int q = warp & 3;
                        const uint32_t row = (uint32_t)(q * 32 + lane);
                        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + C::A_TMEM_COL0 + s * 64;
#pragma unroll
                        for (int c0 = 0; c0 < 32; c0 += 16) {
                            uint32_t hi[16], lo[16];
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                const float4 v = *reinterpret_cast<const float4*>(a_hi + sw128_offset(row, (uint32_t)(c0 / 4 + j)));
                                const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                                for (int k = 0; k < 4; k++) {
                                    // Round to nearest on this side (it costs nothing here): the remainder is then
                                    // zero-mean, so the dropped lo*lo product carries no bias even though the filter
                                    // side splits by truncation.
                                    const float h = tf32_round(e[k]);
                                    hi[4 * j + k] = __float_as_uint(h);
                                    lo[4 * j + k] = __float_as_uint(tf32_round(e[k] - h));
                                }
                            }
                            tmem_st_32x16(t_row + c0, hi);
                            tmem_st_32x16(t_row + 32 + c0, lo);
                        }
                        tmem_st_wait();
                        tc_fence_before_sync();
                    } else {
#pragma unroll 4
                        for (int i = st_id; i < C::A_BYTES / 16; i += st_threads) split_chunk(a_hi + i * 16, a_lo + i * 16);
                    }
#pragma unroll 4
                    for (int i = st_id; i < C::B_BYTES / 16; i += st_threads) split_chunk(b_hi + i * 16, b_lo + i * 16);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ctl->full[s]);
                }
            }
            if (p.debug && blockIdx.x == 0 && st_id == 0) p.debug[3] = waited;
        }
    } else if (warp == TMA_WARP ? tma_roles : (!tma_roles && warp >= 9)) {
        // ------------------------------------------------------------ producers
        // TMA-fed launches: one lane of the TMA warp issues the copies.  Otherwise warps 9-16 gather with
        // asynchronous 16-byte copies (zero-filled outside the image) straight into the swizzled
        // stage buffers, several stages ahead of the MMA.  Eight consecutive threads copy the
        // eight 16-byte chunks of one operand row, so a warp instruction reads four full 128-byte
        // lines; each thread serves rows (t/8), (t/8)+16, ... of the tile with its fixed chunk t%8.
        const int pt = tma_roles ? lane : (warp - 9) * 32 + lane;   // gather: 0..255; TMA: lane 0 issues
        const T* __restrict__ X0 = reinterpret_cast<const T*>(p.x);
        const T* __restrict__ W0 = reinterpret_cast<const T*>(p.w);
        const bool vec = (p.C % C::EPC) == 0;
        constexpr int RPT = BM / 32;            // A rows per thread
        const int chunk = pt & 7;
        const int row0 = pt >> 3;               // 0..31; this thread serves rows row0 + 32*i
        // (row & 7) == (row0 & 7) for all of them, so the swizzled chunk position is a per-thread constant
        const uint32_t sw_off = (uint32_t)row0 * 128u + (uint32_t)((chunk ^ (row0 & 7)) << 4);
        RingPos ring;
        bool dead = false;
        WorkIter work(p, tiles);
        Seg seg;
        while (!dead && work.next(seg)) {
            const int tile = seg.tile;
            const int bidx = tile / tiles_per_problem;
            const int tloc = tile - bidx * tiles_per_problem;
            const int tm = tloc / p.tiles_n, tn = tloc % p.tiles_n;
            const T* __restrict__ X = X0 + (long long)bidx * p.batch_stride_x;
            const T* __restrict__ Wt = W0 + (long long)bidx * p.batch_stride_w;
            const int kb_begin = seg.kb_begin, kb_end = seg.kb_end;
            if (p.use_tma && p.mode == 1) {
                // Filter gradient fed by TMA (float32).  A k-block is 32 consecutive output pixels; both operands
                // stay pixel-major: four boxes of 32 pixels x 32 output channels of dy, and BN/32 im2col boxes of
                // 32 pixels x 32 input channels of the layer input at this tile's tap.
                if (pt == 0 && sizeof(T) == 4) {
                    const bool multi = p.wg_tpt > 1;
                    const int tap0 = multi ? tn * p.wg_tpt : tn / p.ctiles;
                    const int cbase = multi ? 0 : (tn - tap0 * p.ctiles) * BN;
                    const int taps = p.R * p.S;
                    const int k0 = tm * BM;
                    const int pq = p.P * p.Q;
                    // box g holds 32 columns of the tile: one tap's channels [bc[g], bc[g] + 32); -1: nothing to load
                    // (tap offsets are worked out here, once per tile: the loop below is the copy-issuing thread's
                    // critical path)
                    int bc[BN / 32], nb_boxes = 0;
                    uint16_t boff_w[BN / 32], boff_h[BN / 32];
#pragma unroll
                    for (int g = 0; g < BN / 32; g++) {
                        const int btap = multi ? tap0 + (32 * g) / p.wg_cr : tap0;
                        bc[g] = multi ? (32 * g) % p.wg_cr : cbase + 32 * g;
                        const int fr = btap / p.S, fs = btap - fr * p.S;
                        boff_w[g] = (uint16_t)(fs * p.dil_w);
                        boff_h[g] = (uint16_t)(fr * p.dil_h);
                        if (bc[g] >= p.C || btap >= taps) bc[g] = -1;
                        else nb_boxes++;
                    }
                    // first pixel of the k-block as (image, row, column), carried along from k-block to k-block
                    int n_img, op, oq;
                    {
                        const long long mb = (long long)kb_begin * 32;
                        n_img = (int)(mb / pq);
                        const int rem = (int)(mb - (long long)n_img * pq);
                        op = rem / p.Q;
                        oq = rem - op * p.Q;
                    }
                    for (int kb = kb_begin; kb < kb_end; kb++, ring.advance(stages)) {
                        const int s = ring.s;
                        const long long m0 = (long long)kb * 32;
                        const int cur_n = n_img, cur_p = op, cur_q = oq;
                        oq += 32;
                        while (oq >= p.Q) {
                            oq -= p.Q;
                            if (++op == p.P) { op = 0; n_img++; }
                        }
                        if (!timed_wait(&ctl->empty[s], (ring.ph ^ 1u), abort_flag, waited)) {
                            if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_EMPTY); }
                            dead = true;
                            break;
                        }
                        const uint32_t a_dst = smem_u32(smem + s * stage_bytes);
                        const uint32_t b_dst = a_dst + b_off;
                        mbar_arrive_expect_tx(&ctl->raw_full[s], C::A_BYTES + nb_boxes * 4096);
#pragma unroll
                        for (int g = 0; g < BM / 32; g++) tma_load_tile_2d(a_dst + g * 4096, p.tmap_a, &ctl->raw_full[s], k0 + 32 * g, (int)m0);
#pragma unroll
                        for (int g = 0; g < BN / 32; g++)
                            if (bc[g] >= 0)   // columns past C or past the last tap are never stored
                                tma_load_im2col_4d(b_dst + g * 4096, p.tmap_b, &ctl->raw_full[s], bc[g], cur_q * p.stride_w - p.pad_w,
                                                   cur_p * p.stride_h - p.pad_h, cur_n, boff_w[g], boff_h[g]);
                    }
                } else {
                    break;
                }
                continue;
            }
            if (p.use_tma) {
                // Both operand tiles of a k-block arrive by one TMA copy each, issued by a single thread:
                // 128 im2col rows of the activation (zero outside the image, walking pixels in GEMM row
                // order from the tile's first pixel) and BN filter rows, both landing in the 128-byte
                // swizzled layout the MMA descriptors expect.
                if (pt == 0) {
                    const long long m0 = (long long)tm * BM;
                    const int pq = p.OH * p.OW;
                    const int n_img = (int)(m0 / pq);
                    const int rem = (int)(m0 - (long long)n_img * pq);
                    const int op = rem / p.OW, oq = rem - op * p.OW;
                    const int cw = oq * p.bmul_w + p.tma_base_w, ch = op * p.bmul_h + p.tma_base_h;
                    const int cn = bidx * p.Nb + n_img;
                    // Filter row r, tap ts and channel tc of the k-block are carried along instead of divided out
                    // every time: this loop is the copy-issuing thread's critical path.
                    int r = kb_begin / p.kblocks_per_r;
                    int kb_in_r = kb_begin - r * p.kblocks_per_r;
                    int ts = (kb_in_r * C::BK) / p.C, tc = kb_in_r * C::BK - ts * p.C;
                    for (int kb = kb_begin; kb < kb_end; kb++, ring.advance(stages)) {
                        const int s = ring.s;
                        const int off_h = p.step_h >= 0 ? r * p.step_h : (p.R - 1 - r) * -p.step_h;
                        const int off_w = p.step_w >= 0 ? ts * p.step_w : (p.S - 1 - ts) * -p.step_w;
                        const int cur_r = r, cur_ts = ts, cur_tc = tc;
                        tc += C::BK;                       // next k-block: whole taps per k-block row (C % BK == 0), or one tap
                        if (tc >= p.C) { tc -= p.C; ts++; }
                        if (++kb_in_r == p.kblocks_per_r) { kb_in_r = 0; r++; ts = 0; tc = 0; }
                        if (!timed_wait(&ctl->empty[s], (ring.ph ^ 1u), abort_flag, waited)) {
                            if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_EMPTY); }
                            dead = true;
                            break;
                        }
                        const uint32_t a_dst = smem_u32(smem + s * stage_bytes);
                        const uint32_t b_dst = a_dst + b_off;
                        mbar_arrive_expect_tx(&ctl->raw_full[s], C::A_BYTES + C::B_BYTES);
                        tma_load_im2col_4d(a_dst, p.tmap_a, &ctl->raw_full[s], cur_tc, cw, ch, cn, (uint16_t)off_w, (uint16_t)off_h);
                        tma_load_tile_5d(b_dst, p.tmap_b, &ctl->raw_full[s], cur_tc, cur_ts, cur_r, tn * BN, bidx);
                    }
                } else {
                    break;   // the other producer threads have nothing to do
                }
                continue;
            }
            if (p.mode == 1) {
                // Filter gradient (float32 data).  A k-block is 32 consecutive output pixels.  Both operands
                // have the pixel index as their slow dimension in memory, so they are transposed on the way
                // in: thread (prow, cg) loads, for pixel m = first + prow, every eighth 16-byte chunk of
                // dy[m][k0..k0+127] and of x[pixel of m at this tile's tap][c0..c0+BN-1], and scatters the four
                // values of a chunk to column m of four consecutive K-major operand rows.
                if (sizeof(T) == 4) {
                    const int tap = tn / p.ctiles, cblk = tn - tap * p.ctiles;
                    const int fr = tap / p.S, fs = tap - fr * p.S;
                    const int k0 = tm * BM, c0 = cblk * BN;
                    const int pq = p.P * p.Q;
                    const int prow = pt >> 3, cg = pt & 7;
                    const float* __restrict__ DY = reinterpret_cast<const float*>(X);
                    const float* __restrict__ IN = reinterpret_cast<const float*>(Wt);
                    for (int kb = kb_begin; kb < kb_end; kb++, ring.advance(stages)) {
                        const int s = ring.s;
                        const long long m = (long long)kb * 32 + prow;
                        const bool m_ok = m < p.M;
                        const float* xsrc = nullptr;
                        if (m_ok) {
                            const int n_img = (int)(m / pq);
                            const int rem = (int)(m - (long long)n_img * pq);
                            const int op = rem / p.Q, oq = rem - op * p.Q;
                            const int h = op * p.stride_h - p.pad_h + fr * p.dil_h;
                            const int w = oq * p.stride_w - p.pad_w + fs * p.dil_w;
                            if ((unsigned)h < (unsigned)p.H && (unsigned)w < (unsigned)p.W)
                                xsrc = IN + (((long long)n_img * p.H + h) * p.W + w) * p.C;
                        }
                        float4 av[BM / 32], bv[BN / 32];
#pragma unroll
                        for (int i = 0; i < BM / 32; i++) {
                            const int k = k0 + (cg + 8 * i) * 4;
                            av[i] = (m_ok && k < p.Kout) ? __ldg(reinterpret_cast<const float4*>(DY + m * p.Kout + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int i = 0; i < BN / 32; i++) {
                            const int c = c0 + (cg + 8 * i) * 4;
                            bv[i] = (xsrc != nullptr && c < p.C) ? __ldg(reinterpret_cast<const float4*>(xsrc + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                        if (!timed_wait(&ctl->empty[s], (ring.ph ^ 1u), abort_flag, waited)) {
                            if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_EMPTY); }
                            dead = true;
                            break;
                        }
                        uint8_t* a_dst = smem + s * stage_bytes;
                        uint8_t* b_dst = a_dst + b_off;
                        const uint32_t col_chunk = (uint32_t)prow >> 2, col_word = ((uint32_t)prow & 3u) * 4u;
#pragma unroll
                        for (int i = 0; i < BM / 32; i++) {
                            const uint32_t row = (uint32_t)(cg + 8 * i) * 4u;
                            const float e[4] = {av[i].x, av[i].y, av[i].z, av[i].w};
#pragma unroll
                            for (int q = 0; q < 4; q++)
                                *reinterpret_cast<float*>(a_dst + sw128_offset(row + q, col_chunk) + col_word) = e[q];
                        }
#pragma unroll
                        for (int i = 0; i < BN / 32; i++) {
                            const uint32_t row = (uint32_t)(cg + 8 * i) * 4u;
                            const float e[4] = {bv[i].x, bv[i].y, bv[i].z, bv[i].w};
#pragma unroll
                            for (int q = 0; q < 4; q++)
                                *reinterpret_cast<float*>(b_dst + sw128_offset(row + q, col_chunk) + col_word) = e[q];
                        }
                        if (!C::kSplit) fence_proxy_async_smem();
                        mbar_arrive(&ctl->raw_full[s]);
                    }
                }
                continue;
            }
            if (vec) {
                // Unit-divisor gathers (forward convolution, stride-1 data gradient): xpix is the address of
                // the (possibly out-of-image) tap-0 pixel of row i, and a tap adds a row-independent offset.
                // Strided data gradients keep the image base and compute the pixel per tap.  Null past M.
                const bool unit = p.div_h == 1 && p.div_w == 1;
                const T* xpix[RPT];
                int hb[RPT], wb[RPT];
                const int pq = p.OH * p.OW;
#pragma unroll
                for (int i = 0; i < RPT; i++) {
                    const long long m = (long long)tm * BM + i * 32 + row0;
                    xpix[i] = nullptr;
                    hb[i] = wb[i] = 0;
                    if (m < p.M) {
                        const int n_img = (int)(m / pq);
                        const int rem = (int)(m - (long long)n_img * pq);
                        const int op = rem / p.OW, oq = rem - op * p.OW;
                        hb[i] = op * p.bmul_h + p.badd_h;
                        wb[i] = oq * p.bmul_w + p.badd_w;
                        xpix[i] = X + (long long)n_img * p.IH * p.IW * p.C + (unit ? ((long long)hb[i] * p.IW + wb[i]) * p.C : 0);
                    }
                }
                const T* wrow[BN / 32];
#pragma unroll
                for (int i = 0; i < BN / 32; i++) {
                    const int kout = tn * BN + i * 32 + row0;
                    wrow[i] = kout < p.Kout ? Wt + (long long)kout * p.R * SC : nullptr;
                }
                for (int kb = kb_begin; kb < kb_end; kb++, ring.advance(stages)) {
                    const int s = ring.s;
                    const int r = kb / p.kblocks_per_r;
                    const int kk = (kb - r * p.kblocks_per_r) * C::BK + chunk * C::EPC;
                    const bool k_ok = kk < SC;
                    const int ts = kk / p.C, tc = kk - ts * p.C;
                    const int dh = r * p.step_h, dw = ts * p.step_w;
                    const long long xoff = ((long long)dh * p.IW + dw) * p.C + tc;   // same for every row of the tile
                    const long long woff = (long long)r * SC + kk;
                    if (!timed_wait(&ctl->empty[s], (ring.ph ^ 1u), abort_flag, waited)) {
                        if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_EMPTY); }
                        dead = true;
                        break;
                    }
                    const uint32_t a_dst = smem_u32(smem + s * stage_bytes) + sw_off;
                    const uint32_t b_dst = a_dst + b_off;
                    if (unit) {
#pragma unroll
                        for (int i = 0; i < RPT; i++) {
                            const int h = hb[i] + dh, w = wb[i] + dw;
                            const bool ok = k_ok && xpix[i] != nullptr && (unsigned)h < (unsigned)p.IH && (unsigned)w < (unsigned)p.IW;
                            cp_async_16(a_dst + i * 4096, ok ? (const void*)(xpix[i] + xoff) : (const void*)X, ok);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < RPT; i++) {
                            const int hn = hb[i] + dh, wn = wb[i] + dw;
                            const int h = hn / p.div_h, w = wn / p.div_w;
                            const bool ok = k_ok && xpix[i] != nullptr && hn >= 0 && wn >= 0 && h * p.div_h == hn && w * p.div_w == wn &&
                                            h < p.IH && w < p.IW;
                            cp_async_16(a_dst + i * 4096, ok ? (const void*)(xpix[i] + ((long long)h * p.IW + w) * p.C + tc) : (const void*)X, ok);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < BN / 32; i++) {
                        const bool ok = k_ok && wrow[i] != nullptr;
                        cp_async_16(b_dst + i * 4096, ok ? (const void*)(wrow[i] + woff) : (const void*)Wt, ok);
                    }
                    cp_async_arrive_noinc(&ctl->raw_full[s]);
                }
            } else {
                // Channel counts that are not a multiple of the 16-byte chunk (the 3-channel stem):
                // scalar gather, one thread per operand row.
                const int row = pt & 127;
                const bool worker = pt < 128;   // one thread per operand row; the other producer warps only arrive
                const long long m = (long long)tm * BM + row;
                const bool m_ok = worker && m < p.M;
                int n_img = 0, h_base = 0, w_base = 0;
                if (m_ok) {
                    const int pq = p.OH * p.OW;
                    n_img = (int)(m / pq);
                    const int rem = (int)(m - (long long)n_img * pq);
                    const int op = rem / p.OW, oq = rem - op * p.OW;
                    h_base = op * p.bmul_h + p.badd_h;
                    w_base = oq * p.bmul_w + p.badd_w;
                }
                const int kout = tn * BN + row;
                const bool b_ok = worker && row < BN && kout < p.Kout;
                for (int kb = kb_begin; kb < kb_end; kb++, ring.advance(stages)) {
                    const int s = ring.s;
                    const int r = kb / p.kblocks_per_r;
                    const int kk0 = (kb - r * p.kblocks_per_r) * C::BK;
                    const int hn = h_base + r * p.step_h;
                    const int h = hn / p.div_h;
                    const bool h_ok = m_ok && hn >= 0 && h * p.div_h == hn && h < p.IH;
                    const T* xrow = X + ((long long)n_img * p.IH + (h_ok ? h : 0)) * p.IW * p.C;
                    const T* wrow = Wt + ((long long)(b_ok ? kout : 0) * p.R + r) * SC;
                    if (!timed_wait(&ctl->empty[s], (ring.ph ^ 1u), abort_flag, waited)) {
                        if (!*abort_flag) { ctl->abort_flag = 1; if (p.status) atomicExch(p.status, OB200_ERR_WAIT_EMPTY); }
                        dead = true;
                        break;
                    }
                    uint8_t* st = smem + s * stage_bytes;
                    uint8_t* a_dst = st;
                    uint8_t* b_dst = st + b_off;
                    int ts = kk0 / p.C, tc = kk0 - ts * p.C;
#pragma unroll 1
                    for (int j = 0; j < (worker ? 8 : 0); j++) {
                        const uint32_t off = sw128_offset((uint32_t)row, (uint32_t)j);
#pragma unroll
                        for (int e = 0; e < C::EPC; e++) {
                            const int kk = kk0 + j * C::EPC + e;
                            const int wn = w_base + ts * p.step_w;
                            const int w = wn / p.div_w;
                            T av = T(0.f), bv = T(0.f);
                            if (h_ok && kk < SC && wn >= 0 && w * p.div_w == wn && w < p.IW) av = xrow[(long long)w * p.C + tc];
                            if (b_ok && kk < SC) bv = wrow[kk];
                            reinterpret_cast<T*>(a_dst + off)[e] = av;
                            if (row < BN) reinterpret_cast<T*>(b_dst + off)[e] = bv;
                            tc++;
                            if (tc >= p.C) { tc = 0; ts++; }
                        }
                    }
                    if (!C::kSplit) fence_proxy_async_smem();
                    mbar_arrive(&ctl->raw_full[s]);
                }
            }
        }
    }

    if (p.debug && blockIdx.x == 0) {
        if (warp == (tma_roles ? TMA_WARP : 9) && lane == 0) p.debug[4] = waited;   // TMA issuer / producer warp 0
        if (tid == 0) p.debug[5] = clock64() - t_start;
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

template <typename T, int BN, int PASSES, bool ATMEM = false>
static cudaError_t launch_cfg(const IgemmParams& p, int num_ctas, cudaStream_t stream) {
    using C = Cfg<T, BN, PASSES, ATMEM>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(igemm_fprop_kernel<T, BN, PASSES, ATMEM>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    // Every role derives its share of the work from gridDim.x (WorkIter), in all three schedules.
    OB200_ELASTIC((igemm_fprop_kernel<T, BN, PASSES, ATMEM>), 1);
    static const bool pdl = [] {   // ORION_PDL=0: plain stream order between consecutive kernels
        const char* e = getenv("ORION_PDL");
        return !(e && e[0] == '0');
    }();
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3((unsigned)num_ctas);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, igemm_fprop_kernel<T, BN, PASSES, ATMEM>, p);
}

}  // namespace ob200

namespace ob200 {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
using EncodeIm2colFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct TmaApi {
    EncodeTiledFn tiled = nullptr;
    EncodeIm2colFn im2col = nullptr;
    bool ok = false;
};

// The two driver entry points, looked up once through the runtime (no link against the driver library).
static const TmaApi& tma_api() {
    static const TmaApi api = [] {
        TmaApi a;
        const char* off = getenv("ORION_NO_TMA");
        if (off && off[0] == '1') return a;
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess && f &&
            q == cudaDriverEntryPointSuccess)
            a.tiled = reinterpret_cast<EncodeTiledFn>(f);
        f = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &f, cudaEnableDefault, &q) == cudaSuccess && f &&
            q == cudaDriverEntryPointSuccess)
            a.im2col = reinterpret_cast<EncodeIm2colFn>(f);
        a.ok = a.tiled && a.im2col;
        return a;
    }();
    return api;
}

// Decides whether this launch can feed both operands by TMA and, if so, encodes the two tensor maps.
// Needs unit-divisor gathers (forward, stride-1 data gradient, GEMM), channels that fill whole 16-byte
// chunks, and k-blocks that never straddle two filter taps (1x1 filters, or C a multiple of the k-block).
static bool setup_tma(IgemmParams& p, int bn) {
    static_assert(sizeof(CUtensorMap) == sizeof(p.tmap_a), "tensor map size");
    p.use_tma = 0;
    const TmaApi& api = tma_api();
    if (!api.ok) return false;
    if (p.mode == 1) {
        // Filter gradient: dy as a plain [pixels, Kout] matrix in boxes of 32 x 32, the layer input through an
        // im2col map that walks 32 output pixels per box.
        if (p.dtype == 1 || p.C < 32 || (p.C & 3) || (p.Kout & 3) || ((uintptr_t)p.x | (uintptr_t)p.w) % 16) return false;
        if (p.stride_h > 8 || p.stride_w > 8) return false;
        int lower[2] = {-p.pad_w, -p.pad_h};
        int upper[2] = {-p.pad_w + (p.Q - 1) * p.stride_w + 1 - p.W, -p.pad_h + (p.P - 1) * p.stride_h + 1 - p.H};
        for (int i = 0; i < 2; i++)
            if (lower[i] < -128 || lower[i] > 127 || upper[i] < -128 || upper[i] > 127) return false;
        if ((p.R - 1) * p.dil_h > 127 || (p.S - 1) * p.dil_w > 127) return false;
        const CUtensorMapSwizzle wg_swz = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
        {
            cuuint64_t dims[2] = {(cuuint64_t)p.Kout, (cuuint64_t)p.M};
            cuuint64_t strides[1] = {(cuuint64_t)p.Kout * 4};
            cuuint32_t box[2] = {32, 32};
            cuuint32_t steps[2] = {1, 1};
            if (api.tiled(reinterpret_cast<CUtensorMap*>(p.tmap_a), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(p.x), dims,
                          strides, box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE, wg_swz,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return false;
        }
        {
            cuuint64_t dims[4] = {(cuuint64_t)p.C, (cuuint64_t)p.W, (cuuint64_t)p.H, (cuuint64_t)p.Nb};
            cuuint64_t strides[3] = {(cuuint64_t)p.C * 4, (cuuint64_t)p.W * p.C * 4, (cuuint64_t)p.H * p.W * p.C * 4};
            cuuint32_t steps[4] = {1, (cuuint32_t)p.stride_w, (cuuint32_t)p.stride_h, 1};
            if (api.im2col(reinterpret_cast<CUtensorMap*>(p.tmap_b), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(p.w), dims,
                           strides, lower, upper, 32, 32, steps, CU_TENSOR_MAP_INTERLEAVE_NONE, wg_swz,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return false;
        }
        // Operand descriptor above the address: float32 MN-major operands use the 128-byte swizzle with
        // 32-byte atoms (layout type 1; the pattern repeats every four 128-byte rows), groups of four
        // reduction indices 512 bytes apart (stride byte offset), the next 32 M/N indices 4096 bytes on
        // (leading byte offset) -- what the boxes of 32 pixels x 128 bytes written by TMA look like.
        p.mn_desc_bits = ((4096ull >> 4) << 16) | ((512ull >> 4) << 32) | (1ull << 46) | (1ull << 61);
        p.use_tma = 1;
        return true;
    }
    if (p.mode != 0 || p.div_h != 1 || p.div_w != 1) return false;
    const int elem = p.dtype == 1 ? 2 : 4;
    const int bk = 128 / elem;
    if (p.C < bk || (p.C * elem) % 16) return false;
    if (p.R * p.S != 1 && p.C % bk != 0) return false;
    if (p.bmul_h < 1 || p.bmul_h > 8 || p.bmul_w < 1 || p.bmul_w > 8) return false;
    if (((uintptr_t)p.x | (uintptr_t)p.w) % 16) return false;
    const int batch = p.batch > 1 ? p.batch : 1;
    if (batch > 1 && (p.batch_stride_x != (long long)p.Nb * p.IH * p.IW * p.C || (p.batch_stride_w * elem) % 16)) return false;
    const int base_h = p.badd_h + (p.step_h < 0 ? (p.R - 1) * p.step_h : 0);
    const int base_w = p.badd_w + (p.step_w < 0 ? (p.S - 1) * p.step_w : 0);
    const int span_h = (p.R - 1) * (p.step_h < 0 ? -p.step_h : p.step_h);
    const int span_w = (p.S - 1) * (p.step_w < 0 ? -p.step_w : p.step_w);
    // Base pixels run from the lower corner to (extent - 1 + upper corner): exactly OH x OW of them.
    int lower[2] = {base_w, base_h};
    int upper[2] = {base_w + (p.OW - 1) * p.bmul_w + 1 - p.IW, base_h + (p.OH - 1) * p.bmul_h + 1 - p.IH};
    for (int i = 0; i < 2; i++)
        if (lower[i] < -128 || lower[i] > 127 || upper[i] < -128 || upper[i] > 127) return false;
    if (span_h > 127 || span_w > 127) return false;
    const CUtensorMapDataType dt = p.dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    {
        cuuint64_t dims[4] = {(cuuint64_t)p.C, (cuuint64_t)p.IW, (cuuint64_t)p.IH, (cuuint64_t)p.Nb * batch};
        cuuint64_t strides[3] = {(cuuint64_t)p.C * elem, (cuuint64_t)p.IW * p.C * elem, (cuuint64_t)p.IH * p.IW * p.C * elem};
        cuuint32_t steps[4] = {1, (cuuint32_t)p.bmul_w, (cuuint32_t)p.bmul_h, 1};
        if (api.im2col(reinterpret_cast<CUtensorMap*>(p.tmap_a), dt, 4, const_cast<void*>(p.x), dims, strides, lower, upper,
                       (cuuint32_t)bk, (cuuint32_t)BM, steps, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    {
        // Filter as [batch, Kout, R, S, C]; a tap subset changes the base address and the tap strides.
        const bool subset = p.w_R > 0;
        const cuuint64_t wR = subset ? p.w_R : p.R, wS = subset ? p.w_S : p.S;
        const cuuint64_t rstep = subset ? p.w_rstep : 1, sstep = subset ? p.w_sstep : 1;
        const char* base = reinterpret_cast<const char*>(p.w) + (subset ? ((size_t)p.w_r0 * wS + p.w_s0) * p.C * elem : 0);
        cuuint64_t dims[5] = {(cuuint64_t)p.C, (cuuint64_t)p.S, (cuuint64_t)p.R, (cuuint64_t)p.Kout, (cuuint64_t)batch};
        cuuint64_t strides[4] = {sstep * p.C * elem, rstep * wS * p.C * elem, wR * wS * p.C * elem,
                                 (batch > 1 ? (cuuint64_t)p.batch_stride_w : wR * wS * p.C * p.Kout) * elem};
        cuuint32_t box[5] = {(cuuint32_t)bk, 1, 1, (cuuint32_t)bn, 1};
        cuuint32_t steps[5] = {1, 1, 1, 1, 1};
        if (api.tiled(reinterpret_cast<CUtensorMap*>(p.tmap_b), dt, 5, const_cast<char*>(base), dims, strides, box, steps,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    p.tma_base_h = base_h;
    p.tma_base_w = base_w;
    p.use_tma = 1;
    return true;
}

}  // namespace ob200

static std::atomic<long long> g_tma_launches{0};

extern "C" long long ob200_tma_launch_count(void) { return g_tma_launches.load(std::memory_order_relaxed); }

extern "C" int ob200_igemm_launch(const IgemmParams* params, int bn, int num_ctas, void* stream) {
    using namespace ob200;
    IgemmParams p = *params;
    if (bn != 64 && bn != 128 && !(bn == 256 && p.dtype != 0)) return -1;
    static const bool a_tmem_off = [] {   // ORION_A_TMEM=0: activation parts through shared memory (for measurements)
        const char* e = getenv("ORION_A_TMEM");
        return e && e[0] == '0';
    }();
    p.a_in_tmem = (p.dtype == 0 && p.mode == 0 && !a_tmem_off) ? 1 : 0;
    {   // Cross-term accumulator where no CTA of a whole-device launch computes more than two pieces (see
        // IgemmParams::cross_acc); decided from the problem and the device, not from this call's CTA count, so that the
        // arithmetic does not change with the SM quota.  ORION_CROSS_ACC=0/1 pins it.
        static const int device_sms = [] {
            int dev = 0, v = 0;
            if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
            return v;
        }();
        static const char force = [] {
            const char* e = getenv("ORION_CROSS_ACC");
            return e ? e[0] : '\0';
        }();
        const long long units = (long long)p.tiles_m * p.tiles_n * (p.splits > 1 ? p.splits : 1) * (p.batch > 1 ? p.batch : 1);
        p.cross_acc = (p.a_in_tmem && (force == '1' || (force != '0' && !p.stream_k && units <= 2LL * device_sms))) ? 1 : 0;
    }
    if (setup_tma(p, bn)) g_tma_launches.fetch_add(1, std::memory_order_relaxed);
    else if (p.require_tma || p.w_R > 0) return -4;   // tap subsets exist only on the TMA path
    {   // class of this launch for the scheduler's profiles: arithmetic intensity of the problem against the device's
        const double batch = p.batch > 1 ? p.batch : 1;
        const double elem = p.dtype == 1 ? 2.0 : 4.0;
        const double flop = 2.0 * p.M * (double)p.Kout * p.C * p.R * p.S * batch;
        const double bytes = p.mode == 1 ? ((double)p.M * p.Kout + (double)p.Nb * p.H * p.W * p.C) * elem + (double)p.Kout * p.R * p.S * p.C * 4.0
                                         : ((double)p.Nb * p.IH * p.IW * p.C + (double)p.Kout * p.R * p.S * p.C + (double)p.M * p.Kout) * elem * batch;
        annotate_launch(flop >= ai_threshold(p.dtype) * bytes ? 1 : 0, flop, bytes);
    }
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (p.dtype == 0) {
        if (p.a_in_tmem) return (int)(bn == 64 ? launch_cfg<float, 64, 3, true>(p, num_ctas, s) : launch_cfg<float, 128, 3, true>(p, num_ctas, s));
        return (int)(bn == 64 ? launch_cfg<float, 64, 3>(p, num_ctas, s) : launch_cfg<float, 128, 3>(p, num_ctas, s));
    } else if (p.dtype == 1) {
        // 128 x 256 tiles (single-pass modes only: 3xTF32 needs the tensor-memory columns for the activation parts)
        if (bn == 256) return p.mode == 0 ? (int)launch_cfg<__nv_bfloat16, 256, 1>(p, num_ctas, s) : -1;
        return (int)(bn == 64 ? launch_cfg<__nv_bfloat16, 64, 1>(p, num_ctas, s) : launch_cfg<__nv_bfloat16, 128, 1>(p, num_ctas, s));
    } else if (p.dtype == 2) {   // float32 data, one TF32 pass (the precision cuDNN uses by default on tensor cores)
        if (bn == 256) return p.mode == 0 ? (int)launch_cfg<float, 256, 1>(p, num_ctas, s) : -1;
        return (int)(bn == 64 ? launch_cfg<float, 64, 1>(p, num_ctas, s) : launch_cfg<float, 128, 1>(p, num_ctas, s));
    }
    return -1;
}
