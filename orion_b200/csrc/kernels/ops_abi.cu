// C-ABI front of the tensor-core kernels: argument checks, tile / split-K choice,
// per-stream scratch, and the device status word.  Declarations and the reference
// call each entry point replaces are in include/orion_kernels.h.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "igemm_params.h"

namespace {

struct Scratch {
    int* counters = nullptr;     // arrival counters: zero between launches
    float* slabs = nullptr;      // partial tiles of cut tiles (split-K: one per unit; stream-K: two per CTA); contents
                                 // arbitrary between launches
    size_t slab_bytes = 0;
};
constexpr size_t kSlabBytes = 40u << 20;                // 128 x 128 float slabs for up to 640 pieces
constexpr int kMaxTilesSplit = 4096;                    // counters per stream

std::mutex g_mu;
std::unordered_map<uint64_t, Scratch> g_scratch;        // key: device << 56 ^ stream
std::unordered_map<int, int*> g_status;                 // per device

long long* g_debug = nullptr;   // optional role-wait counters, see ob200_set_debug_buffer

int* status_word(int dev) {
    thread_local int cached_dev = -1;
    thread_local int* cached = nullptr;
    if (dev == cached_dev && cached) return cached;
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_status.find(dev);
    if (it != g_status.end()) {
        cached_dev = dev;
        cached = it->second;
        return cached;
    }
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(int));
    g_status[dev] = p;
    return p;
}

// Split-K scratch is private to a stream: two clients that run split-K convolutions
// at the same time on different streams must not share partial sums.
Scratch* scratch_for(int dev, cudaStream_t s) {
    uint64_t key = ((uint64_t)dev << 56) ^ (uint64_t)(uintptr_t)s;
    thread_local uint64_t cached_key = ~0ull;
    thread_local Scratch* cached = nullptr;
    if (key == cached_key && cached) return cached;   // entries are never erased; unordered_map nodes do not move
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_scratch.find(key);
    if (it != g_scratch.end()) {
        cached_key = key;
        cached = &it->second;
        return cached;
    }
    Scratch sc;
    if (cudaMalloc(&sc.counters, kMaxTilesSplit * sizeof(int)) != cudaSuccess) return nullptr;
    if (cudaMalloc(&sc.slabs, kSlabBytes) != cudaSuccess) return nullptr;
    sc.slab_bytes = kSlabBytes;
    cudaMemsetAsync(sc.counters, 0, kMaxTilesSplit * sizeof(int), s);
    g_scratch[key] = sc;
    return &g_scratch[key];
}

}  // namespace

// Number of SMs the schedule of a problem is planned for.  The plan (tile width, split-K factor, stream-K or not)
// depends on the device alone, never on the SM quota of the call: the quota only sets how many CTAs walk the
// planned work units, so a split-K result is bit-identical for every quota (the scheduler may cut a launch to
// its granted quota at the last moment).
static int plan_sm_count() {
    static const int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
            v = 148;
        return v;
    }();
    return n;
}

// For the other translation units of the library: the planning SM count and the calling stream's scratch for partial
// sums (contents arbitrary between launches; launches of one stream use it one after the other).
extern "C" int ob200_plan_sm_count(void) { return plan_sm_count(); }
extern "C" float* ob200_stream_slabs(void* stream, size_t* bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    Scratch* sc = scratch_for(dev, (cudaStream_t)stream);
    if (!sc) return nullptr;
    if (bytes) *bytes = sc->slab_bytes;
    return sc->slabs;
}

// Device status word of the current device, for the other translation units of the library.
extern "C" int* ob200_status_word_for_current_device(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    return status_word(dev);
}

extern "C" int ob200_plan_conv(int dtype, long long M, int Kout, int R, int S, int C, int num_ctas, int* bn_out, int* splits_out) {
    const int bk = dtype == 1 ? 64 : 32;
    const int kblocks = R * ((S * C + bk - 1) / bk);
    const int tiles_m = (int)((M + 127) / 128);
    int bn = 128;
    const int rem = Kout % 128;
    if (Kout <= 64 || (rem > 0 && rem <= 64 && Kout < 256)) bn = 64;
    // Narrow tiles only while wide ones would leave more than half of the CTAs idle: a wide tile
    // re-reads and re-splits the activation operand half as often, which outweighs a partial wave.
    if ((long long)tiles_m * ((Kout + 127) / 128) * 2 <= num_ctas && Kout >= 128) bn = 64;
    const int tiles = tiles_m * ((Kout + bn - 1) / bn);
    int splits = 1;
    if (tiles * 2 <= num_ctas && kblocks >= 4) {
        splits = num_ctas / tiles;
        if (splits > kblocks / 4) splits = kblocks / 4;   // chains of at least four k-blocks
        if (splits > 16) splits = 16;
        if (splits < 1) splits = 1;
    }
    *bn_out = bn;
    *splits_out = splits;
    return 0;
}

namespace {

// Tile width when the schedule balances the load by itself (stream-K): wide tiles halve the re-reads of
// the activation operand; narrow ones only where the output is narrow or its last wide tile would be
// mostly padding.
int streamk_bn(int Kout) {
    const int rem = Kout % 128;
    return (Kout <= 64 || (rem > 0 && rem <= 64 && Kout < 256)) ? 64 : 128;
}

// Single-pass modes (bf16, one TF32 pass) are bound by L2->SM operand traffic at 128 x 128; a 128 x 256 tile moves a
// quarter less per FLOP.  Taken when the output is wide enough and the wide tiles still fill the granted SMs.
bool wide_tiles_pay(int dtype, long long M, int Kout, int num_ctas) {
    if (dtype == 0 || Kout < 256 || (Kout % 256 != 0 && Kout % 256 <= 128)) return false;
    static const bool off = [] {
        const char* e = getenv("ORION_WIDE_TILES");
        return e && e[0] == '0';
    }();
    if (off) return false;
    return ((M + 127) / 128) * ((Kout + 255) / 256) >= num_ctas;
}

// Whether stream-K beats one unit per tile, in units of one k-block of MMA work per CTA: a tile costs its
// k-blocks plus about four for the epilogue; stream-K gives every CTA an equal share of all k-blocks but
// pays about twelve for writing and re-reading the two tiles a CTA shares with its neighbours.  It wins
// where the tiles are deep and the last wave would be partly empty (3x3 layers at moderate batch), and
// loses on shallow 1x1 layers and where a tile would be cut into many pieces.
bool stream_k_pays(long long tiles, int num_kblocks, int num_ctas) {
    static const char force = [] {   // ORION_SCHEDULE=streamk / tiles pins the schedule (for measurements); read once
        const char* e = getenv("ORION_SCHEDULE");
        return e ? e[0] : '\0';
    }();
    if (force == 's') return true;
    if (force == 't') return false;
    if (tiles * 4 < num_ctas || num_kblocks < 8) return false;
    const double waves = (double)((tiles + num_ctas - 1) / num_ctas);
    const double tiles_cost = waves * (num_kblocks + 4);
    const double sk_cost = (double)tiles * num_kblocks / num_ctas + 4 + 12;
    return sk_cost < 0.9 * tiles_cost;
}

// Puts a mode-0 launch on the stream-K schedule if it pays and the stream's scratch has two slabs per CTA;
// returns the grid, or 0 to keep the caller's schedule.
int schedule_stream_k(IgemmParams& p, int bn, int num_ctas, int dev, cudaStream_t stream) {
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    if (!stream_k_pays(tiles, p.num_kblocks, plan_sm_count())) return 0;
    const long long work = tiles * p.num_kblocks;
    long long grid = work / 4;
    if (grid > num_ctas) grid = num_ctas;
    if (grid < 1) grid = 1;
    Scratch* sc = grid > 1 ? scratch_for(dev, stream) : nullptr;
    if (grid > 1 && (!sc || grid > kMaxTilesSplit || (size_t)grid * 2 * 128 * bn * sizeof(float) > sc->slab_bytes)) return 0;
    p.stream_k = 1;
    p.splits = 1;
    if (sc) {
        p.slabs = sc->slabs;
        p.counters = sc->counters;
    }
    return (int)grid;
}

}  // namespace

// The schedule ob200_conv2d_fprop picks for a problem (host logic only, no launch): tile width, split-K factor
// and whether the stream-K schedule is used (then splits = 1 and the tile width is the wide-tile preference).
extern "C" int ob200_plan_schedule(int dtype, long long M, int Kout, int R, int S, int C, int num_ctas, int* bn_out, int* splits_out,
                                   int* stream_k_out) {
    if (M <= 0 || Kout <= 0 || R <= 0 || S <= 0 || C <= 0 || num_ctas <= 0 || !bn_out || !splits_out || !stream_k_out) return -1;
    const int bk = dtype == 1 ? 64 : 32;
    const int bn = streamk_bn(Kout);
    const long long tiles = ((M + 127) / 128) * ((Kout + bn - 1) / bn);
    if (stream_k_pays(tiles, R * ((S * C + bk - 1) / bk), num_ctas)) {
        *bn_out = bn;
        *splits_out = 1;
        *stream_k_out = 1;
        return 0;
    }
    *stream_k_out = 0;
    return ob200_plan_conv(dtype, M, Kout, R, S, C, num_ctas, bn_out, splits_out);
}

namespace {

int fprop_impl(const void* x, const void* w, void* y, const float* scale, const float* shift, const void* residual, int relu,
               int dtype, int Nb, int H, int W, int C, int Kout, int R, int S, int stride_h, int stride_w, int pad_h, int pad_w,
               int dil_h, int dil_w, int bn, int splits, bool stream_k, float* scratch, int* counters, int num_ctas, void* stream) {
    if (dtype < 0 || dtype > 2) return -1;
    if (Nb < 0 || H <= 0 || W <= 0 || C <= 0 || Kout <= 0 || R <= 0 || S <= 0 || stride_h <= 0 || stride_w <= 0 || dil_h <= 0 ||
        dil_w <= 0 || pad_h < 0 || pad_w < 0 || num_ctas <= 0)
        return -1;
    if (Nb == 0) return 0;
    const int P = (H + 2 * pad_h - dil_h * (R - 1) - 1) / stride_h + 1;
    const int Q = (W + 2 * pad_w - dil_w * (S - 1) - 1) / stride_w + 1;
    if (P <= 0 || Q <= 0) return -1;
    const int elem = dtype == 1 ? 2 : 4;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y | (uintptr_t)residual) % 16) return -2;   // 128-bit accesses
    int dev = 0;
    cudaGetDevice(&dev);
    IgemmParams p;
    memset(&p, 0, sizeof p);
    p.x = x; p.w = w; p.y = y; p.scale = scale; p.shift = shift; p.residual = residual;
    p.relu = relu; p.dtype = dtype;
    p.Nb = Nb; p.H = H; p.W = W; p.C = C; p.Kout = Kout; p.R = R; p.S = S; p.P = P; p.Q = Q;
    p.stride_h = stride_h; p.stride_w = stride_w; p.pad_h = pad_h; p.pad_w = pad_w; p.dil_h = dil_h; p.dil_w = dil_w;
    const long long M = (long long)Nb * P * Q;
    if (M > 0x7fffffffLL) return -1;
    p.M = (int)M;
    const int bk = 128 / elem;
    p.kblocks_per_r = (S * C + bk - 1) / bk;
    p.num_kblocks = R * p.kblocks_per_r;
    if (bn != 64 && bn != 128 && !(bn == 256 && dtype != 0)) return -1;
    p.tiles_m = (int)((M + 127) / 128);
    p.tiles_n = (Kout + bn - 1) / bn;
    if (splits < 1 || splits > p.num_kblocks) return -1;
    p.splits = splits;
    igemm_set_fprop(&p);
    p.status = status_word(dev);
    p.debug = g_debug;
    if (stream_k) {
        const int grid = schedule_stream_k(p, bn, num_ctas, dev, (cudaStream_t)stream);
        if (grid > 0) return ob200_igemm_launch(&p, bn, grid, stream);
    }
    if (splits > 1) {
        if (!scratch || !counters) return -1;
        p.slabs = scratch;      // one 128 x bn slab per (tile, split)
        p.counters = counters;
    }
    const int units = p.tiles_m * p.tiles_n * splits;
    const int grid = units < num_ctas ? units : num_ctas;
    return ob200_igemm_launch(&p, bn, grid, stream);
}

}  // namespace

extern "C" int ob200_conv2d_fprop_ex(const void* x, const void* w, void* y, const float* scale, const float* shift,
                                     const void* residual, int relu, int dtype, int Nb, int H, int W, int C, int Kout, int R,
                                     int S, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int bn,
                                     int splits, float* scratch, int* counters, int num_ctas, void* stream) {
    return fprop_impl(x, w, y, scale, shift, residual, relu, dtype, Nb, H, W, C, Kout, R, S, stride_h, stride_w, pad_h, pad_w, dil_h,
                      dil_w, bn, splits, false, scratch, counters, num_ctas, stream);
}

extern "C" int ob200_conv2d_fprop(const void* x, const void* w, void* y, const float* scale, const float* shift,
                                  const void* residual, int relu, int dtype, int Nb, int H, int W, int C, int Kout, int R, int S,
                                  int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int num_ctas,
                                  void* stream) {
    if (Nb <= 0 || H <= 0 || W <= 0) return Nb == 0 ? 0 : -1;
    if (num_ctas <= 0) return -1;
    const int P = (H + 2 * pad_h - dil_h * (R - 1) - 1) / (stride_h > 0 ? stride_h : 1) + 1;
    const int Q = (W + 2 * pad_w - dil_w * (S - 1) - 1) / (stride_w > 0 ? stride_w : 1) + 1;
    const long long M = (long long)Nb * P * Q;
    const int plan_ctas = plan_sm_count();
    if (wide_tiles_pay(dtype, M, Kout, plan_ctas))
        return fprop_impl(x, w, y, scale, shift, residual, relu, dtype, Nb, H, W, C, Kout, R, S, stride_h, stride_w, pad_h, pad_w, dil_h,
                          dil_w, 256, 1, true, nullptr, nullptr, num_ctas, stream);
    {   // stream-K with the tile width it prefers, where it pays
        const int bn = streamk_bn(Kout);
        const int bk = dtype == 1 ? 64 : 32;
        const long long tiles = ((M + 127) / 128) * ((Kout + bn - 1) / bn);
        if (stream_k_pays(tiles, R * ((S * C + bk - 1) / bk), plan_ctas))
            return fprop_impl(x, w, y, scale, shift, residual, relu, dtype, Nb, H, W, C, Kout, R, S, stride_h, stride_w, pad_h, pad_w,
                              dil_h, dil_w, bn, 1, true, nullptr, nullptr, num_ctas, stream);
    }
    // otherwise one unit per tile, or split-K where the tiles are few
    int bn = 128, splits = 1;
    ob200_plan_conv(dtype, M, Kout, R, S, C, plan_ctas, &bn, &splits);
    float* scratch = nullptr;
    int* counters = nullptr;
    if (splits > 1) {
        int dev = 0;
        cudaGetDevice(&dev);
        const long long tiles = ((M + 127) / 128) * ((Kout + bn - 1) / bn);
        Scratch* sc = scratch_for(dev, (cudaStream_t)stream);
        if (!sc || tiles > kMaxTilesSplit || (size_t)tiles * splits * 128 * bn * sizeof(float) > sc->slab_bytes) {
            splits = 1;
        } else {
            scratch = sc->slabs;
            counters = sc->counters;
        }
    }
    return fprop_impl(x, w, y, scale, shift, residual, relu, dtype, Nb, H, W, C, Kout, R, S, stride_h, stride_w, pad_h, pad_w, dil_h,
                      dil_w, bn, splits, false, scratch, counters, num_ctas, stream);
}

// Data gradient of the convolution: dx[n,h,w,c] = sum_{r,s,k} dy[n,(h+pad-r*dil)/stride,(w+pad-s*dil)/stride,k] * w[k,r,s,c]
// over the taps whose division is exact.  wt is the filter re-laid out as [C, R, S, Kout]
// (ob200_filter_transpose).  Same kernel as the forward pass, with the gather geometry of
// Strided data gradient as one dense problem per parity class of the input pixel.  Input pixel
// h = a + stride*i receives only from taps r = r0 + stride*t with r0 = (a + pad) mod stride, and reads
// dy row i + (a + pad - r0)/stride - t: a unit-stride gather over that class's pixels and taps, with
// no multiplications by structural zeros (a stride-2 gradient spends a quarter of the dense work).
// Classes without taps (1x1 filters) keep the zeros of the initial clear.  Returns -4 when a class
// cannot be fed by TMA (the caller then runs the single dense launch).
static int dgrad_by_parity_class(const void* dy, const void* wt, void* dx, int dtype, int Nb, int H, int W, int C, int Kout,
                                 int R, int S, int stride_h, int stride_w, int pad_h, int pad_w, int P, int Q, int num_ctas,
                                 void* stream, int dev) {
    const int elem = dtype == 1 ? 2 : 4;
    const int bk = 128 / elem;
    if (Kout % bk != 0) return -4;
    cudaStream_t st = (cudaStream_t)stream;
    if (R < stride_h || S < stride_w)
        if (cudaMemsetAsync(dx, 0, (size_t)Nb * H * W * C * elem, st) != cudaSuccess) return -1;
    for (int a = 0; a < stride_h && a < H; a++) {
        for (int b = 0; b < stride_w && b < W; b++) {
            const int Hc = (H - a + stride_h - 1) / stride_h, Wc = (W - b + stride_w - 1) / stride_w;
            const int r0 = (a + pad_h) % stride_h, s0 = (b + pad_w) % stride_w;
            const int Rc = r0 < R ? (R - r0 + stride_h - 1) / stride_h : 0;
            const int Sc = s0 < S ? (S - s0 + stride_w - 1) / stride_w : 0;
            if (Rc == 0 || Sc == 0) {
                if (!(R < stride_h || S < stride_w)) return -1;   // unreachable: an empty class implies the clear above
                continue;
            }
            const long long M = (long long)Nb * Hc * Wc;
            const int bn = streamk_bn(C);
            IgemmParams p;
            memset(&p, 0, sizeof p);
            p.x = dy; p.w = wt; p.y = dx;
            p.dtype = dtype;
            p.Nb = Nb; p.H = H; p.W = W; p.P = P; p.Q = Q; p.R = Rc; p.S = Sc;
            p.C = Kout; p.Kout = C;
            p.stride_h = stride_h; p.stride_w = stride_w; p.pad_h = pad_h; p.pad_w = pad_w; p.dil_h = p.dil_w = 1;
            p.M = (int)M;
            p.kblocks_per_r = (Sc * Kout + bk - 1) / bk;
            p.num_kblocks = Rc * p.kblocks_per_r;
            p.tiles_m = (int)((M + 127) / 128);
            p.tiles_n = (C + bn - 1) / bn;
            p.status = status_word(dev);
            p.debug = g_debug;
            p.splits = 1;
            p.OH = Hc; p.OW = Wc; p.IH = P; p.IW = Q;
            p.bmul_h = p.bmul_w = 1;
            p.badd_h = (a + pad_h - r0) / stride_h; p.badd_w = (b + pad_w - s0) / stride_w;
            p.step_h = p.step_w = -1;
            p.div_h = p.div_w = 1;
            p.w_R = R; p.w_S = S; p.w_r0 = r0; p.w_s0 = s0; p.w_rstep = stride_h; p.w_sstep = stride_w;
            p.out_map = 1; p.out_H = H; p.out_W = W;
            p.out_mul_h = stride_h; p.out_mul_w = stride_w; p.out_add_h = a; p.out_add_w = b;
            p.require_tma = 1;
            int grid = schedule_stream_k(p, bn, num_ctas, dev, st);
            if (grid <= 0) {
                const long long units = (long long)p.tiles_m * p.tiles_n;
                grid = units < num_ctas ? (int)units : num_ctas;
            }
            const int rc = ob200_igemm_launch(&p, bn, grid, stream);
            if (rc != 0) return rc;
        }
    }
    return 0;
}

// igemm_set_dgrad: GEMM rows are input pixels, the reduction runs over (r, s, k).
extern "C" int ob200_conv2d_dgrad(const void* dy, const void* wt, void* dx, int dtype, int Nb, int H, int W, int C, int Kout, int R,
                                  int S, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int num_ctas,
                                  void* stream) {
    if (dtype < 0 || dtype > 2) return -1;
    if (Nb < 0 || H <= 0 || W <= 0 || C <= 0 || Kout <= 0 || R <= 0 || S <= 0 || stride_h <= 0 || stride_w <= 0 || dil_h <= 0 ||
        dil_w <= 0 || pad_h < 0 || pad_w < 0 || num_ctas <= 0)
        return -1;
    if (Nb == 0) return 0;
    const int P = (H + 2 * pad_h - dil_h * (R - 1) - 1) / stride_h + 1;
    const int Q = (W + 2 * pad_w - dil_w * (S - 1) - 1) / stride_w + 1;
    if (P <= 0 || Q <= 0) return -1;
    if (((uintptr_t)dy | (uintptr_t)wt | (uintptr_t)dx) % 16) return -2;
    const long long M = (long long)Nb * H * W;
    if (M > 0x7fffffffLL) return -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if ((stride_h > 1 || stride_w > 1) && dil_h == 1 && dil_w == 1) {
        const int rc = dgrad_by_parity_class(dy, wt, dx, dtype, Nb, H, W, C, Kout, R, S, stride_h, stride_w, pad_h, pad_w, P, Q,
                                             num_ctas, stream, dev);
        if (rc != -4) return rc;
    }
    const int bn = streamk_bn(C);
    IgemmParams p;
    memset(&p, 0, sizeof p);
    p.x = dy; p.w = wt; p.y = dx;
    p.dtype = dtype;
    p.Nb = Nb; p.H = H; p.W = W; p.P = P; p.Q = Q; p.R = R; p.S = S;
    p.C = Kout;      // reduction channels: those of dy
    p.Kout = C;      // GEMM columns: the channels of dx
    p.stride_h = stride_h; p.stride_w = stride_w; p.pad_h = pad_h; p.pad_w = pad_w; p.dil_h = dil_h; p.dil_w = dil_w;
    p.M = (int)M;
    const int bk = dtype == 1 ? 64 : 32;
    p.kblocks_per_r = (S * Kout + bk - 1) / bk;
    p.num_kblocks = R * p.kblocks_per_r;
    p.tiles_m = (int)((M + 127) / 128);
    p.tiles_n = (C + bn - 1) / bn;
    p.status = status_word(dev);
    p.debug = g_debug;
    p.splits = 1;
    igemm_set_dgrad(&p, H, W, P, Q);
    int grid = schedule_stream_k(p, bn, num_ctas, dev, (cudaStream_t)stream);
    if (grid <= 0) {
        const long long units = (long long)p.tiles_m * p.tiles_n;
        grid = units < num_ctas ? (int)units : num_ctas;
    }
    return ob200_igemm_launch(&p, bn, grid, stream);
}

// Filter gradient of the convolution: dw[k,r,s,c] = sum_{n,p,q} dy[n,p,q,k] * x[n, p*stride-pad+r*dil, q*stride-pad+s*dil, c].
// float32 only (dtype 0: 3xTF32, 2: one TF32 pass); C and Kout multiples of 4.  The reduction over the
// N*P*Q pixels is split across CTAs and summed with atomic adds, so dw is cleared on `stream` first.
extern "C" int ob200_conv2d_wgrad(const void* x, const void* dy, float* dw, int dtype, int Nb, int H, int W, int C, int Kout, int R,
                                  int S, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int num_ctas,
                                  void* stream) {
    if (dtype != 0 && dtype != 2) return -1;
    if (Nb < 0 || H <= 0 || W <= 0 || C <= 0 || Kout <= 0 || R <= 0 || S <= 0 || stride_h <= 0 || stride_w <= 0 || dil_h <= 0 ||
        dil_w <= 0 || pad_h < 0 || pad_w < 0 || num_ctas <= 0 || (C & 3) || (Kout & 3))
        return -1;
    const int P = (H + 2 * pad_h - dil_h * (R - 1) - 1) / stride_h + 1;
    const int Q = (W + 2 * pad_w - dil_w * (S - 1) - 1) / stride_w + 1;
    if (P <= 0 || Q <= 0) return -1;
    if (((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dw) % 16) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t dw_bytes = (size_t)Kout * R * S * C * sizeof(float);
    if (Nb == 0) return (int)cudaMemsetAsync(dw, 0, dw_bytes, s);
    const long long Mpix = (long long)Nb * P * Q;
    if (Mpix > 0x7fffffffLL) return -1;
    int dev = 0;
    cudaGetDevice(&dev);
    IgemmParams p;
    memset(&p, 0, sizeof p);
    p.mode = 1;
    p.x = dy; p.w = x; p.y = dw;
    p.dtype = dtype;
    p.Nb = Nb; p.H = H; p.W = W; p.C = C; p.Kout = Kout; p.R = R; p.S = S; p.P = P; p.Q = Q;
    p.stride_h = stride_h; p.stride_w = stride_w; p.pad_h = pad_h; p.pad_w = pad_w; p.dil_h = dil_h; p.dil_w = dil_w;
    p.M = (int)Mpix;
    // Few input channels and several taps: a 128-column tile covers 128 / roundup(C, 32) consecutive taps, so dy is
    // read once per group of taps (TMA-fed launches only; `multi_tap` falls back below if TMA is not available).
    const bool multi_tap = C >= 32 && C <= 64 && R * S > 1;
    const int bn = (C > 64 || multi_tap) ? 128 : 64;
    p.ctiles = (C + bn - 1) / bn;
    p.tiles_m = (Kout + 127) / 128;
    p.tiles_n = R * S * p.ctiles;
    if (multi_tap) {
        p.wg_cr = (C + 31) / 32 * 32;
        p.wg_tpt = 128 / p.wg_cr;
        p.ctiles = 1;
        p.tiles_n = (R * S + p.wg_tpt - 1) / p.wg_tpt;
        p.require_tma = 1;
    }
    p.kblocks_per_r = (int)((Mpix + 31) / 32);
    p.num_kblocks = p.kblocks_per_r;
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    long long splits = (2LL * num_ctas + tiles - 1) / tiles;       // about two units per granted SM
    if (splits > p.num_kblocks / 2) splits = p.num_kblocks / 2;    // at least two k-blocks per unit
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    p.splits = (int)splits;
    p.status = status_word(dev);
    p.debug = g_debug;
    igemm_set_fprop(&p);
    if (p.splits > 1) {
        cudaError_t e = cudaMemsetAsync(dw, 0, dw_bytes, s);
        if (e != cudaSuccess) return (int)e;
    }
    const long long units = tiles * p.splits;
    const int grid = units < num_ctas ? (int)units : num_ctas;
    const int rc = ob200_igemm_launch(&p, bn, grid, stream);
    if (rc == -4 && multi_tap) {   // no TMA for this problem: one tap per 64-column tile through the gathering producers
        p.wg_tpt = p.wg_cr = p.require_tma = 0;
        p.ctiles = 1;
        p.tiles_n = R * S;
        const long long tiles1 = (long long)p.tiles_m * p.tiles_n;
        long long sp = (2LL * num_ctas + tiles1 - 1) / tiles1;
        if (sp > p.num_kblocks / 2) sp = p.num_kblocks / 2;
        if (sp > 64) sp = 64;
        if (sp < 1) sp = 1;
        p.splits = (int)sp;
        if (p.splits > 1 && cudaMemsetAsync(dw, 0, dw_bytes, s) != cudaSuccess) return -1;
        const long long units1 = tiles1 * p.splits;
        return ob200_igemm_launch(&p, 64, units1 < num_ctas ? (int)units1 : num_ctas, stream);
    }
    return rc;
}

// y[M, N] = x[M, K] . w[N, K]^T (+ bias) (+ ReLU): a 1x1 convolution over M "pixels".
extern "C" int ob200_linear(const void* x, const void* w, void* y, const float* bias, int relu, int dtype, int M, int N, int K,
                            int num_ctas, void* stream) {
    if (M == 0) return 0;
    return ob200_conv2d_fprop(x, w, y, nullptr, bias, nullptr, relu, dtype, M, 1, 1, K, N, 1, 1, 1, 1, 0, 0, 1, 1, num_ctas, stream);
}

// `batch` independent GEMMs of one shape: y_b[M, N] = x_b[M, K] . w_b[N, K]^T, operands `stride_*` elements
// apart.  Takes the place of cublasSgemmStridedBatched (attention scores and context products).
extern "C" int ob200_linear_batched(const void* x, const void* w, void* y, int dtype, int batch, int M, int N, int K,
                                    long long stride_x, long long stride_w, long long stride_y, int num_ctas, void* stream) {
    if (dtype < 0 || dtype > 2 || batch < 0 || M < 0 || N <= 0 || K <= 0 || num_ctas <= 0) return -1;
    if (batch == 0 || M == 0) return 0;
    const int elem = dtype == 1 ? 2 : 4;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) % 16) return -2;
    if ((stride_x * elem) % 16 || (stride_w * elem) % 16 || (stride_y * elem) % 16) return -2;
    int dev = 0;
    cudaGetDevice(&dev);
    IgemmParams p;
    memset(&p, 0, sizeof p);
    p.x = x; p.w = w; p.y = y;
    p.dtype = dtype;
    p.Nb = M; p.H = p.W = p.P = p.Q = p.R = p.S = 1;
    p.C = K; p.Kout = N;
    p.stride_h = p.stride_w = p.dil_h = p.dil_w = 1;
    p.M = M;
    const int bk = 128 / elem;
    p.kblocks_per_r = (K + bk - 1) / bk;
    p.num_kblocks = p.kblocks_per_r;
    const int bn = N <= 64 ? 64 : wide_tiles_pay(dtype, (long long)M * batch, N, num_ctas) ? 256 : 128;
    p.tiles_m = (M + 127) / 128;
    p.tiles_n = (N + bn - 1) / bn;
    p.splits = 1;
    p.status = status_word(dev);
    p.debug = g_debug;
    p.batch = batch;
    p.batch_stride_x = stride_x; p.batch_stride_w = stride_w; p.batch_stride_y = stride_y;
    igemm_set_fprop(&p);
    const long long units = (long long)p.tiles_m * p.tiles_n * batch;
    if (units > 0x7fffffffLL) return -1;
    const int grid = units < num_ctas ? (int)units : num_ctas;
    return ob200_igemm_launch(&p, bn, grid, stream);
}

// Reads and clears the device status word of the current device (synchronises the
// device).  0 = no kernel reported a timed-out wait since the last call.
extern "C" int ob200_read_status(void) {
    int dev = 0;
    cudaGetDevice(&dev);
    int* p = status_word(dev);
    if (!p) return -1;
    int v = 0;
    if (cudaMemcpy(&v, p, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) {
        cudaMemset(p, 0, sizeof v);
        // A kernel that gave up a wait left early: the arrival counters of its stream's split-K scratch may not be back
        // at zero, and a later split-K launch would count from there.  The copy above drained the device; clear them all.
        std::lock_guard<std::mutex> lk(g_mu);
        for (auto& kv : g_scratch)
            if ((int)(kv.first >> 56) == dev && kv.second.counters) cudaMemset(kv.second.counters, 0, kMaxTilesSplit * sizeof(int));
    }
    return v;
}

// Tuning aid: device buffer of 8 long longs that receives, from CTA 0 of every implicit-GEMM launch,
// the cycles each warp role spent waiting: [0] epilogue, [1] MMA on operands, [2] MMA on a free
// accumulator, [3] splitter, [4] producer, [5] whole kernel.  NULL switches it off.
extern "C" void ob200_set_debug_buffer(long long* dev_buf) { g_debug = dev_buf; }

extern "C" int ob200_sm_count(void) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    return n;
}
