// Split-K convolution for callers that must not allocate device memory.
//
// ob200_conv2d_fprop and ob200_conv2d_fprop_ex get their split-K scratch either from a
// cudaMalloc made on first use or from the caller.  Some callers can do neither: code
// that runs while a stream is being captured, code inside a memory-pool callback or a
// framework hook where allocating would re-enter the allocator, and embedders whose
// device memory is carved up front and who forbid any later cudaMalloc.  For them this
// file offers one more entry point whose scratch is a fixed array compiled into the
// library.  It calls no cudaMalloc, no cudaFree and no allocating library routine.
//
// Cost and limits:
//   * the array (kScratchFloats floats + kCounterInts ints, 8 MiB + 1 KiB) is part of
//     the module image, so every GPU that loads the library holds it until exit;
//   * a problem whose split-K partial tiles (tiles * splits * 128 * bn floats) or tile
//     count do not fit is rejected with OB200_ERR_STATIC_SCRATCH_TOO_SMALL (-3);
//   * all calls share the one array.  It keeps whatever the previous call left: the
//     partial tiles need no particular start value (every unit overwrites its own),
//     the tile counters must start at zero and are cleared on the call's stream before
//     its kernel runs; two calls that overlap on the GPU (different streams, no
//     ordering) race on the array;
//   * the first call on each device looks up the array's device address (a set-up step
//     that is not a stream operation): make that first call before any stream capture.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "igemm_params.h"

namespace {

constexpr size_t kScratchFloats = 2u * 1024 * 1024;   // 8 MiB of split-K partial tiles
constexpr int kCounterInts = 256;                     // one arrival counter per output tile
constexpr int kMaxDevices = 64;

struct StaticScratch {
    float partial[kScratchFloats];
    int counters[kCounterInts];
    int status;   // receives the code of a bounded wait that expired inside a kernel launched from here (0: none)
};

// Device-resident.  In host code this name is only a handle for the runtime's symbol
// calls — it is NOT a device address and must never be handed to a kernel; the address
// comes from cudaGetSymbolAddress below, once per device.
static __device__ __align__(256) StaticScratch g_static_scratch;

StaticScratch* g_dev_ptr[kMaxDevices];   // device address of the array, per device

// Look the array up on the current device (idempotent; no allocation, no stream work).
int scratch_for_current_device(StaticScratch** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return -1;
    if (!g_dev_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);   // resolves the symbol in the CURRENT device's module
        if (e != cudaSuccess) return (int)e;
        if (!p) return -1;
        g_dev_ptr[dev] = static_cast<StaticScratch*>(p);
    }
    *out = g_dev_ptr[dev];
    return 0;
}

}  // namespace

// Same arguments and result as ob200_conv2d_fprop_ex without the scratch pointers.
// Returns 0, a cudaError_t (> 0), -1/-2 for invalid arguments / misaligned pointers, or
// -3 when the split-K scratch of this problem exceeds the built-in array.
extern "C" int ob200_conv2d_fprop_noalloc(const void* x, const void* w, void* y, const float* scale, const float* shift,
                                          const void* residual, int relu, int dtype, int Nb, int H, int W, int C, int Kout, int R,
                                          int S, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int bn,
                                          int splits, int num_ctas, void* stream) {
    if (dtype < 0 || dtype > 2) return -1;
    if (Nb < 0 || H <= 0 || W <= 0 || C <= 0 || Kout <= 0 || R <= 0 || S <= 0 || stride_h <= 0 || stride_w <= 0 || dil_h <= 0 ||
        dil_w <= 0 || pad_h < 0 || pad_w < 0 || num_ctas <= 0 || (bn != 64 && bn != 128))
        return -1;
    if (Nb == 0) return 0;
    const int P = (H + 2 * pad_h - dil_h * (R - 1) - 1) / stride_h + 1;
    const int Q = (W + 2 * pad_w - dil_w * (S - 1) - 1) / stride_w + 1;
    if (P <= 0 || Q <= 0) return -1;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y | (uintptr_t)residual) % 16) return -2;
    const long long M = (long long)Nb * P * Q;
    if (M > 0x7fffffffLL) return -1;
    const int bk = dtype == 1 ? 64 : 32;

    IgemmParams p;
    memset(&p, 0, sizeof p);
    p.x = x; p.w = w; p.y = y; p.scale = scale; p.shift = shift; p.residual = residual;
    p.relu = relu; p.dtype = dtype;
    p.Nb = Nb; p.H = H; p.W = W; p.C = C; p.Kout = Kout; p.R = R; p.S = S; p.P = P; p.Q = Q;
    p.stride_h = stride_h; p.stride_w = stride_w; p.pad_h = pad_h; p.pad_w = pad_w; p.dil_h = dil_h; p.dil_w = dil_w;
    p.M = (int)M;
    p.kblocks_per_r = (S * C + bk - 1) / bk;
    p.num_kblocks = R * p.kblocks_per_r;
    p.tiles_m = (int)((M + 127) / 128);
    p.tiles_n = (Kout + bn - 1) / bn;
    if (splits < 1 || splits > p.num_kblocks) return -1;
    p.splits = splits;
    igemm_set_fprop(&p);

    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    const unsigned long long need = (unsigned long long)tiles * (unsigned long long)splits * 128ull * (unsigned long long)bn;
    if (splits > 1 && (tiles > kCounterInts || need > kScratchFloats)) return -3;   // OB200_ERR_STATIC_SCRATCH_TOO_SMALL

    StaticScratch* sc = nullptr;
    int rc = scratch_for_current_device(&sc);
    if (rc != 0) return rc;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    p.status = &sc->status;   // device address inside the static array: the other entry points' status word is heap-allocated
    if (splits > 1) {
        // The array still holds the previous call's leftovers.  Every unit overwrites its own partial tile before
        // anyone reads it, so only the arrival counters have to start at zero.
        cudaError_t e = cudaMemsetAsync(sc->counters, 0, (size_t)tiles * sizeof(int), s);
        if (e != cudaSuccess) return (int)e;
        p.slabs = sc->partial;
        p.counters = sc->counters;
    }
    const long long units = tiles * splits;
    const int grid = units < num_ctas ? (int)units : num_ctas;
    return ob200_igemm_launch(&p, bn, grid, stream);
}

// Reads and clears the status word of the allocation-free entry point on the current device (synchronises the device; no
// allocation).  0 = no kernel launched through ob200_conv2d_fprop_noalloc reported a timed-out wait since the last call.
extern "C" int ob200_conv2d_fprop_noalloc_status(void) {
    StaticScratch* sc = nullptr;
    int rc = scratch_for_current_device(&sc);
    if (rc != 0) return -1;
    int v = 0;
    if (cudaMemcpy(&v, &sc->status, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v && cudaMemset(&sc->status, 0, sizeof v) != cudaSuccess) return -1;
    return v;
}
