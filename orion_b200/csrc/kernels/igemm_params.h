// Launch parameters of the implicit-GEMM kernels (plain C so that the C-ABI layer,
// the kernels and host-side tests share one definition).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

#ifdef __cplusplus
#define OB200_ALIGN64 alignas(64)
#else
#define OB200_ALIGN64 _Alignas(64)
#endif

typedef struct IgemmParams {
    const void* x;          /* activations, NHWC [Nb, H, W, C] */
    const void* w;          /* filters, KRSC [Kout, R, S, C] */
    void* y;                /* output, NHWC [Nb, P, Q, Kout] */
    const float* scale;     /* optional per-output-channel multiplier */
    const float* shift;     /* optional per-output-channel addend (bias) */
    const void* residual;   /* optional tensor of y's shape added before the ReLU */
    float* scratch;         /* filter gradient only: unused (its partial sums are added into y) */
    int* counters;          /* arrival counters of cut tiles (split-K: one per tile; stream-K: see below), zero on entry and exit */
    int* status;            /* optional device word that receives an error code */
    long long* debug;       /* optional: 8 cycle counters written by CTA 0 (role wait times) */
    int relu;               /* 0 none, 1 ReLU, 2 ReLU6 */
    int dtype;              /* 0 = fp32 (3xTF32), 1 = bf16, 2 = fp32 data with a single TF32 pass */
    int Nb, H, W, C, Kout, R, S, P, Q;
    int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
    int M;                  /* Nb*P*Q */
    int kblocks_per_r;      /* ceil(S*C / BK) */
    int num_kblocks;        /* R * kblocks_per_r */
    int tiles_m, tiles_n;
    /* Split-K factor, <= num_kblocks.  splits > 1 (mode 0): unit (tile, split) covers a contiguous range of the
     * tile's k-blocks and writes its partial accumulator to slab tile*splits + split of `slabs` (128 x BN floats
     * each, contents arbitrary on entry and exit); the unit that arrives last on the tile's counter adds the
     * slabs in split order -- the sum does not depend on arrival order -- and applies the epilogue. */
    int splits;
    /* stream_k = 1 (mode 0 only): the k-blocks of all tiles, laid end to end, are cut into one equal contiguous
     * range per CTA, so a CTA may finish a tile another one began.  Each piece of a cut tile is written to its
     * own slab of `slabs` (two slabs of 128 x BN floats per CTA, contents arbitrary on entry and exit); the piece
     * that arrives last on the tile's counter (index: first CTA that starts inside the tile; zero on entry and
     * exit) adds the slabs in CTA order -- the sum does not depend on arrival order -- and applies the epilogue.
     * splits is ignored. */
    int stream_k;
    float* slabs;
    /* Gather geometry (filled by igemm_set_fprop / igemm_set_dgrad).  GEMM row m = (n*OH + oh)*OW + ow;
     * for tap (r, s) the source pixel of tensor x [Nb, IH, IW, C] is
     *   ih = (oh*bmul_h + badd_h + r*step_h) / div_h   (valid only if the division is exact), same for w. */
    int OH, OW, IH, IW;
    /* Batched GEMM: `batch` independent problems of one shape; tile index runs over (b, tile_m, tile_n)
     * and problem b reads x + b*batch_stride_x, w + b*batch_stride_w, writes y + b*batch_stride_y
     * (strides in elements).  batch <= 1 means a single problem. */
    int batch;
    long long batch_stride_x, batch_stride_w, batch_stride_y;
    /* mode 0: forward / data gradient / GEMM (operands K-major).  mode 1: filter gradient:
     *   dw[k][r][s][c] = sum over pixels m of dy[m][k] * x[pixel of m at tap (r,s)][c]
     * with x = dy [Nb*P*Q, Kout], w = the layer input [Nb, H, W, C], y = dw (float32, accumulated with
     * atomic adds when splits > 1, so it must be zero on entry then); the reduction runs over pixels (the
     * producers transpose both operands into K-major tiles), tiles_m covers Kout and tiles_n covers
     * (tap, channel block). */
    int mode;
    int ctiles;             /* filter gradient: channel blocks per tap, ceil(C / BN) */
    /* Filter gradient with few input channels (TMA-fed only): a tile's BN columns cover wg_tpt consecutive taps of
     * wg_cr columns each (wg_cr = C rounded up to 32), so dy is read once per wg_tpt taps.  wg_tpt <= 1: one tap
     * (and one channel block) per tile. */
    int wg_tpt, wg_cr;
    int bmul_h, bmul_w, badd_h, badd_w, step_h, step_w, div_h, div_w;
    /* Tap subset (TMA-fed launches only): the filter in memory has w_R x w_S taps and the launch iterates
     * R x S of them, tap (t, u) being filter tap (w_r0 + w_rstep*t, w_s0 + w_sstep*u).  w_R = 0: the launch
     * iterates the whole filter.  One parity class of a strided data gradient uses this. */
    int w_R, w_S, w_r0, w_s0, w_rstep, w_sstep;
    /* Output row map: out_map = 0 stores GEMM row m at row m of y; 1 stores row m = (n*OH + i)*OW + j at
     * pixel (n, i*out_mul_h + out_add_h, j*out_mul_w + out_add_w) of an [Nb, out_H, out_W, Kout] tensor. */
    int out_map, out_H, out_W, out_mul_h, out_mul_w, out_add_h, out_add_w;
    /* require_tma = 1: ob200_igemm_launch returns -4 instead of falling back to the gathering producers. */
    int require_tma;
    /* Filled by ob200_igemm_launch.  use_tma = 1: both operands arrive by TMA, the activation through an
     * im2col tensor map over [Nb, IH, IW, C] whose traversal starts at pixel (oh*bmul_h + tma_base_h,
     * ow*bmul_w + tma_base_w) and whose per-tap offsets are non-negative, the filter through a tiled map
     * over [batch, Kout, R, S, C].  0: the producer warps gather with 16-byte asynchronous copies. */
    int use_tma;
    int a_in_tmem;     /* 3xTF32, mode 0: the splitters put both parts of the activation tile into tensor memory */
    /* 3xTF32 with a_in_tmem: the two small cross products (lo*hi, hi*lo) accumulate in a second accumulator and are
     * added to the main one in the epilogue.  The tensor core adds into its fp32 accumulator by truncation; with the
     * cross terms elsewhere the large accumulator takes one addition per k-step instead of three, which cuts the
     * systematic shrinkage of long reductions threefold.  The second accumulator takes the place of the second
     * output buffer, so the epilogue of a tile no longer overlaps the next tile's MMAs: set by the launcher where a
     * CTA computes at most two tiles anyway (small batches). */
    int cross_acc;
    int tma_base_h, tma_base_w;
    unsigned long long mn_desc_bits;   /* filter gradient on TMA: the operand descriptors' bits above the address */
    OB200_ALIGN64 unsigned char tmap_a[128];
    OB200_ALIGN64 unsigned char tmap_b[128];
} IgemmParams;

/* Forward convolution: rows are output pixels (P x Q), the source is the input image. */
static inline void igemm_set_fprop(IgemmParams* p) {
    p->OH = p->P; p->OW = p->Q; p->IH = p->H; p->IW = p->W;
    p->bmul_h = p->stride_h; p->bmul_w = p->stride_w;
    p->badd_h = -p->pad_h; p->badd_w = -p->pad_w;
    p->step_h = p->dil_h; p->step_w = p->dil_w;
    p->div_h = 1; p->div_w = 1;
}

/* Data gradient: rows are input pixels (H x W), the source is dy [Nb, P, Q, C] (C = the
 * convolution's output channels), and tap (r, s) reads dy at ((h + pad - r*dil) / stride). */
static inline void igemm_set_dgrad(IgemmParams* p, int conv_H, int conv_W, int conv_P, int conv_Q) {
    p->OH = conv_H; p->OW = conv_W; p->IH = conv_P; p->IW = conv_Q;
    p->bmul_h = 1; p->bmul_w = 1;
    p->badd_h = p->pad_h; p->badd_w = p->pad_w;
    p->step_h = -p->dil_h; p->step_w = -p->dil_w;
    p->div_h = p->stride_h; p->div_w = p->stride_w;
}

int ob200_igemm_launch(const IgemmParams* params, int bn, int num_ctas, void* stream);

#ifdef __cplusplus
}
#endif
