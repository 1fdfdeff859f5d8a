// Launch parameters of the implicit-GEMM kernels (plain C so that the C-ABI layer,
// the kernels and host-side tests share one definition).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

typedef struct IgemmParams {
    const void* x;          /* activations, NHWC [Nb, H, W, C] */
    const void* w;          /* filters, KRSC [Kout, R, S, C] */
    void* y;                /* output, NHWC [Nb, P, Q, Kout] */
    const float* scale;     /* optional per-output-channel multiplier */
    const float* shift;     /* optional per-output-channel addend (bias) */
    const void* residual;   /* optional tensor of y's shape added before the ReLU */
    float* scratch;         /* split-K partial sums, zero on entry, zero on exit */
    int* counters;          /* split-K arrival counters, one per tile, zero on entry and exit */
    int* status;            /* optional device word that receives an error code */
    long long* debug;       /* optional: 8 cycle counters written by CTA 0 (role wait times) */
    int relu;               /* 0 none, 1 ReLU, 2 ReLU6 */
    int dtype;              /* 0 = fp32 (3xTF32), 1 = bf16 */
    int Nb, H, W, C, Kout, R, S, P, Q;
    int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
    int M;                  /* Nb*P*Q */
    int kblocks_per_r;      /* ceil(S*C / BK) */
    int num_kblocks;        /* R * kblocks_per_r */
    int tiles_m, tiles_n;
    int splits;             /* split-K factor, <= num_kblocks */
} IgemmParams;

int ob200_igemm_launch(const IgemmParams* params, int bn, int num_ctas, void* stream);

#ifdef __cplusplus
}
#endif
