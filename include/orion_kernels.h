/* liborion_kernels.so — C ABI of the sm_100a workload kernels.
 *
 * Plain pointers and sizes only.  Every entry point launches on `stream`
 * (a cudaStream_t) with at most `num_ctas` persistent CTAs (the SM quota granted to
 * the caller) and returns 0 on success, a cudaError_t value (> 0) if the launch
 * failed, or a negative number for invalid arguments.  Layouts: activations NHWC,
 * filters KRSC (a torch tensor in channels_last memory format).  dtype: 0 = float32
 * (computed as 3xTF32 with fp32 accumulation, ~1e-6 relative error), 1 = bfloat16 (fp32
 * accumulation), 2 = float32 data multiplied in a single TF32 pass (10-bit mantissa products:
 * what cuDNN does by default on tensor cores; about three times less tensor work).
 * There is no CPU fallback.
 */
#ifndef ORION_KERNELS_H
#define ORION_KERNELS_H

#ifdef __cplusplus
extern "C" {
#endif

/* y = act(conv(x, w) * scale[k] + shift[k] + residual).  Takes the place of the
 * cudnnConvolutionForward call the reference replays (reference
 * src/scheduler/utils_sched.cpp:284-296, trapped at src/cuda_capture/intercept_cudnn.cpp:6-62).
 * scale / shift / residual may be NULL; relu: 0 none, 1 ReLU, 2 ReLU6.  Chooses the
 * tile width and a split-K factor itself; split-K partial sums live in a scratch
 * buffer that is allocated once per stream on first use. */
int ob200_conv2d_fprop(const void* x, const void* w, void* y, const float* scale, const float* shift, const void* residual,
                       int relu, int dtype, int Nb, int H, int W, int C, int Kout, int R, int S, int stride_h, int stride_w,
                       int pad_h, int pad_w, int dil_h, int dil_w, int num_ctas, void* stream);

/* Same with the tile width (bn: 64 or 128), the split-K factor and the scratch
 * passed by the caller: scratch = tiles*splits*128*bn floats (one partial tile per split, any
 * contents), counters = tiles ints, zero on entry (the kernel leaves them zero); unused when
 * splits == 1.  The partial tiles are added in split order, so the result is reproducible bit for bit. */
int ob200_conv2d_fprop_ex(const void* x, const void* w, void* y, const float* scale, const float* shift, const void* residual,
                          int relu, int dtype, int Nb, int H, int W, int C, int Kout, int R, int S, int stride_h, int stride_w,
                          int pad_h, int pad_w, int dil_h, int dil_w, int bn, int splits, float* scratch, int* counters,
                          int num_ctas, void* stream);

/* No counterpart in the reference.  ob200_conv2d_fprop_ex for callers that cannot allocate device
 * memory at the moment of the call — code running under stream capture, inside an allocator or
 * framework hook where a cudaMalloc would re-enter the allocator, or an embedder that hands out all
 * device memory up front.  The split-K scratch is a fixed 8 MiB (+1 KiB of tile counters) array
 * compiled into the library (held by every GPU that loads it, until exit); the call performs no
 * cudaMalloc / cudaFree and uses no allocating library routine.  Limits: tiles*splits*128*bn floats must fit
 * in 2 Mi floats and tiles (ceil(M/128)*ceil(Kout/bn)) in 256, else the call returns -3 and launches
 * nothing.  All calls share the array: each call clears the tile counters it uses on `stream` first, and calls
 * that overlap on the GPU without an ordering between their streams race on it.  The first call on a
 * device resolves the array's device address (not a stream operation): make it before any capture. */
int ob200_conv2d_fprop_noalloc(const void* x, const void* w, void* y, const float* scale, const float* shift,
                               const void* residual, int relu, int dtype, int Nb, int H, int W, int C, int Kout, int R, int S,
                               int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int bn, int splits,
                               int num_ctas, void* stream);
/* Its status word (kept inside the same built-in array; reading it synchronises the device and allocates nothing): the code
 * of a bounded in-kernel wait that expired since the last call, 0 if none.  No counterpart in the reference. */
int ob200_conv2d_fprop_noalloc_status(void);

/* Tile width and split-K factor of the one-unit-per-tile / split-K schedule for a problem size (host logic only). */
int ob200_plan_conv(int dtype, long long M, int Kout, int R, int S, int C, int num_ctas, int* bn_out, int* splits_out);
/* The schedule ob200_conv2d_fprop picks (host logic only): stream_k_out = 1 means the k-blocks of all tiles are cut
 * into one equal range per CTA (then splits_out = 1); otherwise the ob200_plan_conv choice.  No counterpart in the
 * reference (cuDNN picks its own algorithm behind cudnnConvolutionForward). */
int ob200_plan_schedule(int dtype, long long M, int Kout, int R, int S, int C, int num_ctas, int* bn_out, int* splits_out,
                        int* stream_k_out);

/* Data gradient of the convolution, dx [Nb,H,W,C] from dy [Nb,P,Q,Kout] and the re-laid-out filter
 * wt [C,R,S,Kout] (ob200_filter_transpose).  Takes the place of cudnnConvolutionBackwardData
 * (reference src/scheduler/utils_sched.cpp:439-464, trapped at src/cuda_capture/intercept_cudnn.cpp:482-558). */
int ob200_conv2d_dgrad(const void* dy, const void* wt, void* dx, int dtype, int Nb, int H, int W, int C, int Kout, int R, int S,
                       int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int num_ctas, void* stream);
/* Filter gradient dw [Kout,R,S,C] (float32) from the layer input x [Nb,H,W,C] and dy [Nb,P,Q,Kout]; dtype 0 or 2
 * (float32 data), C and Kout multiples of 4.  Takes the place of cudnnConvolutionBackwardFilter (reference
 * src/scheduler/utils_sched.cpp:465-489, trapped at src/cuda_capture/intercept_cudnn.cpp:560-640). */
int ob200_conv2d_wgrad(const void* x, const void* dy, float* dw, int dtype, int Nb, int H, int W, int C, int Kout, int R, int S,
                       int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int num_ctas, void* stream);
/* w [K, R*S, C] -> wt [C, R*S, K]; elem_bytes 4 or 2.  No counterpart in the reference (cuDNN re-lays filters internally). */
int ob200_filter_transpose(const void* w, void* wt, int K, int RS, int C, int elem_bytes, void* stream);

/* Batch-norm training forward over [rows, C] float32 (C % 4 == 0): batch statistics, normalisation,
 * running-statistics update; save_mean / save_invstd feed the backward pass.  `sums` is a scratch of
 * 2*C doubles that must be zero on entry.  Takes the place of cudnnBatchNormalizationForwardTrainingEx
 * (reference src/scheduler/utils_sched.cpp:297-339). */
int ob200_bn_train_forward_f32(const float* x, float* y, const float* gamma, const float* beta, float* running_mean,
                               float* running_var, float* save_mean, float* save_invstd, double* sums, float eps, float momentum,
                               long long rows, int C, int num_ctas, void* stream);
/* Batch-norm backward: dx, dgamma, dbeta (the last two may be NULL); `sums` as above.  Takes the place of
 * cudnnBatchNormalizationBackwardEx (reference src/scheduler/utils_sched.cpp:398-438). */
int ob200_bn_backward_f32(const float* dy, const float* x, float* dx, const float* gamma, const float* save_mean,
                          const float* save_invstd, float* dgamma, float* dbeta, double* sums, long long rows, int C, int num_ctas,
                          void* stream);

/* Training batch norm fused with the residual add and the activation around it: y = act(batch_norm(x) [+ residual]),
 * act 0 none / 1 ReLU / 2 ReLU6, x [rows, C] float32, C % 4 == 0, C <= 8192.  Two launches per direction (a reduction
 * whose last-arriving CTA finishes the statistics and cleans its own scratch, then one elementwise pass); the scratch
 * belongs to the library (allocated once per stream).  The backward pass recomputes the activation's input from x, or
 * reads it from the saved output `yout` when a residual was added (yout = NULL otherwise); dres receives the residual's
 * gradient (NULL when there was none).  They take the place of cudnnBatchNormalizationForwardTrainingEx /
 * cudnnBatchNormalizationBackwardEx (reference src/scheduler/utils_sched.cpp:297-339,398-438) plus the add / ReLU /
 * ReLU-backward elementwise kernels that follow them in the reference's profiles
 * (reference benchmarking/model_kernels/resnet50_32_fb1). */
int ob200_bn_act_train_forward_f32(const float* x, const float* residual, float* y, const float* gamma, const float* beta,
                                   float* running_mean, float* running_var, float* save_mean, float* save_invstd, float eps,
                                   float momentum, long long rows, int C, int act, int num_ctas, void* stream);
int ob200_bn_act_backward_f32(const float* dy, const float* x, const float* yout, float* dx, float* dres, const float* gamma,
                              const float* beta, const float* save_mean, const float* save_invstd, float* dgamma, float* dbeta,
                              long long rows, int C, int act, int num_ctas, void* stream);
/* dx = dy where y > 0, else 0 (threshold_backward kernels behind the reference's cudaLaunchKernel trap). */
int ob200_relu_backward_f32(const float* dy, const float* y, float* dx, long long n, int num_ctas, void* stream);
/* torch.optim.SGD step with momentum on one parameter tensor (the foreach kernels behind the same trap). */
int ob200_sgd_momentum_f32(float* p, const float* g, float* m, long long n, float lr, float mu, float wd, int nesterov,
                           int first_step, int num_ctas, void* stream);
/* The same update over `count` tensors (host arrays of device pointers and element counts) in ceil(count / 96) launches:
 * the role of the multi-tensor (foreach) optimizer kernels in the reference's training profiles. */
int ob200_sgd_momentum_multi_f32(float* const* p, const float* const* g, float* const* m, const long long* n, int count, float lr,
                                 float mu, float wd, int nesterov, int first_step, int num_ctas, void* stream);

/* y[M,N] = x[M,K] . w[N,K]^T + bias, optional ReLU.  Takes the place of cublasSgemm_v2
 * (reference src/scheduler/utils_sched.cpp:490-501, trapped at src/cuda_capture/intercept_cublas.cpp:5-56). */
int ob200_linear(const void* x, const void* w, void* y, const float* bias, int relu, int dtype, int M, int N, int K,
                 int num_ctas, void* stream);

/* `batch` independent GEMMs of one shape, operands stride_* elements apart (strides multiples of 16 bytes).
 * Takes the place of cublasSgemmStridedBatched (reference src/scheduler/utils_sched.cpp:502-513, trapped at
 * src/cuda_capture/intercept_cublas.cpp:114-170): attention scores Q.K^T and, with V pre-transposed, P.V. */
int ob200_linear_batched(const void* x, const void* w, void* y, int dtype, int batch, int M, int N, int K, long long stride_x,
                         long long stride_w, long long stride_y, int num_ctas, void* stream);

/* bfloat16 GEMM with transpose flags, strides and two batch levels (float32 accumulation):
 *   C[bo][bi][m, n] = alpha * sum_k A[bo][bi][m, k] * B[bo][bi][n, k] (+ bias[n]),   bi < batch_inner, bo < batch_outer.
 * a_mn = 0: A lies as [M, K] rows `lda` elements apart; a_mn = 1: as [K, M] rows (the reduction index is the slow one).
 * b_mn likewise for B ([N, K] rows or [K, N] rows).  C rows are `ldc` apart; *_si / *_so are the element offsets between
 * problems of the inner / outer batch level.  lda, ldb and the operand batch offsets must be multiples of 8 elements, the
 * operand pointers 16-byte aligned.  out_f32 selects a float32 or bfloat16 C.  Few output tiles with a long reduction are cut
 * along K into float32 partial matrices summed in split order (same result for every num_ctas).
 * Takes the place of cublasSgemm_v2 / cublasSgemmStridedBatched with CUBLAS_OP_T / CUBLAS_OP_N operands (reference
 * src/scheduler/utils_sched.cpp:490-513, trapped at src/cuda_capture/intercept_cublas.cpp:5-56,114-170): the data and weight
 * gradients of linear layers and the attention products of training (the sgemm rows of benchmarking/model_kernels/bert_8_fb1). */
int ob200_gemm_bf16(const void* a, const void* b, void* c, const float* bias, int M, int N, int K, int a_mn, int b_mn, long long lda,
                    long long ldb, long long ldc, int batch_inner, int batch_outer, long long a_si, long long a_so, long long b_si,
                    long long b_so, long long c_si, long long c_so, float alpha, int out_f32, int num_ctas, void* stream);

/* ob200_gemm_bf16 with two more epilogue addends: the bias given in bfloat16 (a parameter of a bfloat16 model; either bias
 * pointer may be NULL) and a bfloat16 `residual` laid out like C, added in float32 before the result is rounded (the
 * residual stream of a transformer layer: the elementwise add rows of benchmarking/model_kernels/bert_8_fb1), and `tri` for the
 * products of causal attention, whose probability matrix P[q, key] is zero for key > q: 0 = plain; 1 = only output tiles that
 * reach n <= m are computed, the others are left unwritten (scores, dP); 2 = A[m, k] is zero for k > m, the reduction stops
 * behind the tile's last row (P.V, dS.K); 3 = A[m, k] is zero for k < m, the reduction starts at the tile's first row
 * (P^T.dO, dS^T.Q). */
int ob200_gemm_bf16_ex(const void* a, const void* b, void* c, const float* bias, const void* bias_bf16, const void* residual, int M,
                       int N, int K, int a_mn, int b_mn, long long lda, long long ldb, long long ldc, int batch_inner,
                       int batch_outer, long long a_si, long long a_so, long long b_si, long long b_so, long long c_si,
                       long long c_so, float alpha, int out_f32, int tri, int num_ctas, void* stream);

/* out[col] = sum over rows of x[row, col] (rows `ld` elements apart), summed in a fixed order: the bias gradient of a linear
 * layer.  dtype 0 float32, 1 bfloat16.  Stands where the reference's clients launch ATen's reduce_kernel
 * (benchmarking/model_kernels/bert_8_fb1), trapped at src/cuda_capture/intercept_temp.cpp:418-458 like the three below. */
int ob200_colsum(const void* x, void* out, long long rows, int D, long long ld, int dtype, int num_ctas, void* stream);

/* ds = scale * prob * (dprob - rowsum(prob * dprob)): gradient of softmax(scale * s) with respect to s; ds may alias dprob.
 * causal_period > 0: row r belongs to query position r % causal_period; columns behind it are not read (dprob may be
 * unwritten there) and get ds = 0.  Stands for softmax_warp_backward of the same profile. */
int ob200_softmax_backward(const void* prob, const void* dprob, void* ds, long long rows, int D, float scale, int causal_period,
                           int dtype, int num_ctas, void* stream);

/* out[t, :] = sum of up to three embedding rows: table_k[ids_k[t], :], or table_k[t % periods[k], :] where ids_k is NULL
 * (position table).  Stands for vectorized_gather_kernel + the adds behind it. */
int ob200_embedding_sum(const void* const* tables, const long long* const* ids, const long long* periods, int count, void* out,
                        long long tokens, int D, int dtype, int num_ctas, void* stream);

/* dtable = 0; dtable[row(t), :] += dy[t, :] with atomic adds.  Stands for embedding_backward_feature_kernel. */
int ob200_embedding_backward(const void* dy, const long long* ids, long long period, void* dtable, long long table_rows,
                             long long tokens, int D, int dtype, int num_ctas, void* stream);

/* Batch-norm inference over the innermost (channel) dimension.  Takes the place of
 * cudnnBatchNormalizationForwardInference (reference src/scheduler/utils_sched.cpp:340-353). */
int ob200_bn_inference_f32(const float* x, float* y, const float* gamma, const float* beta, const float* mean, const float* var,
                           float eps, long long n_elems, int C, int relu, int num_ctas, void* stream);

/* mode 0: y = relu(a); 1: y = a + b; 2: y = relu(a + b).  Takes the place of the
 * at::native elementwise kernels that reach the reference through its cudaLaunchKernel
 * trap (reference src/cuda_capture/intercept_temp.cpp:418-458). */
int ob200_binary_f32(const float* a, const float* b, float* y, long long n_elems, int mode, int num_ctas, void* stream);

/* NHWC max-pool / global average pool (same trap as above: max_pool_forward_nchw and
 * the mean reduce kernel in the reference's profiles). */
int ob200_maxpool_nhwc_f32(const float* x, float* y, int Nb, int H, int W, int C, int k, int stride, int pad, int num_ctas,
                           void* stream);
/* Gradient of the max-pool: the output gradient goes to the first largest element of each window in row-major order (the
 * element the stock forward kernel records; ties are frequent behind a ReLU); dx is cleared on `stream` first.  Stands in for
 * the max_pool_backward_nhwc kernel that reaches the reference through its cudaLaunchKernel trap
 * (reference src/cuda_capture/intercept_temp.cpp:418-458). */
int ob200_maxpool_backward_nhwc_f32(const float* dy, const float* x, float* dx, int Nb, int H, int W, int C, int k, int stride,
                                    int pad, int num_ctas, void* stream);
int ob200_avgpool_nhwc_f32(const float* x, float* y, int Nb, int HW, int C, int num_ctas, void* stream);

/* Row kernels of the transformer clients; dtype 0 = float32, 1 = bfloat16 (float32 math), D a multiple of
 * 4 / 8 elements.  They take the place of the at::native kernels that reach the reference through its
 * cudaLaunchKernel trap (reference src/cuda_capture/intercept_temp.cpp:418-458): vectorized_layer_norm_kernel,
 * softmax_warp_forward, the bias + GELU elementwise kernels, and the optimizer's elementwise update kernels. */
int ob200_layernorm(const void* x, void* y, const float* gamma, const float* beta, float* mean_out, float* rstd_out,
                    long long rows, int D, float eps, int dtype, int num_ctas, void* stream);
int ob200_softmax(const void* x, void* y, long long rows, int D, float scale, int dtype, int num_ctas, void* stream);
/* The same with the causal mask of a decoder: row r holds the scores of query position r % causal_period against keys
 * 0..D-1, and keys after the query position get probability 0 (causal_period = 0: no mask). */
int ob200_softmax_causal(const void* x, void* y, long long rows, int D, float scale, int causal_period, int dtype, int num_ctas,
                         void* stream);
/* Fused self-attention forward (bfloat16, head dimension 64, S <= 384): ctx [B, S, H*64] = softmax(Q K^T * scale [+ causal
 * mask]) V, read straight from the fused projection output qkv [B, S, 3, H, 64]; scores and probabilities stay in tensor
 * memory / shared memory.  Takes the place of the two cublasSgemmStridedBatched calls around a softmax kernel
 * (reference src/scheduler/utils_sched.cpp:502-513). */
int ob200_attention_fwd_bf16(const void* qkv, void* ctx, int B, int S, int H, int head_dim, float scale, int causal, int num_ctas,
                             void* stream);

/* Training side of the transformer clients (dtype 0 float32, 1 bfloat16; parameters in the activations' type).  They
 * stand in for the kernels the reference's BERT training profile lists (reference benchmarking/model_kernels/bert_8_fb1:
 * vectorized_layer_norm_kernel, layer_norm_grad_input_kernel, GammaBetaBackwardCUDAKernel, the GELU elementwise kernels,
 * softmax / nll_loss forward and backward, multi_tensor_apply_kernel), which reach the reference through its cudaLaunchKernel
 * trap (reference src/cuda_capture/intercept_temp.cpp:418-458).  Per-column parameter gradients are summed in a fixed order. */
int ob200_layernorm_train_forward(const void* x, void* y, const void* gamma, const void* beta, float* mean, float* rstd, long long rows,
                                  int D, float eps, int dtype, int num_ctas, void* stream);
int ob200_layernorm_backward(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                             void* dgamma, void* dbeta, long long rows, int D, int dtype, int num_ctas, void* stream);
int ob200_bias_gelu_train_forward(const void* x, const void* bias, void* y, long long rows, int D, int dtype, int num_ctas, void* stream);
int ob200_bias_gelu_backward(const void* dy, const void* x, const void* bias, void* dx, void* dbias, long long rows, int D, int dtype,
                             int num_ctas, void* stream);
/* Cross-entropy over a large vocabulary straight from the logits' own type: loss[row] and logsumexp[row]; the gradient of the
 * mean loss, (softmax - onehot) * grad[0] / rows, is written in the logits' type. */
int ob200_cross_entropy_forward(const void* logits, const long long* target, float* loss, float* lse, long long rows, int V, int dtype,
                                void* stream);
int ob200_cross_entropy_backward(const void* logits, const long long* target, const float* lse, const float* grad, void* dlogits,
                                 long long rows, int V, int dtype, void* stream);
/* torch.optim.AdamW over `count` tensors of one type (host arrays of device pointers; state in the parameters' type) in
 * ceil(count / 72) launches. */
int ob200_adamw_multi(void* const* p, const void* const* g, void* const* m, void* const* v, const long long* n, int count, float lr,
                      float beta1, float beta2, float eps, float weight_decay, int step, int dtype, int num_ctas, void* stream);
int ob200_bias_gelu(const void* x, void* y, const float* bias, long long rows, int D, int dtype, int num_ctas, void* stream);
/* torch.optim.AdamW step number `step` (>= 1) on one float32 tensor. */
int ob200_adamw_f32(float* p, const float* g, float* m, float* v, long long n, float lr, float beta1, float beta2, float eps,
                    float weight_decay, int step, int num_ctas, void* stream);

/* Device status word of the current device (synchronises the device): 0, or the code of
 * the bounded wait a kernel gave up on.  Clears the word; after a non-zero status it also clears the split-K arrival
 * counters of every stream of the device, which the kernel that gave up may have left above zero.  No counterpart in the
 * reference. */
int ob200_read_status(void);
/* Tuning aid, no counterpart in the reference: `dev_buf` (8 long longs in device memory, or NULL to
 * switch off) receives from CTA 0 of every implicit-GEMM launch the cycles each warp role spent
 * waiting: [0] epilogue, [1] MMA on operands, [2] MMA on a free accumulator, [3] splitter,
 * [4] producer, [5] whole kernel. */
void ob200_set_debug_buffer(long long* dev_buf);
/* Depthwise convolution (groups = C, channel multiplier 1), NHWC float32, C a multiple of 4, with the same
 * fused epilogue as ob200_conv2d_fprop (scale, shift, relu 0/1/2 = none/ReLU/ReLU6).  w_tap_major = 0: filter
 * [C][R][S] as torch holds a [C,1,R,S] weight; 1: [R][S][C].  Stands in for the grouped cudnnConvolutionForward
 * calls of MobileNetV2 that the reference replays (src/scheduler/utils_sched.cpp:284-296). */
int ob200_depthwise_conv2d_f32(const float* x, const float* w, float* y, const float* scale, const float* shift, int relu, int Nb,
                               int H, int W, int C, int R, int S, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h,
                               int dil_w, int w_tap_major, int num_ctas, void* stream);
/* Its gradients (filter [C][R][S], dilation 1): the data gradient for any filter size and stride, the filter gradient for
 * 3x3 filters (dw is cleared on `stream` and accumulated with atomic adds).  They stand in for the
 * conv_depthwise2d_backward_kernel / conv_depthwise2d_grad_weight_kernel rows of the reference's MobileNetV2 training profile
 * (reference benchmarking/model_kernels/mobilenetv2_64_fb1). */
int ob200_depthwise_conv2d_dgrad_f32(const float* dy, const float* w, float* dx, int Nb, int H, int W, int C, int R, int S,
                                     int stride_h, int stride_w, int pad_h, int pad_w, int num_ctas, void* stream);
int ob200_depthwise_conv2d_wgrad3x3_f32(const float* dy, const float* x, float* dw, int Nb, int H, int W, int C, int stride, int pad,
                                        int num_ctas, void* stream);
/* Number of implicit-GEMM launches of this process whose operands were fed by TMA tensor maps (the others
 * gathered with 16-byte asynchronous copies: strided data gradients, filter gradients, channel counts below
 * one k-block or k-blocks that straddle filter taps).  No counterpart in the reference. */
long long ob200_tma_launch_count(void);
/* SM count of the current device.  No counterpart in the reference. */
int ob200_sm_count(void);
/* Copies [pixels, C] to [pixels, Cpad] (Cpad > C) with zeros in the added channels; elem_bytes 2 or 4.
 * Lets a 3-channel stem convolution (torchvision resnet / mobilenet conv1, which the reference hands to
 * cudnnConvolutionForward, src/cuda_capture/intercept_cudnn.cpp:17) use 16-byte operand chunks.
 * No counterpart in the reference. */
int ob200_pad_channels(const void* src, void* dst, long long pixels, int C, int Cpad, int elem_bytes, int num_ctas,
                       void* stream);

#ifdef __cplusplus
}
#endif
#endif
