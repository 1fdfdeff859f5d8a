Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::elementwise_kernel,1,0,1638,103332
volta_sgemm_128x64_tn,0,0,24,413483
volta_sgemm_128x64_tn,1,0,24,301867
void at::native::reduce_kernel,0,0,105,15150
void at::native::reduce_kernel,1,0,88,395819
void at::native::reduce_kernel,0,0,148,7358
void at::native::vectorized_elementwise_kernel,-1,0,3744,816357
BatchNorm,-1,0,109,462996
Conv,0,0,121,779854
void at::native::vectorized_elementwise_kernel,1,0,145,694821
void at::native::reduce_kernel,0,0,131,3042
volta_sgemm_128x64_tn,1,0,138,2578
volta_sgemm_128x64_tn,0,0,157,9622
void at::native::vectorized_elementwise_kernel,0,0,71,834823.5
Conv,1,0,138,68189
Conv,1,0,49,2460
void at::native::vectorized_elementwise_kernel,-1,0,34,744206
void at::native::vectorized_elementwise_kernel,1,0,1532,3855.5
void at::native::elementwise_kernel,1,0,3152,408174
void at::native::elementwise_kernel,1,0,115,16025
Conv,1,0,844,16933
void at::native::vectorized_elementwise_kernel,-1,0,65,2243
volta_sgemm_128x64_tn,0,0,74,825749
BatchNorm,1,0,100,695814
volta_sgemm_128x64_tn,1,0,19,4336.5
