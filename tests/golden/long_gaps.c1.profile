Name,Profile,Memory_footprint,SM_usage,Duration
Conv,-1,0,17,618757
Conv,-1,0,8,503947
Conv,1,0,9,5103
Conv,0,0,38,8905
BatchNorm,1,0,71,2646
volta_sgemm_128x64_tn,-1,0,25,9124
void at::native::elementwise_kernel,0,0,2594,262324
void at::native::vectorized_elementwise_kernel,0,0,3035,641222
void at::native::reduce_kernel,0,0,44,14286
void at::native::elementwise_kernel,0,0,23,4377
void at::native::elementwise_kernel,1,0,27,162885
void at::native::elementwise_kernel,1,0,3587,60319
void at::native::vectorized_elementwise_kernel,-1,0,80,2593
volta_sgemm_128x64_tn,1,0,50,16272.5
void at::native::elementwise_kernel,1,0,26,736265
void at::native::vectorized_elementwise_kernel,1,0,54,3309
void at::native::vectorized_elementwise_kernel,-1,0,52,13954
void at::native::reduce_kernel,1,0,73,9225
BatchNorm,1,0,47,17032
Conv,0,0,39,774086
void at::native::vectorized_elementwise_kernel,0,0,61,18478
void at::native::reduce_kernel,-1,0,68,19826
void at::native::vectorized_elementwise_kernel,1,0,58,262165
void at::native::elementwise_kernel,1,0,3673,10918.5
Conv,1,0,3738,393024
