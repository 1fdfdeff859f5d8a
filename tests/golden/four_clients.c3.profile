Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::reduce_kernel,1,0,82,48139
BatchNorm,1,0,3271,112014
BatchNorm,-1,0,65,681054
Conv,0,0,62,752149
void at::native::reduce_kernel,0,0,2766,476467
void at::native::vectorized_elementwise_kernel,1,0,16,353814
volta_sgemm_128x64_tn,0,0,67,280183.5
volta_sgemm_128x64_tn,1,0,3786,249578
void at::native::vectorized_elementwise_kernel,1,0,43,9837
void at::native::elementwise_kernel,-1,0,68,733505
void at::native::elementwise_kernel,1,0,40,8945
Conv,-1,0,19,36512
BatchNorm,0,0,4,34369
void at::native::elementwise_kernel,1,0,6,70959
volta_sgemm_128x64_tn,1,0,50,114319
Conv,1,0,12,11416.5
Conv,1,0,44,446350
void at::native::vectorized_elementwise_kernel,1,0,48,18506
volta_sgemm_128x64_tn,1,0,4,459650
void at::native::elementwise_kernel,1,0,28,4978
Conv,-1,0,7,13396.5
void at::native::elementwise_kernel,1,0,76,18880
BatchNorm,0,0,30,524521
Conv,0,0,72,5426
void at::native::reduce_kernel,0,0,12,2824
