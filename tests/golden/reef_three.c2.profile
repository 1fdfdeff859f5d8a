Name,Profile,Memory_footprint,SM_usage,Duration
BatchNorm,0,0,6,9990.5
BatchNorm,-1,0,42,854839
BatchNorm,0,0,39,8294
void at::native::elementwise_kernel,0,0,33,766142
void at::native::reduce_kernel,0,0,25,11044
BatchNorm,-1,0,54,15832
BatchNorm,0,0,49,18758
volta_sgemm_128x64_tn,1,0,14,649190
void at::native::reduce_kernel,1,0,925,19338
volta_sgemm_128x64_tn,1,0,2533,865572
void at::native::vectorized_elementwise_kernel,0,0,35,713141
BatchNorm,0,0,358,16862
void at::native::elementwise_kernel,1,0,52,561886
BatchNorm,0,0,72,890517
void at::native::vectorized_elementwise_kernel,1,0,25,418185
volta_sgemm_128x64_tn,1,0,15,6728
Conv,1,0,25,19240.5
void at::native::elementwise_kernel,1,0,1198,48958
void at::native::vectorized_elementwise_kernel,1,0,9,17590
volta_sgemm_128x64_tn,0,0,35,577626
void at::native::reduce_kernel,1,0,56,16181
void at::native::reduce_kernel,0,0,37,9627.5
volta_sgemm_128x64_tn,-1,0,3435,114188
void at::native::elementwise_kernel,1,0,48,866521
void at::native::reduce_kernel,1,0,2145,9814
