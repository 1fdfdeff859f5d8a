Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::vectorized_elementwise_kernel,0,0,24,685681
void at::native::elementwise_kernel,1,0,2257,9009.5
BatchNorm,-1,0,36,876912
void at::native::vectorized_elementwise_kernel,0,0,18,10411
void at::native::reduce_kernel,-1,0,55,13934
void at::native::elementwise_kernel,1,0,77,10614
void at::native::elementwise_kernel,1,0,57,7787
volta_sgemm_128x64_tn,0,0,59,11179
volta_sgemm_128x64_tn,0,0,73,8372
void at::native::reduce_kernel,0,0,55,47307
void at::native::elementwise_kernel,0,0,21,15549
void at::native::vectorized_elementwise_kernel,1,0,48,547629
BatchNorm,-1,0,2955,3266
volta_sgemm_128x64_tn,0,0,871,174473
void at::native::reduce_kernel,-1,0,70,3272
void at::native::elementwise_kernel,1,0,17,5981
void at::native::vectorized_elementwise_kernel,-1,0,10,19105
Conv,1,0,20,19457
BatchNorm,0,0,49,527731
void at::native::elementwise_kernel,1,0,76,249219
void at::native::reduce_kernel,1,0,55,12385
Conv,1,0,1,687076
volta_sgemm_128x64_tn,0,0,38,555708
Conv,1,0,21,12091
void at::native::vectorized_elementwise_kernel,1,0,13,18085
