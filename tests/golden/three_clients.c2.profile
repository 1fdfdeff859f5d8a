Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::reduce_kernel,1,0,43,8404.5
volta_sgemm_128x64_tn,0,0,57,15996
BatchNorm,0,0,59,4324
volta_sgemm_128x64_tn,1,0,40,18414
void at::native::reduce_kernel,0,0,63,6832
void at::native::elementwise_kernel,-1,0,6,5546
void at::native::vectorized_elementwise_kernel,0,0,3629,11624.5
Conv,-1,0,3842,9750
void at::native::reduce_kernel,1,0,45,9499
void at::native::vectorized_elementwise_kernel,1,0,43,12680
BatchNorm,1,0,23,852875
volta_sgemm_128x64_tn,1,0,39,12655
void at::native::elementwise_kernel,0,0,2528,7129.5
volta_sgemm_128x64_tn,1,0,2124,4830
BatchNorm,0,0,18,722007
void at::native::reduce_kernel,0,0,989,182562
void at::native::vectorized_elementwise_kernel,1,0,57,13519
volta_sgemm_128x64_tn,0,0,30,886546
void at::native::elementwise_kernel,0,0,241,13733
void at::native::vectorized_elementwise_kernel,1,0,2,9264.5
void at::native::elementwise_kernel,-1,0,31,20767
Conv,0,0,22,3415
void at::native::reduce_kernel,0,0,65,6744
void at::native::vectorized_elementwise_kernel,1,0,52,115626
void at::native::elementwise_kernel,1,0,32,313411
