Name,Profile,Memory_footprint,SM_usage,Duration
BatchNorm,0,0,17,204497
volta_sgemm_128x64_tn,1,0,4,17971
volta_sgemm_128x64_tn,1,0,52,95916
void at::native::elementwise_kernel,0,0,61,5726.5
Conv,0,0,49,3902
Conv,0,0,67,220016
Conv,0,0,19,16950
void at::native::vectorized_elementwise_kernel,0,0,3211,5198
void at::native::elementwise_kernel,0,0,26,6920
volta_sgemm_128x64_tn,1,0,65,737360
Conv,0,0,35,15874
void at::native::elementwise_kernel,0,0,1704,123909
BatchNorm,0,0,3343,14466
volta_sgemm_128x64_tn,0,0,18,16616
volta_sgemm_128x64_tn,1,0,13,37686
volta_sgemm_128x64_tn,0,0,3916,531450
Conv,1,0,656,359347
void at::native::vectorized_elementwise_kernel,0,0,1,679219.5
volta_sgemm_128x64_tn,1,0,75,7826
void at::native::reduce_kernel,1,0,2560,18292
void at::native::reduce_kernel,1,0,3034,6143
Conv,0,0,47,479454
void at::native::reduce_kernel,1,0,3051,2741
volta_sgemm_128x64_tn,1,0,77,528996
void at::native::reduce_kernel,-1,0,1,305623
