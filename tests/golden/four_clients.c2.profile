Name,Profile,Memory_footprint,SM_usage,Duration
volta_sgemm_128x64_tn,0,0,2802,14406
void at::native::reduce_kernel,1,0,401,4646
Conv,-1,0,27,13686
void at::native::reduce_kernel,1,0,2020,14213
void at::native::vectorized_elementwise_kernel,0,0,1763,262060
void at::native::reduce_kernel,1,0,8,271500
void at::native::vectorized_elementwise_kernel,0,0,3987,3428
void at::native::elementwise_kernel,0,0,39,5954
Conv,0,0,60,14665
void at::native::reduce_kernel,1,0,24,11128
void at::native::vectorized_elementwise_kernel,0,0,77,84853
BatchNorm,1,0,5,19845
void at::native::reduce_kernel,1,0,34,656942.5
void at::native::reduce_kernel,0,0,625,439089
void at::native::elementwise_kernel,1,0,38,11155
void at::native::elementwise_kernel,0,0,1094,196758
volta_sgemm_128x64_tn,1,0,51,265878
Conv,0,0,14,6710
void at::native::vectorized_elementwise_kernel,1,0,30,127007
volta_sgemm_128x64_tn,1,0,48,7824
void at::native::elementwise_kernel,1,0,2522,746180.5
void at::native::vectorized_elementwise_kernel,1,0,1125,42093
void at::native::reduce_kernel,0,0,1359,83720
volta_sgemm_128x64_tn,0,0,496,836502
Conv,1,0,35,11283
Conv,0,0,46,436194
void at::native::vectorized_elementwise_kernel,1,0,52,2192
void at::native::reduce_kernel,1,0,52,13951
BatchNorm,1,0,664,673787
void at::native::vectorized_elementwise_kernel,-1,0,1506,299056
