Name,Profile,Memory_footprint,SM_usage,Duration
BatchNorm,-1,0,9,5863
void at::native::reduce_kernel,0,0,13,2928
Conv,0,0,3365,5349.5
Conv,-1,0,3690,9097
volta_sgemm_128x64_tn,1,0,64,9637
BatchNorm,0,0,3,438396
void at::native::elementwise_kernel,0,0,1443,18410
void at::native::elementwise_kernel,1,0,76,18557
Conv,0,0,3347,425926
void at::native::elementwise_kernel,0,0,2799,535123
void at::native::reduce_kernel,0,0,4,3424
volta_sgemm_128x64_tn,-1,0,22,178783
BatchNorm,-1,0,71,15253
volta_sgemm_128x64_tn,0,0,35,693236
void at::native::elementwise_kernel,-1,0,67,8733
void at::native::reduce_kernel,0,0,26,15546
void at::native::reduce_kernel,0,0,2293,12850
BatchNorm,1,0,24,98051
void at::native::elementwise_kernel,1,0,149,2477
Conv,-1,0,1270,74892
BatchNorm,0,0,38,12551
Conv,0,0,54,8161
void at::native::elementwise_kernel,-1,0,78,454623.5
BatchNorm,1,0,21,18590
BatchNorm,-1,0,68,3005
void at::native::vectorized_elementwise_kernel,0,0,1304,133788
Conv,0,0,39,7184
BatchNorm,1,0,5,9130
void at::native::elementwise_kernel,-1,0,49,212142
void at::native::elementwise_kernel,0,0,64,14781
Conv,0,0,52,297018
void at::native::vectorized_elementwise_kernel,-1,0,44,8980
void at::native::reduce_kernel,-1,0,69,510033.5
Conv,1,0,763,8978
volta_sgemm_128x64_tn,-1,0,48,357311
volta_sgemm_128x64_tn,0,0,2338,5416.5
Conv,0,0,19,6096
volta_sgemm_128x64_tn,0,0,2334,4678
void at::native::vectorized_elementwise_kernel,-1,0,15,482005
void at::native::vectorized_elementwise_kernel,1,0,2,98136
Conv,1,0,2484,443464
void at::native::elementwise_kernel,1,0,3542,16257
volta_sgemm_128x64_tn,0,0,62,331734
Conv,1,0,3872,12493
void at::native::reduce_kernel,1,0,1380,632662
volta_sgemm_128x64_tn,-1,0,61,13659
BatchNorm,0,0,1557,87321
void at::native::reduce_kernel,1,0,44,14795.5
BatchNorm,0,0,75,10055
volta_sgemm_128x64_tn,-1,0,12,259003
void at::native::reduce_kernel,1,0,3634,76361
void at::native::vectorized_elementwise_kernel,0,0,20,18430.5
void at::native::elementwise_kernel,1,0,693,12478
volta_sgemm_128x64_tn,-1,0,3741,218783
volta_sgemm_128x64_tn,-1,0,27,11795
Conv,1,0,344,16637
volta_sgemm_128x64_tn,0,0,59,14966
void at::native::reduce_kernel,1,0,54,600321
volta_sgemm_128x64_tn,1,0,18,11073
BatchNorm,-1,0,2071,7818
