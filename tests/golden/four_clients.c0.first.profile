Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::vectorized_elementwise_kernel,1,0,7,77954
Conv,-1,0,433,456710
volta_sgemm_128x64_tn,0,0,2397,131815
void at::native::reduce_kernel,1,0,6,6363
volta_sgemm_128x64_tn,1,0,72,857770
void at::native::elementwise_kernel,1,0,71,748702
void at::native::reduce_kernel,-1,0,41,16849
BatchNorm,1,0,1310,18223
void at::native::vectorized_elementwise_kernel,-1,0,16,538800
BatchNorm,0,0,10,12280
volta_sgemm_128x64_tn,0,0,59,5066
void at::native::elementwise_kernel,1,0,2954,16602
void at::native::elementwise_kernel,0,0,1972,374731
BatchNorm,0,0,1095,14810.5
void at::native::reduce_kernel,0,0,18,16107
void at::native::vectorized_elementwise_kernel,0,0,20,89015
BatchNorm,1,0,76,10609.5
void at::native::reduce_kernel,-1,0,73,336088
void at::native::elementwise_kernel,-1,0,52,5392
Conv,1,0,936,464030
