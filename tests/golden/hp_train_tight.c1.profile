Name,Profile,Memory_footprint,SM_usage,Duration
BatchNorm,0,0,72,202034
BatchNorm,1,0,47,506607
void at::native::elementwise_kernel,1,0,67,737659.5
void at::native::reduce_kernel,-1,0,2139,12735
volta_sgemm_128x64_tn,1,0,61,14303
Conv,0,0,12,260608
void at::native::vectorized_elementwise_kernel,1,0,44,11383
void at::native::vectorized_elementwise_kernel,-1,0,17,737001
void at::native::reduce_kernel,1,0,79,650921
void at::native::reduce_kernel,1,0,9,4563
void at::native::vectorized_elementwise_kernel,1,0,8,465206
Conv,1,0,68,19542
volta_sgemm_128x64_tn,0,0,18,12902.5
void at::native::vectorized_elementwise_kernel,0,0,72,10283
void at::native::reduce_kernel,0,0,556,159694
void at::native::vectorized_elementwise_kernel,0,0,21,330724.5
volta_sgemm_128x64_tn,1,0,71,3981
void at::native::reduce_kernel,0,0,33,8527
void at::native::elementwise_kernel,1,0,32,466237
void at::native::vectorized_elementwise_kernel,-1,0,7,18456
void at::native::vectorized_elementwise_kernel,0,0,8,12961
volta_sgemm_128x64_tn,0,0,48,266041
BatchNorm,0,0,36,112728.5
void at::native::vectorized_elementwise_kernel,0,0,70,716711
void at::native::vectorized_elementwise_kernel,1,0,25,622675
void at::native::vectorized_elementwise_kernel,0,0,305,625644.5
volta_sgemm_128x64_tn,0,0,67,620870
void at::native::elementwise_kernel,0,0,39,51999
void at::native::elementwise_kernel,1,0,53,639367
volta_sgemm_128x64_tn,1,0,36,8288
