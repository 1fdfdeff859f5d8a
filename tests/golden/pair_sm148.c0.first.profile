Name,Profile,Memory_footprint,SM_usage,Duration
BatchNorm,0,0,1771,504140.5
void at::native::reduce_kernel,-1,0,16,19050
BatchNorm,1,0,3947,10528
void at::native::vectorized_elementwise_kernel,0,0,96,13056
BatchNorm,1,0,23,19945.5
void at::native::vectorized_elementwise_kernel,-1,0,80,891238
volta_sgemm_128x64_tn,0,0,42,11997
Conv,1,0,2714,19002
BatchNorm,1,0,3890,16455
void at::native::reduce_kernel,-1,0,143,210364
void at::native::elementwise_kernel,1,0,2533,647327
BatchNorm,0,0,11,4706
void at::native::vectorized_elementwise_kernel,1,0,83,162337
BatchNorm,0,0,1173,7206
void at::native::vectorized_elementwise_kernel,1,0,94,13885
void at::native::reduce_kernel,1,0,54,121137.5
BatchNorm,-1,0,39,3339
void at::native::vectorized_elementwise_kernel,1,0,2316,309135
BatchNorm,0,0,10,15802
void at::native::reduce_kernel,1,0,9,10335
BatchNorm,1,0,67,150585
void at::native::vectorized_elementwise_kernel,-1,0,2482,3327
void at::native::reduce_kernel,1,0,147,13029
void at::native::elementwise_kernel,0,0,136,10791
void at::native::reduce_kernel,1,0,72,660359
volta_sgemm_128x64_tn,1,0,69,701599
void at::native::reduce_kernel,-1,0,104,411408
BatchNorm,1,0,66,14969
volta_sgemm_128x64_tn,1,0,52,12834
void at::native::reduce_kernel,1,0,2997,5700
void at::native::vectorized_elementwise_kernel,-1,0,11,382181
void at::native::vectorized_elementwise_kernel,1,0,2374,477812
void at::native::vectorized_elementwise_kernel,0,0,2142,899030.5
volta_sgemm_128x64_tn,0,0,112,438095
BatchNorm,0,0,123,444986
BatchNorm,1,0,84,13094
Conv,1,0,1426,128828
void at::native::elementwise_kernel,-1,0,20,10042
void at::native::vectorized_elementwise_kernel,1,0,1,3734
void at::native::reduce_kernel,-1,0,130,16442
