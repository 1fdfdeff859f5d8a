Name,Profile,Memory_footprint,SM_usage,Duration
Conv,1,0,30,381493
void at::native::elementwise_kernel,1,0,32,234755
volta_sgemm_128x64_tn,0,0,24,3876
void at::native::vectorized_elementwise_kernel,0,0,1714,16799.5
void at::native::vectorized_elementwise_kernel,1,0,5,6449
void at::native::vectorized_elementwise_kernel,1,0,67,2795
Conv,1,0,13,105513
void at::native::vectorized_elementwise_kernel,1,0,58,245589
volta_sgemm_128x64_tn,0,0,2049,684145
void at::native::vectorized_elementwise_kernel,1,0,2361,10563.5
void at::native::reduce_kernel,-1,0,3020,2142
void at::native::reduce_kernel,1,0,22,16325
void at::native::vectorized_elementwise_kernel,-1,0,2028,5200
Conv,-1,0,56,19856
void at::native::reduce_kernel,-1,0,71,361626
volta_sgemm_128x64_tn,1,0,67,14129
Conv,1,0,2270,729807
void at::native::reduce_kernel,1,0,2796,692059
void at::native::reduce_kernel,1,0,50,543163
void at::native::elementwise_kernel,1,0,62,6265
Conv,1,0,63,17416
void at::native::reduce_kernel,-1,0,2080,13654
BatchNorm,-1,0,3174,19992
void at::native::reduce_kernel,1,0,15,172197
volta_sgemm_128x64_tn,-1,0,48,15463
