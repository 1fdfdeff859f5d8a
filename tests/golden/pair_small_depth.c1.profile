Name,Profile,Memory_footprint,SM_usage,Duration
volta_sgemm_128x64_tn,0,0,9,637300
Conv,0,0,57,90276
void at::native::elementwise_kernel,1,0,79,19554
BatchNorm,-1,0,62,15335
Conv,0,0,3,195551
void at::native::vectorized_elementwise_kernel,-1,0,61,44532
void at::native::reduce_kernel,1,0,26,785067
void at::native::vectorized_elementwise_kernel,0,0,27,17968
void at::native::elementwise_kernel,0,0,56,17176
volta_sgemm_128x64_tn,1,0,37,2963
void at::native::vectorized_elementwise_kernel,0,0,67,12546
BatchNorm,-1,0,3972,54701
void at::native::reduce_kernel,0,0,47,3150
Conv,0,0,44,878119
void at::native::vectorized_elementwise_kernel,1,0,64,10531.5
void at::native::reduce_kernel,1,0,22,800364
void at::native::reduce_kernel,-1,0,44,6381.5
Conv,1,0,8,17075
volta_sgemm_128x64_tn,-1,0,67,7596
void at::native::elementwise_kernel,1,0,71,15374
void at::native::vectorized_elementwise_kernel,0,0,68,164848
void at::native::reduce_kernel,0,0,59,615944
volta_sgemm_128x64_tn,-1,0,593,295443
Conv,0,0,2075,791103
void at::native::vectorized_elementwise_kernel,1,0,51,3615
