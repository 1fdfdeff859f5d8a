Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::vectorized_elementwise_kernel,0,0,54,239654
void at::native::elementwise_kernel,0,0,992,11718
void at::native::elementwise_kernel,1,0,78,327172
void at::native::vectorized_elementwise_kernel,1,0,78,2896
void at::native::elementwise_kernel,0,0,40,10461
void at::native::vectorized_elementwise_kernel,0,0,23,591975
Conv,1,0,31,7062
void at::native::reduce_kernel,0,0,2945,2428
void at::native::reduce_kernel,1,0,61,6028
Conv,0,0,19,9610
Conv,-1,0,2744,12465
void at::native::elementwise_kernel,1,0,494,743946
void at::native::reduce_kernel,1,0,15,3580
void at::native::elementwise_kernel,0,0,2465,13681
Conv,1,0,1748,15270
void at::native::reduce_kernel,0,0,323,8494
volta_sgemm_128x64_tn,0,0,965,121212
void at::native::reduce_kernel,0,0,1718,251077
void at::native::reduce_kernel,-1,0,837,381914
BatchNorm,0,0,63,321457
void at::native::vectorized_elementwise_kernel,0,0,2720,8853
void at::native::reduce_kernel,-1,0,2671,5516.5
Conv,0,0,7,540290.5
void at::native::vectorized_elementwise_kernel,0,0,346,8253
Conv,1,0,1699,638299
void at::native::elementwise_kernel,1,0,8,156462
void at::native::elementwise_kernel,-1,0,35,540713
void at::native::reduce_kernel,0,0,1968,786404
Conv,0,0,13,164891
void at::native::elementwise_kernel,1,0,30,8670.5
Conv,0,0,214,604016
BatchNorm,1,0,46,15207
volta_sgemm_128x64_tn,0,0,46,16454
void at::native::vectorized_elementwise_kernel,1,0,28,404276
void at::native::reduce_kernel,-1,0,67,427549
void at::native::reduce_kernel,1,0,22,3846.5
void at::native::reduce_kernel,0,0,5,152016
BatchNorm,-1,0,2817,620591.5
volta_sgemm_128x64_tn,-1,0,594,4619
volta_sgemm_128x64_tn,0,0,73,641582
BatchNorm,-1,0,1156,16556.5
void at::native::elementwise_kernel,0,0,73,826300
void at::native::vectorized_elementwise_kernel,0,0,3625,473555
Conv,0,0,26,88427
BatchNorm,0,0,14,781174
BatchNorm,0,0,38,384174
void at::native::elementwise_kernel,-1,0,423,293891
void at::native::elementwise_kernel,0,0,569,18183.5
Conv,0,0,16,15745
BatchNorm,-1,0,734,235504
void at::native::vectorized_elementwise_kernel,1,0,2722,6723.5
void at::native::vectorized_elementwise_kernel,0,0,44,12656
BatchNorm,0,0,159,2704
void at::native::reduce_kernel,-1,0,76,95257
volta_sgemm_128x64_tn,1,0,258,180304
Conv,0,0,32,17364
void at::native::vectorized_elementwise_kernel,0,0,1776,2323
BatchNorm,0,0,1,225415
volta_sgemm_128x64_tn,1,0,52,2506.5
void at::native::vectorized_elementwise_kernel,0,0,43,820604.5
