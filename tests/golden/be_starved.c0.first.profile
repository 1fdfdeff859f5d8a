Name,Profile,Memory_footprint,SM_usage,Duration
BatchNorm,1,0,229,167688.5
void at::native::elementwise_kernel,1,0,1585,5838
void at::native::vectorized_elementwise_kernel,0,0,1491,8762
BatchNorm,0,0,66,9582
void at::native::reduce_kernel,1,0,3353,16395
void at::native::elementwise_kernel,0,0,3618,4157
Conv,1,0,786,2569
BatchNorm,1,0,1700,4411
volta_sgemm_128x64_tn,0,0,2137,7872.5
void at::native::vectorized_elementwise_kernel,0,0,2645,14677
void at::native::reduce_kernel,1,0,3512,10927
void at::native::elementwise_kernel,0,0,144,882806
Conv,0,0,3949,7189
void at::native::reduce_kernel,1,0,2024,4677
volta_sgemm_128x64_tn,0,0,1128,713206.5
void at::native::elementwise_kernel,0,0,310,11906
Conv,0,0,3737,2492
volta_sgemm_128x64_tn,1,0,1102,18796
BatchNorm,-1,0,1386,4666
Conv,1,0,2151,5547
BatchNorm,0,0,1488,19949
Conv,0,0,75,6802
void at::native::reduce_kernel,1,0,2451,12557
volta_sgemm_128x64_tn,-1,0,2252,760653
void at::native::elementwise_kernel,0,0,2557,596181
BatchNorm,0,0,845,65357.5
void at::native::elementwise_kernel,0,0,2853,76196
BatchNorm,0,0,3626,14068
void at::native::elementwise_kernel,1,0,2413,155773
void at::native::reduce_kernel,0,0,781,4241
void at::native::reduce_kernel,1,0,178,12895
BatchNorm,1,0,96,17057.5
void at::native::reduce_kernel,0,0,1153,16890
void at::native::elementwise_kernel,-1,0,761,12258
void at::native::vectorized_elementwise_kernel,-1,0,427,225973
volta_sgemm_128x64_tn,0,0,2929,12861
void at::native::reduce_kernel,0,0,3633,286169
void at::native::elementwise_kernel,1,0,2436,274722
volta_sgemm_128x64_tn,1,0,62,545055
void at::native::reduce_kernel,0,0,1255,15354
