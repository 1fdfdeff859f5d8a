Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::reduce_kernel,-1,0,18,2210
volta_sgemm_128x64_tn,1,0,79,3340
void at::native::reduce_kernel,0,0,31,55827
volta_sgemm_128x64_tn,1,0,50,5331
BatchNorm,0,0,35,14993
Conv,1,0,1,3795
BatchNorm,1,0,15,627838
BatchNorm,1,0,11,141652
volta_sgemm_128x64_tn,0,0,26,4255
Conv,-1,0,78,756592
void at::native::elementwise_kernel,-1,0,35,774677
void at::native::reduce_kernel,1,0,65,47121
Conv,-1,0,27,423706
volta_sgemm_128x64_tn,0,0,538,9264
Conv,0,0,14,544642
volta_sgemm_128x64_tn,0,0,32,4171
Conv,0,0,72,6559
void at::native::vectorized_elementwise_kernel,1,0,3397,183147
volta_sgemm_128x64_tn,1,0,330,8835
Conv,0,0,62,591228
void at::native::elementwise_kernel,-1,0,16,15760
volta_sgemm_128x64_tn,0,0,22,10983
Conv,0,0,23,839194
BatchNorm,1,0,61,19875.5
volta_sgemm_128x64_tn,0,0,34,563438
volta_sgemm_128x64_tn,0,0,68,554590
volta_sgemm_128x64_tn,-1,0,9,762141
void at::native::elementwise_kernel,0,0,63,669692
void at::native::reduce_kernel,1,0,74,657345.5
volta_sgemm_128x64_tn,1,0,53,428431
volta_sgemm_128x64_tn,1,0,203,17408.5
Conv,0,0,1397,17199
void at::native::reduce_kernel,0,0,14,9579
BatchNorm,1,0,7,127924
void at::native::elementwise_kernel,1,0,67,212427
void at::native::vectorized_elementwise_kernel,-1,0,2,462593
volta_sgemm_128x64_tn,0,0,1110,500679
void at::native::elementwise_kernel,0,0,5,8117
void at::native::reduce_kernel,1,0,39,2965
void at::native::reduce_kernel,-1,0,73,15077
