Name,Profile,Memory_footprint,SM_usage,Duration
volta_sgemm_128x64_tn,0,0,68,32414
BatchNorm,1,0,32,401253
Conv,1,0,24,804921
Conv,1,0,57,134853
Conv,1,0,22,11479
volta_sgemm_128x64_tn,1,0,26,403838
BatchNorm,1,0,43,2110.5
void at::native::vectorized_elementwise_kernel,0,0,41,17768
Conv,0,0,3,13719.5
void at::native::reduce_kernel,0,0,2,476818
BatchNorm,1,0,60,18793
void at::native::vectorized_elementwise_kernel,0,0,48,3200
Conv,1,0,79,6856
void at::native::elementwise_kernel,-1,0,41,323043
void at::native::elementwise_kernel,0,0,21,757109
volta_sgemm_128x64_tn,0,0,77,10198
BatchNorm,1,0,5,18173
BatchNorm,-1,0,53,7531
Conv,0,0,59,7547
void at::native::elementwise_kernel,0,0,38,494915
volta_sgemm_128x64_tn,1,0,64,356920
volta_sgemm_128x64_tn,-1,0,47,68174
void at::native::vectorized_elementwise_kernel,-1,0,36,17914
void at::native::elementwise_kernel,0,0,44,683251
void at::native::vectorized_elementwise_kernel,0,0,60,18395
void at::native::elementwise_kernel,0,0,53,7651
void at::native::vectorized_elementwise_kernel,-1,0,22,13862
Conv,0,0,75,15788
void at::native::elementwise_kernel,0,0,4,7243
BatchNorm,1,0,24,3371
BatchNorm,1,0,15,7948
Conv,0,0,49,696706
void at::native::vectorized_elementwise_kernel,1,0,36,899428
volta_sgemm_128x64_tn,0,0,71,645368
volta_sgemm_128x64_tn,0,0,38,6232
volta_sgemm_128x64_tn,-1,0,19,14541
BatchNorm,-1,0,1,5536
volta_sgemm_128x64_tn,-1,0,73,16064
void at::native::reduce_kernel,0,0,49,7211
void at::native::vectorized_elementwise_kernel,0,0,3,12075
BatchNorm,0,0,80,10044.5
BatchNorm,0,0,69,589533
Conv,1,0,20,11362
void at::native::reduce_kernel,-1,0,78,781588
void at::native::vectorized_elementwise_kernel,0,0,44,645376
void at::native::vectorized_elementwise_kernel,-1,0,1,266684
volta_sgemm_128x64_tn,1,0,55,17790
void at::native::elementwise_kernel,1,0,60,4164
void at::native::elementwise_kernel,0,0,61,328055
volta_sgemm_128x64_tn,0,0,69,162985.5
BatchNorm,0,0,9,2837
Conv,0,0,7,131368
Conv,1,0,57,159003
BatchNorm,1,0,6,5545
void at::native::vectorized_elementwise_kernel,1,0,16,780397.5
Conv,0,0,63,13580
BatchNorm,0,0,65,9228.5
BatchNorm,0,0,37,544109
void at::native::reduce_kernel,0,0,3,688831
Conv,1,0,65,624827
