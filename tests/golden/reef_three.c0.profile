Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::reduce_kernel,0,0,45,151527
void at::native::reduce_kernel,0,0,59,726138
BatchNorm,0,0,44,222464.5
void at::native::elementwise_kernel,0,0,12,21508.5
void at::native::reduce_kernel,0,0,1814,19678
volta_sgemm_128x64_tn,1,0,7,584117
void at::native::reduce_kernel,-1,0,78,405262
Conv,1,0,34,13898
Conv,0,0,1569,391300.5
void at::native::reduce_kernel,1,0,29,710474
volta_sgemm_128x64_tn,1,0,29,4555.5
void at::native::vectorized_elementwise_kernel,0,0,7,17049
void at::native::vectorized_elementwise_kernel,0,0,62,7490
void at::native::vectorized_elementwise_kernel,1,0,3146,2218
void at::native::vectorized_elementwise_kernel,1,0,116,527762
void at::native::vectorized_elementwise_kernel,-1,0,4,340120
volta_sgemm_128x64_tn,-1,0,46,277437
volta_sgemm_128x64_tn,1,0,3947,542197
volta_sgemm_128x64_tn,0,0,96,729821
void at::native::vectorized_elementwise_kernel,0,0,901,458423
volta_sgemm_128x64_tn,0,0,54,5043
volta_sgemm_128x64_tn,-1,0,48,671058.5
void at::native::elementwise_kernel,1,0,5,78536
void at::native::reduce_kernel,1,0,25,10870
Conv,1,0,51,610890
void at::native::vectorized_elementwise_kernel,1,0,19,4966
BatchNorm,0,0,4,17984
Conv,-1,0,31,345355.5
void at::native::vectorized_elementwise_kernel,0,0,905,16170
BatchNorm,-1,0,43,18407
volta_sgemm_128x64_tn,1,0,7,9454
void at::native::reduce_kernel,-1,0,7,12225
Conv,0,0,47,665260
BatchNorm,-1,0,2106,16060
void at::native::elementwise_kernel,-1,0,3410,829770
void at::native::elementwise_kernel,1,0,78,14400
void at::native::elementwise_kernel,0,0,49,14604
BatchNorm,1,0,33,116979
void at::native::elementwise_kernel,0,0,40,6498
BatchNorm,1,0,6,15584
void at::native::elementwise_kernel,0,0,24,813071
Conv,0,0,69,211977
void at::native::elementwise_kernel,1,0,65,11614
void at::native::reduce_kernel,0,0,4,751744
void at::native::reduce_kernel,0,0,55,15299
BatchNorm,0,0,523,445611
BatchNorm,1,0,2887,594226
void at::native::reduce_kernel,1,0,44,19796
void at::native::reduce_kernel,1,0,44,63581
void at::native::reduce_kernel,-1,0,1218,15149
void at::native::reduce_kernel,0,0,41,14505
volta_sgemm_128x64_tn,-1,0,9,13185
volta_sgemm_128x64_tn,1,0,57,11143
Conv,1,0,64,183218
volta_sgemm_128x64_tn,0,0,40,13627
volta_sgemm_128x64_tn,0,0,2639,8716
volta_sgemm_128x64_tn,0,0,19,13020
void at::native::elementwise_kernel,0,0,1426,680997
volta_sgemm_128x64_tn,1,0,21,851109
BatchNorm,0,0,356,884030
