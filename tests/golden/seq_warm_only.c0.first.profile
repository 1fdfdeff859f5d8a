Name,Profile,Memory_footprint,SM_usage,Duration
Conv,-1,0,68,10883
Conv,0,0,51,5879
void at::native::vectorized_elementwise_kernel,0,0,47,845350
void at::native::elementwise_kernel,0,0,2750,6031.5
void at::native::vectorized_elementwise_kernel,1,0,49,425284
void at::native::elementwise_kernel,1,0,47,5102
BatchNorm,0,0,28,11218
Conv,0,0,195,171571
volta_sgemm_128x64_tn,1,0,22,14671
void at::native::reduce_kernel,0,0,13,17549
volta_sgemm_128x64_tn,0,0,667,10742.5
void at::native::elementwise_kernel,0,0,55,13386
void at::native::vectorized_elementwise_kernel,0,0,25,17376.5
Conv,1,0,184,18602
void at::native::vectorized_elementwise_kernel,0,0,3998,155302
volta_sgemm_128x64_tn,0,0,932,12879
void at::native::vectorized_elementwise_kernel,1,0,77,779268
void at::native::reduce_kernel,1,0,70,12303
volta_sgemm_128x64_tn,1,0,3905,17365.5
Conv,1,0,2916,8932
BatchNorm,-1,0,7,5485
volta_sgemm_128x64_tn,0,0,57,235112
BatchNorm,1,0,3801,234822
void at::native::reduce_kernel,0,0,42,82439
void at::native::elementwise_kernel,-1,0,9,449049
BatchNorm,1,0,2852,322007
volta_sgemm_128x64_tn,1,0,1922,493472
void at::native::vectorized_elementwise_kernel,1,0,2511,679210
BatchNorm,1,0,15,6044
void at::native::vectorized_elementwise_kernel,0,0,43,32679
volta_sgemm_128x64_tn,0,0,68,614588
Conv,0,0,50,15844
void at::native::reduce_kernel,1,0,49,752264
volta_sgemm_128x64_tn,1,0,31,206614
Conv,0,0,72,54689
void at::native::elementwise_kernel,-1,0,55,483903
void at::native::elementwise_kernel,1,0,59,8636
void at::native::vectorized_elementwise_kernel,0,0,2872,12943
void at::native::vectorized_elementwise_kernel,1,0,2688,6362
void at::native::vectorized_elementwise_kernel,-1,0,308,2998
