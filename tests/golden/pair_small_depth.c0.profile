Name,Profile,Memory_footprint,SM_usage,Duration
BatchNorm,-1,0,48,635256
void at::native::reduce_kernel,0,0,25,17409
BatchNorm,1,0,67,410878
volta_sgemm_128x64_tn,1,0,4,10828
void at::native::reduce_kernel,0,0,74,6395.5
BatchNorm,0,0,2833,11864
void at::native::reduce_kernel,-1,0,75,9614
Conv,0,0,21,734551
BatchNorm,-1,0,590,17794.5
Conv,0,0,3,15996
Conv,-1,0,6,12844
Conv,0,0,523,630896
void at::native::reduce_kernel,0,0,20,3390
BatchNorm,0,0,67,5361
void at::native::elementwise_kernel,1,0,56,19076
Conv,0,0,41,23026.5
void at::native::elementwise_kernel,0,0,46,11139.5
Conv,1,0,33,16952
void at::native::vectorized_elementwise_kernel,1,0,41,14096
void at::native::reduce_kernel,1,0,4,6306
void at::native::elementwise_kernel,0,0,848,713001
void at::native::vectorized_elementwise_kernel,0,0,29,461727
void at::native::elementwise_kernel,1,0,58,285744.5
BatchNorm,0,0,74,11128
void at::native::elementwise_kernel,1,0,45,6249
void at::native::vectorized_elementwise_kernel,0,0,54,15755.5
void at::native::reduce_kernel,1,0,2036,18716
void at::native::elementwise_kernel,1,0,1951,19007
BatchNorm,1,0,37,127825.5
void at::native::elementwise_kernel,-1,0,56,606979
Conv,1,0,31,2650.5
volta_sgemm_128x64_tn,1,0,33,569259
BatchNorm,1,0,16,9846
BatchNorm,1,0,74,3636
volta_sgemm_128x64_tn,-1,0,7,497871
BatchNorm,1,0,361,508266
void at::native::reduce_kernel,0,0,374,14641
void at::native::vectorized_elementwise_kernel,0,0,1427,451524
void at::native::elementwise_kernel,0,0,73,3407
void at::native::elementwise_kernel,-1,0,6,655185
void at::native::reduce_kernel,0,0,54,485225
void at::native::vectorized_elementwise_kernel,-1,0,1821,237343
void at::native::vectorized_elementwise_kernel,0,0,72,831336
Conv,-1,0,14,771377
void at::native::elementwise_kernel,1,0,31,813916
volta_sgemm_128x64_tn,1,0,49,2769
Conv,1,0,62,11322
Conv,-1,0,31,113928
volta_sgemm_128x64_tn,1,0,31,10190
void at::native::reduce_kernel,0,0,51,369299
BatchNorm,0,0,21,18944
void at::native::reduce_kernel,1,0,2120,17843
BatchNorm,1,0,896,18895
void at::native::elementwise_kernel,-1,0,38,15539
void at::native::vectorized_elementwise_kernel,1,0,3374,403342
BatchNorm,0,0,19,440741
void at::native::elementwise_kernel,-1,0,3033,77890
BatchNorm,1,0,9,229930
void at::native::vectorized_elementwise_kernel,1,0,2967,3204
Conv,0,0,453,766378.5
