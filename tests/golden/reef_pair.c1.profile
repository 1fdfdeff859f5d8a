Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::elementwise_kernel,1,0,6,432551
Conv,0,0,4,551302
void at::native::reduce_kernel,0,0,32,7316
void at::native::vectorized_elementwise_kernel,1,0,68,308209
void at::native::elementwise_kernel,1,0,20,815626
Conv,-1,0,5,329733
BatchNorm,-1,0,61,625678
void at::native::vectorized_elementwise_kernel,0,0,3183,19964
void at::native::reduce_kernel,0,0,44,694322
BatchNorm,0,0,3962,14614
Conv,1,0,61,391609
volta_sgemm_128x64_tn,1,0,42,153769
volta_sgemm_128x64_tn,0,0,7,159971
BatchNorm,1,0,1186,646730
void at::native::elementwise_kernel,0,0,3147,19806.5
BatchNorm,0,0,2875,97363.5
void at::native::reduce_kernel,-1,0,40,12182.5
void at::native::vectorized_elementwise_kernel,0,0,9,379182
void at::native::reduce_kernel,0,0,16,687702
void at::native::elementwise_kernel,0,0,73,120829
void at::native::elementwise_kernel,1,0,20,14320
void at::native::reduce_kernel,-1,0,33,8551
void at::native::vectorized_elementwise_kernel,0,0,73,12867
Conv,1,0,467,139824
Conv,0,0,12,107310
