Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::reduce_kernel,0,0,14,558432.5
volta_sgemm_128x64_tn,1,0,35,18682
BatchNorm,0,0,6,17596
Conv,0,0,4,9531
void at::native::elementwise_kernel,1,0,27,8484
void at::native::vectorized_elementwise_kernel,1,0,72,38809
void at::native::vectorized_elementwise_kernel,0,0,13,3575
void at::native::reduce_kernel,1,0,29,760668
void at::native::elementwise_kernel,1,0,44,14584
Conv,0,0,3284,12322.5
void at::native::elementwise_kernel,1,0,18,189908
Conv,0,0,11,5739
BatchNorm,-1,0,78,4982
void at::native::elementwise_kernel,0,0,70,565648
BatchNorm,0,0,764,16843
void at::native::reduce_kernel,-1,0,68,366182
BatchNorm,0,0,30,153159
void at::native::elementwise_kernel,1,0,17,344419
BatchNorm,1,0,26,300114
BatchNorm,1,0,61,3401
Conv,0,0,29,585420
void at::native::elementwise_kernel,0,0,18,14362
void at::native::vectorized_elementwise_kernel,1,0,19,18996.5
void at::native::reduce_kernel,0,0,14,520637
void at::native::vectorized_elementwise_kernel,1,0,547,269008
