Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::vectorized_elementwise_kernel,1,0,14,13406
void at::native::elementwise_kernel,0,0,37,536075.5
void at::native::reduce_kernel,1,0,69,752084
volta_sgemm_128x64_tn,-1,0,55,441784
Conv,1,0,46,7944.5
Conv,1,0,29,4074
volta_sgemm_128x64_tn,1,0,71,201145
Conv,-1,0,75,685298
volta_sgemm_128x64_tn,0,0,17,164311
void at::native::vectorized_elementwise_kernel,1,0,74,18921
volta_sgemm_128x64_tn,0,0,2516,136046.5
void at::native::elementwise_kernel,1,0,53,10205
BatchNorm,0,0,29,3029
Conv,0,0,4,17639
BatchNorm,0,0,47,549309
volta_sgemm_128x64_tn,1,0,47,442213
void at::native::elementwise_kernel,0,0,2530,19081.5
void at::native::elementwise_kernel,0,0,47,838989
void at::native::elementwise_kernel,1,0,64,7657
void at::native::vectorized_elementwise_kernel,-1,0,39,10668
void at::native::reduce_kernel,-1,0,1943,108266
void at::native::vectorized_elementwise_kernel,0,0,52,189308
void at::native::reduce_kernel,0,0,31,468279
void at::native::vectorized_elementwise_kernel,0,0,2977,2308
void at::native::elementwise_kernel,-1,0,62,671914
