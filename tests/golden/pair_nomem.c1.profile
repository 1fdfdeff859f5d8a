Name,Profile,Memory_footprint,SM_usage,Duration
volta_sgemm_128x64_tn,1,0,22,82398
Conv,-1,0,70,15337
void at::native::reduce_kernel,-1,0,32,15706.5
void at::native::vectorized_elementwise_kernel,1,0,20,123211
void at::native::vectorized_elementwise_kernel,-1,0,3303,725753.5
void at::native::reduce_kernel,1,0,10,8204
BatchNorm,-1,0,62,882709
BatchNorm,1,0,703,5437
BatchNorm,-1,0,14,385083
void at::native::vectorized_elementwise_kernel,0,0,3730,715556
volta_sgemm_128x64_tn,0,0,16,628089
void at::native::reduce_kernel,0,0,10,516522
void at::native::reduce_kernel,0,0,26,362329
void at::native::reduce_kernel,1,0,38,429926
Conv,1,0,31,286226
Conv,-1,0,24,569656.5
void at::native::vectorized_elementwise_kernel,1,0,1,6614
Conv,0,0,50,543870
BatchNorm,0,0,2207,11147
Conv,1,0,65,457811.5
void at::native::elementwise_kernel,0,0,56,398927
BatchNorm,0,0,55,4514
void at::native::reduce_kernel,1,0,61,383067
Conv,1,0,10,79497
BatchNorm,1,0,64,335093
