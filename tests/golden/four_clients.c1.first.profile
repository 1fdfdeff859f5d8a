Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::elementwise_kernel,1,0,3372,21045.5
void at::native::elementwise_kernel,-1,0,25,541214
Conv,0,0,70,14880
BatchNorm,0,0,3693,6578
Conv,1,0,2642,10375
Conv,0,0,37,9936.5
BatchNorm,1,0,95,13932
volta_sgemm_128x64_tn,0,0,3695,9139
void at::native::vectorized_elementwise_kernel,0,0,1223,529186
Conv,1,0,448,152853
void at::native::vectorized_elementwise_kernel,0,0,11,616028
void at::native::elementwise_kernel,-1,0,42,757684
volta_sgemm_128x64_tn,1,0,3502,18809
volta_sgemm_128x64_tn,1,0,65,598093.5
Conv,1,0,14,396912
void at::native::elementwise_kernel,-1,0,63,2108
void at::native::elementwise_kernel,-1,0,12,693325
void at::native::reduce_kernel,0,0,34,248190
void at::native::reduce_kernel,0,0,10,504278
void at::native::elementwise_kernel,1,0,684,10321
