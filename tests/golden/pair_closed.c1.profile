Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::reduce_kernel,-1,0,41,44066
BatchNorm,0,0,58,19187.5
void at::native::vectorized_elementwise_kernel,1,0,50,10552
void at::native::vectorized_elementwise_kernel,0,0,39,100627
BatchNorm,0,0,66,14815
void at::native::elementwise_kernel,0,0,72,756326
void at::native::vectorized_elementwise_kernel,1,0,1675,548389
BatchNorm,-1,0,1311,19487
void at::native::vectorized_elementwise_kernel,0,0,67,527396
void at::native::elementwise_kernel,0,0,74,16805
void at::native::vectorized_elementwise_kernel,0,0,11,609091.5
void at::native::reduce_kernel,-1,0,33,10040
void at::native::elementwise_kernel,0,0,60,629322.5
void at::native::vectorized_elementwise_kernel,1,0,15,195567
volta_sgemm_128x64_tn,0,0,27,276409
BatchNorm,1,0,56,14062
void at::native::vectorized_elementwise_kernel,1,0,77,9707
void at::native::vectorized_elementwise_kernel,-1,0,25,838932
void at::native::vectorized_elementwise_kernel,0,0,69,14475.5
volta_sgemm_128x64_tn,-1,0,75,3314
void at::native::reduce_kernel,1,0,1307,731804
volta_sgemm_128x64_tn,0,0,70,11257
volta_sgemm_128x64_tn,0,0,75,16828
void at::native::reduce_kernel,-1,0,3245,172887
void at::native::elementwise_kernel,-1,0,1804,423673
