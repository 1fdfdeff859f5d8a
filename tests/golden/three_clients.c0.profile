Name,Profile,Memory_footprint,SM_usage,Duration
volta_sgemm_128x64_tn,1,0,34,40611
void at::native::reduce_kernel,0,0,3,287944
void at::native::reduce_kernel,-1,0,13,204359
void at::native::vectorized_elementwise_kernel,1,0,53,10207
BatchNorm,0,0,268,8582
BatchNorm,-1,0,65,31802
void at::native::vectorized_elementwise_kernel,0,0,12,526452
void at::native::elementwise_kernel,0,0,26,400256
BatchNorm,-1,0,3267,2558
void at::native::elementwise_kernel,-1,0,48,19280
void at::native::elementwise_kernel,0,0,1813,624780
BatchNorm,1,0,58,470917
void at::native::reduce_kernel,0,0,53,8296
void at::native::elementwise_kernel,1,0,2284,10229
volta_sgemm_128x64_tn,0,0,67,15453
void at::native::vectorized_elementwise_kernel,-1,0,62,6659
void at::native::elementwise_kernel,0,0,21,14322
void at::native::reduce_kernel,0,0,21,869896
Conv,1,0,3249,5674
void at::native::reduce_kernel,-1,0,870,163887
volta_sgemm_128x64_tn,0,0,1031,14154
void at::native::elementwise_kernel,1,0,19,41510.5
void at::native::reduce_kernel,0,0,9,661761
Conv,1,0,34,16810
void at::native::elementwise_kernel,1,0,25,17701
void at::native::vectorized_elementwise_kernel,0,0,9,11560
Conv,1,0,36,10982
void at::native::vectorized_elementwise_kernel,1,0,32,858027
void at::native::vectorized_elementwise_kernel,0,0,3979,8854
Conv,1,0,15,421066
void at::native::reduce_kernel,1,0,1516,547539
BatchNorm,1,0,699,533964
void at::native::elementwise_kernel,-1,0,17,7347
volta_sgemm_128x64_tn,-1,0,3378,598550
void at::native::reduce_kernel,-1,0,51,887910
void at::native::elementwise_kernel,-1,0,48,287107
void at::native::elementwise_kernel,1,0,8,3306
Conv,-1,0,1586,626552
void at::native::reduce_kernel,1,0,38,99216
Conv,1,0,57,127890.5
Conv,0,0,37,270109
void at::native::elementwise_kernel,-1,0,28,2429
void at::native::elementwise_kernel,0,0,12,3072
Conv,1,0,4,13160
Conv,0,0,121,4231.5
void at::native::vectorized_elementwise_kernel,1,0,79,288501
volta_sgemm_128x64_tn,1,0,2796,16060
void at::native::vectorized_elementwise_kernel,1,0,215,203883
volta_sgemm_128x64_tn,1,0,1,540515
void at::native::reduce_kernel,0,0,68,19743
void at::native::elementwise_kernel,0,0,3845,2349
void at::native::vectorized_elementwise_kernel,1,0,2490,898562.5
void at::native::vectorized_elementwise_kernel,1,0,2630,652468
void at::native::reduce_kernel,1,0,19,3649
void at::native::vectorized_elementwise_kernel,-1,0,35,4186
Conv,-1,0,20,861791
Conv,1,0,16,13502
void at::native::elementwise_kernel,1,0,834,6112
void at::native::reduce_kernel,-1,0,2596,145328
void at::native::elementwise_kernel,1,0,34,73597.5
