Name,Profile,Memory_footprint,SM_usage,Duration
BatchNorm,0,0,27,4262
Conv,-1,0,41,15375
void at::native::elementwise_kernel,1,0,2765,589415
void at::native::vectorized_elementwise_kernel,1,0,46,301484.5
volta_sgemm_128x64_tn,-1,0,15,3302
void at::native::reduce_kernel,0,0,31,15865
void at::native::reduce_kernel,0,0,70,627852
Conv,0,0,51,18764
volta_sgemm_128x64_tn,1,0,378,105864
void at::native::elementwise_kernel,1,0,1,377258.5
Conv,0,0,79,8582
Conv,0,0,46,6761
volta_sgemm_128x64_tn,1,0,28,5781
void at::native::elementwise_kernel,1,0,2400,595543
BatchNorm,0,0,77,11995
void at::native::elementwise_kernel,0,0,45,5837
void at::native::vectorized_elementwise_kernel,1,0,2175,872236
Conv,1,0,65,2576.5
BatchNorm,1,0,36,181260
volta_sgemm_128x64_tn,1,0,2,12616.5
Conv,0,0,21,889238
volta_sgemm_128x64_tn,0,0,2391,14576
void at::native::reduce_kernel,-1,0,76,2012
Conv,1,0,608,2102
void at::native::elementwise_kernel,-1,0,1499,15336
Conv,1,0,570,482604
void at::native::elementwise_kernel,1,0,3665,276056.5
void at::native::elementwise_kernel,1,0,41,80716
void at::native::vectorized_elementwise_kernel,0,0,1101,19358
Conv,1,0,558,14966
void at::native::reduce_kernel,0,0,3549,6852
BatchNorm,0,0,49,367677
Conv,0,0,22,734398
BatchNorm,0,0,32,433658
void at::native::reduce_kernel,-1,0,5,5937.5
void at::native::vectorized_elementwise_kernel,-1,0,60,839771
void at::native::reduce_kernel,1,0,19,19804.5
Conv,1,0,964,213498
BatchNorm,1,0,77,18749
Conv,-1,0,43,665593
volta_sgemm_128x64_tn,0,0,3793,9505
BatchNorm,0,0,2329,87699
Conv,1,0,80,4049
void at::native::vectorized_elementwise_kernel,0,0,21,29175
Conv,1,0,39,16294.5
void at::native::vectorized_elementwise_kernel,1,0,1067,15944
void at::native::elementwise_kernel,0,0,36,5880
volta_sgemm_128x64_tn,0,0,3865,265231
void at::native::reduce_kernel,0,0,3599,9048
void at::native::reduce_kernel,1,0,55,194344
void at::native::vectorized_elementwise_kernel,0,0,27,563309
volta_sgemm_128x64_tn,0,0,18,14079
void at::native::elementwise_kernel,0,0,3579,91520
void at::native::vectorized_elementwise_kernel,1,0,3561,875246
void at::native::elementwise_kernel,0,0,35,9092
Conv,-1,0,3786,3614
void at::native::vectorized_elementwise_kernel,0,0,65,5459
BatchNorm,0,0,72,16172
void at::native::vectorized_elementwise_kernel,1,0,21,11915
volta_sgemm_128x64_tn,-1,0,2488,10139
