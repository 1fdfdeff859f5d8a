Name,Profile,Memory_footprint,SM_usage,Duration
void at::native::reduce_kernel,-1,0,60,475780
volta_sgemm_128x64_tn,0,0,24,16633
volta_sgemm_128x64_tn,1,0,51,476999
Conv,1,0,3683,2985
volta_sgemm_128x64_tn,1,0,38,526050
void at::native::vectorized_elementwise_kernel,0,0,11,10322
volta_sgemm_128x64_tn,0,0,2387,5536
void at::native::vectorized_elementwise_kernel,0,0,150,890468
Conv,0,0,51,442183
void at::native::vectorized_elementwise_kernel,0,0,1443,17885
void at::native::elementwise_kernel,1,0,1985,837737
BatchNorm,0,0,17,441595
BatchNorm,1,0,3371,623533
void at::native::reduce_kernel,-1,0,13,46153
Conv,-1,0,38,406928.5
volta_sgemm_128x64_tn,1,0,1591,391759
void at::native::reduce_kernel,-1,0,1662,7050
volta_sgemm_128x64_tn,1,0,21,8441
volta_sgemm_128x64_tn,1,0,14,3268
void at::native::elementwise_kernel,0,0,3454,18089
void at::native::elementwise_kernel,1,0,2044,4429
BatchNorm,1,0,1766,469356.5
void at::native::vectorized_elementwise_kernel,0,0,17,98670
void at::native::vectorized_elementwise_kernel,-1,0,18,620529
void at::native::vectorized_elementwise_kernel,0,0,3,4452.5
void at::native::vectorized_elementwise_kernel,0,0,377,16846
void at::native::elementwise_kernel,1,0,44,4782
void at::native::reduce_kernel,1,0,74,14528
volta_sgemm_128x64_tn,1,0,2700,10428
void at::native::reduce_kernel,-1,0,60,881094
volta_sgemm_128x64_tn,1,0,12,506319
Conv,0,0,63,2370
void at::native::elementwise_kernel,-1,0,775,13223
BatchNorm,0,0,33,210148
void at::native::reduce_kernel,1,0,41,222088
Conv,1,0,36,863780
void at::native::vectorized_elementwise_kernel,1,0,49,19038
void at::native::elementwise_kernel,-1,0,10,3031
Conv,0,0,40,682826
BatchNorm,1,0,35,250941
