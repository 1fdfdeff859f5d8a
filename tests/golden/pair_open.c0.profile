Name,Profile,Memory_footprint,SM_usage,Duration
Conv,1,0,3503,12097
volta_sgemm_128x64_tn,1,0,21,14895
void at::native::reduce_kernel,-1,0,228,13928
void at::native::reduce_kernel,0,0,68,174478
BatchNorm,0,0,2170,537008
void at::native::reduce_kernel,0,0,47,13592
void at::native::reduce_kernel,1,0,52,751890
void at::native::reduce_kernel,-1,0,46,16899
void at::native::elementwise_kernel,-1,0,63,9268
BatchNorm,-1,0,3814,12143
void at::native::elementwise_kernel,-1,0,65,15325
void at::native::reduce_kernel,-1,0,80,81036
BatchNorm,1,0,2755,53285
Conv,-1,0,1169,258724
void at::native::elementwise_kernel,1,0,1556,182230.5
Conv,1,0,3843,14225
BatchNorm,1,0,1,406295
Conv,1,0,79,5706
Conv,0,0,78,3499
volta_sgemm_128x64_tn,1,0,29,99993.5
BatchNorm,-1,0,51,18869
void at::native::vectorized_elementwise_kernel,0,0,1800,687050
void at::native::vectorized_elementwise_kernel,1,0,780,102529
void at::native::elementwise_kernel,1,0,30,750544
volta_sgemm_128x64_tn,1,0,80,13790
void at::native::vectorized_elementwise_kernel,-1,0,20,14607
volta_sgemm_128x64_tn,1,0,489,22763
Conv,-1,0,59,19548
BatchNorm,0,0,3,3678
volta_sgemm_128x64_tn,1,0,62,385971
void at::native::vectorized_elementwise_kernel,0,0,53,5441
void at::native::elementwise_kernel,1,0,8,17920
volta_sgemm_128x64_tn,-1,0,1245,14219
Conv,1,0,25,14235
BatchNorm,0,0,16,268508.5
void at::native::vectorized_elementwise_kernel,0,0,14,27867
void at::native::reduce_kernel,0,0,59,14285
void at::native::reduce_kernel,0,0,38,415843
void at::native::vectorized_elementwise_kernel,-1,0,11,616361
volta_sgemm_128x64_tn,1,0,9,839361
void at::native::vectorized_elementwise_kernel,0,0,2828,12794
void at::native::vectorized_elementwise_kernel,1,0,3971,794489
BatchNorm,-1,0,3746,167162
void at::native::vectorized_elementwise_kernel,-1,0,60,2962
BatchNorm,0,0,62,15268
void at::native::reduce_kernel,0,0,71,348792
BatchNorm,0,0,49,2380
void at::native::elementwise_kernel,0,0,13,19969
volta_sgemm_128x64_tn,0,0,13,8538
volta_sgemm_128x64_tn,-1,0,3374,643650
void at::native::reduce_kernel,0,0,2399,183998
Conv,0,0,2069,4144
void at::native::vectorized_elementwise_kernel,0,0,2140,484681
void at::native::vectorized_elementwise_kernel,1,0,52,269693
void at::native::reduce_kernel,0,0,20,11262
void at::native::vectorized_elementwise_kernel,1,0,49,593718
void at::native::vectorized_elementwise_kernel,0,0,62,19647.5
void at::native::vectorized_elementwise_kernel,0,0,40,687149
BatchNorm,0,0,20,838621
BatchNorm,0,0,67,292965
