Name,Profile,Memory_footprint,SM_usage,Duration
BatchNorm,0,0,66,331833
Conv,1,0,76,16862
void at::native::elementwise_kernel,-1,0,43,16497.5
Conv,0,0,4,283513
Conv,0,0,1742,118391
void at::native::vectorized_elementwise_kernel,0,0,61,167181.5
void at::native::vectorized_elementwise_kernel,0,0,38,2895
void at::native::reduce_kernel,1,0,31,14504
volta_sgemm_128x64_tn,1,0,62,8352
BatchNorm,-1,0,15,4207
void at::native::vectorized_elementwise_kernel,0,0,25,8735
void at::native::vectorized_elementwise_kernel,-1,0,8,3901
BatchNorm,1,0,29,6524
volta_sgemm_128x64_tn,-1,0,45,7498
BatchNorm,1,0,3971,221732
void at::native::elementwise_kernel,0,0,8,5281.5
void at::native::vectorized_elementwise_kernel,1,0,58,7974
Conv,1,0,11,687012
void at::native::vectorized_elementwise_kernel,1,0,4,17258
Conv,0,0,66,884881
void at::native::elementwise_kernel,-1,0,2270,864220
Conv,0,0,271,124606
volta_sgemm_128x64_tn,1,0,28,617353
BatchNorm,1,0,433,802748
void at::native::reduce_kernel,0,0,4,299067
Conv,0,0,50,259984
Conv,-1,0,49,808634.5
volta_sgemm_128x64_tn,1,0,1078,655754
Conv,1,0,76,9028
void at::native::vectorized_elementwise_kernel,0,0,47,4974
void at::native::vectorized_elementwise_kernel,0,0,39,6278
void at::native::reduce_kernel,-1,0,28,4543
BatchNorm,-1,0,3364,2981.5
BatchNorm,1,0,14,787837
Conv,1,0,38,335131
void at::native::elementwise_kernel,1,0,2950,18230
void at::native::vectorized_elementwise_kernel,0,0,46,671274
void at::native::reduce_kernel,0,0,19,19225.5
void at::native::elementwise_kernel,1,0,20,28294
void at::native::vectorized_elementwise_kernel,-1,0,66,449271
