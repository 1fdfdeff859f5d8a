Name,Profile,Memory_footprint,SM_usage,Duration
volta_sgemm_128x64_tn,1,0,74,8753
void at::native::vectorized_elementwise_kernel,1,0,2088,345694
void at::native::elementwise_kernel,0,0,3604,13635
void at::native::elementwise_kernel,0,0,39,695996
BatchNorm,0,0,6,613248
void at::native::vectorized_elementwise_kernel,-1,0,31,19989
Conv,-1,0,65,9349
Conv,0,0,78,691848
volta_sgemm_128x64_tn,0,0,20,5165
BatchNorm,0,0,54,10043
volta_sgemm_128x64_tn,1,0,35,479872
BatchNorm,1,0,45,345999.5
void at::native::elementwise_kernel,1,0,41,4618
volta_sgemm_128x64_tn,1,0,64,9910
volta_sgemm_128x64_tn,0,0,63,17120
volta_sgemm_128x64_tn,-1,0,50,7432.5
void at::native::reduce_kernel,1,0,57,563426
BatchNorm,1,0,63,17028
void at::native::reduce_kernel,0,0,59,445873
void at::native::vectorized_elementwise_kernel,-1,0,882,675815
void at::native::vectorized_elementwise_kernel,0,0,32,755131.5
volta_sgemm_128x64_tn,1,0,37,172533
void at::native::reduce_kernel,1,0,24,8378
Conv,0,0,60,19119
void at::native::elementwise_kernel,-1,0,77,384023
volta_sgemm_128x64_tn,0,0,26,75581
void at::native::vectorized_elementwise_kernel,0,0,55,8344
void at::native::vectorized_elementwise_kernel,-1,0,34,16471
void at::native::vectorized_elementwise_kernel,0,0,62,617710
void at::native::elementwise_kernel,0,0,52,7521
Conv,-1,0,40,12736.5
void at::native::reduce_kernel,-1,0,78,197418
volta_sgemm_128x64_tn,1,0,10,8282
volta_sgemm_128x64_tn,1,0,44,8251
void at::native::elementwise_kernel,-1,0,73,15009
BatchNorm,1,0,45,3020.5
void at::native::reduce_kernel,-1,0,8,16573
void at::native::elementwise_kernel,0,0,23,15879
volta_sgemm_128x64_tn,0,0,13,455926
BatchNorm,1,0,47,588276
BatchNorm,0,0,29,53948
void at::native::vectorized_elementwise_kernel,1,0,6,417034
BatchNorm,0,0,52,17342
BatchNorm,1,0,54,18821
void at::native::reduce_kernel,1,0,55,12185
Conv,0,0,67,651846
Conv,1,0,50,729092
void at::native::reduce_kernel,1,0,52,9138
BatchNorm,-1,0,68,4453
Conv,0,0,23,3552
void at::native::reduce_kernel,1,0,602,305249
void at::native::reduce_kernel,-1,0,77,441079.5
Conv,1,0,23,132692.5
void at::native::reduce_kernel,1,0,7,580490
volta_sgemm_128x64_tn,0,0,24,15069
void at::native::elementwise_kernel,0,0,18,280201.5
Conv,1,0,68,325458
void at::native::vectorized_elementwise_kernel,-1,0,1,10508
BatchNorm,1,0,78,65263
void at::native::vectorized_elementwise_kernel,0,0,4,394295
