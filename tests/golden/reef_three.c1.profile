Name,Profile,Memory_footprint,SM_usage,Duration
Conv,0,0,12,387605
volta_sgemm_128x64_tn,1,0,412,13540
void at::native::elementwise_kernel,1,0,44,450158
void at::native::vectorized_elementwise_kernel,0,0,8,31589.5
void at::native::elementwise_kernel,1,0,2,7430
Conv,0,0,6,512203
void at::native::elementwise_kernel,0,0,75,19324
void at::native::reduce_kernel,-1,0,2031,426705
void at::native::reduce_kernel,0,0,1038,17779
void at::native::elementwise_kernel,1,0,3460,193562
void at::native::elementwise_kernel,0,0,77,15479
void at::native::elementwise_kernel,0,0,71,522630
BatchNorm,1,0,70,10088
void at::native::reduce_kernel,-1,0,1457,16960
void at::native::elementwise_kernel,-1,0,2699,695908
volta_sgemm_128x64_tn,1,0,882,560568
Conv,0,0,80,16647.5
void at::native::vectorized_elementwise_kernel,1,0,1715,10828
BatchNorm,0,0,1083,115861
volta_sgemm_128x64_tn,0,0,25,802848
Conv,-1,0,3322,14323
void at::native::reduce_kernel,-1,0,64,641498
BatchNorm,0,0,58,12854.5
BatchNorm,-1,0,79,856161.5
void at::native::reduce_kernel,1,0,36,323657.5
volta_sgemm_128x64_tn,0,0,79,3424.5
Conv,1,0,3361,654898
void at::native::reduce_kernel,0,0,77,841259
void at::native::vectorized_elementwise_kernel,0,0,51,15735
void at::native::vectorized_elementwise_kernel,0,0,3490,14960
BatchNorm,1,0,30,71844
volta_sgemm_128x64_tn,0,0,3569,5162
volta_sgemm_128x64_tn,1,0,42,8637
void at::native::elementwise_kernel,1,0,77,10073
void at::native::reduce_kernel,0,0,35,157434
BatchNorm,1,0,42,13030
BatchNorm,0,0,79,5908
BatchNorm,-1,0,52,17975
void at::native::reduce_kernel,0,0,79,366865
BatchNorm,-1,0,58,30370
volta_sgemm_128x64_tn,0,0,19,710589
void at::native::reduce_kernel,1,0,1320,11068.5
BatchNorm,-1,0,55,18318
BatchNorm,0,0,57,373938
void at::native::elementwise_kernel,0,0,21,5935
Conv,-1,0,2112,446345
BatchNorm,-1,0,78,15323
volta_sgemm_128x64_tn,-1,0,3199,15273
Conv,1,0,1142,95422
void at::native::elementwise_kernel,1,0,2061,9433
volta_sgemm_128x64_tn,1,0,3306,15942
volta_sgemm_128x64_tn,1,0,66,333183
void at::native::elementwise_kernel,0,0,3,17048
void at::native::elementwise_kernel,0,0,4,16398
void at::native::reduce_kernel,-1,0,17,13939
void at::native::elementwise_kernel,-1,0,72,2386
Conv,0,0,29,115100.5
Conv,-1,0,18,265843.5
void at::native::vectorized_elementwise_kernel,-1,0,33,102662
volta_sgemm_128x64_tn,-1,0,66,4397
