// Placeholder until the tcgen05 grouped GEMMs are in: report "not my sizes".
#include "common.cuh"

int ftk_moe_gemm1_act_tc(const void*, const void*, const int32_t*, int, int, int, int, int, float, float, void*,
                         cudaStream_t) {
  return -1;
}
int ftk_moe_gemm2_tc(const void*, const void*, const int32_t*, const int32_t*, const float*, int, int, int, int, void*,
                     cudaStream_t) {
  return -1;
}
