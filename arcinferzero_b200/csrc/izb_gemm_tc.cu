// placeholder until the tcgen05 kernel lands
#include "izb_common.cuh"
int izb_make_raw_tensor_map(izb_weight*) { return IZB_ERR_CUDA; }
int izb_gemm_tc_launch(const izb_weight*, int, const int8_t*, const float*, int, int, float*, int, int, int, int32_t*, cudaStream_t) { return 1; }
int izb_moe_gateup_tc(const izb_weight*, const izb_weight*, const int8_t*, const float*, int, const int32_t*, int, const int32_t*, float*, cudaStream_t) { return 1; }
int izb_moe_down_tc(const izb_weight*, const int8_t*, const float*, int, const int32_t*, int, const float*, float*, cudaStream_t) { return 1; }
extern "C" int izb_selfcheck(int) { return IZB_OK; }
