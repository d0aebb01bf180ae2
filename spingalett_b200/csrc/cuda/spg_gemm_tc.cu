// placeholder: replaced by the tcgen05 GEMM
#include "spg_common.cuh"
extern "C" {
int spgk_gemm_tc_supported(const spgk_layer *) { return 0; }
uint32_t spgk_gemm_tc_softmax_max(void) { return 0; }
int spgk_layer_gemm_tc(const spgk_layer *, const void *, uint32_t, uint64_t, int, int, void *, uint32_t, uint64_t, int,
                       float *, uint32_t, uint32_t, int, int32_t *, void *) { return SPGK_E_UNSUPPORTED; }
}
