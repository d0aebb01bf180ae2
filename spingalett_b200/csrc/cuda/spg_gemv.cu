// placeholder: replaced by the fused dequant-GEMV
#include "spg_common.cuh"
extern "C" {
size_t spgk_gemv_scratch_bytes(const spgk_layer *, uint32_t) { return 0; }
int spgk_layer_gemv(const spgk_layer *, const float *, uint32_t, float *, uint32_t, uint32_t, void *, void *) { return SPGK_E_UNSUPPORTED; }
}
