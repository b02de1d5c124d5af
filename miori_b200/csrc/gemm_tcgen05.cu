// placeholder until the tcgen05 GEMM lands
#include "common.cuh"
using namespace miori_b200;
MIORI_API int miori_gemm_bf16_cache(const void*, const void*, void*, uint32_t, uint32_t, uint32_t, uint32_t, void*) { return fail(MIORI_E_STATE, "miori_gemm_bf16_cache: not built yet"); }
