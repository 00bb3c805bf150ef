// placeholder, replaced below
#include "attention_common.cuh"
#include "fxp_common.cuh"
namespace fxpr {
bool attention_mma_supported(const AttnParams&, int) { return false; }
int attention_mma(const AttnParams&, int, int, cudaStream_t) { return FXPR_ERR_UNSUPPORTED; }
}
