// placeholder, replaced below
#include "fxp_common.cuh"
#include "gemm_common.cuh"
namespace fxpr {
bool gemm_tc_supported(const GemmArgs&) { return false; }
int gemm_tc(const GemmArgs&, cudaStream_t) { return FXPR_ERR_UNSUPPORTED; }
int64_t gemm_tc_scratch_bytes(int64_t M, int64_t N, int int_bits) { return M * N * 8 + 4096; }
}
