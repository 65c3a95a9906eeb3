// Tensor-core (tcgen05 / TMEM) dequant GEMM for batched decode and prefill.
#include "pi_common.cuh"

bool pi_gemm_tc_supported(const pi_ctx*, const pi_linear*, const pi_linear_args&) { return false; }
pi_status pi_launch_gemm_tc(pi_ctx* ctx, const pi_linear*, const pi_linear_args&) {
  return pi_fail(ctx, PI_ERR_UNSUPPORTED, "tensor-core GEMM is not available for this shape");
}
