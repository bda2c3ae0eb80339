// Fused-RoPE flash-attention backward for sm_100a (tensor-core path).
#include "common.cuh"

namespace corope {

bool rope_bwd_tc_supported(int, int, int, int, int, int) { return false; }

int launch_rope_bwd_tc(const RopeParams&, int, cudaStream_t) { return COROPE_ERR_BAD_SHAPE; }

}  // namespace corope
