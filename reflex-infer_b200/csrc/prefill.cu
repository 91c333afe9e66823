// Tensor-core path of dense fused_attention (placeholder until the tcgen05 kernel lands:
// every shape reports NotImplemented and the caller takes the scalar kernel).
#include "common.cuh"

namespace rfx {
int launch_dense_tensor(const RfxAttentionArgs*) { return RFX_NOT_IMPLEMENTED; }
}  // namespace rfx
