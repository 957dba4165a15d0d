// Tensor-core implicit GEMM (TMA + tcgen05.mma kind::i8).  Placeholder plan: no geometry accepted yet.
#include "internal.h"

namespace enn_b200 {
bool tc_available(const enn_b200_context *ctx) { return false && ctx != nullptr; }
int32_t tc_plan_conv(enn_b200_op *op, const void *weights_hwio_host) {
    (void)op; (void)weights_hwio_host;
    return ENN_B200_INVALID_PARAMS;
}
int32_t tc_execute(enn_b200_op *op, const void *in, void *out) {
    (void)op; (void)in; (void)out;
    return ENN_B200_FAILURE;
}
void tc_release(enn_b200_op *op) { (void)op; }
}  // namespace enn_b200
