// Tensor-core store kernel (placeholder until the split-operand GEMM lands):
// reports "not handled" so tq_store runs the fp32 kernel.
#include "tq_common.cuh"

int tq_store_tc_launch(const tq_consts*, const void*, const void*, tq_dtype, int64_t, int32_t, int64_t, int64_t,
                       const int64_t*, const int32_t*, int64_t, const tq_pool*, cudaStream_t, int* handled) {
    *handled = 0;
    return TQ_OK;
}
