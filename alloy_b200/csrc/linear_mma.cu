// Tensor-core dequant-GEMV family (placeholder routing until the kernels land).
#include "linear.cuh"

namespace alloyb {

int try_linear_fast(const void*, int, int, int, const WeightSeg*, int, const void*, cudaStream_t) {
    return ALLOYB_NOT_TAKEN;
}
int try_gated_fast(const void*, const void*, const void*, const void*, const void*, void*, int, int,
                   int, int, int, int, cudaStream_t) {
    return ALLOYB_NOT_TAKEN;
}

}  // namespace alloyb
