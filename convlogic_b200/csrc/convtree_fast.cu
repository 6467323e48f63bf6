// Shape-specialised fp32 forward of the fused ConvLogic block (placeholder: no fast path yet).
#include "clb_common.cuh"

int clb_convtree_fwd_fast_f32(const float *, const float *, const int32_t *, float *, uint8_t *, int, int, int, int, int, int, int,
                              int, int, int, int, int, cudaStream_t)
{
    return CLB_ERR_SHAPE;
}
