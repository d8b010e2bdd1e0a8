// Instantiates the segment-reduction kernels (segment_reduce_kernels.cuh) for one operator.
#include "segment_reduce_kernels.cuh"

namespace texb {
TEXB_DEFINE_REDUCE_UNIT(sum_max, OpSumMax)
}  // namespace texb
