// Instantiation of the staged forward kernels for T = float, 1 channel(s) per lane.
#include "uvu_fast_fwd.cuh"
namespace luna {
namespace fastk {
template int launch_fast_fwd<float, 1>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const float*, const float*,
                                     const float*, float*, bool, cudaStream_t);
}  // namespace fastk
}  // namespace luna
