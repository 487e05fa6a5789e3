// Instantiation of the staged backward kernels for T = float, 1 channel(s) per lane.
#include "uvu_fast_bwd.cuh"
namespace luna {
namespace fastk {
template int launch_fast_bwd<float, 1>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const float*, const float*,
                                     const float*, const float*, float*, bool, float*, bool, float*, bool, void*, int64_t,
                                     cudaStream_t);
}  // namespace fastk
}  // namespace luna
