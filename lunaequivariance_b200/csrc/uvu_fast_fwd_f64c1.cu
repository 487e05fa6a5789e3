// Instantiation of the staged forward kernels for T = double, 1 channel(s) per lane.
#include "uvu_fast_fwd.cuh"
namespace luna {
namespace fastk {
template int launch_fast_fwd<double, 1>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const double*, const double*,
                                     const double*, double*, bool, cudaStream_t);
}  // namespace fastk
}  // namespace luna
