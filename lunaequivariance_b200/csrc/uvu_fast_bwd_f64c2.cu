// Instantiation of the staged backward kernels for T = double, 2 channel(s) per lane.
#include "uvu_fast_bwd.cuh"
namespace luna {
namespace fastk {
template int launch_fast_bwd<double, 2>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const double*, const double*,
                                     const double*, const double*, double*, bool, double*, bool, double*, bool, void*, int64_t,
                                     cudaStream_t);
}  // namespace fastk
}  // namespace luna
