// Instantiation of the compile-time-layout backward kernels for T = float, 1 channel(s) per lane: one warp per
// edge (TW = 1) and two warps that split an edge's paths (TW = 2), for the degree shapes with unrolled kernels.
#include "uvu_fast_bwd_plain.cuh"

namespace luna {
namespace fastk {

template <>
int launch_fast_bwd_plain_any<float, 1>(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph,
                                        const BwdParams<float>& P, bool teams, cudaStream_t stream) {
  return dispatch_fast_bwd_plain<float, 1>(plan, dt, graph, P, teams, stream);
}

}  // namespace fastk
}  // namespace luna
