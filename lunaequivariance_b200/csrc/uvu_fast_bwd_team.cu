// Instantiation of the warp-team backward kernel (FP32, two channels per lane, two warps per edge) for the degree
// shapes that have unrolled kernels.
#include "uvu_fast_bwd_team.cuh"

namespace luna {
namespace fastk {

int launch_fast_bwd_team_f32(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph,
                             const BwdParams<float>& P, bool has_gy, bool wxw, cudaStream_t stream) {
  const int lx = plan->fast.LX, lo = plan->fast.LO, l2 = plan->fast.canon_l2;
  if (plan->fast.ch != 32 * 2 * kTeamWarps)
    return fail(LUNA_ERR_UNSUPPORTED, "the warp-team backward covers blocks of %d channels", 32 * 2 * kTeamWarps);
  if (lx == 2 && l2 == 3 && lo == 3) return launch_fast_bwd_team<float, 2, 2, 3, 3>(plan, dt, graph, P, has_gy, wxw, stream);
  if (lx == 2 && l2 == 2 && lo == 2) return launch_fast_bwd_team<float, 2, 2, 2, 2>(plan, dt, graph, P, has_gy, wxw, stream);
  if (lx == 3 && l2 == 3 && lo == 3) return launch_fast_bwd_team<float, 2, 3, 3, 3>(plan, dt, graph, P, has_gy, wxw, stream);
  if (lx == 1 && l2 == 1 && lo == 1) return launch_fast_bwd_team<float, 2, 1, 1, 1>(plan, dt, graph, P, has_gy, wxw, stream);
  return fail(LUNA_ERR_UNSUPPORTED, "no warp-team backward for degree shape (%d, %d, %d)", lx, l2, lo);
}

}  // namespace fastk
}  // namespace luna
