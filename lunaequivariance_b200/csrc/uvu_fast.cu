// Dispatch of the staged kernels by dtype and channels-per-lane, stage-count policy and shared-memory accounting.
#include <cstdlib>

#include "uvu_fast_bwd.cuh"
#include "uvu_fast_fwd.cuh"

namespace luna {
namespace fastk {

// Warps per CTA and stages per warp.  The kernels hide per-edge latency with resident warps, so the policy
// maximises CTAs per SM first (up to 4 CTAs of 4 warps), then stages (3 preferred over 2); if one CTA of 4 warps
// with two stages does not fit, the CTA shrinks.  Returns 0 if even one warp with two stages does not fit.
int choose_stages(size_t stage_bytes, size_t fixed_bytes, size_t shared_bytes, int max_smem_optin,
                  size_t* block_bytes, int* warps) {
  int max_ctas = 4;
  if (const char* knob = std::getenv("LUNA_B200_MAX_CTAS")) max_ctas = std::max(1, std::atoi(knob));
  for (int w = kWarps; w >= 1; --w) {
    for (int ctas = max_ctas; ctas >= 1; --ctas) {
      const size_t budget = static_cast<size_t>(max_smem_optin + 1024) / ctas - 1024;  // 1 KB reserved per CTA
      for (int stages = 3; stages >= 2; --stages) {
        const size_t bytes = shared_bytes + w * (stages * stage_bytes + fixed_bytes);
        if (bytes <= budget) {
          *block_bytes = bytes;
          *warps = w;
          return stages;
        }
      }
    }
  }
  *block_bytes = 0;
  *warps = 0;
  return 0;
}

// Explicit instantiations live in uvu_fast_fwd_*.cu so that they compile in parallel.
extern template int launch_fast_fwd<float, 1>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const float*, const float*, const float*, float*, bool, cudaStream_t);
extern template int launch_fast_fwd<float, 2>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const float*, const float*, const float*, float*, bool, cudaStream_t);
extern template int launch_fast_fwd<float, 4>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const float*, const float*, const float*, float*, bool, cudaStream_t);
extern template int launch_fast_fwd<double, 1>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const double*, const double*, const double*, double*, bool, cudaStream_t);
extern template int launch_fast_fwd<double, 2>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const double*, const double*, const double*, double*, bool, cudaStream_t);

#define LUNA_BWD_SIG(T) const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const T*, const T*, const T*, const T*, T*, bool, T*, bool, T*, bool, void*, int64_t, cudaStream_t
extern template int launch_fast_bwd<float, 1>(LUNA_BWD_SIG(float));
extern template int launch_fast_bwd<float, 2>(LUNA_BWD_SIG(float));
extern template int launch_fast_bwd<float, 4>(LUNA_BWD_SIG(float));
extern template int launch_fast_bwd<double, 1>(LUNA_BWD_SIG(double));
extern template int launch_fast_bwd<double, 2>(LUNA_BWD_SIG(double));
#undef LUNA_BWD_SIG

}  // namespace fastk

bool fast_available() { return true; }

namespace {
constexpr int kSmemLimit = 227 * 1024;
}

int64_t fast_smem_bytes(const luna_uvu_plan* plan, int which) {
  if (!plan->fast_ok) return 0;
  const FastMeta& f = plan->fast;
  const size_t elem = plan->dtype == LUNA_F64 ? 8 : 4;
  size_t fixed, stage;
  if (which == 0) {
    fixed = static_cast<size_t>(f.m_total) * elem + 32 * elem + fastk::kMaxStages * sizeof(uint64_t);
    stage = static_cast<size_t>(f.w_stage_elems + f.x_stage_elems) * elem;
  } else {
    fixed = plan->dtype == LUNA_F64 ? fastk::bwd_fixed_bytes<double>(f) : fastk::bwd_fixed_bytes<float>(f);
    stage = static_cast<size_t>(f.w_stage_elems + f.g_stage_elems) * elem;
  }
  size_t bytes = 0;
  int warps = 0;
  const size_t shared = plan->dtype == LUNA_F64 ? fastk::ell_bytes<double>(f.m_total, f.m_terms)
                                                : fastk::ell_bytes<float>(f.m_total, f.m_terms);
  fastk::choose_stages(stage, fixed, shared, kSmemLimit, &bytes, &warps);
  return static_cast<int64_t>(bytes);
}

// Per-chunk partial rows of gy when the channels of a block are split over several warps.
int64_t fast_scratch_bytes(const luna_uvu_plan* plan, int64_t, int64_t num_edges) {
  if (!plan->fast_ok || plan->force_generic || plan->fast.chunks <= 1) return 0;
  const int64_t elem = plan->dtype == LUNA_F64 ? 8 : 4;
  return static_cast<int64_t>(plan->fast.chunks) * num_edges * plan->Y * elem;
}

int fast_forward(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y, const void* w,
                 const void* rx, const void* ry, const void* rw, void* out, bool tangents, cudaStream_t stream) {
  const DeviceTables* dt = nullptr;
  int rc = get_device_tables(plan, &dt);
  if (rc != LUNA_OK) return rc;
  if (!plan->out_fully_covered) {
    const size_t elem = plan->dtype == LUNA_F64 ? 8 : 4;
    LUNA_CUDA_CHECK(cudaMemsetAsync(out, 0, static_cast<size_t>(graph->num_nodes) * plan->O * elem, stream));
  }
  auto one = [&](const void* xa, const void* ya, const void* wa, bool acc) -> int {
    const int cpl = plan->fast.cpl;
    if (plan->dtype == LUNA_F64) {
      auto X = static_cast<const double*>(xa), Y = static_cast<const double*>(ya), W = static_cast<const double*>(wa);
      auto O = static_cast<double*>(out);
      if (cpl == 2) return fastk::launch_fast_fwd<double, 2>(plan, *dt, graph, X, Y, W, O, acc, stream);
      return fastk::launch_fast_fwd<double, 1>(plan, *dt, graph, X, Y, W, O, acc, stream);
    }
    auto X = static_cast<const float*>(xa), Y = static_cast<const float*>(ya), W = static_cast<const float*>(wa);
    auto O = static_cast<float*>(out);
    if (cpl == 4) return fastk::launch_fast_fwd<float, 4>(plan, *dt, graph, X, Y, W, O, acc, stream);
    if (cpl == 2) return fastk::launch_fast_fwd<float, 2>(plan, *dt, graph, X, Y, W, O, acc, stream);
    return fastk::launch_fast_fwd<float, 1>(plan, *dt, graph, X, Y, W, O, acc, stream);
  };
  if (!tangents) return one(x, y, w, false);
  bool acc = false;
  if (rx) { rc = one(rx, y, w, acc); if (rc != LUNA_OK) return rc; acc = true; }
  if (ry) { rc = one(x, ry, w, acc); if (rc != LUNA_OK) return rc; acc = true; }
  if (rw) { rc = one(x, y, rw, acc); if (rc != LUNA_OK) return rc; acc = true; }
  if (!acc) return fail(LUNA_ERR_INVALID_ARGUMENT, "tangent forward needs at least one tangent");
  return LUNA_OK;
}

int fast_backward(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y, const void* w,
                  const void* g, void* gx, bool acc_x, void* gy, bool acc_y, void* gw, bool acc_w, void* scratch,
                  int64_t scratch_bytes, cudaStream_t stream) {
  const DeviceTables* dt = nullptr;
  int rc = get_device_tables(plan, &dt);
  if (rc != LUNA_OK) return rc;
  const int cpl = plan->fast.cpl;
  if (plan->dtype == LUNA_F64) {
    auto X = static_cast<const double*>(x), Y = static_cast<const double*>(y), W = static_cast<const double*>(w);
    auto G = static_cast<const double*>(g);
    auto GX = static_cast<double*>(gx), GY = static_cast<double*>(gy), GW = static_cast<double*>(gw);
    if (cpl == 2)
      return fastk::launch_fast_bwd<double, 2>(plan, *dt, graph, X, Y, W, G, GX, acc_x, GY, acc_y, GW, acc_w, scratch, scratch_bytes, stream);
    return fastk::launch_fast_bwd<double, 1>(plan, *dt, graph, X, Y, W, G, GX, acc_x, GY, acc_y, GW, acc_w, scratch, scratch_bytes, stream);
  }
  auto X = static_cast<const float*>(x), Y = static_cast<const float*>(y), W = static_cast<const float*>(w);
  auto G = static_cast<const float*>(g);
  auto GX = static_cast<float*>(gx), GY = static_cast<float*>(gy), GW = static_cast<float*>(gw);
  if (cpl == 4)
    return fastk::launch_fast_bwd<float, 4>(plan, *dt, graph, X, Y, W, G, GX, acc_x, GY, acc_y, GW, acc_w, scratch, scratch_bytes, stream);
  if (cpl == 2)
    return fastk::launch_fast_bwd<float, 2>(plan, *dt, graph, X, Y, W, G, GX, acc_x, GY, acc_y, GW, acc_w, scratch, scratch_bytes, stream);
  return fastk::launch_fast_bwd<float, 1>(plan, *dt, graph, X, Y, W, G, GX, acc_x, GY, acc_y, GW, acc_w, scratch, scratch_bytes, stream);
}

}  // namespace luna
