// Dispatch of the staged kernels by dtype and channels-per-lane, stage-count policy and shared-memory accounting.
#include <cstdlib>

#include "uvu_fast_bwd.cuh"
#include "uvu_fast_fwd.cuh"

namespace luna {
namespace fastk {

// Warps per CTA (at most 8), CTAs per SM and stages per warp (2 or 3).  The kernels hide per-edge latency with
// resident warps, so the policy maximises warps per SM (up to 16); ties go to more stages, then to fewer CTAs.
// Returns 0 if even one warp with two stages does not fit.
int choose_stages(size_t stage_bytes, size_t fixed_bytes, size_t shared_bytes, int max_smem_optin,
                  size_t* block_bytes, int* warps) {
  int max_ctas = 4;
  if (const char* knob = std::getenv("LUNA_B200_MAX_CTAS")) max_ctas = std::max(1, std::atoi(knob));
  int best_score = 0, best_stages = 0, best_warps = 0, best_ctas = 0;
  size_t best_bytes = 0;
  for (int ctas = 1; ctas <= max_ctas; ++ctas) {
    const size_t budget = static_cast<size_t>(max_smem_optin + 1024) / ctas - 1024;  // 1 KB reserved per CTA
    for (int w = 1; w <= kMaxWarps; ++w) {
      for (int stages = 2; stages <= 3; ++stages) {
        const size_t bytes = shared_bytes + w * (stages * stage_bytes + fixed_bytes);
        if (bytes > budget) continue;
        const int score = std::min(16, w * ctas) * 4 + (stages - 2) * 2 + (ctas == 1 ? 1 : 0);
        if (score > best_score) {
          best_score = score;
          best_stages = stages;
          best_warps = w;
          best_ctas = ctas;
          best_bytes = bytes;
        }
      }
    }
  }
  (void)best_ctas;
  *block_bytes = best_bytes;
  *warps = best_warps;
  return best_stages;
}

int choose_slots(size_t slot_bytes, size_t fixed_bytes, size_t shared_bytes, int max_smem_optin, int max_warps_by_regs,
                 int nkinds, size_t* block_bytes, int* warps) {
  int max_ctas = 4;
  if (const char* knob = std::getenv("LUNA_B200_MAX_CTAS")) max_ctas = std::max(1, std::atoi(knob));
  int slot_cap = std::min(kMaxSlots, 2 * nkinds);
  if (const char* knob = std::getenv("LUNA_B200_SLOTS")) slot_cap = std::max(2, std::min(slot_cap, std::atoi(knob)));
  const int slot_min = std::min(slot_cap, std::max(2, nkinds));
  int best_score = 0, best_slots = 0, best_warps = 0;
  size_t best_bytes = 0;
  for (int ctas = 1; ctas <= max_ctas; ++ctas) {
    const size_t budget = static_cast<size_t>(max_smem_optin + 1024) / ctas - 1024;  // 1 KB reserved per CTA
    for (int w = 1; w <= kMaxWarps; ++w) {
      if (w * ctas > std::max(1, max_warps_by_regs)) continue;
      for (int slots = slot_min; slots <= slot_cap; ++slots) {
        const size_t bytes = shared_bytes + w * (slots * slot_bytes + fixed_bytes);
        if (bytes > budget) continue;
        const int score = w * ctas * 64 + (slots - slot_min) * 4 + (max_ctas - ctas);
        if (score > best_score) {
          best_score = score;
          best_slots = slots;
          best_warps = w;
          best_bytes = bytes;
        }
      }
    }
  }
  *block_bytes = best_bytes;
  *warps = best_warps;
  return best_slots;
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
    if (plan->dtype == LUNA_F64)
      fixed = f.cpl == 2 ? fastk::fwd_fixed_bytes<double, 2>(f) : fastk::fwd_fixed_bytes<double, 1>(f);
    else
      fixed = f.cpl == 4 ? fastk::fwd_fixed_bytes<float, 4>(f)
                         : (f.cpl == 2 ? fastk::fwd_fixed_bytes<float, 2>(f) : fastk::fwd_fixed_bytes<float, 1>(f));
    stage = static_cast<size_t>(f.w_stage_elems + f.x_stage_elems) * elem;
  } else {
    if (plan->dtype == LUNA_F64)
      fixed = f.cpl == 2 ? fastk::bwd_fixed_bytes<double, 2>(f) : fastk::bwd_fixed_bytes<double, 1>(f);
    else
      fixed = f.cpl == 4 ? fastk::bwd_fixed_bytes<float, 4>(f)
                         : (f.cpl == 2 ? fastk::bwd_fixed_bytes<float, 2>(f) : fastk::bwd_fixed_bytes<float, 1>(f));
    size_t bytes = 0;
    int warps = 0;
    fastk::choose_slots(static_cast<size_t>(f.slot_elems) * elem, fixed, fastk::bwd_shared_bytes(f), kSmemLimit, 8,
                        f.nkinds, &bytes, &warps);
    return static_cast<int64_t>(bytes);
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
