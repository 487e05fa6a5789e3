// Dispatch of the staged kernels by dtype and channels-per-lane, stage-count policy and shared-memory accounting.
#include "uvu_fast_fwd.cuh"

namespace luna {
namespace fastk {

// Largest stage count in [2, 4] that still lets two CTAs share an SM; otherwise the largest that fits one CTA.
int choose_stages(size_t stage_bytes, size_t fixed_bytes, int max_smem_optin, size_t* block_bytes) {
  const size_t two_per_sm = static_cast<size_t>(max_smem_optin) / 2 - 1024;
  for (int stages = kMaxStages; stages >= 2; --stages) {
    const size_t bytes = kWarps * (stages * stage_bytes + fixed_bytes);
    if (bytes <= two_per_sm) {
      *block_bytes = bytes;
      return stages;
    }
  }
  for (int stages = 3; stages >= 2; --stages) {
    const size_t bytes = kWarps * (stages * stage_bytes + fixed_bytes);
    if (bytes <= static_cast<size_t>(max_smem_optin)) {
      *block_bytes = bytes;
      return stages;
    }
  }
  *block_bytes = 0;
  return 0;
}

// Explicit instantiations live in uvu_fast_fwd_*.cu so that they compile in parallel.
extern template int launch_fast_fwd<float, 1>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const float*, const float*, const float*, float*, bool, cudaStream_t);
extern template int launch_fast_fwd<float, 2>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const float*, const float*, const float*, float*, bool, cudaStream_t);
extern template int launch_fast_fwd<float, 4>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const float*, const float*, const float*, float*, bool, cudaStream_t);
extern template int launch_fast_fwd<double, 1>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const double*, const double*, const double*, double*, bool, cudaStream_t);
extern template int launch_fast_fwd<double, 2>(const luna_uvu_plan*, const DeviceTables&, const luna_graph*, const double*, const double*, const double*, double*, bool, cudaStream_t);

}  // namespace fastk

bool fast_available() { return true; }

namespace {
constexpr int kSmemLimit = 227 * 1024;
}

int64_t fast_smem_bytes(const luna_uvu_plan* plan, int which) {
  if (!plan->fast_ok) return 0;
  const FastMeta& f = plan->fast;
  const size_t elem = plan->dtype == LUNA_F64 ? 8 : 4;
  const size_t fixed = static_cast<size_t>(f.m_total) * elem + 32 * elem + fastk::kMaxStages * sizeof(uint64_t);
  const size_t stage = static_cast<size_t>(f.w_stage_elems + (which == 0 ? f.x_stage_elems : f.g_stage_elems)) * elem;
  size_t bytes = 0;
  fastk::choose_stages(stage, fixed, kSmemLimit, &bytes);
  return static_cast<int64_t>(bytes);
}

int64_t fast_scratch_bytes(const luna_uvu_plan*, int64_t, int64_t) { return 0; }

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

// Until the staged source-major kernel is linked, the first-order outputs come from the table-driven kernels.
int fast_backward(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y, const void* w,
                  const void* g, void* gx, bool acc_x, void* gy, bool acc_y, void* gw, bool acc_w, void*, int64_t,
                  cudaStream_t stream) {
  int rc = LUNA_OK;
  if (gx && (rc = generic_contract(plan, graph, kFreeX, nullptr, y, w, g, gx, acc_x, stream)) != LUNA_OK) return rc;
  if (gy && (rc = generic_contract(plan, graph, kFreeY, x, nullptr, w, g, gy, acc_y, stream)) != LUNA_OK) return rc;
  if (gw && (rc = generic_contract(plan, graph, kFreeW, x, y, nullptr, g, gw, acc_w, stream)) != LUNA_OK) return rc;
  return LUNA_OK;
}

}  // namespace luna
