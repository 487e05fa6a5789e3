// Dispatch of the staged kernels by dtype and channels-per-lane, stage-count policy and shared-memory accounting.
#include <cstdlib>

#include "uvu_fast_bwd.cuh"
#include "uvu_fast_fwd.cuh"

namespace luna {
namespace fastk {

Residency choose_residency(size_t ring_bytes, size_t fixed_bytes, size_t shared_bytes, int max_smem_optin,
                           int regs_per_thread, int max_warps, int min_depth, int max_depth) {
  const int max_ctas = 4;
  const int regs_per_warp = (std::max(regs_per_thread, 1) + 7) / 8 * 8 * 32;
  const int warp_slots = std::max(1, 16384 / regs_per_warp);  // per sub-partition
  Residency best;
  int best_score = 0;
  for (int ctas = 1; ctas <= max_ctas; ++ctas) {
    const size_t budget = static_cast<size_t>(max_smem_optin + 1024) / ctas - 1024;  // 1 KB reserved per CTA
    for (int w = 1; w <= std::min(max_warps, kMaxWarps); ++w) {
      if (ctas * ((w + 3) / 4) > warp_slots) continue;
      for (int depth = min_depth; depth <= max_depth; ++depth) {
        const size_t bytes = shared_bytes + w * (depth * ring_bytes + fixed_bytes);
        if (bytes > budget) continue;
        // issue-rate model: a sub-partition with n resident warps runs at n / (n + 2) of its peak
        int score = 0;
        for (int part = 0; part < 4; ++part) {
          const int n = ctas * (w / 4 + (part < w % 4 ? 1 : 0));
          score += 4096 * n / (n + 2);
        }
        score = score * 16 + (depth - min_depth) * 4 + (max_ctas - ctas);
        if (score > best_score) {
          best_score = score;
          best.depth = depth;
          best.warps = w;
          best.ctas = ctas;
          best.block_bytes = bytes;
        }
      }
    }
  }
  return best;
}

int64_t grid_blocks(int64_t num_edges, int64_t target, const Residency& r, int sm_count) {
  const int64_t wave = static_cast<int64_t>(sm_count) * r.ctas;  // CTAs resident at once
  const int64_t wave_warps = wave * r.warps;
  const int64_t per_warp = target;
  if (num_edges > per_warp * wave_warps) {  // several waves of about `target` edges per warp, whole waves only
    const int64_t blocks = ceil_div(ceil_div(num_edges, per_warp), r.warps);
    return ceil_div(blocks, wave) * wave;
  }
  // a small graph gets exactly one wave (fewer edges per warp rather than idle SMs), or less if even 48 edges per
  // warp do not fill one
  if (num_edges >= 48 * wave_warps) return wave;
  return std::max<int64_t>(1, ceil_div(ceil_div(num_edges, 48), r.warps));
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

int fast_bwd_variant(const luna_uvu_plan* plan) {
  if (!plan->fast_ok || plan->force_generic) return LUNA_BWD_TABLE_DRIVEN;
  const FastMeta& f = plan->fast;
  const int lx = f.LX, lo = f.LO, l2 = f.canon_l2;
  // shapes with kernels unrolled for the canonical full path list (see launch_fast_bwd)
  const bool compiled_shape = !plan->tuning.no_canon && ((lx == 2 && l2 == 3 && lo == 3) || (lx == 2 && l2 == 2 && lo == 2) ||
                                                         (lx == 3 && l2 == 3 && lo == 3) || (lx == 1 && l2 == 1 && lo == 1));
  if (!compiled_shape || f.sparse_terms <= 0 || plan->tuning.no_sparse) return LUNA_BWD_STAGED_TABLES;
  const size_t elem = plan->dtype == LUNA_F64 ? 8 : 4;
  // Row stages pay off when an edge's weight row is one long contiguous piece for the CTA; short rows and rows
  // split into channel chunks go through the unit ring.
  const bool rows_ok = f.chunks == 1;
  int variant = rows_ok && static_cast<size_t>(f.w_stage_elems) * elem >= 2560 ? LUNA_BWD_ROW_STAGES : LUNA_BWD_UNIT_RING;
  if (plan->tuning.bwd_kernel == 1) variant = LUNA_BWD_ROW_STAGES;
  if (plan->tuning.bwd_kernel == 2) variant = LUNA_BWD_UNIT_RING;
  return variant;
}

namespace {
constexpr int kSmemLimit = 227 * 1024;
}

int64_t fast_smem_bytes(const luna_uvu_plan* plan, int which) {
  if (!plan->fast_ok) return 0;
  const FastMeta& f = plan->fast;
  const size_t elem = plan->dtype == LUNA_F64 ? 8 : 4;
  // an upper bound for callers that size things before a launch: the launch itself knows the register count
  size_t fixed;
  fastk::Residency r;
  if (which == 0) {
    if (plan->dtype == LUNA_F64)
      fixed = f.cpl == 2 ? fastk::fwd_fixed_bytes<double, 2>(f) : fastk::fwd_fixed_bytes<double, 1>(f);
    else
      fixed = f.cpl == 4 ? fastk::fwd_fixed_bytes<float, 4>(f)
                         : (f.cpl == 2 ? fastk::fwd_fixed_bytes<float, 2>(f) : fastk::fwd_fixed_bytes<float, 1>(f));
    const size_t shared = plan->dtype == LUNA_F64 ? fastk::ell_bytes<double>(f.m_total, f.m_terms)
                                                  : fastk::ell_bytes<float>(f.m_total, f.m_terms);
    r = fastk::choose_residency(static_cast<size_t>(f.w_stage_elems + f.x_stage_elems) * elem, fixed, shared, kSmemLimit,
                                255, fastk::kFwdMaxWarps, 2, 3);
  } else {
    if (plan->dtype == LUNA_F64)
      fixed = f.cpl == 2 ? fastk::bwd_fixed_bytes<double, 2>(f) : fastk::bwd_fixed_bytes<double, 1>(f);
    else
      fixed = f.cpl == 4 ? fastk::bwd_fixed_bytes<float, 4>(f)
                         : (f.cpl == 2 ? fastk::bwd_fixed_bytes<float, 2>(f) : fastk::bwd_fixed_bytes<float, 1>(f));
    r = fastk::choose_residency(static_cast<size_t>(f.slot_elems) * elem, fixed, fastk::bwd_shared_bytes(f), kSmemLimit,
                                255, 8, 2, std::min(fastk::kMaxSlots, 2 * f.nkinds));
  }
  return static_cast<int64_t>(r.block_bytes);
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
