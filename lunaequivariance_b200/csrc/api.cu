// extern "C" entry points of the UVU convolution: argument checks, choice between the staged and the table-driven
// kernels, and composition of the second-order outputs from first-order contractions.
#include "plan.h"

#include <initializer_list>
#include <utility>

using namespace luna;

namespace {

size_t elem_size(const luna_uvu_plan* plan) { return plan->dtype == LUNA_F64 ? 8 : 4; }
int64_t src_rows(const luna_graph* graph) { return graph->num_src_nodes > 0 ? graph->num_src_nodes : graph->num_nodes; }

int check_common(const luna_uvu_plan* plan, const luna_graph* graph) {
  if (!plan) return fail(LUNA_ERR_INVALID_ARGUMENT, "null plan");
  if (!graph) return fail(LUNA_ERR_INVALID_ARGUMENT, "null graph");
  if (graph->num_nodes < 0 || graph->num_edges < 0 || graph->num_src_nodes < 0)
    return fail(LUNA_ERR_INVALID_ARGUMENT, "negative graph size");
  if (graph->num_nodes >= (1LL << 31) - 1024 || graph->num_src_nodes >= (1LL << 31) - 1024 ||
      graph->num_edges >= (1LL << 31) - 1024)
    return fail(LUNA_ERR_OVERFLOW, "graph exceeds the 32-bit index range of this build");
  if (graph->num_nodes > 0 && (!graph->dst_rowptr || !graph->src_rowptr))
    return fail(LUNA_ERR_INVALID_ARGUMENT, "graph row pointers missing");
  if (graph->num_edges > 0 && (!graph->src || !graph->dst || !graph->edge_ids_by_src))
    return fail(LUNA_ERR_INVALID_ARGUMENT, "graph edge tables missing");
  return LUNA_OK;
}

int check_ptr(const luna_uvu_plan* plan, const void* p, const char* name, bool required, int64_t numel) {
  if (!p) {
    if (required && numel > 0) return fail(LUNA_ERR_INVALID_ARGUMENT, "%s is null", name);
    return LUNA_OK;
  }
  if (!aligned_to(p, elem_size(plan))) return fail(LUNA_ERR_MISALIGNED, "%s is not aligned to its element size", name);
  return LUNA_OK;
}

bool use_fast(const luna_uvu_plan* plan, std::initializer_list<const void*> pointers) {
  if (!plan->fast_ok || plan->force_generic || !fast_available()) return false;
  for (const void* p : pointers)
    if (p && !aligned_to(p, 16)) return false;  // bulk copies and 128-bit accesses need 16-byte rows
  return true;
}

int zero_fill(void* p, int64_t numel, size_t elem, cudaStream_t stream) {
  if (p && numel > 0) LUNA_CUDA_CHECK(cudaMemsetAsync(p, 0, static_cast<size_t>(numel) * elem, stream));
  return LUNA_OK;
}

#define LUNA_TRY(expr)            \
  do {                            \
    int luna_rc_ = (expr);        \
    if (luna_rc_ != LUNA_OK) return luna_rc_; \
  } while (0)

}  // namespace

extern "C" int64_t luna_uvu_plan_query(const luna_uvu_plan* plan, int what) {
  if (!plan) return -1;
  switch (what) {
    case LUNA_PLAN_FAST_PATH: return plan->fast_ok && !plan->force_generic;
    case LUNA_PLAN_CHANNELS_PER_LANE: return plan->fast_ok ? plan->fast.cpl : 0;
    case LUNA_PLAN_CHANNEL_CHUNKS: return plan->fast_ok ? plan->fast.chunks : 0;
    case LUNA_PLAN_FWD_SMEM_BYTES: return fast_smem_bytes(plan, 0);
    case LUNA_PLAN_BWD_SMEM_BYTES: return fast_smem_bytes(plan, 1);
    case LUNA_PLAN_CANONICAL_L2: return plan->fast_ok ? plan->fast.canon_l2 : -1;
    case LUNA_PLAN_SPARSE_TERMS: return plan->fast_ok ? plan->fast.sparse_terms : 0;
    case LUNA_PLAN_BWD_VARIANT: return fast_bwd_variant(plan);
    default: return -1;
  }
}

extern "C" int64_t luna_uvu_conv_scratch_bytes(const luna_uvu_plan* plan, int64_t num_nodes, int64_t num_edges) {
  if (!plan || num_nodes < 0 || num_edges < 0) return -1;
  return fast_scratch_bytes(plan, num_nodes, num_edges);
}

extern "C" int luna_uvu_conv_fwd(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y,
                                 const void* w, void* out, void* stream_) {
  clear_error();
  auto stream = static_cast<cudaStream_t>(stream_);
  LUNA_TRY(check_common(plan, graph));
  const int64_t N = graph->num_nodes, E = graph->num_edges;
  LUNA_TRY(check_ptr(plan, x, "x", true, N));
  LUNA_TRY(check_ptr(plan, y, "y", true, E));
  LUNA_TRY(check_ptr(plan, w, "w", true, E));
  LUNA_TRY(check_ptr(plan, out, "out", true, N));
  if (N == 0) return LUNA_OK;
  if (E == 0) return zero_fill(out, N * plan->O, elem_size(plan), stream);
  if (use_fast(plan, {x, w, out})) return fast_forward(plan, graph, x, y, w, nullptr, nullptr, nullptr, out, false, stream);
  return generic_contract(plan, graph, kFreeG, x, y, w, nullptr, out, false, stream);
}

namespace {
int backward_entry(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y, const void* w,
                   const void* g, void* gx, bool add_gx, void* gy, void* gw, void* scratch, int64_t scratch_bytes,
                   void* stream_) {
  clear_error();
  auto stream = static_cast<cudaStream_t>(stream_);
  LUNA_TRY(check_common(plan, graph));
  const int64_t N = graph->num_nodes, E = graph->num_edges;
  LUNA_TRY(check_ptr(plan, x, "x", true, N));
  LUNA_TRY(check_ptr(plan, y, "y", true, E));
  LUNA_TRY(check_ptr(plan, w, "w", true, E));
  LUNA_TRY(check_ptr(plan, g, "g", true, N));
  LUNA_TRY(check_ptr(plan, gx, "gx", false, 0));
  LUNA_TRY(check_ptr(plan, gy, "gy", false, 0));
  LUNA_TRY(check_ptr(plan, gw, "gw", false, 0));
  if (E == 0 || N == 0) return add_gx ? LUNA_OK : zero_fill(gx, src_rows(graph) * plan->X, elem_size(plan), stream);
  if (use_fast(plan, {x, w, g, gx, gw}))
    return fast_backward(plan, graph, x, y, w, g, gx, add_gx, gy, false, gw, false, scratch, scratch_bytes, stream);
  if (gx) LUNA_TRY(generic_contract(plan, graph, kFreeX, nullptr, y, w, g, gx, add_gx, stream));
  if (gy) LUNA_TRY(generic_contract(plan, graph, kFreeY, x, nullptr, w, g, gy, false, stream));
  if (gw) LUNA_TRY(generic_contract(plan, graph, kFreeW, x, y, nullptr, g, gw, false, stream));
  return LUNA_OK;
}
}  // namespace

extern "C" int luna_uvu_conv_bwd(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y,
                                 const void* w, const void* g, void* gx, void* gy, void* gw, void* scratch,
                                 int64_t scratch_bytes, void* stream) {
  return backward_entry(plan, graph, x, y, w, g, gx, false, gy, gw, scratch, scratch_bytes, stream);
}

extern "C" int luna_uvu_conv_bwd_add_gx(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y,
                                        const void* w, const void* g, void* gx, void* gy, void* gw, void* scratch,
                                        int64_t scratch_bytes, void* stream) {
  return backward_entry(plan, graph, x, y, w, g, gx, true, gy, gw, scratch, scratch_bytes, stream);
}

extern "C" int luna_uvu_conv_dbl_bwd(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y,
                                     const void* w, const void* g, const void* rx, const void* ry, const void* rw,
                                     void* hx, void* hy, void* hw, void* hg, void* scratch, int64_t scratch_bytes,
                                     void* stream_) {
  clear_error();
  auto stream = static_cast<cudaStream_t>(stream_);
  LUNA_TRY(check_common(plan, graph));
  const int64_t N = graph->num_nodes, E = graph->num_edges;
  const size_t es = elem_size(plan);
  LUNA_TRY(check_ptr(plan, x, "x", true, N));
  LUNA_TRY(check_ptr(plan, y, "y", true, E));
  LUNA_TRY(check_ptr(plan, w, "w", true, E));
  LUNA_TRY(check_ptr(plan, g, "g", true, N));
  for (auto [p, name] : {std::pair<const void*, const char*>{rx, "rx"}, {ry, "ry"}, {rw, "rw"}, {hx, "hx"},
                         {hy, "hy"}, {hw, "hw"}, {hg, "hg"}})
    LUNA_TRY(check_ptr(plan, p, name, false, 0));
  if (E == 0 || N == 0) {
    LUNA_TRY(zero_fill(hx, src_rows(graph) * plan->X, es, stream));
    return zero_fill(hg, N * plan->O, es, stream);
  }
  const bool fast = use_fast(plan, {x, w, g, rx, rw, hx, hw, hg});

  // hg = F_g(rx, y, w) + F_g(x, ry, w) + F_g(x, y, rw): a forward pass on the tangents.
  if (hg) {
    if (!rx && !ry && !rw) {
      LUNA_TRY(zero_fill(hg, N * plan->O, es, stream));
    } else if (fast) {
      LUNA_TRY(fast_forward(plan, graph, x, y, w, rx, ry, rw, hg, true, stream));
    } else {
      bool acc = false;
      if (rx) { LUNA_TRY(generic_contract(plan, graph, kFreeG, rx, y, w, nullptr, hg, acc, stream)); acc = true; }
      if (ry) { LUNA_TRY(generic_contract(plan, graph, kFreeG, x, ry, w, nullptr, hg, acc, stream)); acc = true; }
      if (rw) { LUNA_TRY(generic_contract(plan, graph, kFreeG, x, y, rw, nullptr, hg, acc, stream)); acc = true; }
    }
  }
  // hx = F_x(ry, w, g) + F_x(y, rw, g);  hy = F_y(rx, w, g) + F_y(x, rw, g);  hw = F_w(rx, y, g) + F_w(x, ry, g)
  if (fast) {
    bool ax = false, ay = false, aw = false;
    if (rx && (hy || hw)) {
      LUNA_TRY(fast_backward(plan, graph, rx, y, w, g, nullptr, false, hy, false, hw, false, scratch, scratch_bytes, stream));
      ay = hy != nullptr;
      aw = hw != nullptr;
    }
    if (ry && (hx || hw)) {
      LUNA_TRY(fast_backward(plan, graph, x, ry, w, g, hx, ax, nullptr, false, hw, aw, scratch, scratch_bytes, stream));
      ax = hx != nullptr;
      aw = hw != nullptr;
    }
    if (rw && (hx || hy)) {
      LUNA_TRY(fast_backward(plan, graph, x, y, rw, g, hx, ax, hy, ay, nullptr, false, scratch, scratch_bytes, stream));
      ax = hx != nullptr;
      ay = hy != nullptr;
    }
    if (hx && !ax) LUNA_TRY(zero_fill(hx, src_rows(graph) * plan->X, es, stream));
    if (hy && !ay) LUNA_TRY(zero_fill(hy, E * plan->Y, es, stream));
    if (hw && !aw) LUNA_TRY(zero_fill(hw, E * plan->W, es, stream));
    return LUNA_OK;
  }
  if (hx) {
    bool acc = false;
    if (ry) { LUNA_TRY(generic_contract(plan, graph, kFreeX, nullptr, ry, w, g, hx, acc, stream)); acc = true; }
    if (rw) { LUNA_TRY(generic_contract(plan, graph, kFreeX, nullptr, y, rw, g, hx, acc, stream)); acc = true; }
    if (!acc) LUNA_TRY(zero_fill(hx, src_rows(graph) * plan->X, es, stream));
  }
  if (hy) {
    bool acc = false;
    if (rx) { LUNA_TRY(generic_contract(plan, graph, kFreeY, rx, nullptr, w, g, hy, acc, stream)); acc = true; }
    if (rw) { LUNA_TRY(generic_contract(plan, graph, kFreeY, x, nullptr, rw, g, hy, acc, stream)); acc = true; }
    if (!acc) LUNA_TRY(zero_fill(hy, E * plan->Y, es, stream));
  }
  if (hw) {
    bool acc = false;
    if (rx) { LUNA_TRY(generic_contract(plan, graph, kFreeW, rx, y, nullptr, g, hw, acc, stream)); acc = true; }
    if (ry) { LUNA_TRY(generic_contract(plan, graph, kFreeW, x, ry, nullptr, g, hw, acc, stream)); acc = true; }
    if (!acc) LUNA_TRY(zero_fill(hw, E * plan->W, es, stream));
  }
  return LUNA_OK;
}

extern "C" int luna_uvu_check_status(luna_uvu_plan* plan, void* stream_) {
  clear_error();
  if (!plan) return fail(LUNA_ERR_INVALID_ARGUMENT, "null plan");
  const DeviceTables* dt = nullptr;
  LUNA_TRY(get_device_tables(plan, &dt));
  auto stream = static_cast<cudaStream_t>(stream_);
  int status = 0;
  LUNA_CUDA_CHECK(cudaMemcpyAsync(&status, dt->status, sizeof(int), cudaMemcpyDeviceToHost, stream));
  LUNA_CUDA_CHECK(cudaStreamSynchronize(stream));
  if (status != 0) {
    LUNA_CUDA_CHECK(cudaMemsetAsync(dt->status, 0, sizeof(int), stream));
    return fail(LUNA_ERR_DEVICE_TIMEOUT, "a bounded wait inside a kernel gave up (code %d)", status);
  }
  return LUNA_OK;
}
