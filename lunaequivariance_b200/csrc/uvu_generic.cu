// Table-driven kernels for any UVU path list: one thread per element of the free argument of
//   F(x, y, w, g) = sum_e sum_p sum_u sum_ijk C^p_ijk x[src e,(u,i)] y[e,j] w[e,(p,u)] g[dst e,(u,k)].
// They are the reference implementation inside the library (any degree, any multiplicity, strided weights,
// unaligned rows) and the fallback for configurations the staged kernels do not cover.  No atomics: every output
// element is produced by exactly one thread, so results are bitwise reproducible.
#include "plan.h"

namespace luna {

namespace {

constexpr int kThreads = 256;

template <typename T>
__device__ __forceinline__ const SlotRec* find_slot(const SlotRec* slots, int n, int col) {
  for (int s = 0; s < n; ++s) {
    const SlotRec& slot = slots[s];
    if (col >= slot.off && col < slot.off + slot.ch * slot.d) return &slots[s];
  }
  return nullptr;
}

// out[t, o] = sum_{e in in(t)} sum_{p -> block(o)} w * sum_{terms with k} c x_i y_j
template <typename T>
__global__ void __launch_bounds__(kThreads)
contract_free_g(GenericTables<T> tb, const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ w,
                const int* __restrict__ src, const int* __restrict__ dst_rowptr, T* __restrict__ out,
                int64_t total, bool accumulate) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (idx >= total) return;
  const int64_t t = idx / tb.O;
  const int o = static_cast<int>(idx - t * tb.O);
  const SlotRec* slot = find_slot<T>(tb.out_slots, tb.num_out_slots, o);
  T acc = T(0);
  if (slot != nullptr) {
    const int u = (o - slot->off) / slot->d;
    const int k = (o - slot->off) - u * slot->d;
    const int e_end = dst_rowptr[t + 1];
    for (int e = dst_rowptr[t]; e < e_end; ++e) {
      const T* xr = x + static_cast<int64_t>(src[e]) * tb.X;
      const T* yr = y + static_cast<int64_t>(e) * tb.Y;
      const T* wr = w + static_cast<int64_t>(e) * tb.W;
      for (int q = slot->path_begin; q < slot->path_end; ++q) {
        const PathRec& p = tb.paths[tb.out_slot_paths[q]];
        T sum = T(0);
        const int tb0 = tb.rowptr_k[p.byk_ptr + k], tb1 = tb.rowptr_k[p.byk_ptr + k + 1];
        for (int tt = tb0; tt < tb1; ++tt) {
          const TermRec<T> term = tb.terms_k[tt];
          sum += term.c * xr[p.x_off + u * p.d1 + term.a] * yr[p.y_off + term.b];
        }
        acc += wr[p.w_off + u * p.w_stride] * sum;
      }
    }
  }
  out[idx] = accumulate ? out[idx] + acc : acc;
}

// gx[s, xi] = sum_{e out of s} sum_{p using block(xi)} w * sum_{terms with i} c y_j g_k
template <typename T>
__global__ void __launch_bounds__(kThreads)
contract_free_x(GenericTables<T> tb, const T* __restrict__ y, const T* __restrict__ w, const T* __restrict__ g,
                const int* __restrict__ dst, const int* __restrict__ src_rowptr,
                const int* __restrict__ edge_ids_by_src, T* __restrict__ out, int64_t total, bool accumulate) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (idx >= total) return;
  const int64_t s = idx / tb.X;
  const int col = static_cast<int>(idx - s * tb.X);
  const SlotRec* slot = find_slot<T>(tb.x_slots, tb.num_x_slots, col);
  T acc = T(0);
  if (slot != nullptr) {
    const int u = (col - slot->off) / slot->d;
    const int i = (col - slot->off) - u * slot->d;
    const int p_end = src_rowptr[s + 1];
    for (int pos = src_rowptr[s]; pos < p_end; ++pos) {
      const int e = edge_ids_by_src[pos];
      const T* gr = g + static_cast<int64_t>(dst[e]) * tb.O;
      const T* yr = y + static_cast<int64_t>(e) * tb.Y;
      const T* wr = w + static_cast<int64_t>(e) * tb.W;
      for (int q = slot->path_begin; q < slot->path_end; ++q) {
        const PathRec& p = tb.paths[tb.x_slot_paths[q]];
        T sum = T(0);
        const int tb0 = tb.rowptr_i[p.byi_ptr + i], tb1 = tb.rowptr_i[p.byi_ptr + i + 1];
        for (int tt = tb0; tt < tb1; ++tt) {
          const TermRec<T> term = tb.terms_i[tt];  // (j, k)
          sum += term.c * yr[p.y_off + term.a] * gr[p.out_off + u * p.d3 + term.b];
        }
        acc += wr[p.w_off + u * p.w_stride] * sum;
      }
    }
  }
  out[idx] = accumulate ? out[idx] + acc : acc;
}

// gy[e, yj] = sum_{p using block(yj)} sum_u w * sum_{terms with j} c x_i g_k
template <typename T>
__global__ void __launch_bounds__(kThreads)
contract_free_y(GenericTables<T> tb, const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ g,
                const int* __restrict__ src, const int* __restrict__ dst, T* __restrict__ out, int64_t total,
                bool accumulate) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (idx >= total) return;
  const int64_t e = idx / tb.Y;
  const int col = static_cast<int>(idx - e * tb.Y);
  const SlotRec* slot = find_slot<T>(tb.y_slots, tb.num_y_slots, col);
  T acc = T(0);
  if (slot != nullptr) {
    const int j = col - slot->off;
    const T* xr = x + static_cast<int64_t>(src[e]) * tb.X;
    const T* gr = g + static_cast<int64_t>(dst[e]) * tb.O;
    const T* wr = w + e * tb.W;
    for (int q = slot->path_begin; q < slot->path_end; ++q) {
      const PathRec& p = tb.paths[tb.y_slot_paths[q]];
      const int tb0 = tb.rowptr_j[p.byj_ptr + j], tb1 = tb.rowptr_j[p.byj_ptr + j + 1];
      if (tb0 == tb1) continue;
      for (int u = 0; u < p.ch; ++u) {
        T sum = T(0);
        for (int tt = tb0; tt < tb1; ++tt) {
          const TermRec<T> term = tb.terms_j[tt];  // (i, k)
          sum += term.c * xr[p.x_off + u * p.d1 + term.a] * gr[p.out_off + u * p.d3 + term.b];
        }
        acc += wr[p.w_off + u * p.w_stride] * sum;
      }
    }
  }
  out[idx] = accumulate ? out[idx] + acc : acc;
}

// gw[e, wi] = sum_{all terms of the owning path} c x_i y_j g_k
template <typename T>
__global__ void __launch_bounds__(kThreads)
contract_free_w(GenericTables<T> tb, const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ g,
                const int* __restrict__ src, const int* __restrict__ dst, T* __restrict__ out, int64_t total,
                bool accumulate) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (idx >= total) return;
  const int64_t e = idx / tb.W;
  const int col = static_cast<int>(idx - e * tb.W);
  const int owner = tb.w_elem_path[col];
  T acc = T(0);
  if (owner >= 0) {
    const PathRec& p = tb.paths[owner];
    const int u = (col - p.w_off) / p.w_stride;
    const T* xr = x + static_cast<int64_t>(src[e]) * tb.X + p.x_off + u * p.d1;
    const T* gr = g + static_cast<int64_t>(dst[e]) * tb.O + p.out_off + u * p.d3;
    const T* yr = y + e * tb.Y + p.y_off;
    const int tb0 = tb.rowptr_k[p.byk_ptr], tb1 = tb.rowptr_k[p.byk_ptr + p.d3];
    int k = 0;
    for (int tt = tb0; tt < tb1; ++tt) {
      while (tt >= tb.rowptr_k[p.byk_ptr + k + 1]) ++k;
      const TermRec<T> term = tb.terms_k[tt];  // (i, j)
      acc += term.c * xr[term.a] * yr[term.b] * gr[k];
    }
  }
  out[idx] = accumulate ? out[idx] + acc : acc;
}

template <typename T>
int launch(luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph, int free_slot, const T* x,
           const T* y, const T* w, const T* g, T* out, bool accumulate, cudaStream_t stream) {
  const GenericTables<T> tb = generic_tables<T>(plan, dt);
  const int64_t N = graph->num_nodes, E = graph->num_edges;
  int64_t total = 0;
  switch (free_slot) {
    case kFreeG: total = N * tb.O; break;
    case kFreeX: total = (graph->num_src_nodes > 0 ? graph->num_src_nodes : N) * tb.X; break;
    case kFreeY: total = E * tb.Y; break;
    case kFreeW: total = E * tb.W; break;
    default: return fail(LUNA_ERR_INVALID_ARGUMENT, "unknown free slot %d", free_slot);
  }
  if (total == 0) return LUNA_OK;
  const int64_t blocks = ceil_div(total, kThreads);
  if (blocks > 2147483647LL) return fail(LUNA_ERR_OVERFLOW, "output has too many elements for one launch");
  const dim3 grid(static_cast<unsigned>(blocks));
  switch (free_slot) {
    case kFreeG:
      contract_free_g<T><<<grid, kThreads, 0, stream>>>(tb, x, y, w, graph->src, graph->dst_rowptr, out, total,
                                                         accumulate);
      break;
    case kFreeX:
      contract_free_x<T><<<grid, kThreads, 0, stream>>>(tb, y, w, g, graph->dst, graph->src_rowptr,
                                                         graph->edge_ids_by_src, out, total, accumulate);
      break;
    case kFreeY:
      contract_free_y<T><<<grid, kThreads, 0, stream>>>(tb, x, w, g, graph->src, graph->dst, out, total, accumulate);
      break;
    case kFreeW:
      contract_free_w<T><<<grid, kThreads, 0, stream>>>(tb, x, y, g, graph->src, graph->dst, out, total, accumulate);
      break;
  }
  LUNA_LAUNCH_CHECK("generic contraction");
  return LUNA_OK;
}

}  // namespace

int generic_contract(luna_uvu_plan* plan, const luna_graph* graph, int free_slot, const void* x, const void* y,
                     const void* w, const void* g, void* out, bool accumulate, cudaStream_t stream) {
  const DeviceTables* dt = nullptr;
  int rc = get_device_tables(plan, &dt);
  if (rc != LUNA_OK) return rc;
  if (plan->dtype == LUNA_F64)
    return launch<double>(plan, *dt, graph, free_slot, static_cast<const double*>(x), static_cast<const double*>(y),
                          static_cast<const double*>(w), static_cast<const double*>(g), static_cast<double*>(out),
                          accumulate, stream);
  return launch<float>(plan, *dt, graph, free_slot, static_cast<const float*>(x), static_cast<const float*>(y),
                       static_cast<const float*>(w), static_cast<const float*>(g), static_cast<float*>(out),
                       accumulate, stream);
}

}  // namespace luna
