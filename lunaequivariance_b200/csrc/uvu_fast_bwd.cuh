// Staged source-major kernel: first derivatives gx, gy, gw in one pass over the weights.
//
// One warp owns a contiguous range of source nodes (balanced by out-edge count) and walks their out-edges through
// the source CSR.  Per edge, bulk copies bring the weight row and the gathered g[dst] row into the warp's stage
// ring.  With M^p = C^p . y[e] (see uvu_fast.cuh) each channel computes
//     s_i   = sum_k M^p[i][k] g_k             (shared by the next two lines)
//     gx_i += w_p * s_i                        (register accumulator of the source node, no atomics)
//     gw_p  = sum_i x_i * s_i                  (streamed straight to global memory)
//     G^p[i][k] += x_i * (w_p g_k)             (summed over the lane's channels, then over the warp)
// The warp-wide sum of G runs through a padded shared-memory tile (write a column per lane, read a row per lane with
// 128-bit loads, conflict-free), batched over the paths of one output degree.  Finally gy[e, j] = sum C^p_ijk G^p[i][k]
// from a small per-j program.  Every output element is written by exactly one thread: deterministic.
#pragma once

#include <algorithm>

#include "uvu_fast.cuh"

namespace luna {
namespace fastk {

constexpr int kRedStride = 36;   // words per tile row: 32 lanes + 4 padding, keeps 128-bit row reads conflict-free
constexpr int kRedEntries = 64;  // tile rows (entries of G summed per flush)

template <typename T>
struct BwdParams {
  FastMeta meta;
  const T* x;
  const T* y;
  const T* w;
  const T* g;
  T* gx;
  T* gy;
  T* gw;
  T* gy_partial;  // [chunks, E, Y] when the channels are split into chunks, else null
  const int* dst;
  const int* src_rowptr;
  const int* edge_ids;
  const unsigned char* ell_j;
  const T* ell_c;
  const int* gy_ptr;
  const int* gy_m;
  const T* gy_c;
  int* status;
  int64_t num_src_nodes, num_edges;
  int stages;
  int acc_x, acc_y, acc_w;
};

template <typename T>
__host__ __device__ inline size_t bwd_fixed_bytes(const FastMeta& f) {
  // M buffer, G buffer, y row, reduction tile, barriers
  return (2 * static_cast<size_t>(f.m_total) + 32 + static_cast<size_t>(kRedEntries) * kRedStride) * sizeof(T) +
         kMaxStages * sizeof(uint64_t);
}

// Sums tile rows [0, count) over the 32 lane columns and writes them to gbuf[0..count).
template <typename T>
__device__ __forceinline__ void flush_tile(const T* red, T* gbuf, int count, int lane) {
  __syncwarp();
  for (int n = lane; n < count; n += 32) {
    constexpr int per = 16 / sizeof(T);
    const Vec<T, per>* row = reinterpret_cast<const Vec<T, per>*>(red + n * kRedStride);
    T a0 = T(0), a1 = T(0);
#pragma unroll
    for (int v = 0; v < 32 / per; v += 2) {
      const Vec<T, per> p = row[v], q = row[v + 1];
#pragma unroll
      for (int c = 0; c < per; ++c) {
        a0 += p.a[c];
        a1 += q.a[c];
      }
    }
    gbuf[n] = a0 + a1;
  }
  __syncwarp();
}

template <typename T, int CPL, int LX, int LO>
__global__ void __launch_bounds__(kMaxWarps * 32, 1) fast_bwd_kernel(const __grid_constant__ BwdParams<T> P) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const FastMeta& F = P.meta;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int stages = P.stages;
  const int stage_elems = F.w_stage_elems + F.g_stage_elems;
  const size_t warp_bytes = static_cast<size_t>(stages) * stage_elems * sizeof(T) + bwd_fixed_bytes<T>(F);
  const T* ell_c;
  const unsigned char* ell_j;
  load_ell<T>(smem_raw, P.ell_c, P.ell_j, F.m_total, F.m_terms, &ell_c, &ell_j);
  unsigned char* base = smem_raw + ell_bytes<T>(F.m_total, F.m_terms) + static_cast<size_t>(warp) * warp_bytes;
  T* stage_mem = reinterpret_cast<T*>(base);
  T* mbuf = stage_mem + static_cast<size_t>(stages) * stage_elems;
  T* gbuf = mbuf + F.m_total;
  T* red = gbuf + F.m_total;
  T* ybuf = red + kRedEntries * kRedStride;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ybuf + 32);

  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
  }
  __syncwarp();

  const int chw = 32 * CPL;
  const int c0 = blockIdx.y * chw;
  const int64_t E = P.num_edges, N = P.num_src_nodes;
  const int nwarps = blockDim.x >> 5;
  const int64_t total_warps = static_cast<int64_t>(gridDim.x) * nwarps;
  const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * nwarps + warp;
  const int64_t bound_lo = E * gwarp / total_warps, bound_hi = E * (gwarp + 1) / total_warps;
  const int64_t n_lo = warp_lower_bound(P.src_rowptr, N, bound_lo, lane);
  const int64_t n_hi = gwarp == total_warps - 1 ? N : warp_lower_bound(P.src_rowptr, N, bound_hi, lane);
  if (n_lo >= n_hi) return;
  const int64_t p_begin = P.src_rowptr[n_lo], p_end = P.src_rowptr[n_hi];
  const bool want_x = P.gx != nullptr, want_y = P.gy != nullptr, want_w = P.gw != nullptr;

  const uint32_t stage_bytes = static_cast<uint32_t>(stage_elems * sizeof(T));
  const int n_pieces = F.n_w_pieces + F.n_g_pieces;
  auto issue = [&](int64_t e, int64_t d_node, int s) {
    uint64_t* bar = &bars[s];
    if (lane == 0) mbar_arrive_expect_tx(bar, stage_bytes);
    __syncwarp();
    T* dstm = stage_mem + static_cast<size_t>(s) * stage_elems;
    for (int pi = lane; pi < n_pieces; pi += 32) {
      if (pi < F.n_w_pieces) {
        const CopyPiece pc = F.pieces_w[pi];
        bulk_copy_g2s(dstm + pc.s_off, P.w + e * F.W + pc.g_off + c0 * pc.comp,
                      static_cast<uint32_t>(pc.n * sizeof(T)), bar);
      } else {
        const CopyPiece pc = F.pieces_g[pi - F.n_w_pieces];
        bulk_copy_g2s(dstm + F.w_stage_elems + pc.s_off, P.g + d_node * F.O + pc.g_off + c0 * pc.comp,
                      static_cast<uint32_t>(pc.n * sizeof(T)), bar);
      }
    }
  };
  for (int s = 0; s < stages; ++s)
    if (p_begin + s < p_end) {
      const int e0 = P.edge_ids[p_begin + s];
      issue(e0, P.dst[e0], s);
    }
  // (edge id, destination) of the edges issued in the next two iterations, fetched early: the two loads depend on
  // each other, so the id runs two iterations ahead and the destination one
  int id_a1 = p_begin + stages < p_end ? P.edge_ids[p_begin + stages] : 0;
  int dst_a1 = p_begin + stages < p_end ? P.dst[id_a1] : 0;
  int id_a2 = p_begin + stages + 1 < p_end ? P.edge_ids[p_begin + stages + 1] : 0;

  int64_t e_next = p_begin < p_end ? P.edge_ids[p_begin] : 0;
  T y_next = (lane < F.Y && p_begin < p_end) ? P.y[e_next * F.Y + lane] : T(0);
  constexpr int XR = (LX + 1) * (LX + 1) * CPL;
  T xr[XR], gxr[XR];
  int64_t pos = p_begin;
  uint32_t it = 0;
  bool alive = true;

  for (int64_t n = n_lo; n < n_hi && alive; ++n) {
    const int64_t pe = P.src_rowptr[n + 1];
    static_for<0, LX + 1>([&](auto l1c) {
      constexpr int l1 = decltype(l1c)::value;
      constexpr int d1 = 2 * l1 + 1;
      if (F.x_off[l1] >= 0 && pos < pe)
        load_vectors<T, CPL, d1>(P.x + n * F.X + F.x_off[l1] + c0 * d1 + lane * (CPL * d1), &xr[l1 * l1 * CPL]);
    });
#pragma unroll
    for (int a = 0; a < XR; ++a) gxr[a] = T(0);

    for (; pos < pe; ++pos, ++it) {
      const int s = it % stages;
      if (!mbar_wait_bounded(&bars[s], (it / stages) & 1u)) {
        if (lane == 0) atomicExch(P.status, 2);
        alive = false;
        break;
      }
      const int64_t e = e_next;
      if (pos + 1 < p_end) e_next = P.edge_ids[pos + 1];
      const T* ws = stage_mem + static_cast<size_t>(s) * stage_elems;
      const T* gs = ws + F.w_stage_elems;
      if (lane < F.Y) ybuf[lane] = y_next;
      __syncwarp();
      compute_m<T>(ell_c, ell_j, F.m_terms, ybuf, mbuf, F.m_total, lane);
      if (pos + 1 < p_end && lane < F.Y) y_next = P.y[e_next * F.Y + lane];
      __syncwarp();

      static_for<0, LO + 1>([&](auto l3c) {
        constexpr int l3 = decltype(l3c)::value;
        constexpr int d3 = 2 * l3 + 1;
        const int q_first = F.pair_ptr[l3 * (kMaxFastL + 1)];
        const int q_last = F.pair_ptr[l3 * (kMaxFastL + 1) + LX + 1];
        if (q_first == q_last) return;
        T gr[CPL * d3];
        load_vectors<T, CPL, d3>(gs + F.gs_off[l3] + lane * (CPL * d3), gr);
        int tile_base = F.m_off[q_first];  // first M/G index held in the reduction tile
        int tile_end = tile_base;          // one past the last index written to the tile
        static_for<0, LX + 1>([&](auto l1c) {
          constexpr int l1 = decltype(l1c)::value;
          constexpr int d1 = 2 * l1 + 1;
          constexpr int cnt = d1 * d3;
          constexpr int cnt_pad = (cnt + 3) / 4 * 4;
          const int q_end = F.pair_ptr[l3 * (kMaxFastL + 1) + l1 + 1];
          for (int q = F.pair_ptr[l3 * (kMaxFastL + 1) + l1]; q < q_end; ++q) {
            T wv[CPL];
            load_vectors<T, CPL, 1>(ws + F.w_soff[q] + lane * CPL, wv);
            T mr[cnt];
            load_matrix<T, cnt>(mbuf + F.m_off[q], mr);
            const T* xl = &xr[l1 * l1 * CPL];
            T* gxl = &gxr[l1 * l1 * CPL];
            T gwv[CPL];
            {
              // s_i = sum_k M[i][k] g_k for every channel first, so the matrix registers die early
              T sv[CPL * d1];
#pragma unroll
              for (int c = 0; c < CPL; ++c) {
#pragma unroll
                for (int i = 0; i < d1; ++i) {
                  T sacc = mr[i * d3] * gr[c * d3];
#pragma unroll
                  for (int k = 1; k < d3; ++k) sacc = fma(mr[i * d3 + k], gr[c * d3 + k], sacc);
                  sv[c * d1 + i] = sacc;
                }
              }
#pragma unroll
              for (int c = 0; c < CPL; ++c) {
#pragma unroll
                for (int i = 0; i < d1; ++i) gxl[c * d1 + i] = fma(wv[c], sv[c * d1 + i], gxl[c * d1 + i]);
                T dot = xl[c * d1] * sv[c * d1];
#pragma unroll
                for (int i = 1; i < d1; ++i) dot = fma(xl[c * d1 + i], sv[c * d1 + i], dot);
                gwv[c] = dot;
              }
            }
            T G[cnt];
            if (want_y) {
#pragma unroll
              for (int c = 0; c < CPL; ++c) {
#pragma unroll
                for (int k = 0; k < d3; ++k) {
                  const T wg = wv[c] * gr[c * d3 + k];
#pragma unroll
                  for (int i = 0; i < d1; ++i)
                    G[i * d3 + k] = c == 0 ? xl[i] * wg : fma(xl[c * d1 + i], wg, G[i * d3 + k]);
                }
              }
            }
            if (want_w) {
              T* dstw = P.gw + e * F.W + F.w_goff[q] + c0 + lane * CPL;
              if (P.acc_w) {
                T old[CPL];
                load_vectors<T, CPL, 1>(dstw, old);
#pragma unroll
                for (int c = 0; c < CPL; ++c) gwv[c] += old[c];
              }
              store_vectors_streaming<T, CPL, 1>(dstw, gwv);
            }
            if (want_y) {
              if (F.m_off[q] + cnt_pad - tile_base > kRedEntries) {  // tile full: reduce what it holds
                flush_tile<T>(red, gbuf + tile_base, tile_end - tile_base, lane);
                tile_base = F.m_off[q];
              }
              T* col = red + (F.m_off[q] - tile_base) * kRedStride + lane;
#pragma unroll
              for (int m = 0; m < cnt; ++m) col[m * kRedStride] = G[m];
              tile_end = F.m_off[q] + cnt;
            }
          }
        });
        if (want_y && tile_end > tile_base) flush_tile<T>(red, gbuf + tile_base, tile_end - tile_base, lane);
      });

      if (want_y) {
        __syncwarp();
        if (lane < F.Y) {
          T acc = T(0);
          const int t1 = __ldg(P.gy_ptr + lane + 1);
          for (int t = __ldg(P.gy_ptr + lane); t < t1; ++t) acc = fma(__ldg(P.gy_c + t), gbuf[__ldg(P.gy_m + t)], acc);
          if (P.gy_partial != nullptr) {
            P.gy_partial[(static_cast<int64_t>(blockIdx.y) * E + e) * F.Y + lane] = acc;
          } else {
            T* dsty = P.gy + e * F.Y + lane;
            *dsty = P.acc_y ? *dsty + acc : acc;
          }
        }
      }
      __syncwarp();
      const int id_now = id_a1, dst_now = dst_a1;
      id_a1 = id_a2;
      if (pos + stages + 1 < p_end) dst_a1 = P.dst[id_a1];
      if (pos + stages + 2 < p_end) id_a2 = P.edge_ids[pos + stages + 2];
      if (pos + stages < p_end) issue(id_now, dst_now, s);
    }
    if (!alive) break;
    if (want_x) {
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        constexpr int d1 = 2 * l1 + 1;
        if (F.x_off[l1] >= 0) {
          T* dstx = P.gx + n * F.X + F.x_off[l1] + c0 * d1 + lane * (CPL * d1);
          T* gxl = &gxr[l1 * l1 * CPL];
          if (P.acc_x) {
            T old[CPL * d1];
            load_vectors<T, CPL, d1>(dstx, old);
#pragma unroll
            for (int a = 0; a < CPL * d1; ++a) gxl[a] += old[a];
          }
          store_vectors<T, CPL, d1>(dstx, gxl);
        }
      });
    }
  }
  if (!alive) {
    for (int d = 1; d < stages; ++d)
      if (pos + d < p_end) mbar_wait_bounded(&bars[(it + d) % stages], ((it + d) / stages) & 1u);
  }
}

// gy[e, j] (+)= sum over channel chunks of the partial rows.
template <typename T>
__global__ void reduce_gy_partial(const T* __restrict__ partial, T* __restrict__ gy, int64_t count, int chunks,
                                  int accumulate) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= count) return;
  T acc = accumulate ? gy[idx] : T(0);
  for (int c = 0; c < chunks; ++c) acc += partial[static_cast<int64_t>(c) * count + idx];
  gy[idx] = acc;
}

int choose_stages(size_t stage_bytes, size_t fixed_bytes, size_t shared_bytes, int max_smem_optin,
                  size_t* block_bytes, int* warps);

template <typename T, int CPL, int LX, int LO>
int launch_fast_bwd_one(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph, const T* x,
                        const T* y, const T* w, const T* g, T* gx, bool acc_x, T* gy, bool acc_y, T* gw, bool acc_w,
                        void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
  const FastMeta& f = plan->fast;
  BwdParams<T> P;
  P.meta = f;
  P.x = x;
  P.y = y;
  P.w = w;
  P.g = g;
  P.gx = gx;
  P.gy = gy;
  P.gw = gw;
  P.gy_partial = nullptr;
  P.dst = graph->dst;
  P.src_rowptr = graph->src_rowptr;
  P.edge_ids = graph->edge_ids_by_src;
  P.ell_j = dt.ell_j;
  P.ell_c = static_cast<const T*>(dt.ell_c);
  P.gy_ptr = dt.gy_ptr;
  P.gy_m = dt.gy_m;
  P.gy_c = static_cast<const T*>(dt.gy_c);
  P.status = dt.status;
  P.num_src_nodes = graph->num_src_nodes > 0 ? graph->num_src_nodes : graph->num_nodes;
  P.num_edges = graph->num_edges;
  P.acc_x = acc_x;
  P.acc_y = acc_y;
  P.acc_w = acc_w;
  const int64_t partial_count = graph->num_edges * f.Y;
  if (gy != nullptr && f.chunks > 1) {
    const int64_t need = static_cast<int64_t>(f.chunks) * partial_count * static_cast<int64_t>(sizeof(T));
    if (scratch == nullptr || scratch_bytes < need)
      return fail(LUNA_ERR_SCRATCH, "backward needs %lld bytes of scratch for per-chunk gy partials",
                  static_cast<long long>(need));
    if (!aligned_to(scratch, 16)) return fail(LUNA_ERR_MISALIGNED, "scratch must be 16-byte aligned");
    P.gy_partial = static_cast<T*>(scratch);
  }
  const size_t stage = static_cast<size_t>(f.w_stage_elems + f.g_stage_elems) * sizeof(T);
  size_t block_bytes = 0;
  int nwarps = kWarps;
  P.stages = choose_stages(stage, bwd_fixed_bytes<T>(f), ell_bytes<T>(f.m_total, f.m_terms), dt.max_smem_optin, &block_bytes, &nwarps);
  if (P.stages == 0) return fail(LUNA_ERR_UNSUPPORTED, "staged backward needs more shared memory than the device has");
  auto kernel = fast_bwd_kernel<T, CPL, LX, LO>;
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(block_bytes)));
  int64_t warps = std::max<int64_t>(1, ceil_div(graph->num_edges, 256));
  int64_t blocks = ceil_div(warps, nwarps);
  const int64_t wave = static_cast<int64_t>(dt.sm_count) * std::max<int64_t>(1, dt.max_smem_optin / std::max<size_t>(block_bytes, 1));
  if (blocks > wave) blocks = ceil_div(blocks, wave) * wave;
  const dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(f.chunks));
  kernel<<<grid, nwarps * 32, block_bytes, stream>>>(P);
  LUNA_LAUNCH_CHECK("staged backward");
  if (P.gy_partial != nullptr) {
    const unsigned rb = static_cast<unsigned>(ceil_div(partial_count, 256));
    reduce_gy_partial<T><<<rb, 256, 0, stream>>>(P.gy_partial, gy, partial_count, f.chunks, acc_y ? 1 : 0);
    LUNA_LAUNCH_CHECK("gy partial reduction");
  }
  return LUNA_OK;
}

template <typename T, int CPL>
int launch_fast_bwd(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph, const T* x,
                    const T* y, const T* w, const T* g, T* gx, bool acc_x, T* gy, bool acc_y, T* gw, bool acc_w,
                    void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
  const int lx = plan->fast.LX, lo = plan->fast.LO;
#define LUNA_BWD_ARGS plan, dt, graph, x, y, w, g, gx, acc_x, gy, acc_y, gw, acc_w, scratch, scratch_bytes, stream
  if (lx <= 1 && lo <= 1) return launch_fast_bwd_one<T, CPL, 1, 1>(LUNA_BWD_ARGS);
  if (lx <= 2 && lo <= 2) return launch_fast_bwd_one<T, CPL, 2, 2>(LUNA_BWD_ARGS);
  if (lx <= 2 && lo <= 3) return launch_fast_bwd_one<T, CPL, 2, 3>(LUNA_BWD_ARGS);
  return launch_fast_bwd_one<T, CPL, 3, 3>(LUNA_BWD_ARGS);
#undef LUNA_BWD_ARGS
}

}  // namespace fastk
}  // namespace luna
