// Staged forward-shaped kernel (free argument g):  out[t] = sum_{e: dst e = t} sum_p w_p * (M^p(y_e)^T x[src e]).
//
// One warp owns a contiguous range of destination nodes (balanced by edge count) and therefore a contiguous range
// of the destination-sorted edge list: a warp-segmented reduction with register accumulators and no atomics.  Per
// edge, lanes issue 1-D bulk copies (cp.async.bulk, completion on an mbarrier) of the edge's weight row and of the
// gathered x[src] row into the warp's ring of shared-memory stages; the warp then reads them with 128-bit shared
// loads while later edges are in flight.  A lane owns CPL consecutive channels of every block.
//
// FP32 arithmetic runs on packed two-wide FMAs (fma.rn.f32x2): on B200 the scalar FFMA rate is about 0.7 of the
// packed rate, and packing halves the instruction count of the loop, which is what limits this kernel (issue slots
// and instruction-cache footprint), not bytes.  Two consecutive channels of a lane form a pair; the per-edge
// coupling matrices are stored duplicated (m, m) in shared memory so that they arrive as ready-made pairs.
#pragma once

#include <algorithm>
#include <cstdlib>

#include "uvu_fast.cuh"

namespace luna {
namespace fastk {

template <typename T>
struct FwdParams {
  FastMeta meta;
  const T* x;
  const T* y;
  const T* w;
  T* out;
  const int* src;
  const int* dst_rowptr;
  const unsigned char* ell_j;
  const T* ell_c;
  int* status;
  int64_t num_nodes, num_edges;
  int stages;
  int accumulate;
};

template <typename T, int CPL>
__host__ __device__ inline size_t fwd_fixed_bytes(const FastMeta& f) {
  // M buffer (duplicated entries on the packed path), y row, barriers
  const size_t m_elems = static_cast<size_t>(f.m_total) * (UsePairs<T, CPL>::value ? 2 : 1);
  return (m_elems + 32) * sizeof(T) + kMaxStages * sizeof(uint64_t);
}

template <typename T, int CPL, int LX, int LO>
__global__ void __launch_bounds__(kFwdMaxWarps * 32, 1) fast_fwd_kernel(const __grid_constant__ FwdParams<T> P) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr bool kPairs = UsePairs<T, CPL>::value;
  constexpr int NP = CPL / 2;  // channel pairs per lane (packed path)
  const FastMeta& F = P.meta;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int stages = P.stages;
  const int stage_elems = F.w_stage_elems + F.x_stage_elems;
  const T* ell_c;
  const unsigned char* ell_j;
  load_ell<T>(smem_raw, P.ell_c, P.ell_j, F.m_total, F.m_terms, &ell_c, &ell_j);
  const size_t warp_bytes = static_cast<size_t>(stages) * stage_elems * sizeof(T) + fwd_fixed_bytes<T, CPL>(F);
  unsigned char* base = smem_raw + ell_bytes<T>(F.m_total, F.m_terms) + static_cast<size_t>(warp) * warp_bytes;
  T* stage_mem = reinterpret_cast<T*>(base);
  T* mbuf = stage_mem + static_cast<size_t>(stages) * stage_elems;
  T* ybuf = mbuf + F.m_total * (kPairs ? 2 : 1);
  uint64_t* bars = reinterpret_cast<uint64_t*>(ybuf + 32);

  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
  }
  __syncwarp();

  const int chw = 32 * CPL;
  const int c0 = blockIdx.y * chw;  // first channel of this warp's chunk
  const int64_t E = P.num_edges, N = P.num_nodes;
  const int nwarps = blockDim.x >> 5;
  const int64_t total_warps = static_cast<int64_t>(gridDim.x) * nwarps;
  const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * nwarps + warp;
  const int64_t bound_lo = E * gwarp / total_warps, bound_hi = E * (gwarp + 1) / total_warps;
  const int64_t n_lo = warp_lower_bound(P.dst_rowptr, N, bound_lo, lane);
  const int64_t n_hi = gwarp == total_warps - 1 ? N : warp_lower_bound(P.dst_rowptr, N, bound_hi, lane);
  if (n_lo >= n_hi) return;
  const int64_t e_begin = P.dst_rowptr[n_lo], e_end = P.dst_rowptr[n_hi];

  // Lane `pi` issues copy piece `pi` of every edge; its description stays in registers.
  const uint32_t stage_bytes = static_cast<uint32_t>(stage_elems * sizeof(T));
  const int n_pieces = F.n_w_pieces + F.n_x_pieces;
  const bool piece_is_w = lane < F.n_w_pieces;
  int64_t piece_goff = 0;
  int piece_soff = 0;
  uint32_t piece_bytes = 0;
  if (lane < n_pieces) {
    const CopyPiece pc = piece_is_w ? F.pieces_w[lane] : F.pieces_x[lane - F.n_w_pieces];
    piece_goff = pc.g_off + static_cast<int64_t>(c0) * pc.comp;
    piece_soff = pc.s_off + (piece_is_w ? 0 : F.w_stage_elems);
    piece_bytes = static_cast<uint32_t>(pc.n * sizeof(T));
  }
  auto issue = [&](int64_t e, int64_t s_node, int s) {
    uint64_t* bar = &bars[s];
    if (lane == 0) mbar_arrive_expect_tx(bar, stage_bytes);
    __syncwarp();
    if (lane < n_pieces) {
      const T* from = piece_is_w ? P.w + e * F.W + piece_goff : P.x + s_node * F.X + piece_goff;
      bulk_copy_g2s(stage_mem + static_cast<size_t>(s) * stage_elems + piece_soff, from, piece_bytes, bar);
    }
  };

  for (int s = 0; s < stages; ++s)
    if (e_begin + s < e_end) issue(e_begin + s, P.src[e_begin + s], s);
  // source node of the edge that will be issued in the next iteration, fetched one iteration early
  int src_ahead = e_begin + stages < e_end ? P.src[e_begin + stages] : 0;

  T y_next = (lane < F.Y && e_begin < e_end) ? P.y[e_begin * F.Y + lane] : T(0);
  constexpr int AR = (LO + 1) * (LO + 1) * CPL;
  T acc[AR];  // packed path: viewed as pairs, element (l3, k, pair) at l3*l3*CPL + (k*NP + pair)*2
  int64_t e = e_begin;
  int s = 0;
  uint32_t parity = 0;
  bool alive = true;

  for (int64_t n = n_lo; n < n_hi && alive; ++n) {
    const int64_t ee = P.dst_rowptr[n + 1];
#pragma unroll
    for (int a = 0; a < AR; ++a) acc[a] = T(0);
#pragma unroll 1
    for (; e < ee; ++e) {
      if (!mbar_wait_bounded(&bars[s], parity)) {
        if (lane == 0) atomicExch(P.status, 1);
        alive = false;
        break;
      }
      const T* ws = stage_mem + static_cast<size_t>(s) * stage_elems;
      const T* xs = ws + F.w_stage_elems;
      // coupling matrices of this edge
      if (lane < F.Y) ybuf[lane] = y_next;
      __syncwarp();
      compute_m_share<T, kPairs>(ell_c, ell_j, ybuf, mbuf, F.m_total, 0, 1, lane);
      if (e + 1 < e_end && lane < F.Y) y_next = P.y[(e + 1) * F.Y + lane];
      __syncwarp();

      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        constexpr int d1 = 2 * l1 + 1;
        if (F.x_off[l1] < 0) return;
        T xl[CPL * d1];
        load_vectors<T, CPL, d1>(xs + F.xs_off[l1] + lane * (CPL * d1), xl);
        static_for<0, LO + 1>([&](auto l3c) {
          constexpr int l3 = decltype(l3c)::value;
          constexpr int d3 = 2 * l3 + 1;
          constexpr int d3p = d3 + 1;  // row stride of the coupling matrices
          const int q_end = F.pair_ptr[l3 * (kMaxFastL + 1) + l1 + 1];
#pragma unroll 1
          for (int q = F.pair_ptr[l3 * (kMaxFastL + 1) + l1]; q < q_end; ++q) {
            T wv[CPL];
            load_vectors<T, CPL, 1>(ws + F.w_soff[q] + lane * CPL, wv);
            T* al = &acc[l3 * l3 * CPL];
            if constexpr (kPairs) {
              // matrix entries arrive duplicated: mr2[m] = (M[m], M[m])
              float2 mr2[d1 * d3p];
              load_matrix<T, 2 * d1 * d3p>(mbuf + 2 * F.m_off[q], reinterpret_cast<T*>(mr2));
#pragma unroll
              for (int p = 0; p < NP; ++p) {
                const float2 w2 = make_float2(wv[2 * p], wv[2 * p + 1]);
#pragma unroll
                for (int k = 0; k < d3; ++k) {
                  float2 t = mul2(mr2[k], make_float2(xl[(2 * p) * d1], xl[(2 * p + 1) * d1]));
#pragma unroll
                  for (int i = 1; i < d1; ++i)
                    t = fma2(mr2[i * d3p + k], make_float2(xl[(2 * p) * d1 + i], xl[(2 * p + 1) * d1 + i]), t);
                  float2* a2 = reinterpret_cast<float2*>(al) + (k * NP + p);
                  *a2 = fma2(w2, t, *a2);
                }
              }
            } else {
              T mr[d1 * d3p];
              load_matrix<T, d1 * d3p>(mbuf + F.m_off[q], mr);
#pragma unroll
              for (int c = 0; c < CPL; ++c) {
#pragma unroll
                for (int k = 0; k < d3; ++k) {
                  T t = mr[k] * xl[c * d1];
#pragma unroll
                  for (int i = 1; i < d1; ++i) t = fma(mr[i * d3p + k], xl[c * d1 + i], t);
                  al[c * d3 + k] = fma(wv[c], t, al[c * d3 + k]);
                }
              }
            }
          }
        });
      });
      __syncwarp();  // every lane is done with this stage, mbuf and ybuf
      const int src_now = src_ahead;
      if (e + stages + 1 < e_end) src_ahead = P.src[e + stages + 1];
      if (e + stages < e_end) issue(e + stages, src_now, s);
      if (++s == stages) {
        s = 0;
        parity ^= 1u;
      }
    }
    if (!alive) break;
    // flush the node's accumulators
    static_for<0, LO + 1>([&](auto l3c) {
      constexpr int l3 = decltype(l3c)::value;
      constexpr int d3 = 2 * l3 + 1;
      if (F.o_off[l3] >= 0) {
        T* dst = P.out + n * F.O + F.o_off[l3] + c0 * d3 + lane * (CPL * d3);
        T* al = &acc[l3 * l3 * CPL];
        T row[CPL * d3];  // memory order: channel-major, component-minor
        if constexpr (kPairs) {
#pragma unroll
          for (int p = 0; p < NP; ++p)
#pragma unroll
            for (int k = 0; k < d3; ++k) {
              row[(2 * p) * d3 + k] = al[(k * NP + p) * 2];
              row[(2 * p + 1) * d3 + k] = al[(k * NP + p) * 2 + 1];
            }
        } else {
#pragma unroll
          for (int a = 0; a < CPL * d3; ++a) row[a] = al[a];
        }
        if (P.accumulate) {
          T old[CPL * d3];
          load_vectors<T, CPL, d3>(dst, old);
#pragma unroll
          for (int a = 0; a < CPL * d3; ++a) row[a] += old[a];
        }
        store_vectors<T, CPL, d3>(dst, row);
      }
    });
  }
  if (!alive) {
    // let copies that are still in flight land before the CTA's shared memory is released
    for (int d = 1; d < stages; ++d) {
      if (++s == stages) {
        s = 0;
        parity ^= 1u;
      }
      if (e + d < e_end) mbar_wait_bounded(&bars[s], parity);
    }
  }
}


template <typename T, int CPL, int LX, int LO>
int launch_fast_fwd_one(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph, const T* x,
                        const T* y, const T* w, T* out, bool accumulate, cudaStream_t stream) {
  const FastMeta& f = plan->fast;
  FwdParams<T> P;
  P.meta = f;
  P.x = x;
  P.y = y;
  P.w = w;
  P.out = out;
  P.src = graph->src;
  P.dst_rowptr = graph->dst_rowptr;
  P.ell_j = dt.ell_j;
  P.ell_c = static_cast<const T*>(dt.ell_c);
  P.status = dt.status;
  P.num_nodes = graph->num_nodes;
  P.num_edges = graph->num_edges;
  P.accumulate = accumulate ? 1 : 0;
  const size_t stage = static_cast<size_t>(f.w_stage_elems + f.x_stage_elems) * sizeof(T);
  auto kernel = fast_fwd_kernel<T, CPL, LX, LO>;
  cudaFuncAttributes attr;
  LUNA_CUDA_CHECK(cudaFuncGetAttributes(&attr, kernel));
  const Residency r = choose_residency(stage, fwd_fixed_bytes<T, CPL>(f), ell_bytes<T>(f.m_total, f.m_terms),
                                       dt.max_smem_optin, attr.numRegs, kFwdMaxWarps, 2, 3);
  if (r.depth == 0) return fail(LUNA_ERR_UNSUPPORTED, "staged forward needs more shared memory than the device has");
  P.stages = r.depth;
  const size_t block_bytes = r.block_bytes;
  const int nwarps = r.warps;
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(block_bytes)));
  // without this the driver may size the shared-memory carve-out for fewer CTAs than planned
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  const int64_t blocks = grid_blocks(graph->num_edges, 1024, r, dt.sm_count);
  const dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(f.chunks));
  kernel<<<grid, nwarps * 32, block_bytes, stream>>>(P);
  LUNA_LAUNCH_CHECK("staged forward");
  return LUNA_OK;
}

// Dispatch on the degree class: the smallest compiled (LX, LO) that covers the plan.
template <typename T, int CPL>
int launch_fast_fwd(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph, const T* x,
                    const T* y, const T* w, T* out, bool accumulate, cudaStream_t stream) {
  const int lx = plan->fast.LX, lo = plan->fast.LO;
  if (lx <= 1 && lo <= 1) return launch_fast_fwd_one<T, CPL, 1, 1>(plan, dt, graph, x, y, w, out, accumulate, stream);
  if (lx <= 2 && lo <= 2) return launch_fast_fwd_one<T, CPL, 2, 2>(plan, dt, graph, x, y, w, out, accumulate, stream);
  if (lx <= 2 && lo <= 3) return launch_fast_fwd_one<T, CPL, 2, 3>(plan, dt, graph, x, y, w, out, accumulate, stream);
  return launch_fast_fwd_one<T, CPL, 3, 3>(plan, dt, graph, x, y, w, out, accumulate, stream);
}

}  // namespace fastk
}  // namespace luna
