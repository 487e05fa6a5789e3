// Staged forward-shaped kernel (free argument g):  out[t] = sum_{e: dst e = t} sum_p w_p * (M^p(y_e)^T x[src e]).
//
// Destination nodes are cut into small tiles of consecutive nodes, handed to the warps in ascending order (the first
// round statically, then from a counter): a tile is a contiguous piece of the destination-sorted edge list, reduced
// by one warp with register accumulators and no atomics on data (results do not depend on which warp took a tile),
// and at any moment the resident warps work on neighbouring destination nodes, so that for a spatially
// ordered graph the x[src] rows they gather are the same few thousand rows and stay in L2.  Per
// edge, lanes issue 1-D bulk copies (cp.async.bulk, completion on an mbarrier) of the edge's weight row and of the
// gathered x[src] row into the warp's ring of shared-memory stages; the warp then reads them with 128-bit shared
// loads while later edges are in flight.  A lane owns CPL consecutive channels of every block.
//
// FP32 arithmetic runs on packed two-wide FMAs (fma.rn.f32x2): on B200 the scalar FFMA rate is about 0.7 of the
// packed rate, and packing halves the instruction count of the loop, which is what limits this kernel (issue slots
// and instruction-cache footprint), not bytes.  Two consecutive channels of a lane form a pair that lives in one
// 64-bit register from the moment it is formed: x pairs are formed once per edge from scalar shared-memory loads,
// weights arrive as ready-made pairs, accumulators are unpacked only when a node is flushed.  The per-edge coupling
// matrices are stored once; a matrix entry enters the packed FMA as a broadcast operand.  Every path is evaluated
// as out_k += sum_i M[i][k] * (x_i * w): the accumulators are the only long-lived operands of the FMAs.
//
// What limits the kernel is the latency of a path's shared-memory loads in front of its arithmetic, with only two
// warps per scheduler to hide it.  For the canonical full path lists (see canon_ok) the loops over paths are
// therefore unrolled from compile-time tables, so that the loads of the next path are issued during the
// arithmetic of the current one; a lane also keeps its share of the coupling-matrix program in registers.
#pragma once

#include <algorithm>
#include <cstdlib>

#include "cg_patterns.h"
#include "uvu_packets.cuh"

namespace luna {
namespace fastk {

// Whether the coupling tensor with pattern PT has a non-zero entry C[i][j][k] for some j: only those (i, k) have a
// non-zero entry in an edge's coupling matrix.
template <typename PT>
__host__ __device__ constexpr bool pattern_has_ik(int i, int k) {
  for (int t = 0; t < PT::n; ++t)
    if (PT::t[t].i == i && PT::t[t].k == k) return true;
  return false;
}

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
  int64_t tile_nodes;  // destination nodes per tile
  unsigned* tile_counters;  // (next tile, warps finished) per channel chunk
  int stages;
  int accumulate;
};

// packet shape of the forward kernel: FP32 pairs whenever a lane has an even number of channels
template <typename T, int CPL>
using FPk = PkT<T, CPL, UsePairs<T, CPL>::value>;

template <typename T, int CPL>
__host__ __device__ inline size_t fwd_fixed_bytes(const FastMeta& f) {
  // M buffer (padded to whole rounds of 32 entries), y row, barriers
  const size_t m_elems = static_cast<size_t>(f.m_total + 31) / 32 * 32;
  return (m_elems + 32) * sizeof(T) + kMaxStages * sizeof(uint64_t);
}

// Register budget of the coupling-matrix program: a lane keeps the two terms of up to this many entries in
// registers (3 registers each); longer programs are read from shared memory.
constexpr int kMaxProgramRounds = 12;

// L2 >= 0: the path list is the canonical full list for (LX, L2, LO) and the loops over paths are unrolled from
// compile-time tables.  L2 < 0: any path list, loops over paths read the tables in FastMeta.
template <typename T, int CPL, int LX, int LO, int L2>
__global__ void __launch_bounds__(kFwdMaxWarps * 32, 1) fast_fwd_kernel(const __grid_constant__ FwdParams<T> P) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  using PK = FPk<T, CPL>;
  using V = typename PK::V;
  constexpr int NP = PK::NP;
  constexpr bool kCanon = L2 >= 0;
  constexpr int kCanonTotal = kCanon ? canon_moff(LX, L2 < 0 ? 0 : L2, LO, -1, -1, -1) : 0;
  constexpr int kRounds = (kCanonTotal + 31) / 32;
  constexpr bool kProgramInRegisters = kCanon && kRounds <= kMaxProgramRounds;
  const FastMeta& F = P.meta;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int stages = P.stages;
  const int stage_elems = F.w_stage_elems + F.x_stage_elems;
  const int m_total = kCanon ? kCanonTotal : F.m_total;
  const T* ell_c;
  const unsigned char* ell_j;
  load_ell<T>(smem_raw, P.ell_c, P.ell_j, m_total, F.m_terms, &ell_c, &ell_j);
  const size_t warp_bytes = static_cast<size_t>(stages) * stage_elems * sizeof(T) + fwd_fixed_bytes<T, CPL>(F);
  unsigned char* base = smem_raw + ell_bytes<T>(m_total, F.m_terms) + static_cast<size_t>(warp) * warp_bytes;
  T* stage_mem = reinterpret_cast<T*>(base);
  T* mbuf = stage_mem + static_cast<size_t>(stages) * stage_elems;
  T* ybuf = mbuf + (m_total + 31) / 32 * 32;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ybuf + 32);

  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
  }
  __syncwarp();

  // the lane's share of the coupling-matrix program: entries lane, lane + 32, ...
  T prog_a[kProgramInRegisters ? kRounds : 1], prog_b[kProgramInRegisters ? kRounds : 1];
  unsigned prog_j[kProgramInRegisters ? kRounds : 1];
  if constexpr (kProgramInRegisters) {
#pragma unroll
    for (int r = 0; r < kRounds; ++r) {
      const int m = r * 32 + lane;
      const bool in = m < m_total;
      prog_a[r] = in ? ell_c[m] : T(0);
      prog_b[r] = in ? ell_c[m_total + m] : T(0);
      prog_j[r] = in ? (static_cast<unsigned>(ell_j[m]) | (static_cast<unsigned>(ell_j[m_total + m]) << 8)) : 0u;
    }
  }

  const int chw = 32 * CPL;
  const int c0 = blockIdx.y * chw;  // first channel of this warp's chunk
  const int64_t N = P.num_nodes;
  const int nwarps = blockDim.x >> 5;
  const int64_t total_warps = static_cast<int64_t>(gridDim.x) * nwarps;
  const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * nwarps + warp;
  const int64_t num_tiles = (N + P.tile_nodes - 1) / P.tile_nodes;

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

  constexpr int AR = (LO + 1) * (LO + 1) * NP;
  constexpr int XR = (LX + 1) * (LX + 1) * NP;
  V acc[AR];  // packet (l3, k, p) at l3 * l3 * NP + k * NP + p
  int64_t e = 0, e_end = 0;
  int s = 0;            // stage of the next edge; the ring keeps turning from one tile to the next
  uint32_t parity = 0;  // phase of that stage's barrier
  bool alive = true;

  // out_k += sum_i M[i][k] * (x_i * w) for one path; the matrix is stored once and broadcast into both halves.
  // With a compile-time degree l2 (canonical lists) the entries that the coupling tensor leaves zero for every y -
  // about a quarter of them - are skipped.
  auto path_body = [&](auto l1c, auto l2c, auto l3c, const T* wq, const T* matrix, const V* xl, V* al) {
    constexpr int l1 = decltype(l1c)::value, l2 = decltype(l2c)::value, l3 = decltype(l3c)::value;
    constexpr int d1 = 2 * l1 + 1, d3 = 2 * l3 + 1, d3p = d3 + 1;
    using PT = CgPattern<l1, (l2 < 0 ? 0 : l2), l3>;
    V w2[NP];  // a lane's consecutive channels are already adjacent in memory
    load_lane_packets<PK, T, CPL>(wq, w2);
    static_for<0, d1>([&](auto ic) {
      constexpr int i = decltype(ic)::value;
      T mrow[d3p];
      load_plain_row<T, d3p, i>(matrix, mrow);
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        const V xw = vmul(xl[i * NP + p], w2[p]);
        static_for<0, d3>([&](auto kc) {
          constexpr int k = decltype(kc)::value;
          if constexpr (l2 < 0 || pattern_has_ik<PT>(i, k))
            al[k * NP + p] = vfma(bcast_packet(mrow[k], V{}), xw, al[k * NP + p]);
        });
      }
    });
  };

  // A warp's first tile is its own number; further tiles are taken from a counter, one ahead of need, so that a warp
  // that started late or met long rows simply takes fewer.
  unsigned* counters = P.tile_counters + 2 * blockIdx.y;
  int64_t tile = gwarp;
#pragma unroll 1
  while (tile < num_tiles && alive) {
  const int64_t tile_after = take_tile(counters, total_warps, lane);
  const int64_t n_lo = tile * P.tile_nodes;
  const int64_t n_hi = n_lo + P.tile_nodes < N ? n_lo + P.tile_nodes : N;
  const int64_t e_begin = P.dst_rowptr[n_lo];
  e_end = P.dst_rowptr[n_hi];
  e = e_begin;
  // all stages are empty here: fill them in ring order from the current one
  for (int d = 0, stage = s; d < stages; ++d) {
    if (e_begin + d < e_end) issue(e_begin + d, P.src[e_begin + d], stage);
    if (++stage == stages) stage = 0;
  }
  // source node of the edge that will be issued in the next iteration, fetched one iteration early
  int src_ahead = e_begin + stages < e_end ? P.src[e_begin + stages] : 0;
  T y_next = (lane < F.Y && e_begin < e_end) ? P.y[e_begin * F.Y + lane] : T(0);

  for (int64_t n = n_lo; n < n_hi && alive; ++n) {
    const int64_t ee = P.dst_rowptr[n + 1];
#pragma unroll
    for (int a = 0; a < AR; ++a) acc[a] = zero_packet<V>();
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
      if constexpr (kProgramInRegisters) {
#pragma unroll
        for (int r = 0; r < kRounds; ++r)
          mbuf[r * 32 + lane] = fma(prog_b[r], ybuf[prog_j[r] >> 8], prog_a[r] * ybuf[prog_j[r] & 255u]);
      } else {
        compute_m_share<T, false>(ell_c, ell_j, ybuf, mbuf, m_total, 0, 1, lane);
      }
      if (e + 1 < e_end && lane < F.Y) y_next = P.y[(e + 1) * F.Y + lane];
      // this lane's x packets, formed once per edge: packet (l1, i, p) at l1 * l1 * NP + i * NP + p
      V xr[XR];
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        constexpr int d1 = 2 * l1 + 1;
        if (kCanon || F.x_off[l1] >= 0)
          load_packets_scalar<PK, T, CPL, d1>(xs + (kCanon ? chw * l1 * l1 : F.xs_off[l1]) + lane * (CPL * d1),
                                              &xr[l1 * l1 * NP]);
      });
      __syncwarp();

      const T* wl = ws + lane * CPL;
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        if (!kCanon && F.x_off[l1] < 0) return;
        const V* xl = &xr[l1 * l1 * NP];
        static_for<0, LO + 1>([&](auto l3c) {
          constexpr int l3 = decltype(l3c)::value;
          V* al = &acc[l3 * l3 * NP];
          if constexpr (kCanon) {
            static_for<0, (L2 < 0 ? 0 : L2) + 1>([&](auto l2c) {
              constexpr int l2 = decltype(l2c)::value;
              if constexpr (canon_ok(LX, L2, LO, l1, l2, l3))
                path_body(l1c, l2c, l3c, wl + canon_wrank(LX, L2, LO, l1, l2, l3) * chw,
                          mbuf + canon_moff(LX, L2, LO, l1, l2, l3), xl, al);
            });
          } else {
            const int q_end = F.pair_ptr[l3 * (kMaxFastL + 1) + l1 + 1];
#pragma unroll 1
            for (int q = F.pair_ptr[l3 * (kMaxFastL + 1) + l1]; q < q_end; ++q)
              path_body(l1c, std::integral_constant<int, -1>{}, l3c, wl + F.w_soff[q], mbuf + F.m_off[q], xl, al);
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
        T row[CPL * d3];  // memory order: channel-major, component-minor
        unpack_packets<PK, T, CPL, d3>(&acc[l3 * l3 * NP], row);
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
  tile = tile_after;
  }
  leave_tiles(counters, total_warps, lane);
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


template <typename T, int CPL, int LX, int LO, int L2>
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
  P.tile_counters = next_tile_counters(plan, dt);
  const size_t stage = static_cast<size_t>(f.w_stage_elems + f.x_stage_elems) * sizeof(T);
  auto kernel = fast_fwd_kernel<T, CPL, LX, LO, L2>;
  cudaFuncAttributes attr;
  LUNA_CUDA_CHECK(cudaFuncGetAttributes(&attr, kernel));
  const Residency r = choose_residency(stage, fwd_fixed_bytes<T, CPL>(f), ell_bytes<T>(f.m_total, f.m_terms),
                                       dt.max_smem_optin, attr.numRegs, capped_warps(plan->tuning, kFwdMaxWarps), 2, 3);
  if (r.depth == 0) return fail(LUNA_ERR_UNSUPPORTED, "staged forward needs more shared memory than the device has");
  P.stages = r.depth;
  const size_t block_bytes = r.block_bytes;
  const int nwarps = r.warps;
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(block_bytes)));
  // without this the driver may size the shared-memory carve-out for fewer CTAs than planned
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  const double degree = static_cast<double>(graph->num_edges) / static_cast<double>(std::max<int64_t>(graph->num_nodes, 1));
  const int64_t tile_edges =
      tile_edges_for(graph->num_edges, static_cast<int64_t>(dt.sm_count) * r.ctas * nwarps,
                     plan->tuning.fwd_tile_edges > 0 ? plan->tuning.fwd_tile_edges : 64);
  P.tile_nodes = std::max<int64_t>(1, static_cast<int64_t>(tile_edges / std::max(degree, 1e-3) + 0.5));
  P.tile_nodes = std::min<int64_t>(P.tile_nodes, 1 << 20);
  const int64_t num_tiles = ceil_div(std::max<int64_t>(graph->num_nodes, 1), P.tile_nodes);
  const int64_t wave = static_cast<int64_t>(dt.sm_count) * r.ctas;  // CTAs resident at once
  const int64_t blocks = std::max<int64_t>(1, std::min<int64_t>(wave, ceil_div(num_tiles, nwarps)));
  const dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(f.chunks));
  kernel<<<grid, nwarps * 32, block_bytes, stream>>>(P);
  LUNA_LAUNCH_CHECK("staged forward");
  return LUNA_OK;
}

// Dispatch: a kernel unrolled for the canonical full path list if the plan has one of the compiled shapes, else
// the smallest compiled degree class (LX, LO) that covers the plan, with loops over the plan's path tables.
template <typename T, int CPL>
int launch_fast_fwd(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph, const T* x,
                    const T* y, const T* w, T* out, bool accumulate, cudaStream_t stream) {
  const int lx = plan->fast.LX, lo = plan->fast.LO, l2 = plan->fast.canon_l2;
#define LUNA_FWD_ARGS plan, dt, graph, x, y, w, out, accumulate, stream
  if (!plan->tuning.no_canon) {
    if (lx == 2 && l2 == 3 && lo == 3) return launch_fast_fwd_one<T, CPL, 2, 3, 3>(LUNA_FWD_ARGS);
    if (lx == 2 && l2 == 2 && lo == 2) return launch_fast_fwd_one<T, CPL, 2, 2, 2>(LUNA_FWD_ARGS);
    if (lx == 3 && l2 == 3 && lo == 3) return launch_fast_fwd_one<T, CPL, 3, 3, 3>(LUNA_FWD_ARGS);
    if (lx == 1 && l2 == 1 && lo == 1) return launch_fast_fwd_one<T, CPL, 1, 1, 1>(LUNA_FWD_ARGS);
  }
  if (lx <= 1 && lo <= 1) return launch_fast_fwd_one<T, CPL, 1, 1, -1>(LUNA_FWD_ARGS);
  if (lx <= 2 && lo <= 2) return launch_fast_fwd_one<T, CPL, 2, 2, -1>(LUNA_FWD_ARGS);
  if (lx <= 2 && lo <= 3) return launch_fast_fwd_one<T, CPL, 2, 3, -1>(LUNA_FWD_ARGS);
  return launch_fast_fwd_one<T, CPL, 3, 3, -1>(LUNA_FWD_ARGS);
#undef LUNA_FWD_ARGS
}

}  // namespace fastk
}  // namespace luna
