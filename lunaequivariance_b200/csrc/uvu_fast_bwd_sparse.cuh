// Staged source-major kernel for canonical full path lists, with the coupling tensors' non-zero patterns compiled in
// (cg_patterns.h): first derivatives gx, gy, gw in one pass over the weights.
//
// Work assignment is that of fast_bwd_kernel (a warp owns a range of source nodes and walks their out-edges).
//
// Data movement.  DRAM is used well only with large contiguous requests, so an edge's whole weight row comes in
// with one bulk copy into one of the warp's two to four row stages, the weight gradients of the edge are written over the
// weights in that stage (every lane overwrites exactly the words it has read) and the row goes back to gw with one
// bulk store; the stage is refilled once the store has read it.  Row copies carry an evict-first L2 hint.  The
// gathered g[dst] row is cut into one block per output degree; these go through a small ring of slots with the
// default L2 priority (an evict-last hint was measured to hurt: the rows of a large graph then crowd each other
// and the next kernel out of L2).
//
// Arithmetic.  With the pattern of C^p known at compile time, a path is a straight line of packed FMAs over its
// terms t = (i, j, k), in (i, k, j) order:
//     s_i   += (c_t y_j) * g_k                         the per-edge scalars c_t y_j come from a small program
//     gx_i  += w_p * s_i,   gw_p += x_i * s_i           at the end of row i
//     P_ik   = sum over the lane's channels of (x_i w_p) * g_k      once per distinct (i, k)
//     gy_j  += c_t * P_ik                               register accumulators of the edge, per lane
// so the edge-attribute gradient is contracted inside each lane and only its in2_dim values cross lanes (one pass
// through the reduction tile per edge), instead of every (path, i, k) entry.  There are no branches, calls or
// shared-memory round trips inside a unit, which lets the compiler overlap the loads of one path with the
// arithmetic of another; with two warps per scheduler that, not the instruction count, decides the speed.
// Every output element is written by exactly one thread in a fixed order: deterministic.
#pragma once

#include "uvu_fast_bwd.cuh"

namespace luna {
namespace fastk {

constexpr int kMaxSparseRounds = 16;  // program entries a lane keeps in registers (two registers each)
constexpr int kSparseTileRows = 8;    // reduction tile: one pair of gy entries per row (in2_dim <= 16)
constexpr int kMaxRowStages = 4;      // weight-row stages per warp (the edge ids of four edges are kept ahead)

template <typename T>
__host__ __device__ inline size_t sparse_fixed_bytes(const FastMeta& f, int row_stages) {
  // weight-row stages, per-edge scalars c_t y_j, reduction tile, reduced gy row, y row, barriers
  const size_t elems = static_cast<size_t>(row_stages) * f.w_stage_elems +
                       static_cast<size_t>(f.sparse_terms + 31) / 32 * 32 +
                       static_cast<size_t>(kSparseTileRows) * red_stride<T>() + 32 + 32;
  return elems * sizeof(T) + (kMaxRowStages + kMaxSlots) * sizeof(uint64_t);
}
// One slot of the g ring: the widest degree block of the row.
template <typename T>
__host__ __device__ inline size_t sparse_slot_bytes(const FastMeta& f) {
  return static_cast<size_t>(32 * f.cpl) * (2 * f.LO + 1) * sizeof(T);
}
// Per-CTA shared tables: the term coefficients.
template <typename T>
__host__ __device__ inline size_t sparse_shared_bytes(const FastMeta& f) {
  return (static_cast<size_t>(f.sparse_terms) * sizeof(T) + 127) / 128 * 128;
}

// Four consecutive entries of a 16-byte aligned table; every lane reads the same address.
template <typename T>
__device__ __forceinline__ void load_four(const T* p, T* out) {
  if constexpr (sizeof(T) == 4) {
    const Vec<T, 4> t = *reinterpret_cast<const Vec<T, 4>*>(p);
#pragma unroll
    for (int c = 0; c < 4; ++c) out[c] = t.a[c];
  } else {
    const Vec<T, 2> a = reinterpret_cast<const Vec<T, 2>*>(p)[0], b = reinterpret_cast<const Vec<T, 2>*>(p)[1];
    out[0] = a.a[0];
    out[1] = a.a[1];
    out[2] = b.a[0];
    out[3] = b.a[1];
  }
}

// Adds the 32 lane contributions of tile rows [0, ROWS) (row r holds the lanes' values of entries 2r and 2r + 1,
// interleaved) and writes the sums to out[0 .. 2 * ROWS).  Four lanes share a row, a quarter each.
template <typename T, int ROWS>
__device__ __forceinline__ void reduce_tile_rows(const T* red, T* out, int lane) {
  static_assert(ROWS <= kSparseTileRows, "tile too small");
  __syncwarp();
  constexpr int per = 16 / static_cast<int>(sizeof(T));
  const int r = lane & 7, part = lane >> 3;
  const T* seg = red + r * red_stride<T>() + part * 16;
  T s0 = T(0), s1 = T(0);
#pragma unroll
  for (int v = 0; v < 16 / per; ++v) {
    const Vec<T, per> q = reinterpret_cast<const Vec<T, per>*>(seg)[v];
#pragma unroll
    for (int c = 0; c < per; c += 2) {
      s0 += q.a[c];
      s1 += q.a[c + 1];
    }
  }
  s0 += __shfl_xor_sync(0xffffffffu, s0, 8);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 8);
  s0 += __shfl_xor_sync(0xffffffffu, s0, 16);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 16);
  if (lane < ROWS) {
    Vec<T, 2> pr{{s0, s1}};
    reinterpret_cast<Vec<T, 2>*>(out)[lane] = pr;
  }
  __syncwarp();
}

// ---- one path of the sparse formulation, row by row ------------------------------------------------------------------
// Positions inside a pattern's term list, which is sorted by (i, k, j): where the row of term t ends, and which
// distinct (i, k) of its row a term belongs to.
template <typename PT>
__host__ __device__ constexpr int pattern_row_end(int t0) {
  int t = t0;
  while (t < PT::n && PT::t[t].i == PT::t[t0].i) ++t;
  return t;
}
template <typename PT>
__host__ __device__ constexpr int pattern_ik_slot(int t0, int t) {
  int slot = 0;
  for (int q = t0 + 1; q <= t; ++q)
    if (PT::t[q].k != PT::t[q - 1].k) ++slot;
  return slot;
}

// Computes one path for a lane's packets.  xl / gxl: the lane's x and gx packets of degree l1; g2: its g packets of
// degree l3; w2: its weights; dot: receives sum_i x_i s_i (the weight gradient before unpacking).
//
// The arithmetic of a row i is issued in three batches of mutually independent instructions, so that the latency of
// one is covered by the others even when few warps are resident:
//   P_ik = sum over the lane's packets of (x_i w) g_k      for every distinct k of the row
//   gy_j += c_t P_ik                                       for every term of the row
//   s_i   = sum_t (c_t y_j) g_k                            in two alternating partial sums
template <typename T, int CPL, int LX, int L2, int LO, int l1, int l2, int l3, bool WXW, bool WY, typename V>
__device__ __forceinline__ void sparse_path_rows(const V* xl, V* gxl, V* gy2, const V* g2, const V* w2, V* dot,
                                                 const T* cybuf, const T* ctab) {
  using PK = PkT<T, CPL, UsePairs<T, CPL>::value>;
  constexpr int NP = PK::NP;
  using PT = CgPattern<l1, l2, l3>;
  constexpr int n = PT::n;
  constexpr int toff = canon_toff(LX, L2, LO, l1, l2, l3);
#pragma unroll
  for (int p = 0; p < NP; ++p) dot[p] = zero_packet<V>();
  static_for<0, n>([&](auto tc) {
    constexpr int t0 = decltype(tc)::value;
    constexpr bool row_first = t0 == 0 || PT::t[t0 == 0 ? 0 : t0 - 1].i != PT::t[t0].i;
    if constexpr (row_first) {
      constexpr int i = PT::t[t0].i;
      constexpr int t1 = pattern_row_end<PT>(t0);
      constexpr int len = t1 - t0;
      constexpr int g_lo = t0 / 4, g_hi = (t1 - 1) / 4;  // groups of four table entries that cover the row
      T cy[WXW ? 4 * (g_hi - g_lo + 1) : 1], cc[WY ? 4 * (g_hi - g_lo + 1) : 1];
      static_for<g_lo, g_hi + 1>([&](auto gc) {
        constexpr int group = decltype(gc)::value;
        if constexpr (WXW) load_four<T>(cybuf + toff + 4 * group, cy + 4 * (group - g_lo));
        if constexpr (WY) load_four<T>(ctab + toff + 4 * group, cc + 4 * (group - g_lo));
      });
      if constexpr (WY) {
        V xw[NP];
#pragma unroll
        for (int p = 0; p < NP; ++p) xw[p] = vmul(xl[i * NP + p], w2[p]);
        constexpr int slots = pattern_ik_slot<PT>(t0, t1 - 1) + 1;
        V pik[slots];
        static_for<t0, t1>([&](auto uc) {
          constexpr int t = decltype(uc)::value;
          constexpr bool ik_first = t == t0 || PT::t[t - 1].k != PT::t[t].k;
          if constexpr (ik_first) {
            constexpr int k = PT::t[t].k, slot = pattern_ik_slot<PT>(t0, t);
            pik[slot] = vmul(xw[0], g2[k * NP]);
#pragma unroll
            for (int p = 1; p < NP; ++p) pik[slot] = vfma(xw[p], g2[k * NP + p], pik[slot]);
          }
        });
        static_for<t0, t1>([&](auto uc) {
          constexpr int t = decltype(uc)::value;
          constexpr int j = PT::t[t].j, slot = pattern_ik_slot<PT>(t0, t);
          gy2[l2 * l2 + j] = vfma(bcast_packet(cc[t - 4 * g_lo], V{}), pik[slot], gy2[l2 * l2 + j]);
        });
      }
      if constexpr (WXW) {
        V sa[NP], sb[NP];
        static_for<t0, t1>([&](auto uc) {
          constexpr int t = decltype(uc)::value;
          constexpr int k = PT::t[t].k, r = t - t0;
          const V c = bcast_packet(cy[t - 4 * g_lo], V{});
#pragma unroll
          for (int p = 0; p < NP; ++p) {
            if constexpr (r == 0) {
              sa[p] = vmul(c, g2[k * NP + p]);
            } else if constexpr (r == 1) {
              sb[p] = vmul(c, g2[k * NP + p]);
            } else if constexpr (r % 2 == 0) {
              sa[p] = vfma(c, g2[k * NP + p], sa[p]);
            } else {
              sb[p] = vfma(c, g2[k * NP + p], sb[p]);
            }
          }
        });
#pragma unroll
        for (int p = 0; p < NP; ++p) {
          if constexpr (len >= 2) sa[p] = vadd(sa[p], sb[p]);
          gxl[i * NP + p] = vfma(w2[p], sa[p], gxl[i * NP + p]);
          dot[p] = vfma(xl[i * NP + p], sa[p], dot[p]);
        }
      }
    }
  });
}

// Warps per CTA at most (caps the registers per thread): FP32 with at most two channels per lane needs fewer
// registers and runs up to 12 warps (168 registers), everything else 8 (255).
#ifndef LUNA_SPARSE_WARPS_SMALL
#define LUNA_SPARSE_WARPS_SMALL 16
#endif
// Shapes up to degree 2 keep far less state per lane (9 x and gx packets, 9 gy accumulators, a short program) and run
// 16 warps at 128 registers (measured on the 64-channel degree-2 workload: 29.4 ms at 12 warps, 26.6 ms at 16).
template <typename T, int CPL, int LX = 3, int L2 = 3, int LO = 3>
__host__ __device__ constexpr int sparse_max_warps() {
  if (sizeof(T) == 4 && CPL <= 2) return (LX <= 2 && L2 <= 2 && LO <= 2) ? LUNA_SPARSE_WARPS_SMALL : 12;
  return 8;
}

template <typename T, int CPL, int LX, int L2, int LO, bool WXW, bool WY>
__global__ void __launch_bounds__(sparse_max_warps<T, CPL, LX, L2, LO>() * 32, 1) fast_bwd_sparse_kernel(const __grid_constant__ BwdParams<T> P) {
  using PK = Pk<T, CPL>;
  using V = typename PK::V;
  constexpr int NP = PK::NP;
  constexpr int TT = canon_toff(LX, L2, LO, -1, -1, -1);  // terms, padded per path
  constexpr int kRounds = (TT + 31) / 32;
  static_assert(kRounds <= kMaxSparseRounds, "coupling program too long for the register budget");
  constexpr int YD = (L2 + 1) * (L2 + 1);
  static_assert((YD + 1) / 2 <= kSparseTileRows, "edge attributes too wide for the reduction tile");
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const FastMeta& F = P.meta;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int R = P.slots;  // slots of the g ring
  constexpr int nk = LO + 1;
  constexpr int chw = 32 * CPL;
  constexpr int gslot_elems = chw * (2 * LO + 1);
  const int c0 = blockIdx.y * chw;
  const int wrow_elems = F.w_stage_elems;

  // CTA-wide table: term coefficients
  T* ctab = reinterpret_cast<T*>(smem_raw);
  for (int i = threadIdx.x; i < TT; i += blockDim.x) ctab[i] = P.sp_c[i];
  __syncthreads();

  const int S = P.row_stages;  // weight-row stages
  const size_t warp_bytes = static_cast<size_t>(R) * gslot_elems * sizeof(T) + sparse_fixed_bytes<T>(F, S);
  T* wst = reinterpret_cast<T*>(smem_raw + sparse_shared_bytes<T>(F) + static_cast<size_t>(warp) * warp_bytes);
  T* gsl = wst + static_cast<size_t>(S) * wrow_elems;
  T* cybuf = gsl + static_cast<size_t>(R) * gslot_elems;
  T* red = cybuf + (TT + 31) / 32 * 32;
  T* gbuf = red + kSparseTileRows * red_stride<T>();
  T* ybuf = gbuf + 32;
  uint64_t* wbar = reinterpret_cast<uint64_t*>(ybuf + 32);
  uint64_t* gbar = wbar + kMaxRowStages;

  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&wbar[s], 1);
    for (int s = 0; s < R; ++s) mbar_init(&gbar[s], 1);
    fence_barrier_init();
  }
  __syncwarp();

  // the lane's share of the per-edge program cy[t] = c_t * y[j_t]: entries lane, lane + 32, ...
  T prog_c[kRounds];
  unsigned prog_j[(kRounds + 3) / 4];  // four 8-bit y indices per register
#pragma unroll
  for (int r = 0; r < (kRounds + 3) / 4; ++r) prog_j[r] = 0u;
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const int t = r * 32 + lane;
    prog_c[r] = t < TT ? ctab[t] : T(0);
    prog_j[r / 4] |= (t < TT ? static_cast<unsigned>(P.sp_j[t]) : 0u) << (8 * (r % 4));
  }

  const int64_t E = P.num_edges, N = P.num_src_nodes;
  const int nwarps = blockDim.x >> 5;
  const int64_t total_warps = static_cast<int64_t>(gridDim.x) * nwarps;
  const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * nwarps + warp;
  const int64_t bound_lo = E * gwarp / total_warps, bound_hi = E * (gwarp + 1) / total_warps;
  const int64_t n_lo = warp_lower_bound(P.src_rowptr, N, bound_lo, lane);
  const int64_t n_hi = gwarp == total_warps - 1 ? N : warp_lower_bound(P.src_rowptr, N, bound_hi, lane);
  if (n_lo >= n_hi) return;
  const int64_t p_begin = P.src_rowptr[n_lo], p_end = P.src_rowptr[n_hi];
  const bool want_x = WXW && P.gx != nullptr, want_w = WXW && P.gw != nullptr;
  const bool stage_gw = want_w && !P.acc_w;  // gradients overwrite the weights in the stage and leave as a row
  const int64_t total_units = (p_end - p_begin) * nk;

  // Weight rows: lane L moves piece L of the row (one piece when the row is contiguous for this CTA's channels).
  const int n_wp = F.n_w_pieces;
  auto load_row = [&](int64_t e, int st) {
    if (lane == 0) mbar_arrive_expect_tx(&wbar[st], static_cast<uint32_t>(wrow_elems * sizeof(T)));
    __syncwarp();
    if (lane < n_wp) {
      const CopyPiece pc = F.pieces_w[lane];
      bulk_copy_g2s_hint(wst + static_cast<size_t>(st) * wrow_elems + pc.s_off,
                         P.w + e * F.W + pc.g_off + static_cast<int64_t>(c0) * pc.comp,
                         static_cast<uint32_t>(pc.n * sizeof(T)), &wbar[st], l2_policy_evict_first());
    }
  };
  auto store_row = [&](int64_t e, int st) {
    fence_async_shared();  // the lanes' gradient writes, before the bulk store reads the stage
    __syncwarp();
    if (lane < n_wp) {
      const CopyPiece pc = F.pieces_w[lane];
      bulk_copy_s2g_hint(P.gw + e * F.W + pc.g_off + static_cast<int64_t>(c0) * pc.comp,
                         wst + static_cast<size_t>(st) * wrow_elems + pc.s_off, static_cast<uint32_t>(pc.n * sizeof(T)),
                         l2_policy_evict_first());
      bulk_commit_group();
    }
  };
  // g ring: one block of the destination's row per unit
  auto load_g = [&](int l3, int64_t d_node, int s) {
    const int d3 = 2 * l3 + 1;
    if (lane == 0) {
      mbar_arrive_expect_tx(&gbar[s], static_cast<uint32_t>(chw * d3 * sizeof(T)));
      bulk_copy_g2s(gsl + static_cast<size_t>(s) * gslot_elems, P.g + d_node * F.O + F.o_off[l3] + c0 * d3,
                    static_cast<uint32_t>(chw * d3 * sizeof(T)), &gbar[s]);
    }
  };

  // ids and destinations of the current and the next two edges; the id after those is fetched one step early
  // because the destination load depends on it
  auto id_at = [&](int64_t p) { return p < p_end ? P.edge_ids[p] : -1; };
  auto dst_of = [&](int e) { return e >= 0 ? P.dst[e] : 0; };
  int e0 = id_at(p_begin), e1 = id_at(p_begin + 1), e2 = id_at(p_begin + 2), e3 = id_at(p_begin + 3);
  int d0 = dst_of(e0), d1n = dst_of(e1), d2n = dst_of(e2);
  load_row(e0, 0);
  if (e1 >= 0) load_row(e1, 1);
  if (S > 2 && e2 >= 0) load_row(e2, 2);
  if (S > 3 && e3 >= 0) load_row(e3, 3);
  for (int v = 0; v < R && v < total_units; ++v) {
    const int de = v / nk, kind = v - de * nk;  // R <= 2 * nk, so de is 0 or 1
    load_g(kind, de == 0 ? d0 : d1n, v);
  }
  T y_next = (lane < F.Y && e0 >= 0) ? P.y[static_cast<int64_t>(e0) * F.Y + lane] : T(0);

  constexpr int XR = (LX + 1) * (LX + 1) * NP;
  V xr[XR], gxr[XR];
  const V ones = runtime_one<V, T>(F.m_terms);
  V gy2[WY ? YD : 1];
  int64_t pos = p_begin;
  int64_t u = 0;  // unit being consumed
  int s = 0;      // its slot in the g ring
  uint32_t gparity = 0;
  int st = 0;  // row stage of the current edge
  uint32_t wparity = 0;  // bit s: parity of stage s
  bool alive = true;
  bool store_pending = false;  // the previous edge's stage has a row store in flight; it is refilled after that
  bool first_edge = true;

  // One path: a straight line over its coupling terms.  wq: the lane's weights in the row stage (overwritten with
  // their gradients when the row is staged back); w_goff: their global offset.
  auto path_body = [&](auto l1c, auto l2c, auto l3c, const V* g2, T* wq, int64_t w_goff) {
    constexpr int l1 = decltype(l1c)::value, l2 = decltype(l2c)::value, l3 = decltype(l3c)::value;
    V w2[NP];  // a lane's consecutive channels are already adjacent in memory
    load_lane_packets<PK, T, CPL>(wq, w2);
    const V* xl = &xr[l1 * l1 * NP];
    V* gxl = &gxr[l1 * l1 * NP];
    V dot[NP];
    sparse_path_rows<T, CPL, LX, L2, LO, l1, l2, l3, WXW, WY, V>(xl, gxl, gy2, g2, w2, dot, cybuf, ctab);
    if (want_w) {
      T gwv[CPL];
      unpack_packets<PK, T, CPL, 1>(dot, gwv);
      if (stage_gw) {
        store_vectors<T, CPL, 1>(wq, gwv);
      } else {
        T* dstw = P.gw + w_goff;
        T old[CPL];
        load_vectors<T, CPL, 1>(dstw, old);
#pragma unroll
        for (int c = 0; c < CPL; ++c) gwv[c] += old[c];
        store_vectors_streaming<T, CPL, 1>(dstw, gwv);
      }
    }
  };

  // One unit = the paths into output degree l3 of the current edge.
  auto unit_body = [&](auto l3c, const T* gblock, T* wrow) {
    constexpr int l3 = decltype(l3c)::value;
    constexpr int d3 = 2 * l3 + 1;
    V g2[d3 * NP];
    load_packets_scalar<PK, T, CPL, d3>(gblock + lane * (CPL * d3), g2);
    settle_packets<d3 * NP>(g2, ones);
    const int64_t w_row = static_cast<int64_t>(e0) * F.W + lane * CPL + c0;
    static_for<0, LX + 1>([&](auto l1c) {
      constexpr int l1 = decltype(l1c)::value;
      static_for<0, L2 + 1>([&](auto l2c) {
        constexpr int l2 = decltype(l2c)::value;
        if constexpr (canon_ok(LX, L2, LO, l1, l2, l3))
          path_body(l1c, l2c, l3c, g2, wrow + canon_wrank(LX, L2, LO, l1, l2, l3) * chw + lane * CPL,
                    w_row + canon_wrank(LX, L2, LO, l1, l2, l3) * F.ch);
      });
    });
  };

  // waits for the unit's g block, runs the unit and refills the slot with the block R units later
  auto run_unit = [&](auto l3c, T* wrow) -> bool {
    constexpr int kind = decltype(l3c)::value;
    if (!mbar_wait_bounded(&gbar[s], gparity)) {
      if (lane == 0) atomicExch(P.status, 2);
      return false;
    }
    unit_body(l3c, gsl + static_cast<size_t>(s) * gslot_elems, wrow);
    __syncwarp();  // every lane is done with this slot
    if (u + R < total_units) {
      int next = kind + R, de = 0;
      if (next >= nk) {
        next -= nk;
        de = 1;
      }
      if (next >= nk) {
        next -= nk;
        de = 2;
      }
      load_g(next, de == 0 ? d0 : (de == 1 ? d1n : d2n), s);
    }
    ++u;
    if (++s == R) {
      s = 0;
      gparity ^= 1u;
    }
    return true;
  };

  for (int64_t n = n_lo; n < n_hi && alive; ++n) {
    const int64_t pe = P.src_rowptr[n + 1];
    if (pos >= pe) {
      // No out-edges: the row of gx was zero-filled (or is left as it is) by the launcher.  A run of such rows (a
      // destination-range shard has hundreds of thousands) is jumped over with one search for the row that holds the
      // warp's next edge, not walked one dependent load at a time.
      if (pos >= p_end) break;
      n = warp_lower_bound(P.src_rowptr, N, pos + 1, lane) - 2;
      continue;
    }
    {
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        constexpr int d1 = 2 * l1 + 1;
        load_packets_scalar<PK, T, CPL, d1>(P.x + n * F.X + F.x_off[l1] + c0 * d1 + lane * (CPL * d1),
                                            &xr[l1 * l1 * NP]);
      });
      settle_packets<XR>(xr, ones);
    }
#pragma unroll
    for (int a = 0; a < XR; ++a) gxr[a] = zero_packet<V>();

#pragma unroll 1
    for (; pos < pe && alive; ++pos) {
      // per-edge scalars, computed while the edge's row may still be in flight
      if (lane < F.Y) ybuf[lane] = y_next;
      __syncwarp();
      if constexpr (WXW) {
#pragma unroll
        for (int r = 0; r < kRounds; ++r)
          cybuf[r * 32 + lane] = prog_c[r] * ybuf[(prog_j[r / 4] >> (8 * (r % 4))) & 255u];
      }
      if (pos + 1 < p_end && lane < F.Y) y_next = P.y[static_cast<int64_t>(e1) * F.Y + lane];
      __syncwarp();
      if constexpr (WY) {
#pragma unroll
        for (int j = 0; j < YD; ++j) gy2[j] = zero_packet<V>();
      }

      // the edge's weight row
      if (!mbar_wait_bounded(&wbar[st], (wparity >> st) & 1u)) {
        if (lane == 0) atomicExch(P.status, 3);
        alive = false;
        break;
      }
      wparity ^= 1u << st;
      T* wrow = wst + static_cast<size_t>(st) * wrow_elems;

      static_for<0, LO + 1>([&](auto l3c) {
        if (alive) alive = run_unit(l3c, wrow);
        if constexpr (decltype(l3c)::value == 0) {
          // the other stage: once the previous edge's row store has read it, fetch the next edge's row into it
          if (store_pending) {
            if (lane < n_wp) bulk_wait_group_read_all();
            __syncwarp();
            store_pending = false;
          }
          // the row S - 1 edges ahead goes into the stage the previous edge has just left
          if (!first_edge && pos + S - 1 < p_end)
            load_row(S == 2 ? e1 : (S == 3 ? e2 : e3), st == 0 ? S - 1 : st - 1);
          first_edge = false;
        }
      });
      if (!alive) break;

      if (stage_gw) {
        store_row(e0, st);
        store_pending = true;
      }

      if constexpr (WY) {
        // the lane's partial gy row goes through the reduction tile: entry pair r in row r
        static_for<0, (YD + 1) / 2>([&](auto rc) {
          constexpr int r = decltype(rc)::value;
          Vec<T, 2> pr;
          pr.a[0] = hsum(gy2[2 * r]);
          if constexpr (2 * r + 1 < YD) {
            pr.a[1] = hsum(gy2[2 * r + 1]);
          } else {
            pr.a[1] = T(0);
          }
          *reinterpret_cast<Vec<T, 2>*>(red + r * red_stride<T>() + lane * 2) = pr;
        });
        reduce_tile_rows<T, (YD + 1) / 2>(red, gbuf, lane);
        if (lane < F.Y) {
          const T acc = lane < YD ? gbuf[lane] : T(0);
          if (P.gy_partial != nullptr) {
            P.gy_partial[(static_cast<int64_t>(blockIdx.y) * E + e0) * F.Y + lane] = acc;
          } else {
            T* dsty = P.gy + static_cast<int64_t>(e0) * F.Y + lane;
            *dsty = P.acc_y ? *dsty + acc : acc;
          }
        }
        __syncwarp();
      }
      e0 = e1;
      d0 = d1n;
      e1 = e2;
      d1n = d2n;
      e2 = e3;
      if (pos + 3 < p_end) d2n = P.dst[e2];
      if (pos + 4 < p_end) e3 = P.edge_ids[pos + 4];
      if (++st == S) st = 0;
    }
    if (!alive) break;
    if (want_x) {
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        constexpr int d1 = 2 * l1 + 1;
        T* dstx = P.gx + n * F.X + F.x_off[l1] + c0 * d1 + lane * (CPL * d1);
        T row[CPL * d1];  // memory order: channel-major, component-minor
        unpack_packets<PK, T, CPL, d1>(&gxr[l1 * l1 * NP], row);
        if (P.acc_x) {
          T old[CPL * d1];
          load_vectors<T, CPL, d1>(dstx, old);
#pragma unroll
          for (int a = 0; a < CPL * d1; ++a) row[a] += old[a];
        }
        store_vectors<T, CPL, d1>(dstx, row);
      });
    }
  }
  // row stores must have read their stages before the CTA's shared memory is released
  if (lane < n_wp) bulk_wait_group_read_all();
  if (!alive) {  // let copies that are still in flight land as well (bounded)
    const int64_t last = u + R < total_units ? u + R : total_units;
    for (int64_t v = u + 1; v < last; ++v) {
      if (++s == R) {
        s = 0;
        gparity ^= 1u;
      }
      mbar_wait_bounded(&gbar[s], gparity);
    }
    for (int v = 0; v < S; ++v) mbar_wait_bounded(&wbar[v], (wparity >> v) & 1u);
  }
}

// Whether the compiled-in program length fits this shape (checked at compile time per instantiation).
template <int LX, int L2, int LO>
constexpr bool sparse_shape_ok() {
  return (canon_toff(LX, L2, LO, -1, -1, -1) + 31) / 32 <= kMaxSparseRounds && (L2 + 1) * (L2 + 1) <= 2 * kSparseTileRows;
}

template <typename T, int CPL, int LX, int L2, int LO>
int launch_fast_bwd_sparse(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph, BwdParams<T> P,
                           bool has_gy, bool wxw, cudaStream_t stream) {
  const FastMeta& f = plan->fast;
  P.sp_c = static_cast<const T*>(dt.sp_c);
  P.sp_j = dt.sp_j;
  auto kernel = !has_gy ? fast_bwd_sparse_kernel<T, CPL, LX, L2, LO, true, false>
                        : (wxw ? fast_bwd_sparse_kernel<T, CPL, LX, L2, LO, true, true>
                               : fast_bwd_sparse_kernel<T, CPL, LX, L2, LO, false, true>);
  cudaFuncAttributes attr;
  LUNA_CUDA_CHECK(cudaFuncGetAttributes(&attr, kernel));
  // One CTA per SM.  As many warps as registers and shared memory allow, then as many row stages as fit (up to
  // four: short rows need the deeper prefetch), then a deeper g ring.
  Residency r;
  int row_stages = 0;
  {
    int max_warps = std::min(sparse_max_warps<T, CPL, LX, L2, LO>(), 65536 / (std::max(attr.numRegs, 1) * 32));
    max_warps = capped_warps(plan->tuning, max_warps);
    int max_stages = kMaxRowStages;
    if (plan->tuning.row_stages > 0) max_stages = std::max(2, std::min(max_stages, plan->tuning.row_stages));
    const size_t budget = static_cast<size_t>(dt.max_smem_optin);
    for (int w = max_warps; w >= 1 && r.depth == 0; --w)
      for (int st = max_stages; st >= 2 && r.depth == 0; --st)
        for (int depth = std::min(4, 2 * f.nkinds); depth >= 2; --depth) {
          const size_t bytes = sparse_shared_bytes<T>(f) + w * (depth * sparse_slot_bytes<T>(f) + sparse_fixed_bytes<T>(f, st));
          if (bytes > budget) continue;
          r.depth = depth;
          r.warps = w;
          r.ctas = 1;
          r.block_bytes = bytes;
          row_stages = st;
          break;
        }
  }
  if (r.depth == 0) return fail(LUNA_ERR_UNSUPPORTED, "staged backward needs more shared memory than the device has");
  P.slots = r.depth;
  P.row_stages = row_stages;
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(r.block_bytes)));
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  const int64_t blocks = grid_blocks(graph->num_edges, edges_per_warp(plan->tuning, 1024), r, dt.sm_count);
  const dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(f.chunks));
  kernel<<<grid, r.warps * 32, r.block_bytes, stream>>>(P);
  LUNA_LAUNCH_CHECK("staged backward (compiled-in coupling patterns)");
  return LUNA_OK;
}

}  // namespace fastk
}  // namespace luna
