// Staged source-major kernel: first derivatives gx, gy, gw in one pass over the weights.
//
// One warp owns a contiguous range of source nodes (balanced by out-edge count) and walks their out-edges through
// the source CSR.  The stream is cut into units, one per (edge, output degree l3): the w chunks of the paths into
// that degree plus the degree's block of the gathered g[dst] row.  Bulk copies bring units into the warp's ring of
// shared-memory slots; a slot is refilled as soon as its unit is consumed, so the ring holds between one and two
// edges and many warps fit on an SM.  With M^p = C^p . y[e] (see uvu_fast.cuh) each channel computes, one matrix
// row i at a time,
//     s_i   = sum_k M^p[i][k] g_k             (shared by the next two lines)
//     gx_i += w_p * s_i                        (register accumulator of the source node, no atomics)
//     gw_p  = sum_i x_i * s_i                  (streamed straight to global memory)
//     G^p[i][k] = sum over the lane's channels of x_i * (w_p g_k)
// The warp-wide sum of G runs through a shared-memory tile of entry pairs: every lane writes its pair into the
// pair's row (64/128-bit stores), one lane per row adds the 32 contributions (128-bit loads, rows padded against
// bank conflicts), batched over up to 32 rows.  Finally gy[e, j] = sum C^p_ijk G^p[i][k] from a small per-j program
// held in shared memory.  Every output element is written by exactly one thread in a fixed order: deterministic.
// FP32 arithmetic with an even number of channels per lane uses packed two-wide FMAs over channel pairs.
#pragma once

#include <algorithm>
#include <cstdlib>

#include "uvu_packets.cuh"

namespace luna {
namespace fastk {

constexpr int kMaxSlots = 8;    // ring slots per warp
constexpr int kRedGroups = 16;  // rows of the reduction tile: one entry pair each, two lanes per row at flush time

// Elements per tile row: 32 lanes x 2 entries plus 16 bytes, so that lanes reading different rows with 128-bit loads
// hit different banks.
template <typename T>
__host__ __device__ constexpr int red_stride() {
  return 64 + 16 / static_cast<int>(sizeof(T));
}

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
  const unsigned char* tables;  // blob described by FastMeta::tb_*
  const T* sp_c;                // sparse term list of a canonical plan (coefficients, y indices), else null
  const unsigned char* sp_j;
  int* status;
  int64_t num_src_nodes, num_edges;
  int slots;
  int row_stages;  // kernel with compiled-in patterns: weight-row stages per warp
  int acc_x, acc_y, acc_w;
};

// packet shape of the backward kernel: FP32 pairs whenever a lane has an even number of channels
template <typename T, int CPL>
using Pk = PkT<T, CPL, UsePairs<T, CPL>::value>;

// Adds the 32 lane contributions of tile rows [0, groups) and writes the entry pairs to gbuf[0 .. 2 * groups).
// Lanes L and L + 16 share row L: each adds one half of the contributions, a shuffle joins the halves.  Called from
// many places of the unrolled kernel, so it stays a real function: the hot loop has to fit the instruction cache.
template <typename T>
__device__ __noinline__ void flush_tile(const T* red, T* gbuf, int groups, int lane) {
  __syncwarp();
  const int r = lane & 15, half = lane >> 4;
  const T* row = red + r * red_stride<T>() + half * 32;
  T s0, s1;
  if constexpr (sizeof(T) == 4) {
    Pair a0{0ull}, a1{0ull};
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      const ulonglong2 q = reinterpret_cast<const ulonglong2*>(row)[v];
      a0 = vadd(a0, Pair{q.x});
      a1 = vadd(a1, Pair{q.y});
    }
    float both[2];
    split_packet(vadd(a0, a1), both);
    s0 = both[0];
    s1 = both[1];
  } else {
    double t0 = 0.0, t1 = 0.0;
    s0 = 0.0;
    s1 = 0.0;
#pragma unroll
    for (int v = 0; v < 16; v += 2) {
      const double2 p = reinterpret_cast<const double2*>(row)[v], q = reinterpret_cast<const double2*>(row)[v + 1];
      s0 += p.x;
      s1 += p.y;
      t0 += q.x;
      t1 += q.y;
    }
    s0 += t0;
    s1 += t1;
  }
  s0 += __shfl_xor_sync(0xffffffffu, s0, 16);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 16);
  if (lane < groups) {
    Vec<T, 2> pr{{s0, s1}};
    reinterpret_cast<Vec<T, 2>*>(gbuf)[lane] = pr;
  }
  __syncwarp();
}

template <typename T, int CPL>
__host__ __device__ inline size_t bwd_fixed_bytes(const FastMeta& f) {
  // coupling matrices (padded to whole rounds of 32 entries), G buffer, reduction tile, y row, barriers
  const size_t elems = static_cast<size_t>(f.m_total + 31) / 32 * 32 + f.m_total +
                       static_cast<size_t>(kRedGroups) * red_stride<T>() + 32;
  return elems * sizeof(T) + kMaxSlots * sizeof(uint64_t);
}
// Per-CTA shared tables: the blob plus one record per path.
__host__ __device__ inline size_t bwd_shared_bytes(const FastMeta& f) {
  return static_cast<size_t>(f.tb_bytes) + kMaxFastPaths * sizeof(int4);
}

// WXW: whether gx and/or gw are produced; WY: whether gy is.  Compiled in or out: each is about half of the kernel,
// and only the first needs the coupling matrices.
// L2 >= 0: canonical full path list for (LX, L2, LO), loops over units and paths unrolled from compile-time tables;
// L2 < 0: any path list, loops read the tables in FastMeta.
// MAXW warps per CTA at most and MINB CTAs per SM at least: together they cap the registers per thread.
template <typename T, int CPL, int LX, int LO, int L2, bool WXW, bool WY, int MAXW, int MINB>
__global__ void __launch_bounds__(MAXW * 32, MINB) fast_bwd_kernel(const __grid_constant__ BwdParams<T> P) {
  using PK = Pk<T, CPL>;
  using V = typename PK::V;
  constexpr int NP = PK::NP;
  constexpr int L1S = kMaxFastL + 1;
  constexpr bool kCanon = L2 >= 0;
  constexpr int L2c = L2 < 0 ? 0 : L2;
  constexpr int kCanonTotal = kCanon ? canon_moff(LX, L2c, LO, -1, -1, -1) : 0;
  constexpr int kRounds = (kCanonTotal + 31) / 32;
  constexpr bool kProgramInRegisters = kCanon && WXW && kRounds <= 12;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const FastMeta& F = P.meta;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int R = P.slots, nk = kCanon ? LO + 1 : F.nkinds;
  const int slot_elems = F.slot_elems;
  const int m_total = kCanon ? kCanonTotal : F.m_total;
  constexpr int chw = 32 * CPL;
  const int c0 = blockIdx.y * chw;

  // CTA-wide tables
  for (int i = threadIdx.x; i < F.tb_bytes / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem_raw)[i] = reinterpret_cast<const uint4*>(P.tables)[i];
  // per path: offset of its w chunk in the unit, offset of its matrix, global w offset for this CTA's channels
  int4* ptab = reinterpret_cast<int4*>(smem_raw + F.tb_bytes);
  for (int q = threadIdx.x; q < F.num_paths; q += blockDim.x)
    ptab[q] = make_int4(F.uw_soff[q], F.m_off[q], F.w_goff[q] + c0, 0);
  __syncthreads();
  const T* ell_c = reinterpret_cast<const T*>(smem_raw);
  const T* gy_c = reinterpret_cast<const T*>(smem_raw + F.tb_gyc);
  const int* gy_ptr = reinterpret_cast<const int*>(smem_raw + F.tb_gyptr);
  const unsigned short* gy_m = reinterpret_cast<const unsigned short*>(smem_raw + F.tb_gym);
  const unsigned char* ell_j = smem_raw + F.tb_ellj;

  const size_t warp_bytes = static_cast<size_t>(R) * slot_elems * sizeof(T) + bwd_fixed_bytes<T, CPL>(F);
  T* slots = reinterpret_cast<T*>(smem_raw + bwd_shared_bytes(F) + static_cast<size_t>(warp) * warp_bytes);
  T* mbuf = slots + static_cast<size_t>(R) * slot_elems;
  T* gbuf = mbuf + (m_total + 31) / 32 * 32;
  T* red = gbuf + m_total;
  T* ybuf = red + kRedGroups * red_stride<T>();
  uint64_t* bars = reinterpret_cast<uint64_t*>(ybuf + 32);

  if (lane == 0) {
    for (int s = 0; s < R; ++s) mbar_init(&bars[s], 1);
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
  constexpr bool want_y = WY;
  const int64_t total_units = (p_end - p_begin) * nk;

  // Lane L copies the w chunk of the unit's L-th path; the lane after the last path copies the g block.
  auto issue = [&](int kind, int64_t e, int64_t d_node, int s) {
    uint64_t* bar = &bars[s];
    const int l3 = F.kind_l3[kind];
    const int q0 = F.pair_ptr[l3 * L1S], np = F.pair_ptr[l3 * L1S + L1S] - q0;
    if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(F.unit_elems[kind] * sizeof(T)));
    __syncwarp();
    T* to = slots + static_cast<size_t>(s) * slot_elems;
    if (lane < np) {
      bulk_copy_g2s(to + lane * chw, P.w + e * F.W + ptab[q0 + lane].z, static_cast<uint32_t>(chw * sizeof(T)), bar);
    } else if (lane == np) {
      const int d3 = 2 * l3 + 1;
      bulk_copy_g2s(to + np * chw, P.g + d_node * F.O + F.o_off[l3] + c0 * d3,
                    static_cast<uint32_t>(chw * d3 * sizeof(T)), bar);
    }
  };

  // ids and destinations of the current and the next two edges; the id after those is fetched one step early
  // because the destination load depends on it
  auto id_at = [&](int64_t p) { return p < p_end ? P.edge_ids[p] : -1; };
  auto dst_of = [&](int e) { return e >= 0 ? P.dst[e] : 0; };
  int e0 = id_at(p_begin), e1 = id_at(p_begin + 1), e2 = id_at(p_begin + 2), e3 = id_at(p_begin + 3);
  int d0 = dst_of(e0), d1n = dst_of(e1), d2n = dst_of(e2);
  for (int v = 0; v < R && v < total_units; ++v) {
    const int de = v / nk, kind = v - de * nk;  // R <= 2 * nk, so de is 0 or 1
    issue(kind, de == 0 ? e0 : e1, de == 0 ? d0 : d1n, v);
  }
  T y_next = (lane < F.Y && e0 >= 0) ? P.y[static_cast<int64_t>(e0) * F.Y + lane] : T(0);

  constexpr int XR = (LX + 1) * (LX + 1) * NP;
  V xr[XR], gxr[XR];
  const V ones = runtime_one<V, T>(F.m_terms);  // see settle_packets
  int64_t pos = p_begin;
  int64_t u = 0;  // unit being consumed
  int s = 0;
  uint32_t parity = 0;
  bool alive = true;
  int tile_base = 0;  // first matrix entry held in the reduction tile
  int tile_end = 0;   // one past the last entry written to the tile

  // One path of a unit.  wq: the lane's weights in the slot; matrix: the path's coupling matrix (stored once);
  // m_off: its first entry (index into the G buffer); w_goff: global offset of the lane's weights (for gw).
  auto path_body = [&](auto l1c, auto l3c, const V* g2, const T* wq, int m_off, int64_t w_goff) {
    constexpr int l1 = decltype(l1c)::value, l3 = decltype(l3c)::value;
    constexpr int d1 = 2 * l1 + 1, d3 = 2 * l3 + 1, d3p = d3 + 1;
    V w2[NP];  // a lane's consecutive channels are already adjacent in memory
    load_lane_packets<PK, T, CPL>(wq, w2);
    const V* xl = &xr[l1 * l1 * NP];
    V* gxl = &gxr[l1 * l1 * NP];
    // rows go to the tile in chunks that fit it; a chunk that does not fit behind what the tile holds first
    // reduces that
    constexpr int rows_per_chunk = (2 * kRedGroups) / d3p < d1 ? (2 * kRedGroups) / d3p : d1;
    T* tile = nullptr;
    V dot[NP];
#pragma unroll
    for (int p = 0; p < NP; ++p) dot[p] = zero_packet<V>();
    const T* matrix = mbuf + m_off;
    static_for<0, d1>([&](auto ic) {
      constexpr int i = decltype(ic)::value;
      if (want_y && i % rows_per_chunk == 0) {
        constexpr int chunk_rows = d1 - i < rows_per_chunk ? d1 - i : rows_per_chunk;
        const int first = m_off + i * d3p;
        if (first + chunk_rows * d3p - tile_base > 2 * kRedGroups) {
          flush_tile<T>(red, gbuf + tile_base, (tile_end - tile_base) / 2, lane);
          tile_base = first;
        }
        tile = red + ((first - tile_base) / 2) * red_stride<T>() + lane * 2;
        tile_end = first + chunk_rows * d3p;
      }
      if constexpr (WXW) {
        T mrow[d3p];
        load_plain_row<T, d3p, i>(matrix, mrow);
#pragma unroll
        for (int p = 0; p < NP; ++p) {
          V sv = vmul(bcast_packet(mrow[0], V{}), g2[p]);
#pragma unroll
          for (int k = 1; k < d3; ++k) sv = vfma(bcast_packet(mrow[k], V{}), g2[k * NP + p], sv);
          gxl[i * NP + p] = vfma(w2[p], sv, gxl[i * NP + p]);
          dot[p] = vfma(xl[i * NP + p], sv, dot[p]);
        }
      }
      if (want_y) {
        V xw[NP];
#pragma unroll
        for (int p = 0; p < NP; ++p) xw[p] = vmul(xl[i * NP + p], w2[p]);
        T grow[d3p];
#pragma unroll
        for (int k = 0; k < d3; ++k) {
          V acc = vmul(xw[0], g2[k * NP]);
#pragma unroll
          for (int p = 1; p < NP; ++p) acc = vfma(xw[p], g2[k * NP + p], acc);
          grow[k] = hsum(acc);
        }
        grow[d3] = T(0);
#pragma unroll
        for (int kk = 0; kk < d3p / 2; ++kk) {
          Vec<T, 2> pr{{grow[2 * kk], grow[2 * kk + 1]}};
          *reinterpret_cast<Vec<T, 2>*>(tile + ((i % rows_per_chunk) * (d3p / 2) + kk) * red_stride<T>()) = pr;
        }
      }
    });
    if (want_w) {
      T gwv[CPL];
      unpack_packets<PK, T, CPL, 1>(dot, gwv);
      T* dstw = P.gw + w_goff;
      if (P.acc_w) {
        T old[CPL];
        load_vectors<T, CPL, 1>(dstw, old);
#pragma unroll
        for (int c = 0; c < CPL; ++c) gwv[c] += old[c];
      }
      store_vectors_streaming<T, CPL, 1>(dstw, gwv);
    }
  };

  // One unit = the paths into output degree l3 of the current edge.
  auto unit_body = [&](auto l3c, const T* unit) {
    constexpr int l3 = decltype(l3c)::value;
    constexpr int d3 = 2 * l3 + 1;
    V g2[d3 * NP];
    const int64_t w_row = static_cast<int64_t>(e0) * F.W + lane * CPL;
    if constexpr (kCanon) {
      constexpr int paths_here = canon_unit_index(LX, L2c, LO, -1, -1, l3);
      load_packets_scalar<PK, T, CPL, d3>(unit + paths_here * chw + lane * (CPL * d3), g2);
      settle_packets<d3 * NP>(g2, ones);
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        static_for<0, L2c + 1>([&](auto l2c) {
          constexpr int l2 = decltype(l2c)::value;
          if constexpr (canon_ok(LX, L2c, LO, l1, l2, l3))
            path_body(l1c, l3c, g2, unit + canon_unit_index(LX, L2c, LO, l1, l2, l3) * chw + lane * CPL,
                      canon_moff(LX, L2c, LO, l1, l2, l3),
                      w_row + canon_wrank(LX, L2c, LO, l1, l2, l3) * F.ch + c0);
        });
      });
    } else {
      load_packets_scalar<PK, T, CPL, d3>(unit + F.ug_soff[l3] + lane * (CPL * d3), g2);
      settle_packets<d3 * NP>(g2, ones);
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        const int q_end = F.pair_ptr[l3 * L1S + l1 + 1];
#pragma unroll 1
        for (int q = F.pair_ptr[l3 * L1S + l1]; q < q_end; ++q) {
          const int4 rec = ptab[q];
          path_body(l1c, l3c, g2, unit + rec.x + lane * CPL, rec.y, w_row + rec.z);
        }
      });
    }
  };

  // waits for the unit in slot s, runs it and refills the slot with the unit R places later
  auto run_unit = [&](auto l3c, int kind) -> bool {
    if (!mbar_wait_bounded(&bars[s], parity)) {
      if (lane == 0) atomicExch(P.status, 2);
      return false;
    }
    unit_body(l3c, slots + static_cast<size_t>(s) * slot_elems);
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
      issue(next, de == 0 ? e0 : (de == 1 ? e1 : e2), de == 0 ? d0 : (de == 1 ? d1n : d2n), s);
    }
    ++u;
    if (++s == R) {
      s = 0;
      parity ^= 1u;
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
        if (kCanon || F.x_off[l1] >= 0)
          load_packets_scalar<PK, T, CPL, d1>(P.x + n * F.X + F.x_off[l1] + c0 * d1 + lane * (CPL * d1),
                                              &xr[l1 * l1 * NP]);
      });
      settle_packets<XR>(xr, ones);
    }
#pragma unroll
    for (int a = 0; a < XR; ++a) gxr[a] = zero_packet<V>();

#pragma unroll 1
    for (; pos < pe && alive; ++pos) {
      // coupling matrices of this edge, computed while its first unit may still be in flight
      if (lane < F.Y) ybuf[lane] = y_next;
      __syncwarp();
      if constexpr (WXW) {
        if constexpr (kProgramInRegisters) {
#pragma unroll
          for (int r = 0; r < kRounds; ++r)
            mbuf[r * 32 + lane] = fma(prog_b[r], ybuf[prog_j[r] >> 8], prog_a[r] * ybuf[prog_j[r] & 255u]);
        } else {
          compute_m_share<T, false>(ell_c, ell_j, ybuf, mbuf, m_total, 0, 1, lane);
        }
      }
      if (pos + 1 < p_end && lane < F.Y) y_next = P.y[static_cast<int64_t>(e1) * F.Y + lane];
      __syncwarp();
      tile_base = 0;
      tile_end = 0;

      if constexpr (kCanon) {
        static_for<0, LO + 1>([&](auto l3c) {
          if (alive) alive = run_unit(l3c, decltype(l3c)::value);
        });
      } else {
        // the per-degree arithmetic is selected by a switch so that the wait and the refill exist once in the loop
#pragma unroll 1
        for (int kind = 0; kind < nk && alive; ++kind) {
          switch (F.kind_l3[kind]) {
            case 0:
              alive = run_unit(std::integral_constant<int, 0>{}, kind);
              break;
            case 1:
              if constexpr (LO >= 1) alive = run_unit(std::integral_constant<int, 1>{}, kind);
              break;
            case 2:
              if constexpr (LO >= 2) alive = run_unit(std::integral_constant<int, 2>{}, kind);
              break;
            default:
              if constexpr (LO >= 3) alive = run_unit(std::integral_constant<int, 3>{}, kind);
              break;
          }
        }
      }
      if (!alive) break;

      if (want_y) {
        if (tile_end > tile_base) flush_tile<T>(red, gbuf + tile_base, (tile_end - tile_base) / 2, lane);
        // gy[e, j] = sum_t c[t] * G[m[t]]; two lanes share a j when the row is short enough
        const int lpj = F.Y <= 16 ? 2 : 1;
        const int j = lpj == 2 ? lane >> 1 : lane, h = lpj == 2 ? lane & 1 : 0;
        T acc = T(0);
        if (j < F.Y) {
          const int t1 = gy_ptr[j + 1];
          for (int t = gy_ptr[j] + h; t < t1; t += lpj) acc = fma(gy_c[t], gbuf[gy_m[t]], acc);
        }
        if (lpj == 2) acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        if (j < F.Y && h == 0) {
          if (P.gy_partial != nullptr) {
            P.gy_partial[(static_cast<int64_t>(blockIdx.y) * E + e0) * F.Y + j] = acc;
          } else {
            T* dsty = P.gy + static_cast<int64_t>(e0) * F.Y + j;
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
    }
    if (!alive) break;
    if (want_x) {
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        constexpr int d1 = 2 * l1 + 1;
        if (F.x_off[l1] >= 0) {
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
        }
      });
    }
  }
  if (!alive) {  // let copies that are still in flight land before the CTA's shared memory is released
    const int64_t last = u + R < total_units ? u + R : total_units;
    for (int64_t v = u + 1; v < last; ++v) {
      if (++s == R) {
        s = 0;
        parity ^= 1u;
      }
      mbar_wait_bounded(&bars[s], parity);
    }
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


}  // namespace fastk
}  // namespace luna

#include "uvu_fast_bwd_sparse.cuh"
#include "uvu_fast_bwd_units.cuh"

namespace luna {
namespace fastk {

// Kernels with a compile-time layout (uvu_fast_bwd_plain.cuh), one translation unit per (T, CPL).  Returns
// LUNA_ERR_UNSUPPORTED if the plan's layout is not the compile-time one.
template <typename T, int CPL>
int launch_fast_bwd_plain_any(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph,
                              const BwdParams<T>& P, cudaStream_t stream);

template <typename T, int CPL, int LX, int LO, int L2>
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
  P.tables = dt.bwd_tables;
  P.sp_c = nullptr;
  P.sp_j = nullptr;
  P.row_stages = 0;
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
  if (gx == nullptr && gy == nullptr && gw == nullptr) return LUNA_OK;
  const bool wxw = gx != nullptr || gw != nullptr;
  // Source rows without out-edges are skipped by the kernels (a long run of them, as in a destination-range shard,
  // would otherwise all land on one warp): their rows of gx are zero-filled here.
  if (gx != nullptr && !acc_x)
    LUNA_CUDA_CHECK(cudaMemsetAsync(gx, 0, static_cast<size_t>(P.num_src_nodes) * f.X * sizeof(T), stream));
  bool launched = false;
  if constexpr (L2 >= 0) {
    // compiled-in coupling patterns, if the plan's terms have them
    if constexpr (sparse_shape_ok<LX, (L2 < 0 ? 0 : L2), LO>()) {
      const int variant = fast_bwd_variant(plan);
      // The call training makes all the time - every gradient, gy and gw not accumulated, one warp pass per block -
      // has kernels with a compile-time layout.
      const bool plain = gx != nullptr && gy != nullptr && gw != nullptr && !acc_y && !acc_w &&
                         f.chunks == 1 && variant == LUNA_BWD_ROW_STAGES && !plan->tuning.no_plain;
      if (plain) {
        const int rc = launch_fast_bwd_plain_any<T, CPL>(plan, dt, graph, P, stream);
        if (rc == LUNA_OK) launched = true;
        else if (rc != LUNA_ERR_UNSUPPORTED) return rc;
      }
      if (!launched && variant != LUNA_BWD_STAGED_TABLES) {
        const bool rows = variant != LUNA_BWD_UNIT_RING;
        const int rc = rows ? launch_fast_bwd_sparse<T, CPL, LX, (L2 < 0 ? 0 : L2), LO>(plan, dt, graph, P, gy != nullptr, wxw, stream)
                            : launch_fast_bwd_units<T, CPL, LX, (L2 < 0 ? 0 : L2), LO>(plan, dt, graph, P, gy != nullptr, wxw, stream);
        if (rc != LUNA_OK) return rc;
        launched = true;
      }
    }
  }
  if (!launched) {
    // Register budget by shape, through the launch bounds: FP32 with four channels per lane or degree-3 blocks runs
    // up to 12 warps in a CTA (168 registers), smaller FP32 shapes up to 16 (128 registers); FP64 and the unrolled
    // canonical kernels keep 8 warps (255).
    constexpr int MAXW = (sizeof(T) == 8 || L2 >= 0) ? 8 : ((CPL == 4 || LX == 3 || LO == 3) ? 12 : 16);
    constexpr int MINB = 1;
    auto kernel = gy == nullptr ? fast_bwd_kernel<T, CPL, LX, LO, L2, true, false, MAXW, MINB>
                                : (wxw ? fast_bwd_kernel<T, CPL, LX, LO, L2, true, true, MAXW, MINB>
                                       : fast_bwd_kernel<T, CPL, LX, LO, L2, false, true, MAXW, MINB>);
    cudaFuncAttributes attr;
    LUNA_CUDA_CHECK(cudaFuncGetAttributes(&attr, kernel));
    // between two units and two edges in a warp's ring
    const Residency r = choose_residency(static_cast<size_t>(f.slot_elems) * sizeof(T), bwd_fixed_bytes<T, CPL>(f),
                                         bwd_shared_bytes(f), dt.max_smem_optin, attr.numRegs, capped_warps(plan->tuning, MAXW), 2,
                                         std::min(kMaxSlots, 2 * f.nkinds));
    if (r.depth == 0) return fail(LUNA_ERR_UNSUPPORTED, "staged backward needs more shared memory than the device has");
    P.slots = r.depth;
    const size_t block_bytes = r.block_bytes;
    const int nwarps = r.warps;
    LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(block_bytes)));
    // without this the driver may size the shared-memory carve-out for fewer CTAs than planned
    LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    const int64_t blocks = grid_blocks(graph->num_edges, edges_per_warp(plan->tuning, 1024), r, dt.sm_count);
    const dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(f.chunks));
    kernel<<<grid, nwarps * 32, block_bytes, stream>>>(P);
    LUNA_LAUNCH_CHECK("staged backward");
  }
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
  const int lx = plan->fast.LX, lo = plan->fast.LO, l2 = plan->fast.canon_l2;
#define LUNA_BWD_ARGS plan, dt, graph, x, y, w, g, gx, acc_x, gy, acc_y, gw, acc_w, scratch, scratch_bytes, stream
  if (!plan->tuning.no_canon) {
    if (lx == 2 && l2 == 3 && lo == 3) return launch_fast_bwd_one<T, CPL, 2, 3, 3>(LUNA_BWD_ARGS);
    if (lx == 2 && l2 == 2 && lo == 2) return launch_fast_bwd_one<T, CPL, 2, 2, 2>(LUNA_BWD_ARGS);
    if (lx == 3 && l2 == 3 && lo == 3) return launch_fast_bwd_one<T, CPL, 3, 3, 3>(LUNA_BWD_ARGS);
    if (lx == 1 && l2 == 1 && lo == 1) return launch_fast_bwd_one<T, CPL, 1, 1, 1>(LUNA_BWD_ARGS);
  }
  if (lx <= 1 && lo <= 1) return launch_fast_bwd_one<T, CPL, 1, 1, -1>(LUNA_BWD_ARGS);
  if (lx <= 2 && lo <= 2) return launch_fast_bwd_one<T, CPL, 2, 2, -1>(LUNA_BWD_ARGS);
  if (lx <= 2 && lo <= 3) return launch_fast_bwd_one<T, CPL, 2, 3, -1>(LUNA_BWD_ARGS);
  return launch_fast_bwd_one<T, CPL, 3, 3, -1>(LUNA_BWD_ARGS);
#undef LUNA_BWD_ARGS
}

}  // namespace fastk
}  // namespace luna
