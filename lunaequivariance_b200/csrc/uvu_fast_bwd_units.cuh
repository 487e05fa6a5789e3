// The kernel of uvu_fast_bwd_sparse.cuh (compiled-in coupling patterns, edge-attribute gradient contracted per lane)
// with the data movement of fast_bwd_kernel: a ring of (edge, output degree) units, each holding the weight chunks of
// the paths into that degree and the degree's block of g[dst]; weight gradients go straight to global memory.  Per
// edge it has less fixed work than the row-stage kernel (no proxy fence, bulk store and store wait), so it is the
// better choice when an edge's weight row is short or is not contiguous for a CTA (channels split into chunks, where
// the row kernel would move one 512-byte piece per path anyway).
#pragma once

#include "uvu_fast_bwd_sparse.cuh"

namespace luna {
namespace fastk {

template <typename T>
__host__ __device__ inline size_t units_fixed_bytes(const FastMeta& f) {
  // per-edge scalars c_t y_j, reduction tile, reduced gy row, y row, barriers
  const size_t elems = static_cast<size_t>(f.sparse_terms + 31) / 32 * 32 +
                       static_cast<size_t>(kRedGroups) * red_stride<T>() + 32 + 32;
  return elems * sizeof(T) + kMaxSlots * sizeof(uint64_t);
}
// Per-CTA shared tables: the term coefficients plus one record per path.
template <typename T>
__host__ __device__ inline size_t units_shared_bytes(const FastMeta& f) {
  return static_cast<size_t>(f.sparse_terms) * sizeof(T) + kMaxFastPaths * sizeof(int4);
}

template <typename T, int CPL, int LX, int L2, int LO, bool WXW, bool WY>
__global__ void __launch_bounds__(sparse_max_warps<T, CPL, LX, L2, LO>() * 32, 1) fast_bwd_units_kernel(const __grid_constant__ BwdParams<T> P) {
  using PK = Pk<T, CPL>;
  using V = typename PK::V;
  constexpr int NP = PK::NP;
  constexpr int L1S = kMaxFastL + 1;
  constexpr int TT = canon_toff(LX, L2, LO, -1, -1, -1);  // terms, padded per path
  constexpr int kRounds = (TT + 31) / 32;
  static_assert(kRounds <= kMaxSparseRounds, "coupling program too long for the register budget");
  constexpr int YD = (L2 + 1) * (L2 + 1);
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const FastMeta& F = P.meta;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int R = P.slots;
  constexpr int nk = LO + 1;
  const int slot_elems = F.slot_elems;
  constexpr int chw = 32 * CPL;
  const int c0 = blockIdx.y * chw;

  // CTA-wide tables: term coefficients, and per path the global w offset for this CTA's channels
  T* ctab = reinterpret_cast<T*>(smem_raw);
  for (int i = threadIdx.x; i < TT; i += blockDim.x) ctab[i] = P.sp_c[i];
  int4* ptab = reinterpret_cast<int4*>(smem_raw + static_cast<size_t>(TT) * sizeof(T));
  for (int q = threadIdx.x; q < F.num_paths; q += blockDim.x)
    ptab[q] = make_int4(F.uw_soff[q], F.m_off[q], F.w_goff[q] + c0, 0);
  __syncthreads();

  const size_t warp_bytes = static_cast<size_t>(R) * slot_elems * sizeof(T) + units_fixed_bytes<T>(F);
  T* slots = reinterpret_cast<T*>(smem_raw + units_shared_bytes<T>(F) + static_cast<size_t>(warp) * warp_bytes);
  T* cybuf = slots + static_cast<size_t>(R) * slot_elems;
  T* red = cybuf + (TT + 31) / 32 * 32;
  T* gbuf = red + kRedGroups * red_stride<T>();
  T* ybuf = gbuf + 32;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ybuf + 32);

  if (lane == 0) {
    for (int s = 0; s < R; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
  }
  __syncwarp();

  // the lane's share of the per-edge program cy[t] = c_t * y[j_t]: entries lane, lane + 32, ...
  T prog_c[kRounds];
  unsigned prog_j[kRounds];
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const int t = r * 32 + lane;
    prog_c[r] = t < TT ? ctab[t] : T(0);
    prog_j[r] = t < TT ? P.sp_j[t] : 0u;
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
  const int64_t total_units = (p_end - p_begin) * nk;

  // Lane L copies the w chunk of the unit's L-th path; the lane after the last path copies the g block.
  auto issue = [&](int l3, int64_t e, int64_t d_node, int s) {
    uint64_t* bar = &bars[s];
    const int q0 = F.pair_ptr[l3 * L1S], np = F.pair_ptr[l3 * L1S + L1S] - q0;
    if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(F.unit_elems[l3] * sizeof(T)));
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
  V gy2[WY ? YD : 1];
  int64_t pos = p_begin;
  int64_t u = 0;  // unit being consumed
  int s = 0;
  uint32_t parity = 0;
  bool alive = true;

  // One path: a straight line over its coupling terms.
  auto path_body = [&](auto l1c, auto l2c, auto l3c, const V* g2, const T* wq, int64_t w_goff) {
    constexpr int l1 = decltype(l1c)::value, l2 = decltype(l2c)::value, l3 = decltype(l3c)::value;
    using PT = CgPattern<l1, l2, l3>;
    constexpr int n = PT::n;
    constexpr int toff = canon_toff(LX, L2, LO, l1, l2, l3);
    V w2[NP];  // a lane's consecutive channels are already adjacent in memory
    load_lane_packets<PK, T, CPL>(wq, w2);
    const V* xl = &xr[l1 * l1 * NP];
    V* gxl = &gxr[l1 * l1 * NP];
    V dot[NP], sv[NP], xw[NP];
    V pik = zero_packet<V>();
#pragma unroll
    for (int p = 0; p < NP; ++p) dot[p] = sv[p] = xw[p] = zero_packet<V>();
    static_for<0, (n + 3) / 4>([&](auto gc) {
      constexpr int group = decltype(gc)::value;
      T cy4[4], cc4[4];
      if constexpr (WXW) load_four<T>(cybuf + toff + 4 * group, cy4);
      if constexpr (WY) load_four<T>(ctab + toff + 4 * group, cc4);
      static_for<0, 4>([&](auto uc) {
        constexpr int t = 4 * group + decltype(uc)::value;
        if constexpr (t < n) {
          constexpr int i = PT::t[t].i, j = PT::t[t].j, k = PT::t[t].k;
          constexpr bool row_first = t == 0 || PT::t[t == 0 ? 0 : t - 1].i != i;
          constexpr bool row_last = t == n - 1 || PT::t[t == n - 1 ? t : t + 1].i != i;
          constexpr bool ik_first = row_first || PT::t[t == 0 ? 0 : t - 1].k != k;
          if constexpr (WY) {
            if constexpr (row_first) {
#pragma unroll
              for (int p = 0; p < NP; ++p) xw[p] = vmul(xl[i * NP + p], w2[p]);
            }
            if constexpr (ik_first) {
              pik = vmul(xw[0], g2[k * NP]);
#pragma unroll
              for (int p = 1; p < NP; ++p) pik = vfma(xw[p], g2[k * NP + p], pik);
            }
            gy2[l2 * l2 + j] = vfma(bcast_packet(cc4[t % 4], V{}), pik, gy2[l2 * l2 + j]);
          }
          if constexpr (WXW) {
#pragma unroll
            for (int p = 0; p < NP; ++p)
              sv[p] = row_first ? vmul(bcast_packet(cy4[t % 4], V{}), g2[k * NP + p])
                                : vfma(bcast_packet(cy4[t % 4], V{}), g2[k * NP + p], sv[p]);
            if constexpr (row_last) {
#pragma unroll
              for (int p = 0; p < NP; ++p) {
                gxl[i * NP + p] = vfma(w2[p], sv[p], gxl[i * NP + p]);
                dot[p] = vfma(xl[i * NP + p], sv[p], dot[p]);
              }
            }
          }
        }
      });
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
    constexpr int paths_here = canon_unit_index(LX, L2, LO, -1, -1, l3);
    V g2[d3 * NP];
    load_packets_scalar<PK, T, CPL, d3>(unit + paths_here * chw + lane * (CPL * d3), g2);
    settle_packets<d3 * NP>(g2, ones);
    const int64_t w_row = static_cast<int64_t>(e0) * F.W + lane * CPL + c0;
    static_for<0, LX + 1>([&](auto l1c) {
      constexpr int l1 = decltype(l1c)::value;
      static_for<0, L2 + 1>([&](auto l2c) {
        constexpr int l2 = decltype(l2c)::value;
        if constexpr (canon_ok(LX, L2, LO, l1, l2, l3))
          path_body(l1c, l2c, l3c, g2, unit + canon_unit_index(LX, L2, LO, l1, l2, l3) * chw + lane * CPL,
                    w_row + canon_wrank(LX, L2, LO, l1, l2, l3) * F.ch);
      });
    });
  };

  // waits for the unit in slot s, runs it and refills the slot with the unit R places later
  auto run_unit = [&](auto l3c) -> bool {
    constexpr int kind = decltype(l3c)::value;
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
        load_packets_scalar<PK, T, CPL, d1>(P.x + n * F.X + F.x_off[l1] + c0 * d1 + lane * (CPL * d1),
                                            &xr[l1 * l1 * NP]);
      });
      settle_packets<XR>(xr, ones);
    }
#pragma unroll
    for (int a = 0; a < XR; ++a) gxr[a] = zero_packet<V>();

#pragma unroll 1
    for (; pos < pe && alive; ++pos) {
      // per-edge scalars, computed while the edge's first unit may still be in flight
      if (lane < F.Y) ybuf[lane] = y_next;
      __syncwarp();
      if constexpr (WXW) {
#pragma unroll
        for (int r = 0; r < kRounds; ++r) cybuf[r * 32 + lane] = prog_c[r] * ybuf[prog_j[r]];
      }
      if (pos + 1 < p_end && lane < F.Y) y_next = P.y[static_cast<int64_t>(e1) * F.Y + lane];
      __syncwarp();
      if constexpr (WY) {
#pragma unroll
        for (int j = 0; j < YD; ++j) gy2[j] = zero_packet<V>();
      }

      static_for<0, LO + 1>([&](auto l3c) {
        if (alive) alive = run_unit(l3c);
      });
      if (!alive) break;

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
        flush_tile<T>(red, gbuf, (YD + 1) / 2, lane);
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

template <typename T, int CPL, int LX, int L2, int LO>
int launch_fast_bwd_units(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph, BwdParams<T> P,
                           bool has_gy, bool wxw, cudaStream_t stream) {
  const FastMeta& f = plan->fast;
  P.sp_c = static_cast<const T*>(dt.sp_c);
  P.sp_j = dt.sp_j;
  auto kernel = !has_gy ? fast_bwd_units_kernel<T, CPL, LX, L2, LO, true, false>
                        : (wxw ? fast_bwd_units_kernel<T, CPL, LX, L2, LO, true, true>
                               : fast_bwd_units_kernel<T, CPL, LX, L2, LO, false, true>);
  cudaFuncAttributes attr;
  LUNA_CUDA_CHECK(cudaFuncGetAttributes(&attr, kernel));
  const Residency r = choose_residency(static_cast<size_t>(f.slot_elems) * sizeof(T), units_fixed_bytes<T>(f),
                                       units_shared_bytes<T>(f), dt.max_smem_optin, attr.numRegs, capped_warps(plan->tuning, sparse_max_warps<T, CPL, LX, L2, LO>()), 2,
                                       std::min(kMaxSlots, 2 * f.nkinds));
  if (r.depth == 0) return fail(LUNA_ERR_UNSUPPORTED, "staged backward needs more shared memory than the device has");
  P.slots = r.depth;
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(r.block_bytes)));
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  const int64_t blocks = grid_blocks(graph->num_edges, edges_per_warp(plan->tuning, 1024), r, dt.sm_count);
  const dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(f.chunks));
  kernel<<<grid, r.warps * 32, r.block_bytes, stream>>>(P);
  LUNA_LAUNCH_CHECK("staged backward (compiled-in coupling patterns, unit ring)");
  return LUNA_OK;
}

}  // namespace fastk
}  // namespace luna
