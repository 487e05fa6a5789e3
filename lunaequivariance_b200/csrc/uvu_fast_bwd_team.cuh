// Source-major first-derivative kernel (gx, gy, gw in one pass) for canonical path lists with 128 FP32 channels, in
// which TEAMS OF TWO WARPS share one edge.
//
// Why teams.  With one warp per edge a lane carries four channels of every block: x, gx, the g block, the gy
// accumulators and the coupling program fill all 255 registers, eight warps fit on an SM, and with two warps per
// scheduler neither the FMA pipe nor DRAM gets more than half busy - the kernel waits on latency.  Here a lane
// carries two channels (one packed pair), which needs about 160 registers, so twelve warps fit; the two warps of a
// team cover channels 0..63 and 64..127 of the same edge and share what is per edge, not per channel:
//   * the edge's weight row: one bulk copy into one of the team's two row stages; both warps overwrite their channels'
//     weights with the weight gradients and the row returns to gw with one bulk store;
//   * the g[dst] row, cut into one block per output degree, in a ring of slots refilled as units are consumed;
//   * the edge-attribute gradient: each warp reduces its 64 channels to in2_dim sums (reduction tile, as in the
//     one-warp kernel), the second warp of the team adds the two sets and writes gy.  No global scratch.
// Hand-offs inside a team never make a warp wait for the other one.  Data arrival is signalled by `full` barriers
// (mbarrier with a byte count), which both warps poll.  Release goes by "the last one out does the chores": each warp
// that is done with a g slot, a row stage or its gy sums bumps a counter in shared memory, and the warp that finds
// itself last refills the slot, sends the row back to gw (and later refills the stage), or adds the two sets of gy
// sums and writes gy.  Whichever warp was last on a tile's final edge also starts the copies of the team's next tile.
// Every wait on a `full` barrier is bounded; a wait that runs out sets the plan's status word and the warp leaves its
// loop (the other warp of the team then runs out of its own waits and leaves too).
//
// Work assignment.  Source nodes are cut into small tiles of consecutive nodes; team q of Q takes tiles q, q + Q,
// q + 2Q, ...  All resident teams therefore work on neighbouring source nodes at any moment, and for a spatially
// ordered graph the g[dst] rows they gather are the same few thousand rows, which stay in L2 (with one far-apart
// node range per warp the gathered rows of the whole graph competed for L2 at once).  gx of a node is accumulated in
// registers by the warp that owns the node's channels: no atomics, results do not depend on the assignment.
#pragma once

#include "uvu_fast_bwd.cuh"

namespace luna {
namespace fastk {

constexpr int kTeamWarps = 2;      // warps that share an edge
constexpr int kTeamMaxStages = 4;  // weight-row stages per team (at most; the launcher picks 2..4)
constexpr int kTeamMaxSlots = 4;   // slots of a team's g ring (at most)
constexpr int kTeamMaxTeams = 6;   // teams per CTA: 12 warps, which caps the registers per thread at 168
constexpr int kTeamSumBuffers = kTeamMaxStages + 1;  // buffers for the warps' gy sums (see the hand-off after an edge)

// Barriers of one team (row landed, per stage; g block landed, per slot), then its counters as 32-bit words (warps
// done with a stage, with a slot, with a gy sum buffer).
constexpr int kTeamBarriers = kTeamMaxStages + kTeamMaxSlots;
constexpr int kTeamCounters = kTeamMaxStages + kTeamMaxSlots + kTeamSumBuffers + 1;

// Shared memory of one warp: per-edge scalars c_t y_j, reduction tile, reduced gy row, y row.
template <typename T>
__host__ __device__ inline size_t team_warp_elems(const FastMeta& f) {
  return static_cast<size_t>(f.sparse_terms + 31) / 32 * 32 + static_cast<size_t>(kSparseTileRows) * red_stride<T>() +
         32 + 32;
}
// Shared memory of one team.
template <typename T>
__host__ __device__ inline size_t team_bytes(const FastMeta& f, int stages, int slots) {
  const size_t gslot = static_cast<size_t>(f.ch) * (2 * f.LO + 1);
  const size_t elems = static_cast<size_t>(stages) * f.W + static_cast<size_t>(slots) * gslot +
                       kTeamWarps * team_warp_elems<T>(f) + kTeamSumBuffers * kTeamWarps * 32;
  return (elems * sizeof(T) + kTeamBarriers * sizeof(uint64_t) + kTeamCounters * sizeof(unsigned) + 127) / 128 * 128;
}

// Called by one lane of a warp that is done with a shared resource.  Returns true for the last of `parties` warps
// (a power of two; the counter only ever counts up), which owns the resource from here on.  The fences order this
// warp's accesses to the resource before the count and the owner's later copies after it.
__device__ __forceinline__ bool last_one_out(unsigned* counter, unsigned parties) {
  __threadfence_block();
  const bool last = (atomicAdd(counter, 1u) & (parties - 1u)) == parties - 1u;
  if (last) __threadfence_block();
  return last;
}

// One path of the sparse formulation for a lane's packets (see uvu_fast_bwd_sparse.cuh for the derivation).
// xl / gxl: the lane's x and gx packets of degree l1; g2: its g packets of degree l3; wq: its weights in the row
// stage, overwritten with their gradients when stage_gw, else added to gw_global.
template <typename T, int CPL, int LX, int L2, int LO, int l1, int l2, int l3, bool WXW, bool WY, typename V>
__device__ __forceinline__ void team_path(const V* xl, V* gxl, V* gy2, const V* g2, T* wq, const T* cybuf,
                                          const T* ctab, bool want_w, bool stage_gw, T* gw_global) {
  using PK = Pk<T, CPL>;
  constexpr int NP = PK::NP;
  using PT = CgPattern<l1, l2, l3>;
  constexpr int n = PT::n;
  constexpr int toff = canon_toff(LX, L2, LO, l1, l2, l3);
  V w2[NP];
  load_lane_packets<PK, T, CPL>(wq, w2);
  V dot[NP];
#ifdef LUNA_PATH_ROWS
  sparse_path_rows<T, CPL, LX, L2, LO, l1, l2, l3, WXW, WY, V>(xl, gxl, gy2, g2, w2, dot, cybuf, ctab);
#else
  V sv[NP], xw[NP];
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
#endif
  if (want_w) {
    T gwv[CPL];
    unpack_packets<PK, T, CPL, 1>(dot, gwv);
    if (stage_gw) {
      store_vectors<T, CPL, 1>(wq, gwv);
    } else {
      T old[CPL];
      load_vectors<T, CPL, 1>(gw_global, old);
#pragma unroll
      for (int c = 0; c < CPL; ++c) gwv[c] += old[c];
      store_vectors_streaming<T, CPL, 1>(gw_global, gwv);
    }
  }
}

template <typename T, int CPL, int LX, int L2, int LO, bool WXW, bool WY>
__global__ void __launch_bounds__(kTeamMaxTeams * kTeamWarps * 32, 1)
    fast_bwd_team_kernel(const __grid_constant__ BwdParams<T> P) {
  using PK = Pk<T, CPL>;
  using V = typename PK::V;
  constexpr int NP = PK::NP;
  constexpr int TW = kTeamWarps;
  constexpr int TT = canon_toff(LX, L2, LO, -1, -1, -1);  // terms, padded per path
  constexpr int kRounds = (TT + 31) / 32;
  static_assert(kRounds <= kMaxSparseRounds, "coupling program too long for the register budget");
  constexpr int YD = (L2 + 1) * (L2 + 1);
  static_assert((YD + 1) / 2 <= kSparseTileRows, "edge attributes too wide for the reduction tile");
  static_assert((kTeamWarps & (kTeamWarps - 1)) == 0, "last_one_out needs a power of two");
  constexpr int nk = LO + 1;
  constexpr int chw = 32 * CPL;      // channels of one warp
  constexpr int cht = chw * TW;      // channels of the team = channels per block
  constexpr int gslot_elems = cht * (2 * LO + 1);
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const FastMeta& F = P.meta;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int team = warp / TW, tw = warp % TW;
  const int nteams = blockDim.x / (32 * TW);
  const int R = P.slots;       // slots of the g ring
  const int S = P.row_stages;  // weight-row stages
  const int W = F.W;
  const int cw0 = tw * chw;  // first channel of this warp

  // ---- shared memory: CTA-wide coefficient table, then one region per team
  T* ctab = reinterpret_cast<T*>(smem_raw);
  unsigned char* team_base = smem_raw + sparse_shared_bytes<T>(F) + static_cast<size_t>(team) * team_bytes<T>(F, S, R);
  T* wst = reinterpret_cast<T*>(team_base);                       // [S][W]
  T* gsl = wst + static_cast<size_t>(S) * W;                      // [R][gslot_elems]
  T* warp_mem = gsl + static_cast<size_t>(R) * gslot_elems + static_cast<size_t>(tw) * team_warp_elems<T>(F);
  T* cybuf = warp_mem;
  T* red = cybuf + (TT + 31) / 32 * 32;
  T* gbuf = red + kSparseTileRows * red_stride<T>();
  T* ybuf = gbuf + 32;
  T* gysum = gsl + static_cast<size_t>(R) * gslot_elems + static_cast<size_t>(TW) * team_warp_elems<T>(F);  // [3][TW][32]
  uint64_t* wfull = reinterpret_cast<uint64_t*>(gysum + kTeamSumBuffers * TW * 32);  // [S] row landed
  uint64_t* gfull = wfull + kTeamMaxStages;                                            // [R] g block landed
  unsigned* wdone = reinterpret_cast<unsigned*>(gfull + kTeamMaxSlots);  // [S] warps done with the row
  unsigned* gdone = wdone + kTeamMaxStages;                              // [R] warps done with the g block
  unsigned* ydone = gdone + kTeamMaxSlots;                               // warps that have written their gy sums

  if (tw == 0 && lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&wfull[s], 1);
    for (int s = 0; s < R; ++s) mbar_init(&gfull[s], 1);
    for (int c = 0; c < kTeamCounters; ++c) wdone[c] = 0u;
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < TT; i += blockDim.x) ctab[i] = P.sp_c[i];
  __syncthreads();

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

  const int64_t N = P.num_src_nodes;
  const int64_t tile_nodes = P.tile_nodes;
  const int64_t num_tiles = (N + tile_nodes - 1) / tile_nodes;
  const int64_t Q = static_cast<int64_t>(gridDim.x) * nteams;
  const bool want_x = WXW && P.gx != nullptr, want_w = WXW && P.gw != nullptr;
  const bool stage_gw = want_w && !P.acc_w;  // gradients overwrite the weights in the stage and leave as a row

  // ---- copies (issued by lane 0 of whichever warp owns the resource at that moment)
  auto load_row = [&](int64_t e, int st) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&wfull[st], static_cast<uint32_t>(W * sizeof(T)));
      bulk_copy_g2s_hint(wst + static_cast<size_t>(st) * W, P.w + e * W, static_cast<uint32_t>(W * sizeof(T)), &wfull[st],
                         l2_policy_evict_first());
    }
  };
  auto store_row = [&](int64_t e, int st) {
    if (lane == 0) {
      bulk_copy_s2g_hint(P.gw + e * W, wst + static_cast<size_t>(st) * W, static_cast<uint32_t>(W * sizeof(T)),
                         l2_policy_evict_first());
      bulk_commit_group();
    }
  };
  auto load_g = [&](int l3, int64_t d_node, int s) {
    const int d3 = 2 * l3 + 1;
    if (lane == 0) {
      mbar_arrive_expect_tx(&gfull[s], static_cast<uint32_t>(cht * d3 * sizeof(T)));
      bulk_copy_g2s(gsl + static_cast<size_t>(s) * gslot_elems, P.g + d_node * F.O + F.o_off[l3],
                    static_cast<uint32_t>(cht * d3 * sizeof(T)), &gfull[s]);
    }
  };

  // ---- state that lives across tiles: positions in the rings, barrier phases
  constexpr int XR = (LX + 1) * (LX + 1) * NP;
  V xr[XR], gxr[XR];
  const V ones = runtime_one<V, T>(F.m_terms);
  V gy2[WY ? YD : 1];
  int s = 0;                  // g slot of the unit being consumed
  int st = 0;                 // row stage of the current edge
  int sumbuf = 0;             // gy sum buffer of the current edge
  uint32_t gfull_par = 0, wfull_par = 0;  // phase bit per barrier
  bool start_next_tile = tw == 0;         // this warp issues the first copies of the team's next tile
  bool alive = true;
  auto give_up = [&](int code) {
    if (lane == 0) atomicExch(P.status, code);
    alive = false;
  };

#pragma unroll 1
  for (int64_t tile = static_cast<int64_t>(blockIdx.x) * nteams + team; tile < num_tiles && alive; tile += Q) {
    const int64_t n_lo = tile * tile_nodes;
    const int64_t n_hi = n_lo + tile_nodes < N ? n_lo + tile_nodes : N;
    const int64_t p_begin = P.src_rowptr[n_lo], p_end = P.src_rowptr[n_hi];
    if (p_begin >= p_end) continue;
    const int total_units = static_cast<int>(p_end - p_begin) * nk;

    // ids and destinations of the current and the next two edges; the id after those is fetched one step early
    // because the destination load depends on it
    auto id_at = [&](int64_t p) { return p < p_end ? P.edge_ids[p] : -1; };
    auto dst_of = [&](int e) { return e >= 0 ? P.dst[e] : 0; };
    int e0 = id_at(p_begin), e1 = id_at(p_begin + 1), e2 = id_at(p_begin + 2), e3 = id_at(p_begin + 3);
    int e4 = id_at(p_begin + 4);  // the row of the edge S <= 4 edges ahead is requested when a stage comes free
    int d0 = dst_of(e0), d1n = dst_of(e1), d2n = dst_of(e2);
    auto edge_ahead = [&](int k) { return k == 1 ? e1 : (k == 2 ? e2 : (k == 3 ? e3 : e4)); };
    if (start_next_tile) {
      load_row(e0, st);
      for (int k = 1, stage = st; k < S; ++k) {
        if (++stage == S) stage = 0;
        if (edge_ahead(k) >= 0) load_row(edge_ahead(k), stage);
      }
      for (int v = 0, slot = s; v < R && v < total_units; ++v) {
        const int de = v / nk, kind = v - de * nk;  // R <= nk, so de is 0
        load_g(kind, de == 0 ? d0 : d1n, slot);
        if (++slot == R) slot = 0;
      }
    }
    T y_next = lane < F.Y ? P.y[static_cast<int64_t>(e0) * F.Y + lane] : T(0);
    int64_t pos = p_begin;
    int u = 0;                 // unit being consumed, counted inside the tile
    int refill_stage = -1;     // this warp sent a row back from that stage and will refill it
    int refill_edge = -1;      // with the row of this edge

    // The paths into output degree l3 of the current edge.
    auto unit_body = [&](auto l3c, const T* gblock, T* wrow) {
      constexpr int l3 = decltype(l3c)::value;
      constexpr int d3 = 2 * l3 + 1;
      V g2[d3 * NP];
      load_packets_scalar<PK, T, CPL, d3>(gblock + (cw0 + lane * CPL) * d3, g2);
      settle_packets<d3 * NP>(g2, ones);
      const int64_t w_row = static_cast<int64_t>(e0) * W + cw0 + lane * CPL;
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        static_for<0, L2 + 1>([&](auto l2c) {
          constexpr int l2 = decltype(l2c)::value;
          if constexpr (canon_ok(LX, L2, LO, l1, l2, l3)) {
            constexpr int rank = canon_wrank(LX, L2, LO, l1, l2, l3);
            team_path<T, CPL, LX, L2, LO, l1, l2, l3, WXW, WY, V>(
                &xr[l1 * l1 * NP], &gxr[l1 * l1 * NP], gy2, g2, wrow + rank * cht + cw0 + lane * CPL, cybuf, ctab,
                want_w, stage_gw, P.gw + w_row + rank * cht);
          }
        });
      });
    };

    // Waits for the unit's g block, runs the unit and hands the slot back; the last warp out refills it with the
    // block R units later.
    auto run_unit = [&](auto l3c, T* wrow) {
      constexpr int kind = decltype(l3c)::value;
      if (!mbar_wait_bounded(&gfull[s], (gfull_par >> s) & 1u)) return give_up(2);
      gfull_par ^= 1u << s;
      unit_body(l3c, gsl + static_cast<size_t>(s) * gslot_elems, wrow);
      __syncwarp();  // every lane is done with this slot
      if (u + R < total_units && lane == 0 && last_one_out(&gdone[s], TW)) {
        int next = kind + R, de = 0;
        if (next >= nk) {  // R <= nk: at most one edge ahead
          next -= nk;
          de = 1;
        }
        load_g(next, de == 0 ? d0 : d1n, s);
      }
      ++u;
      if (++s == R) s = 0;
    };

#pragma unroll 1
    for (int64_t n = n_lo; n < n_hi && alive; ++n) {
      const int64_t pe = P.src_rowptr[n + 1];
      if (pos >= pe) continue;  // no out-edges: the row of gx was zero-filled (or is left as it is) by the launcher
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        constexpr int d1 = 2 * l1 + 1;
        load_packets_scalar<PK, T, CPL, d1>(P.x + n * F.X + F.x_off[l1] + (cw0 + lane * CPL) * d1, &xr[l1 * l1 * NP]);
      });
      settle_packets<XR>(xr, ones);
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
        if (!mbar_wait_bounded(&wfull[st], (wfull_par >> st) & 1u)) {
          give_up(3);
          break;
        }
        wfull_par ^= 1u << st;
        T* wrow = wst + static_cast<size_t>(st) * W;

        static_for<0, LO + 1>([&](auto l3c) {
          constexpr int kind = decltype(l3c)::value;
          if (alive) run_unit(l3c, wrow);
          if constexpr (kind == 0) {
            // This warp sent the previous edge's row back: the store has read the stage by now, so the row of the
            // next edge can come into it.
            if (refill_stage >= 0 && alive) {
              if (lane == 0) {
                bulk_wait_group_read_all();
                if (refill_edge >= 0) load_row(refill_edge, refill_stage);
              }
              refill_stage = -1;
            }
          }
        });
        if (!alive) break;

        // This warp is done with the row.  Its gradient writes must be visible to the bulk store, and a store it
        // issued itself must have read its stage before another warp may refill that stage.
        if (stage_gw) fence_async_shared();
        __syncwarp();
        bool last = false;
        if (lane == 0) {
          bulk_wait_group_read_all();
          last = last_one_out(&wdone[st], TW);
          if (last && stage_gw) store_row(e0, st);
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        const bool final_edge = pos + 1 == p_end;
        if (last && !final_edge) {
          const int ahead = edge_ahead(S);  // the edge that will use this stage next (-1 past the tile's end)
          if (stage_gw) {
            refill_stage = st;  // after the next unit, when the store has read the stage
            refill_edge = ahead;
          } else if (ahead >= 0) {
            load_row(ahead, st);  // nothing to send back: the stage is free now
          }
        }
        if (final_edge) {
          // the warp that is last on the tile's final edge starts the next tile, once its store has read the stage
          start_next_tile = last;
          if (last && lane == 0) bulk_wait_group_read_all();
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
          // Hand-off: both warps put their sums into the edge's buffer; the last one adds them and writes gy.
          // One buffer more than there are row stages, in rotation: a warp cannot run further ahead of the other
          // than the stages reach (it needs a stage the other one releases), so a buffer is never rewritten
          // before it has been read.
          T* sums = gysum + static_cast<size_t>(sumbuf) * TW * 32;
          if (lane < YD) sums[tw * 32 + lane] = gbuf[lane];
          __syncwarp();
          bool add_up = false;
          if (lane == 0) add_up = last_one_out(&ydone[sumbuf], TW);
          add_up = __shfl_sync(0xffffffffu, add_up, 0);
          if (add_up && lane < F.Y) {
            T acc = T(0);
            if (lane < YD) {
#pragma unroll
              for (int t = 0; t < TW; ++t) acc += sums[t * 32 + lane];
            }
            T* dsty = P.gy + static_cast<int64_t>(e0) * F.Y + lane;
            *dsty = P.acc_y ? *dsty + acc : acc;
          }
          if (++sumbuf == kTeamSumBuffers) sumbuf = 0;
        }
        e0 = e1;
        d0 = d1n;
        e1 = e2;
        d1n = d2n;
        e2 = e3;
        e3 = e4;
        if (pos + 3 < p_end) d2n = P.dst[e2];
        e4 = pos + 5 < p_end ? P.edge_ids[pos + 5] : -1;
        if (++st == S) st = 0;
      }
      if (!alive) break;
      if (want_x) {
        static_for<0, LX + 1>([&](auto l1c) {
          constexpr int l1 = decltype(l1c)::value;
          constexpr int d1 = 2 * l1 + 1;
          T* dstx = P.gx + n * F.X + F.x_off[l1] + (cw0 + lane * CPL) * d1;
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
  }
  // row stores must have read their stages before the CTA's shared memory is released
  if (lane == 0) bulk_wait_group_read_all();
  if (!alive) {  // let copies that are still in flight land as well (bounded)
    for (int v = 0; v < R; ++v) mbar_wait_bounded(&gfull[v], (gfull_par >> v) & 1u);
    for (int v = 0; v < S; ++v) mbar_wait_bounded(&wfull[v], (wfull_par >> v) & 1u);
  }
}

template <typename T, int CPL, int LX, int L2, int LO>
int launch_fast_bwd_team(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph, BwdParams<T> P,
                         bool has_gy, bool wxw, cudaStream_t stream) {
  const FastMeta& f = plan->fast;
  P.sp_c = static_cast<const T*>(dt.sp_c);
  P.sp_j = dt.sp_j;
  auto kernel = !has_gy ? fast_bwd_team_kernel<T, CPL, LX, L2, LO, true, false>
                        : (wxw ? fast_bwd_team_kernel<T, CPL, LX, L2, LO, true, true>
                               : fast_bwd_team_kernel<T, CPL, LX, L2, LO, false, true>);
  cudaFuncAttributes attr;
  LUNA_CUDA_CHECK(cudaFuncGetAttributes(&attr, kernel));
  // One CTA per SM with as many teams as registers and shared memory allow, then the deepest g ring that fits
  // (at most one edge's worth of blocks: the refill logic looks at most two edges ahead).
  const int by_registers = 65536 / (std::max(attr.numRegs, 1) * 32) / kTeamWarps;
  int max_teams = std::min(kTeamMaxTeams, std::max(1, by_registers));
  if (plan->tuning.max_warps > 0) max_teams = std::max(1, std::min(max_teams, plan->tuning.max_warps / kTeamWarps));
  const size_t budget = static_cast<size_t>(dt.max_smem_optin);
  // Measured on cfg2: the time follows the number of resident teams (6 teams 16.7 ms, 5 teams 19.2 ms, 4 teams
  // 20.9 ms), not the number of row stages (2, 3 and 4 stages with 4 teams: all 20.9 ms), so shared memory goes to
  // teams first and two stages are the default.
  int want_stages = plan->tuning.row_stages > 0 ? std::max(2, std::min(kTeamMaxStages, plan->tuning.row_stages)) : 2;
  int teams = 0, slots = 0, stages = 0;
  size_t block_bytes = 0;
  for (int st = want_stages; st >= 2 && teams == 0; --st)
    for (int t = max_teams; t >= std::min(max_teams, 4) && teams == 0; --t)
      for (int depth = std::min(kTeamMaxSlots, f.nkinds); depth >= std::min(2, f.nkinds); --depth) {
        const size_t bytes = sparse_shared_bytes<T>(f) + t * team_bytes<T>(f, st, depth);
        if (bytes > budget) continue;
        teams = t;
        slots = depth;
        stages = st;
        block_bytes = bytes;
        break;
      }
  for (int t = std::min(max_teams, 3); t >= 1 && teams == 0; --t) {  // very wide rows: fewer teams, two stages
    const size_t bytes = sparse_shared_bytes<T>(f) + t * team_bytes<T>(f, 2, std::min(2, f.nkinds));
    if (bytes > budget) continue;
    teams = t;
    slots = std::min(2, f.nkinds);
    stages = 2;
    block_bytes = bytes;
  }
  if (teams == 0) return fail(LUNA_ERR_UNSUPPORTED, "team backward needs more shared memory than the device has");
  P.slots = slots;
  P.row_stages = stages;
  // Tiles of about 96 edges: small enough that static round-robin balances the teams, large enough that the few
  // microseconds a team spends filling its pipeline at the start of a tile do not matter.
  const int64_t rows = P.num_src_nodes;
  const double degree = static_cast<double>(graph->num_edges) / static_cast<double>(std::max<int64_t>(rows, 1));
  int64_t tile_edges = edges_per_warp(plan->tuning, 96);
  P.tile_nodes = std::max<int64_t>(1, static_cast<int64_t>(tile_edges / std::max(degree, 1e-3) + 0.5));
  P.tile_nodes = std::min<int64_t>(P.tile_nodes, 1 << 20);
  const int64_t num_tiles = ceil_div(rows, P.tile_nodes);
  const int64_t blocks = std::max<int64_t>(1, std::min<int64_t>(dt.sm_count, ceil_div(num_tiles, teams)));
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(block_bytes)));
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  kernel<<<static_cast<unsigned>(blocks), teams * kTeamWarps * 32, block_bytes, stream>>>(P);
  LUNA_LAUNCH_CHECK("staged backward (warp teams)");
  return LUNA_OK;
}

}  // namespace fastk
}  // namespace luna
