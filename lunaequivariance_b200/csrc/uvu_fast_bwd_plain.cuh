// First-derivative kernel for the case training runs all the time: a canonical path list with compiled-in coupling
// patterns, one warp pass covers the channels of a block (channels == 32 * CPL), all three gradients wanted, nothing
// accumulated.  Everything about the layout is then a compile-time constant - row lengths, block offsets, which
// paths exist - so the kernel carries no layout tables, tests no output flags and computes no addresses from them.
//
// TW == 1: one warp per edge.  TW == 2: two warps share an edge and split its PATHS, not its channels, so the
// instruction count per edge stays what it is for one warp (every lane still owns CPL channels and the per-lane part
// of the edge-attribute gradient is not duplicated) while the lower register need per warp (about 168) lets twelve
// warps reside instead of eight.  The split is made at compile time (TeamSplit):
//   * the gx / gw part of a path (which accumulates into the gx block of degree l1) goes with its l1: each warp owns
//     the gx blocks of some degrees outright, so gx needs no combining;
//   * the gy part of a path (which only adds to the warp's gy partial sums) goes to whichever warp is lighter.
// A path whose two parts sit in different warps has its weights read by one warp and overwritten with their gradients
// by the other; the reader gets them from a second copy that the row copy drops into a small side buffer.
//
// Data movement.  An edge's weight row comes in with one bulk copy into one of the team's row stages (a team is the
// one or two warps that share an edge); the weight gradients overwrite the weights there and the row returns to gw with
// one bulk store.  The gathered g[dst] row is cut into one block per output degree; the blocks go through a small ring
// of slots.  `full` barriers (mbarrier with a byte count) signal arrivals; both warps of a team poll them, every wait
// is bounded, and a wait that runs out sets the plan's status word and ends the warp's loop.
//
// Hand-offs inside a team never make a warp wait for the other one: "the last one out does the chores".  A warp that
// is done with a g slot, a row stage or its gy sums bumps a counter in shared memory, and the warp that finds itself
// last refills the slot, sends the row back (and later refills the stage), or adds the two sets of gy sums and writes
// gy.  Whichever warp was last on a tile's final edge also starts the copies of the team's next tile.
//
// Work assignment.  Source nodes are cut into small tiles of consecutive nodes; team q of Q takes tiles q, q + Q, ...
// All resident teams therefore work on neighbouring source nodes at any moment, and for a spatially ordered graph the
// g[dst] rows they gather are the same few thousand rows, which stay in L2.  gx of a node is accumulated in registers
// by the warp that owns the degree: no atomics, results do not depend on the assignment.
#pragma once

#include "uvu_fast_bwd.cuh"

namespace luna {
namespace fastk {

constexpr int kTeamMaxStages = 4;  // weight-row stages per team (at most; the launcher picks 2..4)
constexpr int kTeamMaxSlots = 4;   // slots of a team's g ring (at most)
constexpr int kTeamSumBuffers = kTeamMaxStages + 1;  // buffers for the warps' gy sums (see the hand-off after an edge)

// Barriers of one team (row landed, per stage; g block landed, per slot), then its counters as 32-bit words (warps
// done with a stage, with a slot, with a gy sum buffer).
constexpr int kTeamBarriers = kTeamMaxStages + kTeamMaxSlots;
constexpr int kTeamCounters = kTeamMaxStages + kTeamMaxSlots + kTeamSumBuffers + 1;

// Called by one lane of a warp that is done with a shared resource.  Returns true for the last of `parties` warps
// (a power of two; the counter only ever counts up), which owns the resource from here on.  The fences order this
// warp's accesses to the resource before the count and the owner's later copies after it.
__device__ __forceinline__ bool last_one_out(unsigned* counter, unsigned parties) {
  __threadfence_block();
  const bool last = (atomicAdd(counter, 1u) & (parties - 1u)) == parties - 1u;
  if (last) __threadfence_block();
  return last;
}

template <typename T>
struct PlainParams {
  const T* x;
  const T* y;
  const T* w;
  const T* g;
  T* gx;
  T* gy;
  T* gw;
  const int* dst;
  const int* src_rowptr;
  const int* edge_ids;
  const T* sp_c;               // term coefficients of the plan (canon_toff order)
  const unsigned char* sp_j;   // y index of each term
  int* status;
  int64_t num_src_nodes;
  int64_t tile_nodes;
  int slots, row_stages;
  int two;                     // always 2: source of the run-time 1.0 that settles freshly assembled pairs
};

// ---- compile-time layout of a canonical list with ch channels per block ---------------------------------------------
template <int LX, int L2, int LO>
struct CanonList {
  static constexpr int paths = canon_wrank(LX, L2, LO, -1, -1, -1);
  static constexpr int terms = canon_toff(LX, L2, LO, -1, -1, -1);  // padded per path
  static constexpr int ydim = (L2 + 1) * (L2 + 1);
};

// ---- split of a canonical list between two warps --------------------------------------------------------------------
// Cost model in packed instructions per lane with two packets per lane: a path with T terms, R = 2 l1 + 1 rows and
// K distinct (i, k) pairs costs 2 T + 4 R for gx / gw and 2 R + 2 K + T for gy.
constexpr int split_wxw_cost(int l1, int l2, int l3) { return 2 * cg_count(l1, l2, l3) + 4 * (2 * l1 + 1); }
constexpr int split_wy_cost(int l1, int l2, int l3) {
  return 2 * (2 * l1 + 1) + 2 * cg_pair_count(l1, l2, l3) + cg_count(l1, l2, l3);
}
template <int LX, int L2, int LO>
constexpr int split_wxw_of_degree(int l1) {
  int c = 0;
  for (int l2 = 0; l2 <= L2; ++l2)
    for (int l3 = 0; l3 <= LO; ++l3)
      if (canon_ok(LX, L2, LO, l1, l2, l3)) c += split_wxw_cost(l1, l2, l3);
  return c;
}
template <int LX, int L2, int LO>
constexpr int split_total() {
  int c = 0;
  for (int l1 = 0; l1 <= LX; ++l1)
    for (int l2 = 0; l2 <= L2; ++l2)
      for (int l3 = 0; l3 <= LO; ++l3)
        if (canon_ok(LX, L2, LO, l1, l2, l3)) c += split_wxw_cost(l1, l2, l3) + split_wy_cost(l1, l2, l3);
  return c;
}
template <int LX, int L2, int LO>
constexpr int split_all_of_degree(int l1) {  // both parts of every path with this l1
  int c = 0;
  for (int l2 = 0; l2 <= L2; ++l2)
    for (int l3 = 0; l3 <= LO; ++l3)
      if (canon_ok(LX, L2, LO, l1, l2, l3)) c += split_wxw_cost(l1, l2, l3) + split_wy_cost(l1, l2, l3);
  return c;
}
// Degrees l1 that warp 0 owns (bit l1): the proper subset that divides the whole paths most evenly.
template <int LX, int L2, int LO>
constexpr unsigned split_degree_mask() {
  unsigned best = 1u;
  int best_gap = 1 << 30;
  for (unsigned mask = 1u; mask + 1u < (1u << (LX + 1)); ++mask) {
    int c = 0;
    for (int l1 = 0; l1 <= LX; ++l1)
      if (mask >> l1 & 1u) c += split_all_of_degree<LX, L2, LO>(l1);
    const int gap = 2 * c > split_total<LX, L2, LO>() ? 2 * c - split_total<LX, L2, LO>() : split_total<LX, L2, LO>() - 2 * c;
    if (gap < best_gap) {
      best_gap = gap;
      best = mask;
    }
  }
  return best;
}
// Owner of every path's gy part (bit = canonical weight rank, set: warp 0).  Every part starts in the warp that owns
// the path's degree; then, while it narrows the gap, the gy part whose cost is closest to half the gap moves from the
// heavier warp to the lighter one.  Few parts move (two for the degree-(2,3,3) list), and only they need a second
// copy of their weights.
template <int LX, int L2, int LO>
constexpr unsigned long long split_gy_mask() {
  constexpr unsigned degrees = split_degree_mask<LX, L2, LO>();
  int load[2] = {0, 0};
  unsigned long long mask = 0ull;
  {
    int rank = 0;
    for (int l1 = 0; l1 <= LX; ++l1) {
      const int owner = (degrees >> l1 & 1u) ? 0 : 1;
      load[owner] += split_all_of_degree<LX, L2, LO>(l1);
      for (int l2 = 0; l2 <= L2; ++l2)
        for (int l3 = 0; l3 <= LO; ++l3)
          if (canon_ok(LX, L2, LO, l1, l2, l3)) {
            if (owner == 0) mask |= 1ull << rank;
            ++rank;  // canonical weight rank: position in (l1, l2, l3) order
          }
    }
  }
  for (int round = 0; round < CanonList<LX, L2, LO>::paths; ++round) {
    const int heavy = load[0] >= load[1] ? 0 : 1;
    const int gap = load[heavy] - load[1 - heavy];
    int pick = -1, pick_cost = 0, pick_left = gap, rank = 0;
    for (int l1 = 0; l1 <= LX; ++l1)
      for (int l2 = 0; l2 <= L2; ++l2)
        for (int l3 = 0; l3 <= LO; ++l3) {
          if (!canon_ok(LX, L2, LO, l1, l2, l3)) continue;
          const int owner = (mask >> rank & 1ull) ? 0 : 1;
          const int home = (degrees >> l1 & 1u) ? 0 : 1;
          const int cost = split_wy_cost(l1, l2, l3);
          const int left = gap > 2 * cost ? gap - 2 * cost : 2 * cost - gap;  // gap after the move
          if (owner == heavy && home == heavy && left < pick_left) {
            pick = rank;
            pick_cost = cost;
            pick_left = left;
          }
          ++rank;
        }
    if (pick < 0) break;
    load[heavy] -= pick_cost;
    load[1 - heavy] += pick_cost;
    mask ^= 1ull << pick;
  }
  return mask;
}

template <int LX, int L2, int LO>
struct TeamSplit {
  static constexpr unsigned degrees = split_degree_mask<LX, L2, LO>();
  static constexpr unsigned long long gy_parts = split_gy_mask<LX, L2, LO>();
  static constexpr int wxw_owner(int l1) { return (degrees >> l1 & 1u) ? 0 : 1; }
  static constexpr int wy_owner(int rank) { return (gy_parts >> rank & 1ull) ? 0 : 1; }
  // paths whose weights one warp reads while the other overwrites them: they get a second copy in the side buffer
  static constexpr bool is_split(int l1, int l2, int l3) {
    return wxw_owner(l1) != wy_owner(canon_wrank(LX, L2, LO, l1, l2, l3));
  }
  static constexpr int side_index(int a, int b, int c) {  // position among the split paths; total for (-1, -1, -1)
    int n = 0;
    for (int l1 = 0; l1 <= LX; ++l1)
      for (int l2 = 0; l2 <= L2; ++l2)
        for (int l3 = 0; l3 <= LO; ++l3) {
          if (l1 == a && l2 == b && l3 == c) return n;
          if (canon_ok(LX, L2, LO, l1, l2, l3) && is_split(l1, l2, l3)) ++n;
        }
    return n;
  }
};

// What a warp does: with one warp per edge everything, else its share of the split.
template <int TW, int ROLE, int LX, int L2, int LO>
struct Role {
  using Split = TeamSplit<LX, L2, LO>;
  static constexpr bool wxw(int l1) { return TW == 1 || Split::wxw_owner(l1) == ROLE; }
  static constexpr bool wy(int l1, int l2, int l3) {
    return TW == 1 || Split::wy_owner(canon_wrank(LX, L2, LO, l1, l2, l3)) == ROLE;
  }
  static constexpr bool reads_x(int l1) {  // x of degree l1 is needed for gw and for the gy part
    if (wxw(l1)) return true;
    for (int l2 = 0; l2 <= L2; ++l2)
      for (int l3 = 0; l3 <= LO; ++l3)
        if (canon_ok(LX, L2, LO, l1, l2, l3) && wy(l1, l2, l3)) return true;
    return false;
  }
  static constexpr bool side(int l1, int l2, int l3) { return TW > 1 && wy(l1, l2, l3) && !wxw(l1); }
  static constexpr int side_paths = TW > 1 ? Split::side_index(-1, -1, -1) : 0;
};

// ---- shared memory --------------------------------------------------------------------------------------------------
template <typename T, int CPL, int TW, int LX, int L2, int LO>
struct PlainLayout {
  static constexpr int ch = 32 * CPL;
  static constexpr int W = CanonList<LX, L2, LO>::paths * ch;
  static constexpr int X = ch * (LX + 1) * (LX + 1);
  static constexpr int O = ch * (LO + 1) * (LO + 1);
  static constexpr int Y = CanonList<LX, L2, LO>::ydim;
  static constexpr int TT = CanonList<LX, L2, LO>::terms;
  static constexpr int gslot = ch * (2 * LO + 1);
  static constexpr int side = (TW > 1 ? TeamSplit<LX, L2, LO>::side_index(-1, -1, -1) : 0) * ch;  // per stage
  static constexpr int warp_elems = (TT + 31) / 32 * 32 + kSparseTileRows * red_stride<T>() + 32 + 32;
  static constexpr size_t table_bytes = (static_cast<size_t>(TT) * sizeof(T) + 127) / 128 * 128;
  static constexpr size_t team_bytes(int stages, int slots) {
    const size_t elems = static_cast<size_t>(stages) * (W + side) + static_cast<size_t>(slots) * gslot +
                         static_cast<size_t>(TW) * warp_elems + kTeamSumBuffers * TW * 32;
    return (elems * sizeof(T) + kTeamBarriers * sizeof(uint64_t) + kTeamCounters * sizeof(unsigned) + 127) / 128 * 128;
  }
};

template <int TW>
__host__ __device__ constexpr int plain_max_warps() {
  return TW == 1 ? 8 : 12;
}

// Pointers into one team's shared memory and the team's coordinates; built once per warp.
template <typename T>
struct TeamMem {
  T* wst;        // [S][W + side]
  T* gsl;        // [R][gslot]
  T* cybuf;      // this warp's per-edge scalars
  T* red;        // this warp's reduction tile
  T* gbuf;       // this warp's reduced gy row
  T* ybuf;       // this warp's y row
  T* gysum;      // [buffers][TW][32]
  uint64_t* wfull;
  uint64_t* gfull;
  unsigned* wdone;
  unsigned* gdone;
  unsigned* ydone;
  const T* ctab;
};

// The edge loop of one warp in its role.
template <typename T, int CPL, int TW, int ROLE, int LX, int L2, int LO>
__device__ __forceinline__ void plain_loop(const PlainParams<T>& P, const TeamMem<T>& M, int lane, int64_t first_tile,
                                           int64_t tile_step) {
  using L = PlainLayout<T, CPL, TW, LX, L2, LO>;
  using RL = Role<TW, ROLE, LX, L2, LO>;
  using PK = Pk<T, CPL>;
  using V = typename PK::V;
  constexpr int NP = PK::NP;
  constexpr int ch = L::ch, W = L::W, X = L::X, O = L::O, Y = L::Y, TT = L::TT;
  constexpr int kRounds = (TT + 31) / 32;
  constexpr int nk = LO + 1;
  constexpr int row_elems = W + L::side;
  const int R = P.slots, S = P.row_stages;

  // the lane's share of the per-edge program cy[t] = c_t * y[j_t]: entries lane, lane + 32, ...
  T prog_c[kRounds];
  unsigned prog_j[(kRounds + 3) / 4];
#pragma unroll
  for (int r = 0; r < (kRounds + 3) / 4; ++r) prog_j[r] = 0u;
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const int t = r * 32 + lane;
    prog_c[r] = t < TT ? M.ctab[t] : T(0);
    prog_j[r / 4] |= (t < TT ? static_cast<unsigned>(P.sp_j[t]) : 0u) << (8 * (r % 4));
  }

  auto load_row = [&](int64_t e, int st) {  // lane 0 only
    mbar_arrive_expect_tx(&M.wfull[st], static_cast<uint32_t>(row_elems * sizeof(T)));
    T* to = M.wst + static_cast<size_t>(st) * row_elems;
    const T* from = P.w + e * W;
    bulk_copy_g2s_hint(to, from, static_cast<uint32_t>(W * sizeof(T)), &M.wfull[st], l2_policy_evict_first());
    if constexpr (TW > 1) {
      // second copies of the weights of the split paths
      static_for<0, LX + 1>([&](auto l1c) {
        static_for<0, L2 + 1>([&](auto l2c) {
          static_for<0, LO + 1>([&](auto l3c) {
            constexpr int l1 = decltype(l1c)::value, l2 = decltype(l2c)::value, l3 = decltype(l3c)::value;
            if constexpr (canon_ok(LX, L2, LO, l1, l2, l3)) {
              if constexpr (TeamSplit<LX, L2, LO>::is_split(l1, l2, l3)) {
                constexpr int k = TeamSplit<LX, L2, LO>::side_index(l1, l2, l3);
                constexpr int rank = canon_wrank(LX, L2, LO, l1, l2, l3);
                bulk_copy_g2s(to + W + k * ch, from + rank * ch, static_cast<uint32_t>(ch * sizeof(T)), &M.wfull[st]);
              }
            }
          });
        });
      });
    }
  };
  auto store_row = [&](int64_t e, int st) {  // lane 0 only
    bulk_copy_s2g_hint(P.gw + e * W, M.wst + static_cast<size_t>(st) * row_elems, static_cast<uint32_t>(W * sizeof(T)),
                       l2_policy_evict_first());
    bulk_commit_group();
  };
  auto load_g = [&](int l3, int64_t d_node, int s) {  // lane 0 only
    const int d3 = 2 * l3 + 1;
    mbar_arrive_expect_tx(&M.gfull[s], static_cast<uint32_t>(ch * d3 * sizeof(T)));
    bulk_copy_g2s(M.gsl + static_cast<size_t>(s) * L::gslot, P.g + d_node * O + ch * l3 * l3,
                  static_cast<uint32_t>(ch * d3 * sizeof(T)), &M.gfull[s]);
  };
  auto last_out = [&](unsigned* counter) -> bool {  // lane 0 only
    if constexpr (TW == 1) {
      return true;
    } else {
      return last_one_out(counter, TW);
    }
  };

  constexpr int XR = (LX + 1) * (LX + 1) * NP;
  V xr[XR], gxr[XR];
  const V ones = runtime_one<V, T>(P.two);
  V gy2[Y];
  int s = 0, st = 0, sumbuf = 0;
  uint32_t gfull_par = 0, wfull_par = 0;
  bool start_next_tile = ROLE == 0;
  bool alive = true;
  auto give_up = [&](int code) {
    if (lane == 0) atomicExch(P.status, code);
    alive = false;
  };
  const int64_t N = P.num_src_nodes;
  const int64_t tile_nodes = P.tile_nodes;
  const int64_t num_tiles = (N + tile_nodes - 1) / tile_nodes;

#pragma unroll 1
  for (int64_t tile = first_tile; tile < num_tiles && alive; tile += tile_step) {
    const int64_t n_lo = tile * tile_nodes;
    const int64_t n_hi = n_lo + tile_nodes < N ? n_lo + tile_nodes : N;
    const int64_t p_begin = P.src_rowptr[n_lo], p_end = P.src_rowptr[n_hi];
    if (p_begin >= p_end) continue;
    const int total_units = static_cast<int>(p_end - p_begin) * nk;

    auto id_at = [&](int64_t p) { return p < p_end ? P.edge_ids[p] : -1; };
    auto dst_of = [&](int e) { return e >= 0 ? P.dst[e] : 0; };
    int e0 = id_at(p_begin), e1 = id_at(p_begin + 1), e2 = id_at(p_begin + 2), e3 = id_at(p_begin + 3);
    int e4 = id_at(p_begin + 4);
    int d0 = dst_of(e0), d1n = dst_of(e1), d2n = dst_of(e2);
    auto edge_ahead = [&](int k) { return k == 1 ? e1 : (k == 2 ? e2 : (k == 3 ? e3 : e4)); };
    if (start_next_tile && lane == 0) {
      load_row(e0, st);
      for (int k = 1, stage = st; k < S; ++k) {
        if (++stage == S) stage = 0;
        if (edge_ahead(k) >= 0) load_row(edge_ahead(k), stage);
      }
      for (int v = 0, slot = s; v < R && v < total_units; ++v) {
        load_g(v, d0, slot);  // R <= nk: all of the first edge
        if (++slot == R) slot = 0;
      }
    }
    T y_next = lane < Y ? P.y[static_cast<int64_t>(e0) * Y + lane] : T(0);
    int64_t pos = p_begin;
    int u = 0;
    int refill_stage = -1, refill_edge = -1;

    auto unit_body = [&](auto l3c, const T* gblock, T* wrow) {
      constexpr int l3 = decltype(l3c)::value;
      constexpr int d3 = 2 * l3 + 1;
      V g2[d3 * NP];
      load_packets_scalar<PK, T, CPL, d3>(gblock + lane * (CPL * d3), g2);
      settle_packets<d3 * NP>(g2, ones);
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        static_for<0, L2 + 1>([&](auto l2c) {
          constexpr int l2 = decltype(l2c)::value;
          if constexpr (canon_ok(LX, L2, LO, l1, l2, l3)) {
            constexpr bool do_wxw = RL::wxw(l1), do_wy = RL::wy(l1, l2, l3);
            if constexpr (do_wxw || do_wy) {
              constexpr int rank = canon_wrank(LX, L2, LO, l1, l2, l3);
              T* wq = wrow + rank * ch + lane * CPL;
              if constexpr (RL::side(l1, l2, l3))
                wq = wrow + W + TeamSplit<LX, L2, LO>::side_index(l1, l2, l3) * ch + lane * CPL;
              V w2[NP], dot[NP];
              load_lane_packets<PK, T, CPL>(wq, w2);
              sparse_path_rows<T, CPL, LX, L2, LO, l1, l2, l3, do_wxw, do_wy, V>(
                  &xr[l1 * l1 * NP], &gxr[l1 * l1 * NP], gy2, g2, w2, dot, M.cybuf, M.ctab);
              if constexpr (do_wxw) {  // the gradients take the weights' place and leave with the row
                T gwv[CPL];
                unpack_packets<PK, T, CPL, 1>(dot, gwv);
                store_vectors<T, CPL, 1>(wq, gwv);
              }
            }
          }
        });
      });
    };

    auto run_unit = [&](auto l3c, T* wrow) {
      constexpr int kind = decltype(l3c)::value;
      if (!mbar_wait_bounded(&M.gfull[s], (gfull_par >> s) & 1u)) return give_up(2);
      gfull_par ^= 1u << s;
      unit_body(l3c, M.gsl + static_cast<size_t>(s) * L::gslot, wrow);
      __syncwarp();
      if (u + R < total_units && lane == 0 && last_out(&M.gdone[s])) {
        int next = kind + R;
        const bool same_edge = next < nk;
        if (!same_edge) next -= nk;
        load_g(next, same_edge ? d0 : d1n, s);
      }
      ++u;
      if (++s == R) s = 0;
    };

#pragma unroll 1
    for (int64_t n = n_lo; n < n_hi && alive; ++n) {
      const int64_t pe = P.src_rowptr[n + 1];
      if (pos >= pe) continue;
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        constexpr int d1 = 2 * l1 + 1;
        if constexpr (RL::reads_x(l1))
          load_packets_scalar<PK, T, CPL, d1>(P.x + n * X + ch * l1 * l1 + lane * (CPL * d1), &xr[l1 * l1 * NP]);
      });
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        if constexpr (RL::reads_x(l1)) settle_packets<(2 * l1 + 1) * NP>(&xr[l1 * l1 * NP], ones);
      });
#pragma unroll
      for (int a = 0; a < XR; ++a) gxr[a] = zero_packet<V>();

#pragma unroll 1
      for (; pos < pe && alive; ++pos) {
        if (lane < Y) M.ybuf[lane] = y_next;
        __syncwarp();
#pragma unroll
        for (int r = 0; r < kRounds; ++r)
          M.cybuf[r * 32 + lane] = prog_c[r] * M.ybuf[(prog_j[r / 4] >> (8 * (r % 4))) & 255u];
        if (pos + 1 < p_end && lane < Y) y_next = P.y[static_cast<int64_t>(e1) * Y + lane];
        __syncwarp();
#pragma unroll
        for (int j = 0; j < Y; ++j) gy2[j] = zero_packet<V>();

        if (!mbar_wait_bounded(&M.wfull[st], (wfull_par >> st) & 1u)) {
          give_up(3);
          break;
        }
        wfull_par ^= 1u << st;
        T* wrow = M.wst + static_cast<size_t>(st) * row_elems;

        static_for<0, LO + 1>([&](auto l3c) {
          constexpr int kind = decltype(l3c)::value;
          if (alive) run_unit(l3c, wrow);
          if constexpr (kind == 0) {
            if (refill_stage >= 0 && alive) {  // the row this warp sent back has been read out of its stage by now
              if (lane == 0) {
                bulk_wait_group_read_all();
                if (refill_edge >= 0) load_row(refill_edge, refill_stage);
              }
              refill_stage = -1;
            }
          }
        });
        if (!alive) break;

        fence_async_shared();  // gradient writes, before the bulk store reads the stage
        __syncwarp();
        bool last = false;
        if (lane == 0) {
          bulk_wait_group_read_all();
          last = last_out(&M.wdone[st]);
          if (last) store_row(e0, st);
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        const bool final_edge = pos + 1 == p_end;
        if (last && !final_edge) {
          refill_stage = st;
          refill_edge = edge_ahead(S);
        }
        if (final_edge) {
          start_next_tile = last;
          if (last && lane == 0) bulk_wait_group_read_all();
        }

        // the lane's partial gy row through the reduction tile: entry pair r in row r
        static_for<0, (Y + 1) / 2>([&](auto rc) {
          constexpr int r = decltype(rc)::value;
          Vec<T, 2> pr;
          pr.a[0] = hsum(gy2[2 * r]);
          if constexpr (2 * r + 1 < Y) {
            pr.a[1] = hsum(gy2[2 * r + 1]);
          } else {
            pr.a[1] = T(0);
          }
          *reinterpret_cast<Vec<T, 2>*>(M.red + r * red_stride<T>() + lane * 2) = pr;
        });
        reduce_tile_rows<T, (Y + 1) / 2>(M.red, M.gbuf, lane);
        if constexpr (TW == 1) {
          if (lane < Y) P.gy[static_cast<int64_t>(e0) * Y + lane] = M.gbuf[lane];
          __syncwarp();
        } else {
          T* sums = M.gysum + static_cast<size_t>(sumbuf) * TW * 32;
          if (lane < Y) sums[ROLE * 32 + lane] = M.gbuf[lane];
          __syncwarp();
          bool add_up = false;
          if (lane == 0) add_up = last_one_out(&M.ydone[sumbuf], TW);
          add_up = __shfl_sync(0xffffffffu, add_up, 0);
          if (add_up && lane < Y) {
            T acc = T(0);
#pragma unroll
            for (int t = 0; t < TW; ++t) acc += sums[t * 32 + lane];
            P.gy[static_cast<int64_t>(e0) * Y + lane] = acc;
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
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        constexpr int d1 = 2 * l1 + 1;
        if constexpr (RL::wxw(l1)) {
          T row[CPL * d1];  // memory order: channel-major, component-minor
          unpack_packets<PK, T, CPL, d1>(&gxr[l1 * l1 * NP], row);
          store_vectors<T, CPL, d1>(P.gx + n * X + ch * l1 * l1 + lane * (CPL * d1), row);
        }
      });
    }
  }
  if (lane == 0) bulk_wait_group_read_all();
  if (!alive) {  // let copies that are still in flight land as well (bounded)
    for (int v = 0; v < R; ++v) mbar_wait_bounded(&M.gfull[v], (gfull_par >> v) & 1u);
    for (int v = 0; v < S; ++v) mbar_wait_bounded(&M.wfull[v], (wfull_par >> v) & 1u);
  }
}

template <typename T, int CPL, int TW, int LX, int L2, int LO>
__global__ void __launch_bounds__(plain_max_warps<TW>() * 32, 1) fast_bwd_plain_kernel(const __grid_constant__ PlainParams<T> P) {
  using L = PlainLayout<T, CPL, TW, LX, L2, LO>;
  static_assert(LO >= 1, "the g ring needs at least two units per edge");
  static_assert((L::TT + 31) / 32 <= kMaxSparseRounds, "coupling program too long for the register budget");
  static_assert((L::Y + 1) / 2 <= kSparseTileRows, "edge attributes too wide for the reduction tile");
  static_assert(TW == 1 || TW == 2, "one warp per edge, or two that split its paths");
  static_assert(CanonList<LX, L2, LO>::paths <= 64, "the split keeps one bit per path");
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int team = warp / TW, tw = warp % TW;
  const int nteams = blockDim.x / (32 * TW);
  const int R = P.slots, S = P.row_stages;

  T* ctab = reinterpret_cast<T*>(smem_raw);
  unsigned char* base = smem_raw + L::table_bytes + static_cast<size_t>(team) * L::team_bytes(S, R);
  TeamMem<T> M;
  M.ctab = ctab;
  M.wst = reinterpret_cast<T*>(base);
  M.gsl = M.wst + static_cast<size_t>(S) * (L::W + L::side);
  T* warp_mem = M.gsl + static_cast<size_t>(R) * L::gslot + static_cast<size_t>(tw) * L::warp_elems;
  M.cybuf = warp_mem;
  M.red = M.cybuf + (L::TT + 31) / 32 * 32;
  M.gbuf = M.red + kSparseTileRows * red_stride<T>();
  M.ybuf = M.gbuf + 32;
  M.gysum = M.gsl + static_cast<size_t>(R) * L::gslot + static_cast<size_t>(TW) * L::warp_elems;
  M.wfull = reinterpret_cast<uint64_t*>(M.gysum + kTeamSumBuffers * TW * 32);
  M.gfull = M.wfull + kTeamMaxStages;
  M.wdone = reinterpret_cast<unsigned*>(M.gfull + kTeamMaxSlots);
  M.gdone = M.wdone + kTeamMaxStages;
  M.ydone = M.gdone + kTeamMaxSlots;

  if (tw == 0 && lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&M.wfull[s], 1);
    for (int s = 0; s < R; ++s) mbar_init(&M.gfull[s], 1);
    for (int c = 0; c < kTeamCounters; ++c) M.wdone[c] = 0u;
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < L::TT; i += blockDim.x) ctab[i] = P.sp_c[i];
  __syncthreads();

  const int64_t first_tile = static_cast<int64_t>(blockIdx.x) * nteams + team;
  const int64_t tile_step = static_cast<int64_t>(gridDim.x) * nteams;
  if constexpr (TW == 1) {
    plain_loop<T, CPL, 1, 0, LX, L2, LO>(P, M, lane, first_tile, tile_step);
  } else {
    if (tw == 0) {
      plain_loop<T, CPL, 2, 0, LX, L2, LO>(P, M, lane, first_tile, tile_step);
    } else {
      plain_loop<T, CPL, 2, 1, LX, L2, LO>(P, M, lane, first_tile, tile_step);
    }
  }
}

// Whether the plan has exactly the layout the kernel assumes (blocks in degree order, weights in path order).
template <typename T, int CPL, int LX, int L2, int LO>
bool plain_layout_matches(const luna_uvu_plan* plan) {
  using L = PlainLayout<T, CPL, 1, LX, L2, LO>;
  const FastMeta& f = plan->fast;
  if (f.chunks != 1 || f.ch != L::ch || f.W != L::W || f.X != L::X || f.O != L::O || f.Y != L::Y) return false;
  if (f.sparse_terms != L::TT) return false;
  for (int l = 0; l <= LX; ++l)
    if (f.x_off[l] != L::ch * l * l) return false;
  for (int l = 0; l <= LO; ++l)
    if (f.o_off[l] != L::ch * l * l) return false;
  return true;
}

template <typename T, int CPL, int TW, int LX, int L2, int LO>
int launch_fast_bwd_plain(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph,
                          const BwdParams<T>& B, cudaStream_t stream) {
  using L = PlainLayout<T, CPL, TW, LX, L2, LO>;
  PlainParams<T> P;
  P.x = B.x;
  P.y = B.y;
  P.w = B.w;
  P.g = B.g;
  P.gx = B.gx;
  P.gy = B.gy;
  P.gw = B.gw;
  P.dst = B.dst;
  P.src_rowptr = B.src_rowptr;
  P.edge_ids = B.edge_ids;
  P.sp_c = static_cast<const T*>(dt.sp_c);
  P.sp_j = dt.sp_j;
  P.status = B.status;
  P.num_src_nodes = B.num_src_nodes;
  P.two = 2;
  auto kernel = fast_bwd_plain_kernel<T, CPL, TW, LX, L2, LO>;
  cudaFuncAttributes attr;
  LUNA_CUDA_CHECK(cudaFuncGetAttributes(&attr, kernel));
  const int by_registers = 65536 / (std::max(attr.numRegs, 1) * 32) / TW;
  int max_teams = std::min(plain_max_warps<TW>() / TW, std::max(1, by_registers));
  if (plan->tuning.max_warps > 0) max_teams = std::max(1, std::min(max_teams, plan->tuning.max_warps / TW));
  const size_t budget = static_cast<size_t>(dt.max_smem_optin);
  const int want_stages = plan->tuning.row_stages > 0 ? std::max(2, std::min(kTeamMaxStages, plan->tuning.row_stages)) : 2;
  constexpr int nk = LO + 1;
  int teams = 0, slots = 0, stages = 0;
  size_t block_bytes = 0;
  // as many teams as fit, then the wanted number of row stages (fewer if need be), then the deepest g ring
  for (int t = max_teams; t >= 1 && teams == 0; --t)
    for (int st = want_stages; st >= 2 && teams == 0; --st)
      for (int depth = std::min(kTeamMaxSlots, nk); depth >= std::min(2, nk); --depth) {
        const size_t bytes = L::table_bytes + t * L::team_bytes(st, depth);
        if (bytes > budget) continue;
        teams = t;
        slots = depth;
        stages = st;
        block_bytes = bytes;
        break;
      }
  if (teams == 0) return fail(LUNA_ERR_UNSUPPORTED, "backward needs more shared memory than the device has");
  P.slots = slots;
  P.row_stages = stages;
  const int64_t rows = P.num_src_nodes;
  const double degree = static_cast<double>(graph->num_edges) / static_cast<double>(std::max<int64_t>(rows, 1));
  const int64_t tile_edges = edges_per_warp(plan->tuning, 96);
  P.tile_nodes = std::max<int64_t>(1, static_cast<int64_t>(tile_edges / std::max(degree, 1e-3) + 0.5));
  P.tile_nodes = std::min<int64_t>(P.tile_nodes, 1 << 20);
  const int64_t num_tiles = ceil_div(rows, P.tile_nodes);
  const int64_t blocks = std::max<int64_t>(1, std::min<int64_t>(dt.sm_count, ceil_div(num_tiles, teams)));
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(block_bytes)));
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  kernel<<<static_cast<unsigned>(blocks), teams * TW * 32, block_bytes, stream>>>(P);
  LUNA_LAUNCH_CHECK("staged backward (compile-time layout)");
  return LUNA_OK;
}

// Dispatch on the degree shape and on one warp / two warps per edge.  LUNA_ERR_UNSUPPORTED (without an error text
// being the caller's concern) if the plan does not have the compile-time layout: the caller then takes the kernel that
// reads the layout from tables.
template <typename T, int CPL>
int dispatch_fast_bwd_plain(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph,
                            const BwdParams<T>& P, bool teams, cudaStream_t stream) {
  const int lx = plan->fast.LX, lo = plan->fast.LO, l2 = plan->fast.canon_l2;
#define LUNA_PLAIN_CASE(A, B, C)                                                                            \
  if (lx == A && l2 == B && lo == C) {                                                                      \
    if (!plain_layout_matches<T, CPL, A, B, C>(plan)) return LUNA_ERR_UNSUPPORTED;                          \
    return teams ? launch_fast_bwd_plain<T, CPL, 2, A, B, C>(plan, dt, graph, P, stream)                    \
                 : launch_fast_bwd_plain<T, CPL, 1, A, B, C>(plan, dt, graph, P, stream);                   \
  }
  LUNA_PLAIN_CASE(2, 3, 3)
  LUNA_PLAIN_CASE(2, 2, 2)
  LUNA_PLAIN_CASE(3, 3, 3)
  LUNA_PLAIN_CASE(1, 1, 1)
#undef LUNA_PLAIN_CASE
  return LUNA_ERR_UNSUPPORTED;
}

}  // namespace fastk
}  // namespace luna
