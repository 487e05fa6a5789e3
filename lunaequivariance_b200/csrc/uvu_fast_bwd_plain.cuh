// First-derivative kernel for the case training runs all the time: a canonical path list with compiled-in coupling
// patterns, one warp pass covers the channels of a block (channels == 32 * CPL), all three gradients wanted, gy and gw
// not accumulated (gx may be: callers that split a graph's edges over several calls add the pieces up).  Everything about the layout is then a compile-time constant - row lengths, block offsets, which
// paths exist - so the kernel carries no layout tables, tests no output flags and computes no addresses from them.
//
// One warp per edge.  Two ways of splitting an edge between two warps were measured on the 128-channel
// degree-(2,3,3) workload and lost to one warp per edge (13.9 ms): splitting the channels (two channels per lane,
// twelve warps: 16.7 ms, because the per-lane part of the edge-attribute gradient and the per-edge bookkeeping are
// duplicated, 40 % more instructions per edge) and splitting the paths (gx / gw by degree, gy parts balanced:
// 28.3 ms, because either half still wants about 230 registers, and at the 168 that twelve warps leave it spills
// inside the edge loop).
//
// Data movement.  An edge's weight row comes in with one bulk copy into one of the warp's row stages; the weight
// gradients overwrite the weights there and the row returns to gw with one bulk store.  The gathered g[dst] row is
// cut into one block per output degree; the blocks go through a small ring of slots.  `full` barriers (mbarrier with
// a byte count) signal arrivals; every wait is bounded, and a wait that runs out sets the plan's status word and ends
// the warp's loop.
//
// Work assignment.  Source nodes are cut into small tiles of consecutive nodes holding about the same number of edges
// (tile t is the nodes whose edge lists begin in the t-th stretch of tile_edges positions of the source-sorted edge
// order, found by a search in the row pointer: rows without edges, as the halo rows of a shard piece have many, cost
// nothing and do not distort the tiles), handed out in ascending order: a
// warp's first tile is its own number, further ones come from a counter (take_tile), so a warp that started late
// takes fewer.  All resident warps work on neighbouring source nodes at any moment, and for a spatially ordered graph the
// g[dst] rows they gather are the same few thousand rows, which stay in L2.  gx of a node is accumulated in registers
// by the one warp that owns the node: no atomics, results do not depend on the assignment.
#pragma once

#include "uvu_fast_bwd.cuh"

namespace luna {
namespace fastk {

// A stage is refilled after the first unit of the next edge: by then the bulk store of the row that was in it has
// read the stage.  Refilling one unit later measured 1 % slower (the row then has less time to arrive).
constexpr int kPlainRefillUnit = 0;
constexpr int kPlainMaxStages = 4;  // weight-row stages per warp (at most; the launcher picks 2..4)
constexpr int kPlainMaxSlots = 4;   // slots of a warp's g ring (at most)
constexpr int kPlainBarriers = kPlainMaxStages + kPlainMaxSlots;  // row landed, per stage; g block landed, per slot

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
  int64_t num_src_nodes, num_edges;
  int64_t tile_edges;          // edges per tile (tiles are cut at node boundaries)
  int64_t tile_nodes;          // > 0: tiles are this many nodes instead (graphs whose rows all have edges)
  int64_t num_tiles;
  unsigned* tile_counters;     // (next tile, warps finished)
  int slots, row_stages;
  int acc_x;                   // gx += instead of gx =
  float rows_per_edge;         // source rows / edges: the average the tile search guesses with
  int two;                     // always 2: source of the run-time 1.0 that settles freshly assembled pairs
};

// ---- compile-time layout of a canonical list with ch channels per block ---------------------------------------------
template <int LX, int L2, int LO>
struct CanonList {
  static constexpr int paths = canon_wrank(LX, L2, LO, -1, -1, -1);
  static constexpr int terms = canon_toff(LX, L2, LO, -1, -1, -1);  // padded per path
  static constexpr int ydim = (L2 + 1) * (L2 + 1);
};

// ---- shared memory --------------------------------------------------------------------------------------------------
template <typename T, int CPL, int LX, int L2, int LO>
struct PlainLayout {
  static constexpr int ch = 32 * CPL;
  static constexpr int W = CanonList<LX, L2, LO>::paths * ch;
  static constexpr int X = ch * (LX + 1) * (LX + 1);
  static constexpr int O = ch * (LO + 1) * (LO + 1);
  static constexpr int Y = CanonList<LX, L2, LO>::ydim;
  static constexpr int TT = CanonList<LX, L2, LO>::terms;
  static constexpr int gslot = ch * (2 * LO + 1);
  static constexpr int scratch_elems = (TT + 31) / 32 * 32 + kSparseTileRows * red_stride<T>() + 32 + 32;
  static constexpr size_t table_bytes = (static_cast<size_t>(TT) * sizeof(T) + 127) / 128 * 128;
  static constexpr size_t warp_bytes(int stages, int slots) {
    const size_t elems = static_cast<size_t>(stages) * W + static_cast<size_t>(slots) * gslot + scratch_elems;
    return (elems * sizeof(T) + kPlainBarriers * sizeof(uint64_t) + 127) / 128 * 128;
  }
};

// Warps per CTA at most (caps the registers per thread), by how much state a lane keeps: four FP32 channels per lane
// or FP64 fill 255 registers (8 warps); with one or two FP32 channels per lane shapes up to degree 2 fit 128
// registers (16 warps) and degree-(2,3,3) 168 (12 warps), while degree-(3,3,3) spills at 168 and is faster with 8
// warps (measured at 64 channels: 20.2 ms against 27.6 ms).
template <typename T, int CPL, int LX, int L2, int LO>
__host__ __device__ constexpr int plain_max_warps() {
  if (sizeof(T) != 4 || CPL > 2) return 8;
  if (LX <= 2 && L2 <= 2 && LO <= 2) return 16;
  return LX + LO >= 6 ? 8 : 12;
}

// Pointers into one warp's shared memory; built once per warp.
template <typename T>
struct PlainMem {
  T* wst;        // [S][W]
  T* gsl;        // [R][gslot]
  T* cybuf;      // per-edge scalars
  T* red;        // reduction tile
  T* gbuf;       // reduced gy row
  T* ybuf;       // y row
  uint64_t* wfull;
  uint64_t* gfull;
  const T* ctab;  // the block's copy of the term coefficients
};

// The edge loop of one warp.
template <typename T, int CPL, int LX, int L2, int LO>
__device__ __forceinline__ void plain_loop(const PlainParams<T>& P, const PlainMem<T>& M, int lane, int64_t first_tile,
                                           int64_t tile_step) {
  using L = PlainLayout<T, CPL, LX, L2, LO>;
  using PK = Pk<T, CPL>;
  using V = typename PK::V;
  constexpr int NP = PK::NP;
  constexpr int ch = L::ch, W = L::W, X = L::X, O = L::O, Y = L::Y, TT = L::TT;
  constexpr int kRounds = (TT + 31) / 32;
  constexpr int nk = LO + 1;
  constexpr int row_elems = W;
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

  constexpr int XR = (LX + 1) * (LX + 1) * NP;
  V xr[XR], gxr[XR];
  const V ones = runtime_one<V, T>(P.two);
  V gy2[Y];
  int s = 0, st = 0;
  uint32_t gfull_par = 0, wfull_par = 0;
  bool alive = true;
  auto give_up = [&](int code) {
    if (lane == 0) atomicExch(P.status, code);
    alive = false;
  };
  const int64_t N = P.num_src_nodes;
  const int64_t tile_edges = P.tile_edges;
  const int64_t num_tiles = P.num_tiles;

  int64_t tile = first_tile, tile_after = first_tile;
  int64_t seen_node = 0, seen_pos = 0;  // a node boundary this warp has seen, and where its edges begin
#pragma unroll 1
  for (; tile < num_tiles && alive; tile = tile_after) {
    tile_after = take_tile(P.tile_counters, tile_step, lane);  // one ahead of need
    int64_t n_lo, n_hi;
    if (P.tile_nodes > 0) {
      n_lo = tile * P.tile_nodes;
      n_hi = n_lo + P.tile_nodes < N ? n_lo + P.tile_nodes : N;
    } else {
      // tile t: the nodes whose edge lists begin in [t, t + 1) * tile_edges of the source-sorted edge order
      // (guessed from where the warp's previous tile ended, assuming rows of average length in between)
      const int64_t guess =
          seen_node + static_cast<int64_t>(static_cast<float>(tile * tile_edges - seen_pos) * P.rows_per_edge);
      n_lo = tile == 0 ? 0 : warp_lower_bound_guess(P.src_rowptr, N, tile * tile_edges, guess, lane);
      n_hi = tile + 1 == num_tiles ? N : warp_lower_bound_near(P.src_rowptr, N, (tile + 1) * tile_edges, n_lo, lane);
    }
    if (n_lo >= n_hi) continue;  // a node with more edges than a tile spans several tile numbers
    const int64_t p_begin = P.src_rowptr[n_lo], p_end = P.src_rowptr[n_hi];
    seen_node = n_hi;
    seen_pos = p_end;
    if (p_begin >= p_end) continue;
    const int total_units = static_cast<int>(p_end - p_begin) * nk;

    auto id_at = [&](int64_t p) { return p < p_end ? P.edge_ids[p] : -1; };
    auto dst_of = [&](int e) { return e >= 0 ? P.dst[e] : 0; };
    int e0 = id_at(p_begin), e1 = id_at(p_begin + 1), e2 = id_at(p_begin + 2), e3 = id_at(p_begin + 3);
    int e4 = id_at(p_begin + 4);
    int d0 = dst_of(e0), d1n = dst_of(e1), d2n = dst_of(e2);
    auto edge_ahead = [&](int k) { return k == 1 ? e1 : (k == 2 ? e2 : (k == 3 ? e3 : e4)); };
    if (lane == 0) {
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
            constexpr int rank = canon_wrank(LX, L2, LO, l1, l2, l3);
            T* wq = wrow + rank * ch + lane * CPL;
            V w2[NP], dot[NP];
            load_lane_packets<PK, T, CPL>(wq, w2);
            sparse_path_rows<T, CPL, LX, L2, LO, l1, l2, l3, true, true, V>(
                &xr[l1 * l1 * NP], &gxr[l1 * l1 * NP], gy2, g2, w2, dot, M.cybuf, M.ctab);
            T gwv[CPL];  // the gradients take the weights' place and leave with the row
            unpack_packets<PK, T, CPL, 1>(dot, gwv);
            store_vectors<T, CPL, 1>(wq, gwv);
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
      if (u + R < total_units && lane == 0) {
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
      if (pos >= pe) {
        // A row without edges.  A shard piece has long runs of them (the sources its destinations do not read):
        // jump to the row that holds the warp's next edge instead of walking the run one dependent load at a time.
        if (pos >= p_end) break;  // nothing but such rows is left in the tile
        n = warp_lower_bound(P.src_rowptr, N, pos + 1, lane) - 2;
        continue;
      }
      static_for<0, LX + 1>([&](auto l1c) {
        constexpr int l1 = decltype(l1c)::value;
        constexpr int d1 = 2 * l1 + 1;
        load_packets_scalar<PK, T, CPL, d1>(P.x + n * X + ch * l1 * l1 + lane * (CPL * d1), &xr[l1 * l1 * NP]);
      });
      settle_packets<XR>(xr, ones);
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
          if constexpr (kind == kPlainRefillUnit) {
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
        if (lane == 0) {
          bulk_wait_group_read_all();
          store_row(e0, st);
        }
        if (pos + 1 < p_end) {  // refill the stage once the row has been read out of it (during the next edge)
          refill_stage = st;
          refill_edge = edge_ahead(S);
        } else if (lane == 0) {
          bulk_wait_group_read_all();  // the next tile's first copies reuse this stage
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
        if (lane < Y) P.gy[static_cast<int64_t>(e0) * Y + lane] = M.gbuf[lane];
        __syncwarp();
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
        T row[CPL * d1];  // memory order: channel-major, component-minor
        unpack_packets<PK, T, CPL, d1>(&gxr[l1 * l1 * NP], row);
        T* to = P.gx + n * X + ch * l1 * l1 + lane * (CPL * d1);
        if (P.acc_x) {
          T old[CPL * d1];
          load_vectors<T, CPL, d1>(to, old);
#pragma unroll
          for (int a = 0; a < CPL * d1; ++a) row[a] += old[a];
        }
        store_vectors<T, CPL, d1>(to, row);
      });
    }
  }
  leave_tiles(P.tile_counters, tile_step, lane);
  if (lane == 0) bulk_wait_group_read_all();
  if (!alive) {  // let copies that are still in flight land as well (bounded)
    for (int v = 0; v < R; ++v) mbar_wait_bounded(&M.gfull[v], (gfull_par >> v) & 1u);
    for (int v = 0; v < S; ++v) mbar_wait_bounded(&M.wfull[v], (wfull_par >> v) & 1u);
  }
}

template <typename T, int CPL, int LX, int L2, int LO>
__global__ void __launch_bounds__(plain_max_warps<T, CPL, LX, L2, LO>() * 32, 1)
    fast_bwd_plain_kernel(const __grid_constant__ PlainParams<T> P) {
  using L = PlainLayout<T, CPL, LX, L2, LO>;
  static_assert(LO >= 1, "the g ring needs at least two units per edge");
  static_assert((L::TT + 31) / 32 <= kMaxSparseRounds, "coupling program too long for the register budget");
  static_assert((L::Y + 1) / 2 <= kSparseTileRows, "edge attributes too wide for the reduction tile");
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int R = P.slots, S = P.row_stages;

  T* ctab = reinterpret_cast<T*>(smem_raw);
  unsigned char* base = smem_raw + L::table_bytes + static_cast<size_t>(warp) * L::warp_bytes(S, R);
  PlainMem<T> M;
  M.ctab = ctab;
  M.wst = reinterpret_cast<T*>(base);
  M.gsl = M.wst + static_cast<size_t>(S) * L::W;
  M.cybuf = M.gsl + static_cast<size_t>(R) * L::gslot;
  M.red = M.cybuf + (L::TT + 31) / 32 * 32;
  M.gbuf = M.red + kSparseTileRows * red_stride<T>();
  M.ybuf = M.gbuf + 32;
  M.wfull = reinterpret_cast<uint64_t*>(M.ybuf + 32);
  M.gfull = M.wfull + kPlainMaxStages;

  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&M.wfull[s], 1);
    for (int s = 0; s < R; ++s) mbar_init(&M.gfull[s], 1);
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < L::TT; i += blockDim.x) ctab[i] = P.sp_c[i];
  __syncthreads();

  const int64_t first_tile = static_cast<int64_t>(blockIdx.x) * nwarps + warp;
  const int64_t tile_step = static_cast<int64_t>(gridDim.x) * nwarps;
  plain_loop<T, CPL, LX, L2, LO>(P, M, lane, first_tile, tile_step);
}

// Whether the plan has exactly the layout the kernel assumes (blocks in degree order, weights in path order).
template <typename T, int CPL, int LX, int L2, int LO>
bool plain_layout_matches(const luna_uvu_plan* plan) {
  using L = PlainLayout<T, CPL, LX, L2, LO>;
  const FastMeta& f = plan->fast;
  if (f.chunks != 1 || f.ch != L::ch || f.W != L::W || f.X != L::X || f.O != L::O || f.Y != L::Y) return false;
  if (f.sparse_terms != L::TT) return false;
  for (int l = 0; l <= LX; ++l)
    if (f.x_off[l] != L::ch * l * l) return false;
  for (int l = 0; l <= LO; ++l)
    if (f.o_off[l] != L::ch * l * l) return false;
  return true;
}

template <typename T, int CPL, int LX, int L2, int LO>
int launch_fast_bwd_plain(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph,
                          const BwdParams<T>& B, cudaStream_t stream) {
  using L = PlainLayout<T, CPL, LX, L2, LO>;
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
  P.acc_x = B.acc_x ? 1 : 0;
  P.tile_counters = next_tile_counters(plan, dt);
  P.two = 2;
  auto kernel = fast_bwd_plain_kernel<T, CPL, LX, L2, LO>;
  cudaFuncAttributes attr;
  LUNA_CUDA_CHECK(cudaFuncGetAttributes(&attr, kernel));
  const int by_registers = 65536 / (std::max(attr.numRegs, 1) * 32);
  int max_warps = std::min(plain_max_warps<T, CPL, LX, L2, LO>(), std::max(1, by_registers));
  if (plan->tuning.max_warps > 0) max_warps = std::max(1, std::min(max_warps, plan->tuning.max_warps));
  const size_t budget = static_cast<size_t>(dt.max_smem_optin);
  const int want_stages =
      plan->tuning.row_stages > 0 ? std::max(2, std::min(kPlainMaxStages, plan->tuning.row_stages)) : 2;
  constexpr int nk = LO + 1;
  int warps = 0, slots = 0, stages = 0;
  size_t block_bytes = 0;
  // as many warps as fit, then the wanted number of row stages (fewer if need be), then the deepest g ring
  for (int t = max_warps; t >= 1 && warps == 0; --t)
    for (int st = want_stages; st >= 2 && warps == 0; --st)
      for (int depth = std::min(kPlainMaxSlots, nk); depth >= std::min(2, nk); --depth) {
        const size_t bytes = L::table_bytes + t * L::warp_bytes(st, depth);
        if (bytes > budget) continue;
        warps = t;
        slots = depth;
        stages = st;
        block_bytes = bytes;
        break;
      }
  if (warps == 0) return fail(LUNA_ERR_UNSUPPORTED, "backward needs more shared memory than the device has");
  P.slots = slots;
  P.row_stages = stages;
  P.num_edges = graph->num_edges;
  P.rows_per_edge = static_cast<float>(static_cast<double>(P.num_src_nodes) / static_cast<double>(std::max<int64_t>(P.num_edges, 1)));
  P.tile_edges = tile_edges_for(P.num_edges, static_cast<int64_t>(dt.sm_count) * warps, edges_per_warp(plan->tuning, 64));
  // A whole graph of some density, or a shard of one (source rows = owned rows plus a halo, at most half as many
  // again as the destination rows), has hardly any rows without edges, and a fixed number of nodes per tile then
  // gives even tiles without any search: measured 5 % faster than edge-count tiles on the 50,000-atom radius graph.
  // Pieces of graphs (a destination sub-range against all source rows) have long runs of rows without edges and get
  // edge-count tiles.
  const bool whole = graph->num_src_nodes <= 0 || graph->num_src_nodes <= graph->num_nodes + graph->num_nodes / 2;
  const double degree = static_cast<double>(P.num_edges) / static_cast<double>(std::max<int64_t>(P.num_src_nodes, 1));
  P.tile_nodes = (whole && degree >= 8.0) ? std::max<int64_t>(1, static_cast<int64_t>(P.tile_edges / degree + 0.5)) : 0;
  const int64_t num_tiles = P.tile_nodes > 0 ? ceil_div(std::max<int64_t>(P.num_src_nodes, 1), P.tile_nodes)
                                             : ceil_div(std::max<int64_t>(P.num_edges, 1), P.tile_edges);
  P.num_tiles = num_tiles;
  const int64_t blocks = std::max<int64_t>(1, std::min<int64_t>(dt.sm_count, ceil_div(num_tiles, warps)));
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(block_bytes)));
  LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  kernel<<<static_cast<unsigned>(blocks), warps * 32, block_bytes, stream>>>(P);
  LUNA_LAUNCH_CHECK("staged backward (compile-time layout)");
  return LUNA_OK;
}

// Dispatch on the degree shape.  LUNA_ERR_UNSUPPORTED if the plan does not have the compile-time layout: the caller
// then takes the kernel that reads the layout from tables.
template <typename T, int CPL>
int dispatch_fast_bwd_plain(const luna_uvu_plan* plan, const DeviceTables& dt, const luna_graph* graph,
                            const BwdParams<T>& P, cudaStream_t stream) {
  const int lx = plan->fast.LX, lo = plan->fast.LO, l2 = plan->fast.canon_l2;
#define LUNA_PLAIN_CASE(A, B, C)                                                                            \
  if (lx == A && l2 == B && lo == C) {                                                                      \
    if (!plain_layout_matches<T, CPL, A, B, C>(plan)) return LUNA_ERR_UNSUPPORTED;                          \
    return launch_fast_bwd_plain<T, CPL, A, B, C>(plan, dt, graph, P, stream);                              \
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
