// UVU convolution plan: host-side analysis of the path list and the lookup tables the kernels read.
#pragma once

#include <array>
#include <cstdint>
#include <map>
#include <atomic>
#include <mutex>
#include <vector>

#include "common.h"

namespace luna {

// ------------------------------------------------------------------------------------------------ generic tables
// One record per path (instruction x edge channel).  *_ptr index the three row-pointer arrays that list a path's
// coupling terms sorted by output component k, by x component i and by y component j.
struct PathRec {
  int x_off, y_off, out_off, w_off, w_stride, ch;
  int d1, d2, d3;
  int byk_ptr, byi_ptr, byj_ptr;  // start of this path's (d+1)-entry row-pointer block in rowptr_{k,i,j}
};

// A block of a feature row shared by several paths (an irrep block of x, y or out).
struct SlotRec {
  int off, ch, d;          // ch = 1 for y slots
  int path_begin, path_end;  // range in the slot's path list
};

template <typename T>
struct TermRec {
  int a, b;  // the two indices other than the sorting one, in (i, j, k) order
  T c;
};

// Pointers into the per-device table buffer.
template <typename T>
struct GenericTables {
  const PathRec* paths;
  int num_paths;
  const SlotRec *out_slots, *x_slots, *y_slots;
  int num_out_slots, num_x_slots, num_y_slots;
  const int *out_slot_paths, *x_slot_paths, *y_slot_paths;
  const int* w_elem_path;  // [weight_numel] path owning each weight column, -1 if none
  const int *rowptr_k, *rowptr_i, *rowptr_j;
  const TermRec<T>*terms_k, *terms_i, *terms_j;
  int X, Y, O, W;
};

// ------------------------------------------------------------------------------------------------ staged ("fast") tables
constexpr int kMaxFastPaths = 64;
constexpr int kMaxFastL = 3;          // degrees 0..3 on x and out
constexpr int kMaxMEntries = 768;     // per-edge coupling-matrix entries (rows padded to an even length)

struct CopyPiece {
  int g_off;   // element offset inside the global row for channel chunk 0
  int comp;    // elements per channel (multiplies the chunk's first channel)
  int s_off;   // element offset inside the shared-memory region
  int n;       // elements
};

// Everything the staged kernels need, small enough to travel as a kernel parameter.  Paths are renumbered
// q = 0.. in (l3, l1) order; the matrix of path q occupies entries m_off[q] + i * (d3 + 1) + k of the per-edge
// coupling-matrix buffer (rows padded to the even length d3 + 1, matrices to a multiple of 4 entries; padding
// entries are zero).
struct FastMeta {
  int LX, LO;                 // highest degree present in x / out
  int canon_l2;               // highest edge-harmonic degree if the path list is the canonical full list, else -1
  int sparse_terms;           // length of the sparse term list (canon_toff total) if the plan's coupling terms have
                              // the compiled-in patterns and y is laid out as degrees 0..L2 in order, else 0
  int cpl;                    // channels per lane
  int chunks;                 // channel chunks per feature block (a warp handles 32 * cpl channels)
  int ch;                     // channels per block (uniform)
  int X, Y, O, W;
  int num_paths;
  int x_off[kMaxFastL + 1];   // global offset of the degree-l block of x, -1 if absent
  int o_off[kMaxFastL + 1];
  int pair_ptr[(kMaxFastL + 1) * (kMaxFastL + 1) + 1];  // first path of (l3, l1); index l3 * 4 + l1
  int w_goff[kMaxFastPaths];  // global weight offset of the path
  int m_off[kMaxFastPaths];
  int m_total;                // entries in the coupling-matrix buffer (multiple of 4)
  int m_terms;                // terms per entry in the padded program (always 2)
  // forward kernel: one stage holds a whole edge, w in global order followed by the x blocks
  int xs_off[kMaxFastL + 1];  // offset of the degree-l block inside the staged x region (elements)
  int w_soff[kMaxFastPaths];  // offset of a path's channel chunk inside the staged w region
  int w_stage_elems, x_stage_elems;
  int n_w_pieces, n_x_pieces;
  CopyPiece pieces_w[kMaxFastPaths];
  CopyPiece pieces_x[kMaxFastL + 1];
  // backward kernel: one ring slot holds one unit = (edge, output degree): the w chunks of the paths into that
  // degree in q order, then the degree's block of the destination's g row
  int nkinds;                       // output degrees present
  int kind_l3[kMaxFastL + 1];       // degree of unit kind 0..nkinds-1 (ascending)
  int kind_of_l3[kMaxFastL + 1];    // inverse, -1 if absent
  int unit_elems[kMaxFastL + 1];    // elements of a unit of that kind
  int slot_elems;                   // largest unit
  int uw_soff[kMaxFastPaths];       // offset of a path's w chunk inside its unit
  int ug_soff[kMaxFastL + 1];       // offset of the g block inside the unit of degree l3
  // byte offsets inside the backward kernel's table blob (copied to shared memory by every CTA)
  int tb_gyc, tb_gyptr, tb_gym, tb_ellj, tb_bytes;
  int gy_terms;
};

// ------------------------------------------------------------------------------------------------ the plan
// Settings that select kernel variants or override a launch policy.  They come from LUNA_B200_* environment
// variables, read once when the plan is created (never on a launch path):
//   LUNA_B200_NO_CANON=1        canonical path lists run the kernels that loop over run-time path tables
//   LUNA_B200_NO_SPARSE=1       backward without the compiled-in coupling patterns
//   LUNA_B200_NO_PLAIN=1        backward without the kernels that have the layout compiled in
//   LUNA_B200_BWD_KERNEL=row|units   data-movement variant of the backward kernel with compiled-in patterns
//   LUNA_B200_MAXW=n            cap on warps per CTA
//   LUNA_B200_ROW_STAGES=n      cap on weight-row stages of the row-staged backward
//   LUNA_B200_EPW=n             backward: edges per tile of source nodes (kernels with a compile-time layout), target
//                               edges per warp when a graph needs several waves (the others)
//   LUNA_B200_FWD_TILE=n        forward: edges per tile of destination nodes
struct Tuning {
  bool no_canon = false, no_sparse = false, no_plain = false;
  int bwd_kernel = 0;  // 0 automatic, 1 row stages, 2 unit ring
  int max_warps = 0;   // 0: no cap
  int row_stages = 0;  // 0: no cap
  int64_t edges_per_warp = 0;  // 0: the kernel's default
  int64_t fwd_tile_edges = 0;  // 0: the kernel's default
};
Tuning tuning_from_environment();

constexpr int kTileCounterSets = 32;    // launches of one plan that may be in flight on a device at a time
constexpr int kTileCounterWords = 64;   // per set: (next tile, warps finished) for up to 32 channel chunks

struct DeviceTables {
  void* buffer = nullptr;  // one allocation holding every table
  size_t bytes = 0;
  int* status = nullptr;   // device status word (inside buffer)
  // Work counters of the kernels that hand out tiles of nodes dynamically: kTileCounterSets sets of
  // kTileCounterWords zero-initialised words (inside buffer).  A launch takes the next set in turn; its last warp
  // to finish puts the set back to zero, so no launch has to clear anything.
  unsigned* tile_counters = nullptr;
  // resolved pointers (type-erased; reinterpret for the plan's dtype)
  const PathRec* paths = nullptr;
  const SlotRec *out_slots = nullptr, *x_slots = nullptr, *y_slots = nullptr;
  const int *out_slot_paths = nullptr, *x_slot_paths = nullptr, *y_slot_paths = nullptr;
  const int* w_elem_path = nullptr;
  const int *rowptr_k = nullptr, *rowptr_i = nullptr, *rowptr_j = nullptr;
  const void *terms_k = nullptr, *terms_i = nullptr, *terms_j = nullptr;
  const unsigned char* ell_j = nullptr;  // [m_terms * m_total] y index of each term (padded form)
  const void* ell_c = nullptr;           // [m_terms * m_total] coefficient of each term, 0 for padding
  // backward kernel's tables in one blob: coefficients of the padded program, coefficients / row pointers /
  // entry indices of the edge-attribute gradient's program (gy[j] = sum_t c[t] * G[m[t]]), y indices of the
  // padded program; offsets in FastMeta::tb_*
  const unsigned char* bwd_tables = nullptr;
  // sparse term list of a canonical plan (FastMeta::sparse_terms entries): coefficient and y index of each term
  const void* sp_c = nullptr;
  const unsigned char* sp_j = nullptr;
  int sm_count = 0;
  int max_smem_optin = 0;
};

}  // namespace luna

struct luna_uvu_plan {
  int dtype = LUNA_F32;
  int X = 0, Y = 0, O = 0, W = 0;
  std::vector<luna::PathRec> paths;
  std::vector<luna::SlotRec> out_slots, x_slots, y_slots;
  std::vector<int> out_slot_paths, x_slot_paths, y_slot_paths;
  std::vector<int> w_elem_path;
  std::vector<int> rowptr_k, rowptr_i, rowptr_j;
  // terms kept in double on the host; narrowed at upload
  struct HostTerm {
    int a, b;
    double c;
  };
  std::vector<HostTerm> terms_k, terms_i, terms_j;
  bool out_fully_covered = false;

  bool fast_ok = false;
  bool force_generic = false;
  luna::Tuning tuning{};
  luna::FastMeta fast{};
  std::vector<double> ell_c;
  std::vector<unsigned char> ell_j;
  std::vector<int> gy_ptr, gy_m;
  std::vector<double> gy_c;
  std::vector<double> sp_c;
  std::vector<unsigned char> sp_j;

  std::mutex mutex;
  std::map<int, luna::DeviceTables> device_tables;
  mutable std::atomic<unsigned> tile_counter_cursor{0};
};

namespace luna {

// Returns the tables for the current device, uploading them on first use.
int get_device_tables(luna_uvu_plan* plan, const DeviceTables** out);

// The set of tile counters for the next launch of this plan on the device of `dt`.
inline unsigned* next_tile_counters(const luna_uvu_plan* plan, const DeviceTables& dt) {
  const unsigned set = plan->tile_counter_cursor.fetch_add(1u, std::memory_order_relaxed) % kTileCounterSets;
  return dt.tile_counters + static_cast<size_t>(set) * kTileCounterWords;
}

template <typename T>
GenericTables<T> generic_tables(const luna_uvu_plan* plan, const DeviceTables& dt) {
  GenericTables<T> t;
  t.paths = dt.paths;
  t.num_paths = static_cast<int>(plan->paths.size());
  t.out_slots = dt.out_slots;
  t.x_slots = dt.x_slots;
  t.y_slots = dt.y_slots;
  t.num_out_slots = static_cast<int>(plan->out_slots.size());
  t.num_x_slots = static_cast<int>(plan->x_slots.size());
  t.num_y_slots = static_cast<int>(plan->y_slots.size());
  t.out_slot_paths = dt.out_slot_paths;
  t.x_slot_paths = dt.x_slot_paths;
  t.y_slot_paths = dt.y_slot_paths;
  t.w_elem_path = dt.w_elem_path;
  t.rowptr_k = dt.rowptr_k;
  t.rowptr_i = dt.rowptr_i;
  t.rowptr_j = dt.rowptr_j;
  t.terms_k = static_cast<const TermRec<T>*>(dt.terms_k);
  t.terms_i = static_cast<const TermRec<T>*>(dt.terms_i);
  t.terms_j = static_cast<const TermRec<T>*>(dt.terms_j);
  t.X = plan->X;
  t.Y = plan->Y;
  t.O = plan->O;
  t.W = plan->W;
  return t;
}

// Which argument of the four-linear form F(x, y, w, g) is left free (differentiated).
enum FreeSlot { kFreeG = 0, kFreeX = 1, kFreeY = 2, kFreeW = 3 };

// Table-driven contraction: out (shaped like the free argument) = or += dF/d(free).  Operands are device
// pointers of the plan's dtype; the pointer in the free position is ignored.
int generic_contract(luna_uvu_plan* plan, const luna_graph* graph, int free_slot, const void* x, const void* y,
                     const void* w, const void* g, void* out, bool accumulate, cudaStream_t stream);

// Staged kernels (bulk-copy pipeline).  fast_available() is false in a build without them.
bool fast_available();
// The luna_bwd_variant the first-order backward takes for this plan (for aligned operands).
int fast_bwd_variant(const luna_uvu_plan* plan);
// which: 0 forward-shaped kernel, 1 backward-shaped kernel.  Dynamic shared memory per block, 0 if not eligible.
int64_t fast_smem_bytes(const luna_uvu_plan* plan, int which);
int64_t fast_scratch_bytes(const luna_uvu_plan* plan, int64_t num_nodes, int64_t num_edges);
// tangents == false: out = F_g(x, y, w).  tangents == true: out = F_g(rx, y, w) + F_g(x, ry, w) + F_g(x, y, rw)
// with null tangents skipped (at least one must be given).
int fast_forward(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y, const void* w,
                 const void* rx, const void* ry, const void* rw, void* out, bool tangents, cudaStream_t stream);
// Any subset of gx, gy, gw (null = skip); acc_* adds to the existing contents instead of overwriting.
int fast_backward(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y, const void* w,
                  const void* g, void* gx, bool acc_x, void* gy, bool acc_y, void* gw, bool acc_w, void* scratch,
                  int64_t scratch_bytes, cudaStream_t stream);

}  // namespace luna
