// Plan creation: validates a path description, builds the lookup tables of the table-driven kernels and, when the
// configuration allows it, the metadata of the staged (bulk-copy) kernels; uploads tables once per device.
#include "plan.h"
#include "uvu_fast.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <string>

namespace luna {

namespace {
thread_local char g_error[512] = "";
}

int fail(int code, const char* format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(g_error, sizeof(g_error), format, args);
  va_end(args);
  return code;
}

void clear_error() { g_error[0] = '\0'; }

namespace {

template <typename Key>
void build_slots(const std::vector<PathRec>& paths, Key key, std::vector<SlotRec>& slots,
                 std::vector<int>& slot_paths) {
  // key(path) -> (off, ch, d)
  std::vector<std::pair<int, int>> order;  // (off, path)
  for (int p = 0; p < static_cast<int>(paths.size()); ++p) order.push_back({key(paths[p]).off, p});
  std::stable_sort(order.begin(), order.end(), [](auto a, auto b) { return a.first < b.first; });
  for (auto [off, p] : order) {
    SlotRec rec = key(paths[p]);
    if (slots.empty() || slots.back().off != off) {
      rec.path_begin = rec.path_end = static_cast<int>(slot_paths.size());
      slots.push_back(rec);
    }
    slot_paths.push_back(p);
    slots.back().path_end = static_cast<int>(slot_paths.size());
  }
}

int round_up(int v, int m) { return (v + m - 1) / m * m; }

// Fills the stage layouts, path order and coupling-matrix program of `f` for `cpl` channels per lane.  Returns false
// if a limit of the staged kernels is exceeded.
bool fill_layout(luna_uvu_plan* plan, FastMeta& f, int cpl) {
  const auto& paths = plan->paths;
  const int elem = plan->dtype == LUNA_F64 ? 8 : 4;
  const int ch = paths[0].ch;
  f.cpl = cpl;
  const int chw = 32 * cpl;
  if (ch % chw != 0) return false;
  f.chunks = ch / chw;
  if (f.chunks > kTileCounterWords / 2) return false;  // one pair of tile counters per channel chunk
  f.ch = ch;
  f.X = plan->X;
  f.Y = plan->Y;
  f.O = plan->O;
  f.W = plan->W;
  f.num_paths = static_cast<int>(paths.size());

  // paths sorted by (l3, l1): all paths into one output degree are contiguous, also in the matrix buffer
  std::vector<int> order(paths.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = static_cast<int>(i);
  const int LO1 = kMaxFastL + 1;  // fixed stride so kernels compiled for larger degrees index the same table
  auto pair_of = [&](int p) { return ((paths[p].d3 - 1) / 2) * LO1 + (paths[p].d1 - 1) / 2; };
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return pair_of(a) < pair_of(b); });
  const int npairs = LO1 * LO1;
  for (int i = 0; i <= npairs; ++i) f.pair_ptr[i] = 0;
  for (int p : order) f.pair_ptr[pair_of(p) + 1]++;
  for (int i = 0; i < npairs; ++i) f.pair_ptr[i + 1] += f.pair_ptr[i];

  // forward stage: w in global weight order
  std::vector<int> by_w(order.size());
  for (size_t q = 0; q < order.size(); ++q) by_w[q] = static_cast<int>(q);
  std::stable_sort(by_w.begin(), by_w.end(),
                   [&](int a, int b) { return paths[order[a]].w_off < paths[order[b]].w_off; });
  f.n_w_pieces = 0;
  for (size_t rank = 0; rank < by_w.size(); ++rank) {
    const int q = by_w[rank];
    const PathRec& p = paths[order[q]];
    f.w_goff[q] = p.w_off;
    f.w_soff[q] = static_cast<int>(rank) * chw;
    CopyPiece piece{p.w_off, 1, f.w_soff[q], chw};
    if (f.chunks == 1 && f.n_w_pieces > 0) {
      CopyPiece& last = f.pieces_w[f.n_w_pieces - 1];
      if (last.g_off + last.n == piece.g_off && last.s_off + last.n == piece.s_off) {
        last.n += piece.n;
        continue;
      }
    }
    f.pieces_w[f.n_w_pieces++] = piece;
  }
  f.w_stage_elems = static_cast<int>(paths.size()) * chw;
  if (f.n_w_pieces + kMaxFastL + 1 > 32) return false;  // one lane issues one copy piece
  {
    std::vector<int> ls;
    for (int l = 0; l <= f.LX; ++l)
      if (f.x_off[l] >= 0) ls.push_back(l);
    std::sort(ls.begin(), ls.end(), [&](int a, int b) { return f.x_off[a] < f.x_off[b]; });
    f.n_x_pieces = 0;
    f.x_stage_elems = 0;
    for (int l : ls) {
      const int d = 2 * l + 1;
      f.xs_off[l] = f.x_stage_elems;
      CopyPiece piece{f.x_off[l], d, f.x_stage_elems, chw * d};
      f.x_stage_elems += chw * d;
      if (f.chunks == 1 && f.n_x_pieces > 0) {
        CopyPiece& last = f.pieces_x[f.n_x_pieces - 1];
        if (last.g_off + last.n == piece.g_off && last.s_off + last.n == piece.s_off) {
          last.n += piece.n;
          continue;
        }
      }
      f.pieces_x[f.n_x_pieces++] = piece;
    }
  }

  // backward units
  f.nkinds = 0;
  f.slot_elems = 0;
  for (int l3 = 0; l3 <= kMaxFastL; ++l3) {
    f.kind_of_l3[l3] = -1;
    f.ug_soff[l3] = 0;
    f.unit_elems[l3] = 0;
    f.kind_l3[l3] = 0;
  }
  for (int l3 = 0; l3 <= f.LO; ++l3) {
    if (f.o_off[l3] < 0) continue;
    const int q0 = f.pair_ptr[l3 * LO1], q1 = f.pair_ptr[l3 * LO1 + LO1];
    if (q1 - q0 + 1 > 32) return false;  // one lane issues one copy piece
    for (int q = q0; q < q1; ++q) f.uw_soff[q] = (q - q0) * chw;
    f.ug_soff[l3] = (q1 - q0) * chw;
    const int kind = f.nkinds++;
    f.kind_l3[kind] = l3;
    f.kind_of_l3[l3] = kind;
    f.unit_elems[kind] = (q1 - q0) * chw + chw * (2 * l3 + 1);
    f.slot_elems = std::max(f.slot_elems, f.unit_elems[kind]);
  }

  // per-edge coupling matrices (path matrices back to back, rows padded to the even length d3 + 1, each matrix
  // padded to a multiple of 4 entries)
  std::vector<int> m_ptr, m_j;
  std::vector<double> m_c;
  int total = 0;
  for (size_t q = 0; q < order.size(); ++q) {
    const PathRec& p = paths[order[q]];
    f.m_off[q] = total;
    // terms sorted by k give (i, j) per k; rebuild a dense (i,k) -> list of (j, c)
    std::vector<std::vector<std::pair<int, double>>> cell(p.d1 * p.d3);
    for (int k = 0; k < p.d3; ++k)
      for (int t = plan->rowptr_k[p.byk_ptr + k]; t < plan->rowptr_k[p.byk_ptr + k + 1]; ++t) {
        const auto& term = plan->terms_k[t];
        cell[term.a * p.d3 + k].push_back({p.y_off + term.b, term.c});
      }
    const int d3p = p.d3 + 1;
    for (int i = 0; i < p.d1; ++i)
      for (int k = 0; k < d3p; ++k) {
        m_ptr.push_back(static_cast<int>(m_j.size()));
        if (k < p.d3)
          for (auto [j, c] : cell[i * p.d3 + k]) {
            m_j.push_back(j);
            m_c.push_back(c);
          }
      }
    total += p.d1 * d3p;
    while (total % 4 != 0) {  // every matrix starts on a 16-byte boundary, also in FP32 without duplication
      m_ptr.push_back(static_cast<int>(m_j.size()));
      ++total;
    }
  }
  m_ptr.push_back(static_cast<int>(m_j.size()));
  f.m_total = total;
  if (total > kMaxMEntries) return false;

  // canonical full path list?  (all degrees 0..LX / 0..LO present, every allowed triple exactly once, weight
  // blocks in (l1, l2, l3) order)
  f.canon_l2 = -1;
  {
    int L2 = 0;
    for (const auto& p : paths) L2 = std::max(L2, (p.d2 - 1) / 2);
    bool canon = f.chunks >= 1 && fastk::canon_wrank(f.LX, L2, f.LO, -1, -1, -1) == static_cast<int>(paths.size()) &&
                 fastk::canon_moff(f.LX, L2, f.LO, -1, -1, -1) == total;
    for (int l = 0; l <= f.LX && canon; ++l) canon = f.x_off[l] >= 0 && f.xs_off[l] == chw * l * l;
    for (int l = 0; l <= f.LO && canon; ++l) canon = f.o_off[l] >= 0;
    for (size_t q = 0; q < order.size() && canon; ++q) {
      const PathRec& p = paths[order[q]];
      const int l1 = (p.d1 - 1) / 2, l2 = (p.d2 - 1) / 2, l3 = (p.d3 - 1) / 2;
      canon = (p.d1 % 2 == 1) && (p.d2 % 2 == 1) && (p.d3 % 2 == 1) && fastk::canon_ok(f.LX, L2, f.LO, l1, l2, l3) &&
              f.w_soff[q] == fastk::canon_wrank(f.LX, L2, f.LO, l1, l2, l3) * chw &&
              p.w_off == fastk::canon_wrank(f.LX, L2, f.LO, l1, l2, l3) * ch &&
              f.m_off[q] == fastk::canon_moff(f.LX, L2, f.LO, l1, l2, l3);
    }
    if (canon) f.canon_l2 = L2;
    // sparse term list: every path's terms must have exactly the compiled-in pattern
    f.sparse_terms = 0;
    plan->sp_c.clear();
    plan->sp_j.clear();
    if (canon && L2 <= 3 && f.LX <= 3 && f.LO <= 3) {
      const int total_terms = fastk::canon_toff(f.LX, L2, f.LO, -1, -1, -1);
      std::vector<double> sc(static_cast<size_t>(total_terms), 0.0);
      std::vector<unsigned char> sj(static_cast<size_t>(total_terms), 0);
      bool match = true;
      for (size_t q = 0; q < order.size() && match; ++q) {
        const PathRec& p = paths[order[q]];
        const int l1 = (p.d1 - 1) / 2, l2 = (p.d2 - 1) / 2, l3 = (p.d3 - 1) / 2;
        const fastk::CgTerm* pattern = fastk::cg_pattern(l1, l2, l3);
        const int n = fastk::cg_count(l1, l2, l3);
        const int toff = fastk::canon_toff(f.LX, L2, f.LO, l1, l2, l3);
        match = pattern != nullptr && p.y_off == l2 * l2;
        int found = 0;
        for (int k = 0; k < p.d3 && match; ++k)
          for (int t = plan->rowptr_k[p.byk_ptr + k]; t < plan->rowptr_k[p.byk_ptr + k + 1] && match; ++t) {
            const auto& term = plan->terms_k[t];  // (a, b) = (i, j)
            int slot = -1;
            for (int u = 0; u < n; ++u)
              if (pattern[u].i == term.a && pattern[u].j == term.b && pattern[u].k == k) slot = u;
            if (slot < 0 || sc[toff + slot] != 0.0) {
              match = false;
            } else {
              sc[toff + slot] = term.c;
              sj[toff + slot] = static_cast<unsigned char>(p.y_off + term.b);
              ++found;
            }
          }
        if (found != n) match = false;  // a pattern entry the plan does not have would be a wasted (zero) term
      }
      if (match) {
        f.sparse_terms = total_terms;
        plan->sp_c = sc;
        plan->sp_j = sj;
      }
    }
  }

  // the program in padded (ELL) form for the kernels: term t of entry m at [t * m_total + m], exactly two
  // (zero-padded) terms per entry, which is enough for l <= 3
  f.m_terms = 2;
  for (int m = 0; m < total; ++m)
    if (m_ptr[m + 1] - m_ptr[m] > 2) return false;
  plan->ell_c.assign(static_cast<size_t>(f.m_terms) * total, 0.0);
  plan->ell_j.assign(static_cast<size_t>(f.m_terms) * total, 0);
  for (int m = 0; m < total; ++m)
    for (int t = m_ptr[m]; t < m_ptr[m + 1]; ++t) {
      const size_t slot = static_cast<size_t>(t - m_ptr[m]) * total + m;
      plan->ell_c[slot] = m_c[t];
      plan->ell_j[slot] = static_cast<unsigned char>(m_j[t]);
    }
  // transposed program for the edge-attribute gradient: gy[j] = sum over (m, c) with that j of c * G[m]
  std::vector<std::vector<std::pair<int, double>>> by_j(plan->Y);
  for (int m = 0; m < total; ++m)
    for (int t = m_ptr[m]; t < m_ptr[m + 1]; ++t) by_j[m_j[t]].push_back({m, m_c[t]});
  plan->gy_ptr.clear();
  plan->gy_m.clear();
  plan->gy_c.clear();
  for (int j = 0; j < plan->Y; ++j) {
    plan->gy_ptr.push_back(static_cast<int>(plan->gy_m.size()));
    for (auto [m, c] : by_j[j]) {
      plan->gy_m.push_back(m);
      plan->gy_c.push_back(c);
    }
  }
  plan->gy_ptr.push_back(static_cast<int>(plan->gy_m.size()));
  f.gy_terms = static_cast<int>(plan->gy_m.size());
  f.tb_gyc = 2 * total * elem;
  f.tb_gyptr = f.tb_gyc + f.gy_terms * elem;
  f.tb_gym = f.tb_gyptr + (plan->Y + 1) * 4;
  f.tb_ellj = f.tb_gym + f.gy_terms * 2;
  f.tb_bytes = round_up(f.tb_ellj + 2 * total, 16);
  return true;
}

// Decide whether the staged kernels apply and fill plan->fast.
void analyse_fast(luna_uvu_plan* plan) {
  plan->fast_ok = false;
  const auto& paths = plan->paths;
  if (paths.empty() || paths.size() > kMaxFastPaths) return;
  const int elem = plan->dtype == LUNA_F64 ? 8 : 4;
  const int align = 16 / elem;  // elements per 16 bytes
  const int ch = paths[0].ch;
  if (ch % 32 != 0) return;
  if (plan->Y > 32) return;
  FastMeta f{};
  f.LX = f.LO = 0;
  for (int l = 0; l <= kMaxFastL; ++l) f.x_off[l] = f.o_off[l] = f.xs_off[l] = -1;
  for (const auto& p : paths) {
    if (p.ch != ch || p.w_stride != 1) return;
    const int l1 = (p.d1 - 1) / 2, l3 = (p.d3 - 1) / 2;
    if (l1 > kMaxFastL || l3 > kMaxFastL) return;
    if (f.x_off[l1] >= 0 && f.x_off[l1] != p.x_off) return;  // two x blocks of the same degree
    if (f.o_off[l3] >= 0 && f.o_off[l3] != p.out_off) return;
    f.x_off[l1] = p.x_off;
    f.o_off[l3] = p.out_off;
    f.LX = std::max(f.LX, l1);
    f.LO = std::max(f.LO, l3);
    if (p.w_off % align || p.x_off % align || p.out_off % align) return;
  }
  // a block offset must not be shared by two different degrees
  for (int a = 0; a <= kMaxFastL; ++a)
    for (int b = a + 1; b <= kMaxFastL; ++b) {
      if (f.x_off[a] >= 0 && f.x_off[a] == f.x_off[b]) return;
      if (f.o_off[a] >= 0 && f.o_off[a] == f.o_off[b]) return;
    }
  if (plan->X % align || plan->O % align || plan->W % align) return;

  int cpl;
  if (plan->dtype == LUNA_F32)
    cpl = ch % 128 == 0 ? 4 : (ch % 64 == 0 ? 2 : 1);
  else
    cpl = ch % 64 == 0 ? 2 : 1;
  if (!fill_layout(plan, f, cpl)) return;
  plan->fast = f;
  plan->fast_ok = true;
}

}  // namespace

Tuning tuning_from_environment() {
  Tuning t;
  auto number = [](const char* name) -> long long {
    const char* value = std::getenv(name);
    return value ? std::atoll(value) : 0;
  };
  t.no_canon = std::getenv("LUNA_B200_NO_CANON") != nullptr;
  t.no_sparse = std::getenv("LUNA_B200_NO_SPARSE") != nullptr;
  t.no_plain = std::getenv("LUNA_B200_NO_PLAIN") != nullptr;
  if (const char* kind = std::getenv("LUNA_B200_BWD_KERNEL"))
    t.bwd_kernel = kind[0] == 'r' ? 1 : (kind[0] == 'u' ? 2 : 0);
  t.max_warps = static_cast<int>(std::max(0ll, number("LUNA_B200_MAXW")));
  t.row_stages = static_cast<int>(std::max(0ll, number("LUNA_B200_ROW_STAGES")));
  t.edges_per_warp = std::max(0ll, number("LUNA_B200_EPW"));
  t.fwd_tile_edges = std::max(0ll, number("LUNA_B200_FWD_TILE"));
  return t;
}

int get_device_tables(luna_uvu_plan* plan, const DeviceTables** out) {
  int device = 0;
  LUNA_CUDA_CHECK(cudaGetDevice(&device));
  std::lock_guard<std::mutex> lock(plan->mutex);
  auto it = plan->device_tables.find(device);
  if (it != plan->device_tables.end()) {
    *out = &it->second;
    return LUNA_OK;
  }
  const bool f64 = plan->dtype == LUNA_F64;
  const size_t term_bytes = f64 ? sizeof(TermRec<double>) : sizeof(TermRec<float>);
  const size_t scalar = f64 ? 8 : 4;

  std::vector<unsigned char> host;
  auto append = [&](const void* data, size_t bytes) {
    size_t offset = (host.size() + 255) / 256 * 256;
    host.resize(offset + std::max<size_t>(bytes, 1));
    if (bytes) std::memcpy(host.data() + offset, data, bytes);
    return offset;
  };
  auto pack_terms = [&](const std::vector<luna_uvu_plan::HostTerm>& terms) {
    std::vector<unsigned char> raw(terms.size() * term_bytes);
    for (size_t i = 0; i < terms.size(); ++i) {
      if (f64) {
        TermRec<double> t{terms[i].a, terms[i].b, terms[i].c};
        std::memcpy(raw.data() + i * term_bytes, &t, term_bytes);
      } else {
        TermRec<float> t{terms[i].a, terms[i].b, static_cast<float>(terms[i].c)};
        std::memcpy(raw.data() + i * term_bytes, &t, term_bytes);
      }
    }
    return raw;
  };
  int zero = 0;
  const size_t o_status = append(&zero, sizeof(int));
  const std::vector<unsigned> no_counts(static_cast<size_t>(kTileCounterSets) * kTileCounterWords, 0u);
  const size_t o_counters = append(no_counts.data(), no_counts.size() * sizeof(unsigned));
  const size_t o_paths = append(plan->paths.data(), plan->paths.size() * sizeof(PathRec));
  const size_t o_os = append(plan->out_slots.data(), plan->out_slots.size() * sizeof(SlotRec));
  const size_t o_xs = append(plan->x_slots.data(), plan->x_slots.size() * sizeof(SlotRec));
  const size_t o_ys = append(plan->y_slots.data(), plan->y_slots.size() * sizeof(SlotRec));
  const size_t o_osp = append(plan->out_slot_paths.data(), plan->out_slot_paths.size() * sizeof(int));
  const size_t o_xsp = append(plan->x_slot_paths.data(), plan->x_slot_paths.size() * sizeof(int));
  const size_t o_ysp = append(plan->y_slot_paths.data(), plan->y_slot_paths.size() * sizeof(int));
  const size_t o_wep = append(plan->w_elem_path.data(), plan->w_elem_path.size() * sizeof(int));
  const size_t o_rk = append(plan->rowptr_k.data(), plan->rowptr_k.size() * sizeof(int));
  const size_t o_ri = append(plan->rowptr_i.data(), plan->rowptr_i.size() * sizeof(int));
  const size_t o_rj = append(plan->rowptr_j.data(), plan->rowptr_j.size() * sizeof(int));
  auto tk = pack_terms(plan->terms_k), ti = pack_terms(plan->terms_i), tj = pack_terms(plan->terms_j);
  const size_t o_tk = append(tk.data(), tk.size());
  const size_t o_ti = append(ti.data(), ti.size());
  const size_t o_tj = append(tj.data(), tj.size());
  const size_t o_mj = append(plan->ell_j.data(), plan->ell_j.size());
  std::vector<unsigned char> mc(plan->ell_c.size() * scalar);
  for (size_t i = 0; i < plan->ell_c.size(); ++i) {
    if (f64) {
      std::memcpy(mc.data() + i * 8, &plan->ell_c[i], 8);
    } else {
      float v = static_cast<float>(plan->ell_c[i]);
      std::memcpy(mc.data() + i * 4, &v, 4);
    }
  }
  const size_t o_mc = append(mc.data(), mc.size());
  // backward kernel's blob
  std::vector<unsigned char> blob;
  if (plan->fast_ok) {
    const FastMeta& f = plan->fast;
    blob.assign(static_cast<size_t>(f.tb_bytes), 0);
    std::memcpy(blob.data(), mc.data(), mc.size());
    for (size_t i = 0; i < plan->gy_c.size(); ++i) {
      if (f64) {
        std::memcpy(blob.data() + f.tb_gyc + i * 8, &plan->gy_c[i], 8);
      } else {
        float v = static_cast<float>(plan->gy_c[i]);
        std::memcpy(blob.data() + f.tb_gyc + i * 4, &v, 4);
      }
      const unsigned short m = static_cast<unsigned short>(plan->gy_m[i]);
      std::memcpy(blob.data() + f.tb_gym + i * 2, &m, 2);
    }
    std::memcpy(blob.data() + f.tb_gyptr, plan->gy_ptr.data(), plan->gy_ptr.size() * sizeof(int));
    std::memcpy(blob.data() + f.tb_ellj, plan->ell_j.data(), plan->ell_j.size());
  }
  const size_t o_blob = append(blob.data(), blob.size());
  std::vector<unsigned char> spc(plan->sp_c.size() * scalar);
  for (size_t i = 0; i < plan->sp_c.size(); ++i) {
    if (f64) {
      std::memcpy(spc.data() + i * 8, &plan->sp_c[i], 8);
    } else {
      float v = static_cast<float>(plan->sp_c[i]);
      std::memcpy(spc.data() + i * 4, &v, 4);
    }
  }
  const size_t o_spc = append(spc.data(), spc.size());
  const size_t o_spj = append(plan->sp_j.data(), plan->sp_j.size());

  DeviceTables dt;
  dt.bytes = host.size();
  LUNA_CUDA_CHECK(cudaMalloc(&dt.buffer, dt.bytes));
  cudaError_t err = cudaMemcpy(dt.buffer, host.data(), dt.bytes, cudaMemcpyHostToDevice);
  if (err != cudaSuccess) {
    cudaFree(dt.buffer);
    return fail(LUNA_ERR_CUDA, "table upload failed: %s", cudaGetErrorString(err));
  }
  auto* base = static_cast<unsigned char*>(dt.buffer);
  dt.status = reinterpret_cast<int*>(base + o_status);
  dt.tile_counters = reinterpret_cast<unsigned*>(base + o_counters);
  dt.paths = reinterpret_cast<const PathRec*>(base + o_paths);
  dt.out_slots = reinterpret_cast<const SlotRec*>(base + o_os);
  dt.x_slots = reinterpret_cast<const SlotRec*>(base + o_xs);
  dt.y_slots = reinterpret_cast<const SlotRec*>(base + o_ys);
  dt.out_slot_paths = reinterpret_cast<const int*>(base + o_osp);
  dt.x_slot_paths = reinterpret_cast<const int*>(base + o_xsp);
  dt.y_slot_paths = reinterpret_cast<const int*>(base + o_ysp);
  dt.w_elem_path = reinterpret_cast<const int*>(base + o_wep);
  dt.rowptr_k = reinterpret_cast<const int*>(base + o_rk);
  dt.rowptr_i = reinterpret_cast<const int*>(base + o_ri);
  dt.rowptr_j = reinterpret_cast<const int*>(base + o_rj);
  dt.terms_k = base + o_tk;
  dt.terms_i = base + o_ti;
  dt.terms_j = base + o_tj;
  dt.ell_j = base + o_mj;
  dt.ell_c = base + o_mc;
  dt.bwd_tables = base + o_blob;
  dt.sp_c = base + o_spc;
  dt.sp_j = base + o_spj;
  LUNA_CUDA_CHECK(cudaDeviceGetAttribute(&dt.sm_count, cudaDevAttrMultiProcessorCount, device));
  LUNA_CUDA_CHECK(cudaDeviceGetAttribute(&dt.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  auto inserted = plan->device_tables.emplace(device, dt);
  *out = &inserted.first->second;
  return LUNA_OK;
}

}  // namespace luna

using namespace luna;

extern "C" const char* luna_last_error(void) { return luna::g_error; }
extern "C" int luna_version(void) { return 100; }
extern "C" int luna_compiled_sm(void) { return 100; }

extern "C" int luna_uvu_plan_create(const luna_uvu_desc* desc, luna_uvu_plan** out) {
  clear_error();
  if (!desc || !out) return fail(LUNA_ERR_INVALID_ARGUMENT, "null description or output pointer");
  *out = nullptr;
  if (desc->dtype != LUNA_F32 && desc->dtype != LUNA_F64)
    return fail(LUNA_ERR_INVALID_ARGUMENT, "dtype must be LUNA_F32 or LUNA_F64");
  if (desc->num_paths <= 0 || !desc->paths) return fail(LUNA_ERR_INVALID_ARGUMENT, "No uvu instructions found.");
  if (desc->in1_dim <= 0 || desc->in2_dim <= 0 || desc->out_dim <= 0 || desc->weight_numel <= 0)
    return fail(LUNA_ERR_INVALID_ARGUMENT, "feature dimensions must be positive");
  if (desc->num_terms < 0 || (desc->num_terms > 0 && (!desc->term_i || !desc->term_j || !desc->term_k || !desc->term_c)))
    return fail(LUNA_ERR_INVALID_ARGUMENT, "term arrays missing");

  auto plan = new luna_uvu_plan();
  plan->tuning = tuning_from_environment();
  plan->dtype = desc->dtype;
  plan->X = desc->in1_dim;
  plan->Y = desc->in2_dim;
  plan->O = desc->out_dim;
  plan->W = desc->weight_numel;
  plan->w_elem_path.assign(plan->W, -1);
  std::vector<char> out_cover(plan->O, 0);

  for (int p = 0; p < desc->num_paths; ++p) {
    const luna_uvu_path& in = desc->paths[p];
    PathRec rec{};
    rec.x_off = in.x_offset;
    rec.y_off = in.y_offset;
    rec.out_off = in.out_offset;
    rec.w_off = in.weight_offset;
    rec.w_stride = in.weight_stride <= 0 ? 1 : in.weight_stride;
    rec.ch = in.channels;
    rec.d1 = 2 * in.l1 + 1;
    rec.d2 = 2 * in.l2 + 1;
    rec.d3 = 2 * in.l3 + 1;
    bool ok = in.l1 >= 0 && in.l2 >= 0 && in.l3 >= 0 && rec.ch > 0 && rec.x_off >= 0 && rec.y_off >= 0 &&
              rec.out_off >= 0 && rec.w_off >= 0 &&
              static_cast<int64_t>(rec.x_off) + static_cast<int64_t>(rec.ch) * rec.d1 <= plan->X &&
              rec.y_off + rec.d2 <= plan->Y &&
              static_cast<int64_t>(rec.out_off) + static_cast<int64_t>(rec.ch) * rec.d3 <= plan->O &&
              static_cast<int64_t>(rec.w_off) + static_cast<int64_t>(rec.ch - 1) * rec.w_stride < plan->W &&
              in.term_begin >= 0 && in.term_end >= in.term_begin && in.term_end <= desc->num_terms;
    if (!ok) {
      delete plan;
      return fail(LUNA_ERR_INVALID_ARGUMENT, "path %d: instruction extent is outside its tensor dimension", p);
    }
    // terms, three orderings
    std::vector<std::array<int, 3>> idx;
    std::vector<double> coef;
    for (int t = in.term_begin; t < in.term_end; ++t) {
      const int i = desc->term_i[t], j = desc->term_j[t], k = desc->term_k[t];
      if (i < 0 || i >= rec.d1 || j < 0 || j >= rec.d2 || k < 0 || k >= rec.d3) {
        delete plan;
        return fail(LUNA_ERR_INVALID_ARGUMENT, "path %d: coupling term index out of range", p);
      }
      idx.push_back({i, j, k});
      coef.push_back(desc->term_c[t]);
    }
    auto emit = [&](int axis, int dim, std::vector<int>& rowptr, std::vector<luna_uvu_plan::HostTerm>& terms) {
      const int start = static_cast<int>(rowptr.size());
      for (int v = 0; v < dim; ++v) {
        rowptr.push_back(static_cast<int>(terms.size()));
        for (size_t t = 0; t < idx.size(); ++t)
          if (idx[t][axis] == v) {
            const int a = axis == 0 ? idx[t][1] : idx[t][0];
            const int b = axis == 2 ? idx[t][1] : idx[t][2];
            terms.push_back({a, b, coef[t]});
          }
      }
      rowptr.push_back(static_cast<int>(terms.size()));
      return start;
    };
    rec.byk_ptr = emit(2, rec.d3, plan->rowptr_k, plan->terms_k);  // (a, b) = (i, j)
    rec.byi_ptr = emit(0, rec.d1, plan->rowptr_i, plan->terms_i);  // (a, b) = (j, k)
    rec.byj_ptr = emit(1, rec.d2, plan->rowptr_j, plan->terms_j);  // (a, b) = (i, k)
    for (int u = 0; u < rec.ch; ++u) {
      int& owner = plan->w_elem_path[rec.w_off + u * rec.w_stride];
      if (owner != -1) {
        delete plan;
        return fail(LUNA_ERR_INVALID_ARGUMENT, "path %d: weight column claimed by two paths", p);
      }
      owner = p;
    }
    for (int c = 0; c < rec.ch * rec.d3; ++c) out_cover[rec.out_off + c] = 1;
    plan->paths.push_back(rec);
  }
  // slots; every path sharing a block offset must agree on the block shape
  build_slots(plan->paths, [](const PathRec& p) { return SlotRec{p.out_off, p.ch, p.d3, 0, 0}; }, plan->out_slots,
              plan->out_slot_paths);
  build_slots(plan->paths, [](const PathRec& p) { return SlotRec{p.x_off, p.ch, p.d1, 0, 0}; }, plan->x_slots,
              plan->x_slot_paths);
  build_slots(plan->paths, [](const PathRec& p) { return SlotRec{p.y_off, 1, p.d2, 0, 0}; }, plan->y_slots,
              plan->y_slot_paths);
  auto consistent = [&](const std::vector<SlotRec>& slots, const std::vector<int>& lists, auto shape) {
    for (size_t s = 0; s < slots.size(); ++s) {
      for (int q = slots[s].path_begin; q < slots[s].path_end; ++q) {
        auto [ch, d] = shape(plan->paths[lists[q]]);
        if (ch != slots[s].ch || d != slots[s].d) return false;
      }
      if (s + 1 < slots.size() && slots[s].off + slots[s].ch * slots[s].d > slots[s + 1].off) return false;
    }
    return true;
  };
  if (!consistent(plan->out_slots, plan->out_slot_paths, [](const PathRec& p) { return std::pair<int, int>{p.ch, p.d3}; }) ||
      !consistent(plan->x_slots, plan->x_slot_paths, [](const PathRec& p) { return std::pair<int, int>{p.ch, p.d1}; }) ||
      !consistent(plan->y_slots, plan->y_slot_paths, [](const PathRec& p) { return std::pair<int, int>{1, p.d2}; })) {
    delete plan;
    return fail(LUNA_ERR_UNSUPPORTED, "paths that share a feature block disagree on its shape or blocks overlap");
  }
  plan->out_fully_covered = std::all_of(out_cover.begin(), out_cover.end(), [](char c) { return c != 0; });
  analyse_fast(plan);
  *out = plan;
  return LUNA_OK;
}

extern "C" void luna_uvu_plan_destroy(luna_uvu_plan* plan) {
  if (!plan) return;
  int current = 0;
  cudaGetDevice(&current);
  for (auto& [device, dt] : plan->device_tables) {
    if (dt.buffer) {
      cudaSetDevice(device);
      cudaFree(dt.buffer);
    }
  }
  cudaSetDevice(current);
  delete plan;
}

extern "C" int luna_uvu_plan_set_generic(luna_uvu_plan* plan, int force_generic) {
  if (!plan) return fail(LUNA_ERR_INVALID_ARGUMENT, "null plan");
  plan->force_generic = force_generic != 0;
  return LUNA_OK;
}
