// Building blocks of the staged kernels: mbarrier / bulk-copy wrappers (1-D TMA copies into this CTA's own shared
// memory), small vector types, compile-time loops, the warp-wide lower-bound search that assigns contiguous node
// ranges to warps, and the per-edge coupling-matrix computation.
//
// Formulation shared by all staged kernels.  For one edge e the edge attributes y[e] are the same for every
// channel, so each path p is first reduced to a small dense matrix
//     M^p[i][k] = sum_j C^p_ijk * y[e, j]                     (d1 x d3, computed once per edge by the warp)
// and the per-channel work becomes dense:
//     forward   out_k  += w_p * sum_i M^p[i][k] * x_i
//     backward  gx_i   += sum_k M^p[i][k] * (w_p * g_k),   gw_p = sum_k g_k * sum_i M^p[i][k] x_i,
//               G^p[i][k] = sum_channels x_i * (w_p * g_k)  and  gy_j = sum_p sum_ik C^p_ijk G^p[i][k].
// The sparse coupling table is only touched in the per-edge (not per-channel) part, so the hot loops depend on the
// degrees (d1, d3) alone and one compiled kernel serves every path list of a given shape class.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <type_traits>

#include "cg_patterns.h"
#include "plan.h"

namespace luna {
namespace fastk {

constexpr int kWarps = 4;           // default warps per CTA; each warp streams its own edge range
constexpr int kMaxWarps = 16;       // upper bound on warps per CTA
constexpr int kFwdMaxWarps = 8;     // forward kernel: its launch bounds leave it 255 registers
constexpr int kMaxStages = 4;
constexpr uint32_t kWaitLimit = 1u << 20;   // bounded mbarrier polling: tries per wait

// ---- shared-memory barriers and bulk copies -------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Polls with an iteration limit; returns false if the barrier never completed.  (A suspend-time hint on try_wait
// was measured to delay the wake-up by the full hint, so none is given.)
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
#pragma unroll 1
  for (uint32_t spin = 0; spin < kWaitLimit; ++spin)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted in bytes on an mbarrier.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// L2 eviction priorities for bulk copies: streamed-once rows (per-edge weights, their gradients) should leave L2
// first so that the gathered node rows, which neighbouring edges read again, stay.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void bulk_copy_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar,
                                                   uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
// 1-D bulk copy from this CTA's shared memory to global memory, tracked by the issuing thread's bulk-copy groups.
__device__ __forceinline__ void bulk_copy_s2g_hint(void* dst, const void* src, uint32_t bytes, uint64_t policy) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;" ::"l"(dst),
               "r"(smem_u32(src)), "r"(bytes), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the issuing thread's bulk stores have finished reading their shared-memory sources.
__device__ __forceinline__ void bulk_wait_group_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Makes this thread's earlier shared-memory writes visible to bulk copies issued afterwards.
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- small vectors ------------------------------------------------------------------------------------------------
template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
  T a[N];
};

// Loads NV vectors of CPL elements from p (aligned to the vector size) into flat[NV * CPL].
template <typename T, int CPL, int NV>
__device__ __forceinline__ void load_vectors(const T* p, T* flat) {
  const Vec<T, CPL>* v = reinterpret_cast<const Vec<T, CPL>*>(p);
#pragma unroll
  for (int n = 0; n < NV; ++n) {
    const Vec<T, CPL> t = v[n];
#pragma unroll
    for (int c = 0; c < CPL; ++c) flat[n * CPL + c] = t.a[c];
  }
}
template <typename T, int CPL, int NV>
__device__ __forceinline__ void store_vectors(T* p, const T* flat) {
  Vec<T, CPL>* v = reinterpret_cast<Vec<T, CPL>*>(p);
#pragma unroll
  for (int n = 0; n < NV; ++n) {
    Vec<T, CPL> t;
#pragma unroll
    for (int c = 0; c < CPL; ++c) t.a[c] = flat[n * CPL + c];
    v[n] = t;
  }
}
// Streaming (evict-first) variant for write-once outputs such as gw.
template <typename T, int CPL, int NV>
__device__ __forceinline__ void store_vectors_streaming(T* p, const T* flat) {
  Vec<T, CPL>* v = reinterpret_cast<Vec<T, CPL>*>(p);
#pragma unroll
  for (int n = 0; n < NV; ++n) {
    Vec<T, CPL> t;
#pragma unroll
    for (int c = 0; c < CPL; ++c) t.a[c] = flat[n * CPL + c];
    if constexpr (sizeof(T) * CPL == 16) {
      __stcs(reinterpret_cast<float4*>(v + n), *reinterpret_cast<const float4*>(&t));
    } else if constexpr (sizeof(T) * CPL == 8) {
      __stcs(reinterpret_cast<float2*>(v + n), *reinterpret_cast<const float2*>(&t));
    } else {
      __stcs(reinterpret_cast<float*>(v + n), *reinterpret_cast<const float*>(&t));
    }
  }
}

// Reads a d1 x d3 matrix (row-major, 16-byte aligned, padded to a multiple of 16 bytes) from shared memory with
// 128-bit loads; every lane reads the same address, so each load is one broadcast.
template <typename T, int COUNT>
__device__ __forceinline__ void load_matrix(const T* m, T* regs) {
  constexpr int per = 16 / sizeof(T);
  constexpr int nv = (COUNT + per - 1) / per;
  const Vec<T, per>* v = reinterpret_cast<const Vec<T, per>*>(m);
#pragma unroll
  for (int n = 0; n < nv; ++n) {
    const Vec<T, per> t = v[n];
#pragma unroll
    for (int c = 0; c < per; ++c)
      if (n * per + c < COUNT) regs[n * per + c] = t.a[c];
  }
}

// ---- compile-time loop ----------------------------------------------------------------------------------------------
template <int I, int N, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, N>(f);
  }
}

// ---- work assignment ------------------------------------------------------------------------------------------------
// First n in [0, count] with rowptr[n] >= bound (rowptr is ascending); all 32 lanes cooperate, 32-ary search.
__device__ __forceinline__ int64_t warp_lower_bound(const int* __restrict__ rowptr, int64_t count, int64_t bound,
                                                    int lane) {
  int64_t lo = 0, hi = count;
  while (hi - lo > 32) {
    const int64_t step = (hi - lo + 31) / 32;
    const int64_t idx = lo + step * lane;
    const bool below = idx < hi && rowptr[idx] < bound;
    const int cnt = __popc(__ballot_sync(0xffffffffu, below));
    if (cnt == 0) {
      hi = lo;
    } else {
      const int64_t new_hi = lo + step * cnt;
      lo = lo + step * (cnt - 1) + 1;
      hi = new_hi < hi ? new_hi : hi;
    }
  }
  const int64_t idx = lo + lane;
  const bool below = idx < hi && rowptr[idx] < bound;
  return lo + __popc(__ballot_sync(0xffffffffu, below));
}

// The same answer as warp_lower_bound(rowptr, count, bound, lane) when it is known to be at or after `from` and is
// expected within 32 entries of it (one coalesced load); falls back to the search otherwise.
__device__ __forceinline__ int64_t warp_lower_bound_near(const int* __restrict__ rowptr, int64_t count, int64_t bound,
                                                         int64_t from, int lane) {
  const int64_t idx = from + lane;
  const bool below = idx < count && rowptr[idx] < bound;
  const unsigned mask = __ballot_sync(0xffffffffu, below);
  if (mask != 0xffffffffu) return from + __popc(mask);  // rowptr is ascending: the lanes below form a prefix
  return warp_lower_bound(rowptr, count, bound, lane);
}

// The same answer again, from a guess of where it lies: one coalesced load of the 32 entries around the guess settles
// it when the answer is among them (the first of them below the bound, not all of them), the search otherwise.
__device__ __forceinline__ int64_t warp_lower_bound_guess(const int* __restrict__ rowptr, int64_t count, int64_t bound,
                                                          int64_t guess, int lane) {
  int64_t base = guess - 16;
  if (base > count - 16) base = count - 16;
  if (base < 0) base = 0;
  const int64_t idx = base + lane;
  const bool below = idx < count && rowptr[idx] < bound;
  const unsigned mask = __ballot_sync(0xffffffffu, below);
  if ((base == 0 || (mask & 1u)) && mask != 0xffffffffu) return base + __popc(mask);
  return warp_lower_bound(rowptr, count, bound, lane);
}

// How a staged kernel is made resident: ring depth per warp, warps per CTA, CTAs per SM, dynamic shared memory.
struct Residency {
  int depth = 0;  // stages / slots per warp, 0 if nothing fits
  int warps = 0;
  int ctas = 0;
  size_t block_bytes = 0;
};
// Picks the configuration with the most resident warps.  Registers are counted per SM sub-partition: a CTA's warps
// are dealt round-robin to the four sub-partitions, each of which holds 16384 registers, so a CTA of w warps takes
// ceil(w / 4) warp slots on the fullest one.  Ties go to the deeper ring (within [min_depth, max_depth]), then to
// fewer CTAs.
Residency choose_residency(size_t ring_bytes, size_t fixed_bytes, size_t shared_bytes, int max_smem_optin,
                           int regs_per_thread, int max_warps, int min_depth, int max_depth);
// CTAs to launch: about `target` edges per warp, rounded up to whole waves of resident CTAs.
int64_t grid_blocks(int64_t num_edges, int64_t target, const Residency& r, int sm_count);

// Target edges per warp when sizing the grid: the plan's override if it has one.
#ifdef __CUDACC__
// Dynamic hand-out of tiles to warps.  counters[0] counts tiles taken beyond every warp's first one, counters[1] the
// warps that are done; the last warp out clears both for the next launch that gets this set.
__device__ __forceinline__ int64_t take_tile(unsigned* counters, int64_t total_warps, int lane) {
  unsigned ticket = 0;
  if (lane == 0) ticket = atomicAdd(&counters[0], 1u);
  ticket = __shfl_sync(0xffffffffu, ticket, 0);
  return total_warps + static_cast<int64_t>(ticket);
}
__device__ __forceinline__ void leave_tiles(unsigned* counters, int64_t total_warps, int lane) {
  if (lane == 0) {
    const unsigned done = atomicAdd(&counters[1], 1u);
    if (static_cast<int64_t>(done) + 1 == total_warps) {  // every other warp has taken its last ticket
      counters[0] = 0u;
      counters[1] = 0u;
      __threadfence();
    }
  }
}
#endif

// Edges per tile for the kernels that hand out tiles dynamically: `wanted` (64 unless overridden), but small enough
// that every resident warp gets about eight tiles, so that a small launch (a piece of a shard, a small graph) does
// not end with most warps idle while a few finish their last tile; never below 16 edges.
inline int64_t tile_edges_for(int64_t num_edges, int64_t resident_warps, int64_t wanted) {
  const int64_t spread = num_edges / std::max<int64_t>(8 * resident_warps, 1);
  return std::max<int64_t>(1, std::min<int64_t>(wanted, std::max<int64_t>(16, spread)));
}

inline int64_t edges_per_warp(const Tuning& tuning, int64_t fallback) {
  return tuning.edges_per_warp > 0 ? tuning.edges_per_warp : fallback;
}
// A kernel's warp limit under the plan's cap.
inline int capped_warps(const Tuning& tuning, int max_warps) {
  return tuning.max_warps > 0 ? std::max(1, std::min(max_warps, tuning.max_warps)) : max_warps;
}

// ---- canonical path lists ---------------------------------------------------------------------------------------
// Most models couple every degree of x with every degree of the edge harmonics into every degree of the output:
// all (l1, l2, l3) with l1 <= LX, l2 <= L2, l3 <= LO that satisfy the triangle rule and have an even degree sum,
// listed in (l1, l2, l3) order, which is also the order of their weight blocks.  For such a list everything the
// inner loops need (which paths exist, where a path's weights sit in a stage, where its coupling matrix sits in
// the per-edge buffer) is known at compile time, so the loops over paths unroll completely and the compiler can
// move shared-memory loads ahead of the arithmetic of the previous path.  These functions define the list; the
// plan checks a configuration against them (FastMeta::canon_l2) and the kernels use them as constants.
__host__ __device__ constexpr bool canon_ok(int LX, int L2, int LO, int l1, int l2, int l3) {
  const int lo = l1 > l2 ? l1 - l2 : l2 - l1;
  return l1 <= LX && l2 <= L2 && l3 <= LO && l3 >= lo && l3 <= l1 + l2 && ((l1 + l2 + l3) % 2 == 0);
}
// position of the path's weight block among the weight blocks
__host__ __device__ constexpr int canon_wrank(int LX, int L2, int LO, int a, int b, int c) {
  int r = 0;
  for (int l1 = 0; l1 <= LX; ++l1)
    for (int l2 = 0; l2 <= L2; ++l2)
      for (int l3 = 0; l3 <= LO; ++l3) {
        if (l1 == a && l2 == b && l3 == c) return r;
        if (canon_ok(LX, L2, LO, l1, l2, l3)) ++r;
      }
  return r;  // (a, b, c) past the end: the number of paths
}
// first entry of the path's coupling matrix in the per-edge buffer: matrices in (l3, l1, l2) order, rows of
// d3 + 1 entries, every matrix padded to a multiple of four entries; past-the-end arguments give the total
__host__ __device__ constexpr int canon_moff(int LX, int L2, int LO, int a, int b, int c) {
  int m = 0;
  for (int l3 = 0; l3 <= LO; ++l3)
    for (int l1 = 0; l1 <= LX; ++l1)
      for (int l2 = 0; l2 <= L2; ++l2) {
        if (!canon_ok(LX, L2, LO, l1, l2, l3)) continue;
        if (l1 == a && l2 == b && l3 == c) return m;
        m += (2 * l1 + 1) * (2 * l3 + 2);
        while (m % 4) ++m;
      }
  return m;
}

// number of canonical paths into degree c that come before (a, b) in (l1, l2) order; past-the-end arguments give
// the number of paths into that degree
__host__ __device__ constexpr int canon_unit_index(int LX, int L2, int LO, int a, int b, int c) {
  int r = 0;
  for (int l1 = 0; l1 <= LX; ++l1)
    for (int l2 = 0; l2 <= L2; ++l2) {
      if (l1 == a && l2 == b) return r;
      if (canon_ok(LX, L2, LO, l1, l2, c)) ++r;
    }
  return r;
}

// first coupling term of the path in the sparse term list: paths in (l3, l1, l2) order, every path's terms (in the
// (i, k, j) order of CgPattern) padded to a multiple of four; past-the-end arguments give the total
__host__ __device__ constexpr int canon_toff(int LX, int L2, int LO, int a, int b, int c) {
  int t = 0;
  for (int l3 = 0; l3 <= LO; ++l3)
    for (int l1 = 0; l1 <= LX; ++l1)
      for (int l2 = 0; l2 <= L2; ++l2) {
        if (!canon_ok(LX, L2, LO, l1, l2, l3)) continue;
        if (l1 == a && l2 == b && l3 == c) return t;
        t += (cg_count(l1, l2, l3) + 3) / 4 * 4;
      }
  return t;
}

// ---- per-edge coupling matrices -------------------------------------------------------------------------------------
// The program that turns an edge's y row into the M matrices lives in shared memory in padded form: term t of
// entry m is (ell_c[t * m_total + m], ell_j[t * m_total + m]); padding terms have coefficient 0.
template <typename T>
__host__ __device__ inline size_t ell_bytes(int m_total, int m_terms) {
  const size_t count = static_cast<size_t>(m_total) * m_terms;
  return count * sizeof(T) + (count + 15) / 16 * 16;
}

// Copies the program from global to the start of the CTA's dynamic shared memory; all threads of the block call it.
template <typename T>
__device__ __forceinline__ void load_ell(unsigned char* smem, const T* __restrict__ gc,
                                         const unsigned char* __restrict__ gj, int m_total, int m_terms,
                                         const T** ell_c, const unsigned char** ell_j) {
  const int count = m_total * m_terms;
  T* c = reinterpret_cast<T*>(smem);
  unsigned char* j = smem + static_cast<size_t>(count) * sizeof(T);
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    c[i] = gc[i];
    j[i] = gj[i];
  }
  *ell_c = c;
  *ell_j = j;
  __syncthreads();
}

// mbuf[m] = sum_t c[t][m] * ybuf[j[t][m]]; lanes stride over the entries, conflict-free shared loads.
template <typename T>
__device__ __forceinline__ void compute_m(const T* ell_c, const unsigned char* ell_j, int m_terms, const T* ybuf,
                                          T* mbuf, int m_total, int lane) {
#pragma unroll 2
  for (int m = lane; m < m_total; m += 32) {
    T a = ell_c[m] * ybuf[ell_j[m]];
    for (int t = 1; t < m_terms; ++t) a = fma(ell_c[t * m_total + m], ybuf[ell_j[t * m_total + m]], a);
    mbuf[m] = a;
  }
}

// FP32 with an even number of channels per lane uses packed two-wide arithmetic; everything else the scalar path.
template <typename T, int CPL>
struct UsePairs {
  static constexpr bool value = sizeof(T) == 4 && (CPL % 2 == 0);
};
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }

// One warp's share of the coupling-matrix computation when `parts` warps split the entries: warp `part` handles
// entries (r * parts + part) * 32 + lane.  Two entries per trip with all loads issued before the arithmetic;
// indices are clamped so the loads are unconditional and only the stores are predicated.  Requires exactly two
// (zero-padded) terms per entry.  With DUP every entry is stored twice, (m, m), ready for packed arithmetic.
template <typename T, bool DUP>
__device__ __forceinline__ void compute_m_share(const T* ell_c, const unsigned char* ell_j, const T* ybuf, T* mbuf,
                                                int m_total, int part, int parts, int lane) {
  const int stride = 32 * parts;
#pragma unroll 1
  for (int m0 = part * 32 + lane; m0 < m_total; m0 += 2 * stride) {
    const int m1 = m0 + stride;
    const int i1 = m1 < m_total ? m1 : m0;
    const unsigned ja0 = ell_j[m0], jb0 = ell_j[m_total + m0], ja1 = ell_j[i1], jb1 = ell_j[m_total + i1];
    const T ca0 = ell_c[m0], cb0 = ell_c[m_total + m0], ca1 = ell_c[i1], cb1 = ell_c[m_total + i1];
    const T r0 = fma(cb0, ybuf[jb0], ca0 * ybuf[ja0]);
    const T r1 = fma(cb1, ybuf[jb1], ca1 * ybuf[ja1]);
    if constexpr (DUP) {
      Vec<T, 2> v0{{r0, r0}}, v1{{r1, r1}};
      reinterpret_cast<Vec<T, 2>*>(mbuf)[m0] = v0;
      if (m1 < m_total) reinterpret_cast<Vec<T, 2>*>(mbuf)[m1] = v1;
    } else {
      mbuf[m0] = r0;
      if (m1 < m_total) mbuf[m1] = r1;
    }
  }
}

}  // namespace fastk
}  // namespace luna
