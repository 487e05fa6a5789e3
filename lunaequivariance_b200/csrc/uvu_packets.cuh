// Arithmetic packets shared by the staged kernels: a lane's channels as scalars or as packed FP32 pairs.
#pragma once

#include "uvu_fast.cuh"

namespace luna {
namespace fastk {

// ---- arithmetic packets ---------------------------------------------------------------------------------------------
// A lane's CPL channels are processed as NP packets of W channels: FP32 pairs with packed two-wide FMAs when CPL is
// even, scalars otherwise.  Coupling-matrix entries are stored W times in shared memory so that one load fills a
// packet.  A pair lives in one 64-bit register from the load to the last use (the packed instructions take 64-bit
// operands; keeping the halves as separate floats costs a register move per operand).
struct Pair {
  unsigned long long v;
};
template <typename T, int CPL, bool PACKED>
struct PkT {
  using V = T;
  static constexpr int W = 1, NP = CPL;
};
template <>
struct PkT<float, 2, true> {
  using V = Pair;
  static constexpr int W = 2, NP = 1;
};
template <>
struct PkT<float, 4, true> {
  using V = Pair;
  static constexpr int W = 2, NP = 2;
};
__device__ __forceinline__ Pair vfma(Pair a, Pair b, Pair c) {
  Pair d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d.v) : "l"(a.v), "l"(b.v), "l"(c.v));
  return d;
}
__device__ __forceinline__ Pair vmul(Pair a, Pair b) {
  Pair d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d.v) : "l"(a.v), "l"(b.v));
  return d;
}
__device__ __forceinline__ Pair vadd(Pair a, Pair b) {
  Pair d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d.v) : "l"(a.v), "l"(b.v));
  return d;
}
__device__ __forceinline__ Pair make_packet(const float* vals, Pair) {
  Pair d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d.v) : "f"(vals[0]), "f"(vals[1]));
  return d;
}
__device__ __forceinline__ void split_packet(Pair a, float* vals) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(vals[0]), "=f"(vals[1]) : "l"(a.v));
}
__device__ __forceinline__ float hsum(Pair a) {
  float v[2];
  split_packet(a, v);
  return v[0] + v[1];
}
__device__ __forceinline__ float vfma(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ double vfma(double a, double b, double c) { return fma(a, b, c); }
__device__ __forceinline__ float vmul(float a, float b) { return a * b; }
__device__ __forceinline__ double vmul(double a, double b) { return a * b; }
__device__ __forceinline__ float vadd(float a, float b) { return a + b; }
__device__ __forceinline__ double vadd(double a, double b) { return a + b; }
__device__ __forceinline__ float hsum(float a) { return a; }
__device__ __forceinline__ double hsum(double a) { return a; }
__device__ __forceinline__ float make_packet(const float* vals, float) { return vals[0]; }
__device__ __forceinline__ double make_packet(const double* vals, double) { return vals[0]; }
__device__ __forceinline__ void split_packet(float a, float* vals) { vals[0] = a; }
__device__ __forceinline__ void split_packet(double a, double* vals) { vals[0] = a; }
template <typename V>
__device__ __forceinline__ V zero_packet() {
  if constexpr (sizeof(V) == sizeof(Pair) && !std::is_floating_point<V>::value) {
    return V{0ull};
  } else {
    return V(0);
  }
}

// Memory row [channel][component] (CPL x D, this lane's channels) -> packets [component][packet].
template <typename PK, typename T, int CPL, int D>
__device__ __forceinline__ void load_packets(const T* p, typename PK::V* out) {
  using V = typename PK::V;
  constexpr int W = PK::W, NP = PK::NP;
  T row[CPL * D];
  load_vectors<T, CPL, D>(p, row);
#pragma unroll
  for (int i = 0; i < D; ++i)
#pragma unroll
    for (int q = 0; q < NP; ++q) {
      T vals[W];
#pragma unroll
      for (int c = 0; c < W; ++c) vals[c] = row[(q * W + c) * D + i];
      out[i * NP + q] = make_packet(vals, V{});
    }
}
template <typename PK, typename T, int CPL, int D>
__device__ __forceinline__ void unpack_packets(const typename PK::V* in, T* row) {
  constexpr int W = PK::W, NP = PK::NP;
#pragma unroll
  for (int i = 0; i < D; ++i)
#pragma unroll
    for (int q = 0; q < NP; ++q) {
      T vals[W];
      split_packet(in[i * NP + q], vals);
#pragma unroll
      for (int c = 0; c < W; ++c) row[(q * W + c) * D + i] = vals[c];
    }
}

// The lane's CPL consecutive channels of one component (already adjacent in memory) as packets.
template <typename PK, typename T, int CPL>
__device__ __forceinline__ void load_lane_packets(const T* p, typename PK::V* out) {
  if constexpr (PK::W == 2) {
    if constexpr (CPL == 4) {
      const ulonglong2 t = *reinterpret_cast<const ulonglong2*>(p);
      out[0].v = t.x;
      out[1].v = t.y;
    } else {
      out[0].v = *reinterpret_cast<const unsigned long long*>(p);
    }
  } else {
    load_vectors<T, CPL, 1>(p, out);
  }
}

// One row of a coupling matrix (D3P entries, each stored W times) from shared memory; every lane reads the same
// address, so each load is one broadcast.  Rows start on 16-byte boundaries except in FP32 without duplication (8).
template <typename T, int W, int D3P, typename V>
__device__ __forceinline__ void load_matrix_row(const T* p, V* row) {
  if constexpr (W == 2) {  // two packets per 128-bit load
    static_assert(D3P % 2 == 0, "row length must be even");
    const ulonglong2* v = reinterpret_cast<const ulonglong2*>(p);
#pragma unroll
    for (int n = 0; n < D3P / 2; ++n) {
      const ulonglong2 t = v[n];
      row[2 * n].v = t.x;
      row[2 * n + 1].v = t.y;
    }
  } else {
    constexpr int per = (sizeof(T) == 4 ? 8 : 16) / sizeof(T);
    static_assert(D3P % per == 0, "row length must be a whole number of vectors");
    const Vec<T, per>* v = reinterpret_cast<const Vec<T, per>*>(p);
#pragma unroll
    for (int n = 0; n < D3P / per; ++n) {
      const Vec<T, per> t = v[n];
#pragma unroll
      for (int c = 0; c < per; ++c) row[n * per + c] = t.a[c];
    }
  }
}


// ---- helpers of the kernels that keep the coupling matrices unduplicated -----------------------------------------
// A scalar as a packet with both halves equal.  The assembler folds this move into the broadcast operand form of
// the packed instruction, so an unduplicated matrix costs no extra instructions and half the shared-memory loads.
__device__ __forceinline__ Pair bcast_packet(float m, Pair) {
  Pair d;
  asm("mov.b64 %0, {%1, %1};" : "=l"(d.v) : "f"(m));
  return d;
}
__device__ __forceinline__ float bcast_packet(float m, float) { return m; }
__device__ __forceinline__ double bcast_packet(double m, double) { return m; }

// Memory row [channel][component] (CPL x D, this lane's channels) -> packets [component][packet], read with scalar
// loads: the two halves of a pair then land directly in the pair's registers.  (Vector loads followed by a pack
// make the assembler re-pack the pair at every use.)
template <typename PK, typename T, int CPL, int D>
__device__ __forceinline__ void load_packets_scalar(const T* p, typename PK::V* out) {
  using V = typename PK::V;
  constexpr int W = PK::W, NP = PK::NP;
#pragma unroll
  for (int i = 0; i < D; ++i)
#pragma unroll
    for (int q = 0; q < NP; ++q) {
      T vals[W];
#pragma unroll
      for (int c = 0; c < W; ++c) vals[c] = p[(q * W + c) * D + i];
      out[i * NP + q] = make_packet(vals, V{});
    }
}

// Row ROW of a coupling matrix stored once (D3P entries per row, D3P even, matrix start 16-byte aligned): 128-bit
// loads where the position is 16-byte aligned, 64-bit loads elsewhere.  Every lane reads the same address.
template <typename T, int D3P, int ROW>
__device__ __forceinline__ void load_plain_row(const T* matrix, T* row) {
  constexpr int per = 16 / static_cast<int>(sizeof(T));  // elements per 128 bits
  const T* p = matrix + ROW * D3P;
  static_for<0, D3P / 2>([&](auto uc) {
    constexpr int u = decltype(uc)::value;  // 2-element unit
    constexpr int pos = 2 * u;
    constexpr bool aligned = (ROW * D3P + pos) % per == 0;
    if constexpr (per == 2) {
      const Vec<T, 2> t = *reinterpret_cast<const Vec<T, 2>*>(p + pos);
      row[pos] = t.a[0];
      row[pos + 1] = t.a[1];
    } else {
      // FP32: an aligned unit that is followed by another one loads both with one 128-bit load
      constexpr bool covered = u > 0 && (ROW * D3P + pos - 2) % per == 0;  // the previous unit was such a unit
      if constexpr (covered) {
        // loaded by the previous unit's 128-bit load
      } else if constexpr (aligned && pos + 4 <= D3P) {
        const Vec<T, 4> t = *reinterpret_cast<const Vec<T, 4>*>(p + pos);
#pragma unroll
        for (int c = 0; c < 4; ++c) row[pos + c] = t.a[c];
      } else {
        const Vec<T, 2> t = *reinterpret_cast<const Vec<T, 2>*>(p + pos);
        row[pos] = t.a[0];
        row[pos + 1] = t.a[1];
      }
    }
  });
}

// A pair that was only assembled from two scalars (mov.b64 {lo, hi}) is not a value of its own for the assembler:
// under register pressure it keeps the halves apart and re-assembles the pair in front of every packed instruction
// that uses it, which costs more moves than arithmetic.  A pair that has gone through one arithmetic instruction
// stays in one 64-bit register.  settle_packets multiplies freshly assembled pairs by a 1.0 the compiler cannot see
// through (derived from a kernel parameter that always holds 2); for scalar packets it does nothing.
template <typename V, typename T>
__device__ __forceinline__ V runtime_one(int two) {
  return bcast_packet(static_cast<T>(two) * T(0.5), V{});
}
template <int N>
__device__ __forceinline__ void settle_packets(Pair* v, Pair one) {
#pragma unroll
  for (int a = 0; a < N; ++a) v[a] = vmul(v[a], one);
}
template <int N, typename S>
__device__ __forceinline__ void settle_packets(S*, S) {}
}  // namespace fastk
}  // namespace luna
