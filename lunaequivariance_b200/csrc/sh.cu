// Real spherical harmonics (e3nn convention, "component" normalised recurrence) with first and second
// derivatives.  One item per thread; the Cartesian recurrence
//   Y_{l,0}    = sqrt((2l+1)/(2l)) (Y_{l-1,0} z + Y_{l-1,2l-2} x)
//   Y_{l,2l}   = sqrt((2l+1)/(2l)) (Y_{l-1,2l-2} z - Y_{l-1,0} x)
//   Y_{l,1}    = sqrt(2l+1) y Y_{l-1,0},   Y_{l,2l-1} = sqrt(2l+1) y Y_{l-1,2l-2}
//   Y_{l,m}    = a(l,m) y Y_{l-1,m-1} - b(l,m) r^2 Y_{l-2,m-2}          (2 <= m <= 2l-2)
// is evaluated on a number type: plain scalars for the values, value+gradient numbers for the first derivative,
// and a directional tangent of value+gradient numbers for the second-order outputs.  Normalisation of the input
// vector (division by max(|v|, 1e-12)) is part of the differentiated chain.  Rows of g / out are staged through
// shared memory so that global traffic is coalesced.
//
// Two evaluators.  The common request - every degree 0..lmax once, lmax <= 6 - runs kernels unrolled for that lmax:
// the recurrence keeps two levels in registers (level l is written over level l-2, highest component first), its
// coefficients are immediates, and the output width is a compile-time constant, so the staging loops have no
// divisions.  Any other degree list (gaps, repeats, lmax up to 12) runs the same recurrence as a run-time loop over
// three rotating level buffers, which the compiler keeps in local memory.
#include <algorithm>
#include <type_traits>

#include "common.h"

namespace luna {
namespace {

constexpr int kBlock = 128;
constexpr int kMaxRepeat = 4;
constexpr int kMaxDegree = 12;

struct ShParams {
  int count[kMaxDegree + 1];              // how many times degree l appears in the output
  int column[kMaxDegree + 1][kMaxRepeat];  // first output column of each appearance
  int C;                                   // output width
  int normalize;
  int normalization;  // 0 component, 1 norm, 2 integral
  int lmax;
};

constexpr double csqrt(double x) {
  double r = x > 1.0 ? x : 1.0;
  for (int i = 0; i < 200; ++i) r = 0.5 * (r + x / r);
  return r;
}
constexpr double coef_edge(int l) { return csqrt((2.0 * l + 1.0) / (2.0 * l)); }
constexpr double coef_diag(int l) { return csqrt(2.0 * l + 1.0); }
constexpr double coef_a(int l, int m) {
  const double mu = m - l;
  return csqrt((2.0 * l + 1.0) * (2.0 * l - 1.0) / (l * l - mu * mu));
}
constexpr double coef_b(int l, int m) {
  const double mu = m - l;
  return csqrt((2.0 * l + 1.0) / (2.0 * l - 3.0) * ((l - 1.0) * (l - 1.0) - mu * mu) / (l * l - mu * mu));
}

// ---- number types ---------------------------------------------------------------------------------------------
template <typename T>
struct G3 {  // value and gradient with respect to the raw input vector
  T v, x, y, z;
};
template <typename N>
struct Du {  // a + eps * b
  N a, b;
};

template <typename T> __device__ __forceinline__ T nadd(T p, T q) { return p + q; }
template <typename T> __device__ __forceinline__ T nsub(T p, T q) { return p - q; }
template <typename T> __device__ __forceinline__ T nmul(T p, T q) { return p * q; }
template <typename T> __device__ __forceinline__ T nscale(T s, T p) { return s * p; }

template <typename T> __device__ __forceinline__ G3<T> nadd(G3<T> p, G3<T> q) { return {p.v + q.v, p.x + q.x, p.y + q.y, p.z + q.z}; }
template <typename T> __device__ __forceinline__ G3<T> nsub(G3<T> p, G3<T> q) { return {p.v - q.v, p.x - q.x, p.y - q.y, p.z - q.z}; }
template <typename T> __device__ __forceinline__ G3<T> nmul(G3<T> p, G3<T> q) {
  return {p.v * q.v, p.v * q.x + p.x * q.v, p.v * q.y + p.y * q.v, p.v * q.z + p.z * q.v};
}
template <typename T> __device__ __forceinline__ G3<T> nscale(T s, G3<T> p) { return {s * p.v, s * p.x, s * p.y, s * p.z}; }

template <typename N> __device__ __forceinline__ Du<N> nadd(Du<N> p, Du<N> q) { return {nadd(p.a, q.a), nadd(p.b, q.b)}; }
template <typename N> __device__ __forceinline__ Du<N> nsub(Du<N> p, Du<N> q) { return {nsub(p.a, q.a), nsub(p.b, q.b)}; }
template <typename N> __device__ __forceinline__ Du<N> nmul(Du<N> p, Du<N> q) {
  return {nmul(p.a, q.a), nadd(nmul(p.a, q.b), nmul(p.b, q.a))};
}
template <typename T, typename N> __device__ __forceinline__ Du<N> nscale(T s, Du<N> p) { return {nscale(s, p.a), nscale(s, p.b)}; }

template <typename T> __device__ __forceinline__ T nscale_neg(T p) { return -p; }
template <typename T> __device__ __forceinline__ G3<T> nscale_neg(G3<T> p) { return {-p.v, -p.x, -p.y, -p.z}; }
template <typename T> __device__ __forceinline__ T nscale_half_neg(T p) { return T(-0.5) * p; }
template <typename T> __device__ __forceinline__ G3<T> nscale_half_neg(G3<T> p) {
  return {T(-0.5) * p.v, T(-0.5) * p.x, T(-0.5) * p.y, T(-0.5) * p.z};
}

// reciprocal square root of a strictly positive number, used for the normalisation x / |x|
template <typename T> __device__ __forceinline__ T nrsqrt(T p) { return T(1) / sqrt(p); }
template <typename T> __device__ __forceinline__ G3<T> nrsqrt(G3<T> p) {
  const T r = T(1) / sqrt(p.v);
  const T d = T(-0.5) * r / p.v;  // d/dp p^(-1/2)
  return {r, d * p.x, d * p.y, d * p.z};
}
template <typename N> __device__ __forceinline__ Du<N> nrsqrt(Du<N> p);
template <typename T> __device__ __forceinline__ T nrecip(T p) { return T(1) / p; }
template <typename T> __device__ __forceinline__ G3<T> nrecip(G3<T> p) {
  const T r = T(1) / p.v;
  const T d = -r * r;
  return {r, d * p.x, d * p.y, d * p.z};
}
template <typename N> __device__ __forceinline__ Du<N> nrecip(Du<N> p) {
  const N r = nrecip(p.a);
  return {r, nmul(nscale_neg(nmul(r, r)), p.b)};
}
template <typename N> __device__ __forceinline__ Du<N> nrsqrt(Du<N> p) {
  const N r = nrsqrt(p.a);                                           // a^(-1/2)
  const N d = nmul(nscale_half_neg(r), nrecip(p.a));                 // -1/2 a^(-3/2)
  return {r, nmul(d, p.b)};
}

template <typename T> __device__ __forceinline__ T value_of(T p) { return p; }
template <typename T> __device__ __forceinline__ T value_of(G3<T> p) { return p.v; }
template <typename N> __device__ __forceinline__ auto value_of(Du<N> p) { return value_of(p.a); }

// ---- the recurrence ---------------------------------------------------------------------------------------------
// Coefficient tables, constant-initialised at compile time and kept in constant memory.
template <typename T>
struct CoefTable {
  T edge[kMaxDegree + 1];
  T diag[kMaxDegree + 1];
  T a[kMaxDegree + 1][2 * kMaxDegree + 1];
  T b[kMaxDegree + 1][2 * kMaxDegree + 1];
};
template <typename T>
constexpr CoefTable<T> make_table() {
  CoefTable<T> t{};
  for (int l = 1; l <= kMaxDegree; ++l) {
    t.edge[l] = T(coef_edge(l));
    t.diag[l] = T(coef_diag(l));
    if (l >= 2)
      for (int m = 2; m <= 2 * l - 2; ++m) {
        t.a[l][m] = T(coef_a(l, m));
        t.b[l][m] = T(coef_b(l, m));
      }
  }
  return t;
}
__constant__ CoefTable<float> kCoefF = make_table<float>();
__constant__ CoefTable<double> kCoefD = make_table<double>();
template <typename T> __device__ __forceinline__ const CoefTable<T>& coef_table();
template <> __device__ __forceinline__ const CoefTable<float>& coef_table<float>() { return kCoefF; }
template <> __device__ __forceinline__ const CoefTable<double>& coef_table<double>() { return kCoefD; }

constexpr int kWidth = 2 * kMaxDegree + 1;

// Walks degrees 0..lmax, handing each finished level to the sink.  Three rotating level buffers.
template <typename T, typename N, typename Sink>
__device__ __forceinline__ void walk(int lmax, const N& one, const N& x, const N& y, const N& z, const N& r2,
                                     Sink& sink) {
  const CoefTable<T>& tb = coef_table<T>();
  N buf[3][kWidth];
  buf[0][0] = one;
  sink.emit(0, buf[0]);
  if (lmax < 1) return;
  buf[1][0] = nscale(tb.diag[1], x);
  buf[1][1] = nscale(tb.diag[1], y);
  buf[1][2] = nscale(tb.diag[1], z);
  sink.emit(1, buf[1]);
  int i2 = 0, i1 = 1, i0 = 2;
  for (int l = 2; l <= lmax; ++l) {
    const N* p1 = buf[i1];
    const N* p2 = buf[i2];
    N* out = buf[i0];
    const T edge = tb.edge[l], diag = tb.diag[l];
    out[0] = nscale(edge, nadd(nmul(p1[0], z), nmul(p1[2 * l - 2], x)));
    out[2 * l] = nscale(edge, nsub(nmul(p1[2 * l - 2], z), nmul(p1[0], x)));
    out[1] = nscale(diag, nmul(y, p1[0]));
    out[2 * l - 1] = nscale(diag, nmul(y, p1[2 * l - 2]));
    for (int m = 2; m <= 2 * l - 2; ++m)
      out[m] = nsub(nscale(tb.a[l][m], nmul(y, p1[m - 1])), nscale(tb.b[l][m], nmul(r2, p2[m - 2])));
    sink.emit(l, out);
    const int t = i2;
    i2 = i1;
    i1 = i0;
    i0 = t;
  }
}

// ---- unrolled recurrence for the degree list 0..LMAX ------------------------------------------------------------
template <int I, int N, typename F>
__device__ __forceinline__ void unroll(F&& f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    unroll<I + 1, N>(f);
  }
}

// Levels of equal parity share an array: level l is computed from level l-1 (the other array) and level l-2 (its own
// array) and written over the latter from the highest component down, so no third buffer is needed and every index
// is a compile-time constant: the arrays live in registers.
template <typename T, typename N, int LMAX, typename Sink>
__device__ __forceinline__ void walk_unrolled(const N& one, const N& x, const N& y, const N& z, const N& r2, Sink& sink) {
  constexpr int kW = 2 * LMAX + 1;
  N even[kW], odd[kW];
  even[0] = one;
  sink.emit(std::integral_constant<int, 0>{}, even);
  if constexpr (LMAX >= 1) {
    odd[0] = nscale(T(coef_diag(1)), x);
    odd[1] = nscale(T(coef_diag(1)), y);
    odd[2] = nscale(T(coef_diag(1)), z);
    sink.emit(std::integral_constant<int, 1>{}, odd);
  }
  unroll<2, LMAX + 1>([&](auto lc) {
    constexpr int l = decltype(lc)::value;
    N* cur = (l % 2 == 0) ? even : odd;        // holds level l-2 on entry
    const N* p1 = (l % 2 == 0) ? odd : even;   // level l-1
    unroll<0, 2 * l - 3>([&](auto dc) {        // interior components m = 2l-2 ... 2
      constexpr int m = 2 * l - 2 - decltype(dc)::value;
      cur[m] = nsub(nscale(T(coef_a(l, m)), nmul(y, p1[m - 1])), nscale(T(coef_b(l, m)), nmul(r2, cur[m - 2])));
    });
    constexpr T edge = T(coef_edge(l)), diag = T(coef_diag(l));
    cur[0] = nscale(edge, nadd(nmul(p1[0], z), nmul(p1[2 * l - 2], x)));
    cur[2 * l] = nscale(edge, nsub(nmul(p1[2 * l - 2], z), nmul(p1[0], x)));
    cur[1] = nscale(diag, nmul(y, p1[0]));
    cur[2 * l - 1] = nscale(diag, nmul(y, p1[2 * l - 2]));
    sink.emit(lc, cur);
  });
}

template <typename T>
__device__ __forceinline__ T degree_scale(int l, int normalization) {
  if (normalization == 1) return T(1) / sqrt(T(2 * l + 1));
  if (normalization == 2) return T(0.28209479177387814);  // 1 / sqrt(4 pi)
  return T(1);
}

// ---- sinks -----------------------------------------------------------------------------------------------------
template <typename T>
struct ForwardSink {
  const ShParams& P;
  T* row;  // this thread's row in the shared tile
  __device__ __forceinline__ void emit(int l, const T* level) {
    const int reps = P.count[l];
    if (reps == 0) return;
    const T scale = degree_scale<T>(l, P.normalization);
    for (int r = 0; r < reps; ++r) {
      T* dst = row + P.column[l][r];
      for (int m = 0; m < 2 * l + 1; ++m) dst[m] = scale * level[m];
    }
  }
};

template <typename T>
struct BackwardSink {
  const ShParams& P;
  const T* row;  // g row in the shared tile
  T dx = T(0), dy = T(0), dz = T(0);
  __device__ __forceinline__ void emit(int l, const G3<T>* level) {
    const int reps = P.count[l];
    if (reps == 0) return;
    const T scale = degree_scale<T>(l, P.normalization);
    for (int m = 0; m < 2 * l + 1; ++m) {
      T gsum = T(0);
      for (int r = 0; r < reps; ++r) gsum += row[P.column[l][r] + m];
      gsum *= scale;
      dx += gsum * level[m].x;
      dy += gsum * level[m].y;
      dz += gsum * level[m].z;
    }
  }
};

template <typename T>
struct DoubleSink {
  const ShParams& P;
  T* row;  // g row on entry; overwritten with sg
  bool write_sg;
  T sx = T(0), sy = T(0), sz = T(0);
  __device__ __forceinline__ void emit(int l, const Du<G3<T>>* level) {
    const int reps = P.count[l];
    if (reps == 0) return;
    const T scale = degree_scale<T>(l, P.normalization);
    for (int m = 0; m < 2 * l + 1; ++m) {
      T gsum = T(0);
      for (int r = 0; r < reps; ++r) gsum += row[P.column[l][r] + m];
      gsum *= scale;
      sx += gsum * level[m].b.x;
      sy += gsum * level[m].b.y;
      sz += gsum * level[m].b.z;
      if (write_sg) {
        const T sg = scale * level[m].b.v;
        for (int r = 0; r < reps; ++r) row[P.column[l][r] + m] = sg;
      }
    }
  }
};

// Builds the (optionally normalised) coordinates as numbers of type N from raw numbers.
template <typename T, typename N>
__device__ __forceinline__ void prepare(const ShParams& P, N& x, N& y, N& z, N& r2) {
  if (P.normalize) {
    const N s = nadd(nadd(nmul(x, x), nmul(y, y)), nmul(z, z));
    const T len2 = value_of(s);
    if (len2 > T(1e-24)) {  // |v| > 1e-12: divide by the length
      const N inv = nrsqrt(s);
      x = nmul(x, inv);
      y = nmul(y, inv);
      z = nmul(z, inv);
    } else {  // clamped denominator is the constant 1e-12
      x = nscale(T(1e12), x);
      y = nscale(T(1e12), y);
      z = nscale(T(1e12), z);
    }
  }
  r2 = nadd(nadd(nmul(x, x), nmul(y, y)), nmul(z, z));
}

// MODE 0: out = Y(v).  MODE 1: dx = J^T g.  MODE 2: sx = d<rx, J^T g>/dv, sg = J rx.
template <typename T, int MODE>
__global__ void __launch_bounds__(kBlock)
sh_kernel(const ShParams P, const T* __restrict__ v, const T* __restrict__ g, const T* __restrict__ rx,
          T* __restrict__ out0, T* __restrict__ out1, int64_t n) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* smem = reinterpret_cast<T*>(smem_raw);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int C = P.C, CP = C | 1;
  T* tile = smem + static_cast<size_t>(warp) * 32 * CP;
  T* row = tile + lane * CP;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * (kBlock / 32);
  for (int64_t base = (static_cast<int64_t>(blockIdx.x) * (kBlock / 32) + warp) * 32; base < n;
       base += warps_total * 32) {
    const int rows = (n - base < 32) ? static_cast<int>(n - base) : 32;
    const int64_t item = base + lane;
    const bool active = lane < rows;
    T vx = T(0), vy = T(1), vz = T(0);
    if (active) {
      vx = v[item * 3 + 0];
      vy = v[item * 3 + 1];
      vz = v[item * 3 + 2];
    }
    if constexpr (MODE != 0) {
      const T* gsrc = g + base * C;
      for (int idx = lane; idx < rows * C; idx += 32) tile[(idx / C) * CP + (idx % C)] = gsrc[idx];
      __syncwarp();
    }
    if constexpr (MODE == 0) {
      T x = vx, y = vy, z = vz, r2;
      prepare<T, T>(P, x, y, z, r2);
      ForwardSink<T> sink{P, row};
      walk<T, T>(P.lmax, T(1), x, y, z, r2, sink);
      __syncwarp();
      T* dst = out0 + base * C;
      for (int idx = lane; idx < rows * C; idx += 32) dst[idx] = tile[(idx / C) * CP + (idx % C)];
    } else if constexpr (MODE == 1) {
      using N = G3<T>;
      N x{vx, T(1), T(0), T(0)}, y{vy, T(0), T(1), T(0)}, z{vz, T(0), T(0), T(1)}, r2;
      prepare<T, N>(P, x, y, z, r2);
      BackwardSink<T> sink{P, row};
      walk<T, N>(P.lmax, N{T(1), T(0), T(0), T(0)}, x, y, z, r2, sink);
      if (active) {
        out0[item * 3 + 0] = sink.dx;
        out0[item * 3 + 1] = sink.dy;
        out0[item * 3 + 2] = sink.dz;
      }
    } else {
      using N = Du<G3<T>>;
      T tx = T(0), ty = T(0), tz = T(0);
      if (active) {
        tx = rx[item * 3 + 0];
        ty = rx[item * 3 + 1];
        tz = rx[item * 3 + 2];
      }
      const G3<T> zero{T(0), T(0), T(0), T(0)};
      N x{{vx, T(1), T(0), T(0)}, {tx, T(0), T(0), T(0)}};
      N y{{vy, T(0), T(1), T(0)}, {ty, T(0), T(0), T(0)}};
      N z{{vz, T(0), T(0), T(1)}, {tz, T(0), T(0), T(0)}};
      N r2;
      prepare<T, N>(P, x, y, z, r2);
      DoubleSink<T> sink{P, row, out1 != nullptr};
      walk<T, N>(P.lmax, N{{T(1), T(0), T(0), T(0)}, zero}, x, y, z, r2, sink);
      if (active && out0 != nullptr) {
        out0[item * 3 + 0] = sink.sx;
        out0[item * 3 + 1] = sink.sy;
        out0[item * 3 + 2] = sink.sz;
      }
      if (out1 != nullptr) {
        __syncwarp();
        T* dst = out1 + base * C;
        for (int idx = lane; idx < rows * C; idx += 32) dst[idx] = tile[(idx / C) * CP + (idx % C)];
      }
    }
    __syncwarp();
  }
}

// Sinks of the unrolled kernels: the degree list is 0..LMAX, so degree l starts at column l * l.
template <typename T>
struct CanonForwardSink {
  int normalization;
  T* row;
  template <int L>
  __device__ __forceinline__ void emit(std::integral_constant<int, L>, const T* level) {
    const T scale = degree_scale<T>(L, normalization);
#pragma unroll
    for (int m = 0; m < 2 * L + 1; ++m) row[L * L + m] = scale * level[m];
  }
};
template <typename T>
struct CanonDoubleSink {
  int normalization;
  T* row;  // g row on entry; overwritten with sg
  bool write_sg;
  T sx = T(0), sy = T(0), sz = T(0);
  template <int L>
  __device__ __forceinline__ void emit(std::integral_constant<int, L>, const Du<G3<T>>* level) {
    const T scale = degree_scale<T>(L, normalization);
#pragma unroll
    for (int m = 0; m < 2 * L + 1; ++m) {
      const T gsum = scale * row[L * L + m];
      sx += gsum * level[m].b.x;
      sy += gsum * level[m].b.y;
      sz += gsum * level[m].b.z;
      if (write_sg) row[L * L + m] = scale * level[m].b.v;
    }
  }
};

// First derivative for the degree list 0..LMAX in reverse mode: dv = J^T g.  The forward sweep keeps every level's
// values in registers; the reverse sweep walks the recurrence from the highest degree down, handing each component's
// adjoint to the components it was computed from and to the coordinates.  About 12 operations per output component,
// against about 30 for carrying a gradient along the forward recurrence, and no wider state than the values
// themselves.  All indices are compile-time constants.
template <typename T, int LMAX>
__device__ __forceinline__ void canon_backward(const ShParams& P, T vx, T vy, T vz, const T* __restrict__ grow,
                                               T& dvx, T& dvy, T& dvz) {
  constexpr int C = (LMAX + 1) * (LMAX + 1);
  // coordinates the polynomials are evaluated at
  T x = vx, y = vy, z = vz, inv = T(1);
  bool unit = false;
  if (P.normalize) {
    const T len2 = vx * vx + vy * vy + vz * vz;
    unit = len2 > T(1e-24);
    inv = unit ? T(1) / sqrt(len2) : T(1e12);
    x *= inv;
    y *= inv;
    z *= inv;
  }
  const T r2 = x * x + y * y + z * z;
  T val[C], adj[C];
  val[0] = T(1);
  if constexpr (LMAX >= 1) {
    val[1] = T(coef_diag(1)) * x;
    val[2] = T(coef_diag(1)) * y;
    val[3] = T(coef_diag(1)) * z;
  }
  unroll<2, LMAX + 1>([&](auto lc) {
    constexpr int l = decltype(lc)::value;
    constexpr int o = l * l, o1 = (l - 1) * (l - 1), o2 = (l - 2) * (l - 2);
    constexpr T edge = T(coef_edge(l)), diag = T(coef_diag(l));
    val[o] = edge * (val[o1] * z + val[o1 + 2 * l - 2] * x);
    val[o + 2 * l] = edge * (val[o1 + 2 * l - 2] * z - val[o1] * x);
    val[o + 1] = diag * y * val[o1];
    val[o + 2 * l - 1] = diag * y * val[o1 + 2 * l - 2];
    unroll<2, 2 * l - 1>([&](auto mc) {
      constexpr int m = decltype(mc)::value;
      val[o + m] = T(coef_a(l, m)) * y * val[o1 + m - 1] - T(coef_b(l, m)) * r2 * val[o2 + m - 2];
    });
  });
  // seeds: the cotangent of every output component, with the degree's normalisation factor
  unroll<0, LMAX + 1>([&](auto lc) {
    constexpr int l = decltype(lc)::value;
    const T scale = degree_scale<T>(l, P.normalization);
#pragma unroll
    for (int m = 0; m < 2 * l + 1; ++m) adj[l * l + m] = scale * grow[l * l + m];
  });
  T ax = T(0), ay = T(0), az = T(0), ar2 = T(0);
  unroll<0, LMAX - 1>([&](auto dc) {
    constexpr int l = LMAX - decltype(dc)::value;  // LMAX ... 2
    constexpr int o = l * l, o1 = (l - 1) * (l - 1), o2 = (l - 2) * (l - 2);
    constexpr T edge = T(coef_edge(l)), diag = T(coef_diag(l));
    unroll<2, 2 * l - 1>([&](auto mc) {
      constexpr int m = decltype(mc)::value;
      const T ma = adj[o + m] * T(coef_a(l, m)), mb = adj[o + m] * T(coef_b(l, m));
      ay += ma * val[o1 + m - 1];
      adj[o1 + m - 1] += ma * y;
      ar2 -= mb * val[o2 + m - 2];
      adj[o2 + m - 2] -= mb * r2;
    });
    const T a0 = adj[o] * edge, a2l = adj[o + 2 * l] * edge, a1 = adj[o + 1] * diag, a2l1 = adj[o + 2 * l - 1] * diag;
    adj[o1] += a0 * z - a2l * x + a1 * y;
    adj[o1 + 2 * l - 2] += a0 * x + a2l * z + a2l1 * y;
    az += a0 * val[o1] + a2l * val[o1 + 2 * l - 2];
    ax += a0 * val[o1 + 2 * l - 2] - a2l * val[o1];
    ay += a1 * val[o1] + a2l1 * val[o1 + 2 * l - 2];
  });
  if constexpr (LMAX >= 1) {
    ax += T(coef_diag(1)) * adj[1];
    ay += T(coef_diag(1)) * adj[2];
    az += T(coef_diag(1)) * adj[3];
  }
  ax += T(2) * x * ar2;
  ay += T(2) * y * ar2;
  az += T(2) * z * ar2;
  if (unit) {  // u = v / |v|: dv = (du - u (u . du)) / |v|
    const T along = x * ax + y * ay + z * az;
    dvx = inv * (ax - x * along);
    dvy = inv * (ay - y * along);
    dvz = inv * (az - z * along);
  } else {  // no normalisation, or the clamped divisor: a constant factor
    dvx = inv * ax;
    dvy = inv * ay;
    dvz = inv * az;
  }
}

// Same three modes as sh_kernel for the degree list 0..LMAX, everything about the list known at compile time.
template <typename T, int MODE, int LMAX>
__global__ void __launch_bounds__(kBlock)
sh_canon_kernel(const ShParams P, const T* __restrict__ v, const T* __restrict__ g, const T* __restrict__ rx,
                T* __restrict__ out0, T* __restrict__ out1, int64_t n) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* smem = reinterpret_cast<T*>(smem_raw);
  constexpr int C = (LMAX + 1) * (LMAX + 1), CP = C | 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T* tile = smem + static_cast<size_t>(warp) * 32 * CP;
  T* row = tile + lane * CP;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * (kBlock / 32);
  for (int64_t base = (static_cast<int64_t>(blockIdx.x) * (kBlock / 32) + warp) * 32; base < n;
       base += warps_total * 32) {
    const int rows = (n - base < 32) ? static_cast<int>(n - base) : 32;
    const int64_t item = base + lane;
    const bool active = lane < rows;
    T vx = T(0), vy = T(1), vz = T(0);
    if (active) {
      vx = v[item * 3 + 0];
      vy = v[item * 3 + 1];
      vz = v[item * 3 + 2];
    }
    if constexpr (MODE != 0) {
      const T* gsrc = g + base * C;
      if (rows == 32) {
        // a full tile: the loads go out in batches of eight per lane before anything is stored, so that a warp has
        // 1 KB (FP32) in flight instead of one row of loads waiting on the next
        constexpr int kBatch = 8;
#pragma unroll
        for (int j0 = 0; j0 < C; j0 += kBatch) {
          T batch[kBatch];
#pragma unroll
          for (int j = 0; j < kBatch; ++j)
            if (j0 + j < C) batch[j] = gsrc[(j0 + j) * 32 + lane];
#pragma unroll
          for (int j = 0; j < kBatch; ++j)
            if (j0 + j < C) {
              const int idx = (j0 + j) * 32 + lane;
              tile[(idx / C) * CP + (idx % C)] = batch[j];
            }
        }
      } else {
#pragma unroll 4
        for (int idx = lane; idx < rows * C; idx += 32) tile[(idx / C) * CP + (idx % C)] = gsrc[idx];
      }
      __syncwarp();
    }
    if constexpr (MODE == 0) {
      T x = vx, y = vy, z = vz, r2;
      prepare<T, T>(P, x, y, z, r2);
      CanonForwardSink<T> sink{P.normalization, row};
      walk_unrolled<T, T, LMAX>(T(1), x, y, z, r2, sink);
      __syncwarp();
      T* dst = out0 + base * C;
#pragma unroll 4
      for (int idx = lane; idx < rows * C; idx += 32) dst[idx] = tile[(idx / C) * CP + (idx % C)];
    } else if constexpr (MODE == 1) {
      T dvx, dvy, dvz;
      canon_backward<T, LMAX>(P, vx, vy, vz, row, dvx, dvy, dvz);
      if (active) {
        out0[item * 3 + 0] = dvx;
        out0[item * 3 + 1] = dvy;
        out0[item * 3 + 2] = dvz;
      }
    } else {
      using N = Du<G3<T>>;
      T tx = T(0), ty = T(0), tz = T(0);
      if (active) {
        tx = rx[item * 3 + 0];
        ty = rx[item * 3 + 1];
        tz = rx[item * 3 + 2];
      }
      const G3<T> zero{T(0), T(0), T(0), T(0)};
      N x{{vx, T(1), T(0), T(0)}, {tx, T(0), T(0), T(0)}};
      N y{{vy, T(0), T(1), T(0)}, {ty, T(0), T(0), T(0)}};
      N z{{vz, T(0), T(0), T(1)}, {tz, T(0), T(0), T(0)}};
      N r2;
      prepare<T, N>(P, x, y, z, r2);
      CanonDoubleSink<T> sink{P.normalization, row, out1 != nullptr};
      walk_unrolled<T, N, LMAX>(N{{T(1), T(0), T(0), T(0)}, zero}, x, y, z, r2, sink);
      if (active && out0 != nullptr) {
        out0[item * 3 + 0] = sink.sx;
        out0[item * 3 + 1] = sink.sy;
        out0[item * 3 + 2] = sink.sz;
      }
      if (out1 != nullptr) {
        __syncwarp();
        T* dst = out1 + base * C;
#pragma unroll 4
        for (int idx = lane; idx < rows * C; idx += 32) dst[idx] = tile[(idx / C) * CP + (idx % C)];
      }
    }
    __syncwarp();
  }
}

template <typename T, int MODE, int LMAX>
int launch_canon(const ShParams& P, const T* v, const T* g, const T* rx, T* out0, T* out1, int64_t n,
                 cudaStream_t stream) {
  constexpr int C = (LMAX + 1) * (LMAX + 1);
  const size_t smem = static_cast<size_t>(kBlock / 32) * 32 * (C | 1) * sizeof(T);
  auto kernel = sh_canon_kernel<T, MODE, LMAX>;
  if (smem > 48 * 1024)
    LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  const int64_t blocks = std::min<int64_t>(ceil_div(n, kBlock), 148 * 16);
  kernel<<<static_cast<unsigned>(blocks), kBlock, smem, stream>>>(P, v, g, rx, out0, out1, n);
  LUNA_LAUNCH_CHECK("spherical harmonics (degrees 0..lmax)");
  return LUNA_OK;
}

// True if the degree list is 0, 1, ..., lmax, each once and in that order.
inline bool is_canonical_list(const ShParams& P, int lmax) {
  for (int l = 0; l <= lmax; ++l)
    if (P.count[l] != 1 || P.column[l][0] != l * l) return false;
  return true;
}

template <typename T, int MODE>
int launch_lmax(int lmax, ShParams P, const T* v, const T* g, const T* rx, T* out0, T* out1, int64_t n,
                cudaStream_t stream) {
  P.lmax = lmax;
  if (lmax >= 1 && lmax <= 6 && is_canonical_list(P, lmax)) {
    switch (lmax) {
      case 1: return launch_canon<T, MODE, 1>(P, v, g, rx, out0, out1, n, stream);
      case 2: return launch_canon<T, MODE, 2>(P, v, g, rx, out0, out1, n, stream);
      case 3: return launch_canon<T, MODE, 3>(P, v, g, rx, out0, out1, n, stream);
      case 4: return launch_canon<T, MODE, 4>(P, v, g, rx, out0, out1, n, stream);
      case 5: return launch_canon<T, MODE, 5>(P, v, g, rx, out0, out1, n, stream);
      default: return launch_canon<T, MODE, 6>(P, v, g, rx, out0, out1, n, stream);
    }
  }
  const size_t smem = static_cast<size_t>(kBlock / 32) * 32 * (P.C | 1) * sizeof(T);
  auto kernel = sh_kernel<T, MODE>;
  if (smem > 48 * 1024)
    LUNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  const int64_t blocks = std::min<int64_t>(ceil_div(n, kBlock), 148 * 16);
  kernel<<<static_cast<unsigned>(blocks), kBlock, smem, stream>>>(P, v, g, rx, out0, out1, n);
  LUNA_LAUNCH_CHECK("spherical harmonics");
  return LUNA_OK;
}

int make_params(const luna_sh_desc* desc, ShParams& P, int& lmax) {
  if (!desc) return fail(LUNA_ERR_INVALID_ARGUMENT, "null description");
  if (desc->dtype != LUNA_F32 && desc->dtype != LUNA_F64) return fail(LUNA_ERR_INVALID_ARGUMENT, "dtype must be LUNA_F32 or LUNA_F64");
  if (desc->num_degrees <= 0 || desc->num_degrees > 32) return fail(LUNA_ERR_INVALID_ARGUMENT, "between 1 and 32 degrees required");
  if (desc->normalization < 0 || desc->normalization > 2) return fail(LUNA_ERR_INVALID_ARGUMENT, "normalization must be component, norm or integral");
  P = ShParams{};
  lmax = 0;
  int column = 0;
  for (int d = 0; d < desc->num_degrees; ++d) {
    const int l = desc->degrees[d];
    if (l < 0) return fail(LUNA_ERR_INVALID_ARGUMENT, "SphericalHarmonics degrees must be nonempty nonnegative integers");
    if (l > kMaxDegree) return fail(LUNA_ERR_UNSUPPORTED, "SphericalHarmonics supports degrees through 12");
    if (P.count[l] >= kMaxRepeat) return fail(LUNA_ERR_UNSUPPORTED, "a degree may appear at most %d times", kMaxRepeat);
    P.column[l][P.count[l]++] = column;
    column += 2 * l + 1;
    lmax = l > lmax ? l : lmax;
  }
  P.C = column;
  P.normalize = desc->normalize != 0;
  P.normalization = desc->normalization;
  return LUNA_OK;
}

template <int MODE>
int dispatch(const luna_sh_desc* desc, const void* v, const void* g, const void* rx, void* out0, void* out1,
             int64_t n, void* stream_) {
  clear_error();
  ShParams P;
  int lmax = 0;
  int rc = make_params(desc, P, lmax);
  if (rc != LUNA_OK) return rc;
  if (n < 0) return fail(LUNA_ERR_INVALID_ARGUMENT, "negative item count");
  if (n == 0) return LUNA_OK;
  if (!v || (MODE != 0 && !g) || (MODE == 2 && !rx) || (MODE != 2 && !out0))
    return fail(LUNA_ERR_INVALID_ARGUMENT, "null tensor pointer");
  auto stream = static_cast<cudaStream_t>(stream_);
  if (desc->dtype == LUNA_F64)
    return launch_lmax<double, MODE>(lmax, P, static_cast<const double*>(v), static_cast<const double*>(g),
                                     static_cast<const double*>(rx), static_cast<double*>(out0),
                                     static_cast<double*>(out1), n, stream);
  return launch_lmax<float, MODE>(lmax, P, static_cast<const float*>(v), static_cast<const float*>(g),
                                  static_cast<const float*>(rx), static_cast<float*>(out0), static_cast<float*>(out1),
                                  n, stream);
}

}  // namespace
}  // namespace luna

extern "C" int luna_sh_fwd(const luna_sh_desc* desc, const void* v, void* out, int64_t n, void* stream) {
  return luna::dispatch<0>(desc, v, nullptr, nullptr, out, nullptr, n, stream);
}
extern "C" int luna_sh_bwd(const luna_sh_desc* desc, const void* v, const void* g, void* dx, int64_t n, void* stream) {
  return luna::dispatch<1>(desc, v, g, nullptr, dx, nullptr, n, stream);
}
extern "C" int luna_sh_dbl_bwd(const luna_sh_desc* desc, const void* v, const void* g, const void* rx, void* sx,
                               void* sg, int64_t n, void* stream) {
  return luna::dispatch<2>(desc, v, g, rx, sx, sg, n, stream);
}
