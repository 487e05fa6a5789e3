// Shared host-side helpers: thread-local error text, CUDA call checking, dtype dispatch.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/luna_b200.h"

namespace luna {

// Stores a printf-formatted message for luna_last_error() and returns `code`.
int fail(int code, const char* format, ...);
void clear_error();

#define LUNA_CUDA_CHECK(expr)                                                                          \
  do {                                                                                                 \
    cudaError_t luna_err_ = (expr);                                                                    \
    if (luna_err_ != cudaSuccess) {                                                                    \
      return ::luna::fail(LUNA_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(luna_err_), \
                          __FILE__, __LINE__);                                                         \
    }                                                                                                  \
  } while (0)

#define LUNA_LAUNCH_CHECK(name)                                                                          \
  do {                                                                                                   \
    cudaError_t luna_err_ = cudaGetLastError();                                                          \
    if (luna_err_ != cudaSuccess) {                                                                      \
      return ::luna::fail(LUNA_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(luna_err_)); \
    }                                                                                                    \
  } while (0)

inline bool aligned_to(const void* p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

template <typename T>
struct dtype_of;
template <>
struct dtype_of<float> {
  static constexpr int value = LUNA_F32;
};
template <>
struct dtype_of<double> {
  static constexpr int value = LUNA_F64;
};

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace luna
