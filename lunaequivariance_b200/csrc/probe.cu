// Arithmetic-peak probe: register-resident chains of fused multiply-adds, nothing else in the loop.  The benchmark
// times it to get this GPU's measured packed-FP32 (fma.rn.f32x2, the instruction the FP32 kernels run on) and FP64
// FMA rates, the denominators of the secondary (arithmetic) roofline next to the HBM one.
#include "common.h"

namespace {

constexpr int kChains = 8;      // independent accumulators per thread: enough to cover the FMA latency
constexpr int kThreads = 512;
constexpr int kCtasPerSm = 4;   // 2048 threads per SM

__global__ void __launch_bounds__(kThreads) probe_f32x2(int iterations, double* sink) {
  const float seed = static_cast<float>(threadIdx.x) * 1e-3f + static_cast<float>(sink[0]);
  unsigned long long acc[kChains], a, b;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(1.0f + seed * 1e-6f), "f"(1.0f - seed * 1e-6f));
  asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(seed * 1e-7f), "f"(-seed * 1e-7f));
#pragma unroll
  for (int c = 0; c < kChains; ++c) asm("mov.b64 %0, {%1, %2};" : "=l"(acc[c]) : "f"(seed + c), "f"(seed - c));
#pragma unroll 1
  for (int it = 0; it < iterations; ++it) {
#pragma unroll
    for (int rep = 0; rep < 4; ++rep)
#pragma unroll
      for (int c = 0; c < kChains; ++c) asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(acc[c]) : "l"(a), "l"(b));
  }
  float total = 0.f;
#pragma unroll
  for (int c = 0; c < kChains; ++c) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc[c]));
    total += lo + hi;
  }
  if (total == 123.456f) sink[1 + (blockIdx.x * kThreads + threadIdx.x) % 1024] = total;  // keeps the chains alive
}

__global__ void __launch_bounds__(kThreads) probe_f64(int iterations, double* sink) {
  const double seed = threadIdx.x * 1e-3 + sink[0];
  const double a = 1.0 + seed * 1e-9, b = seed * 1e-10;
  double acc[kChains];
#pragma unroll
  for (int c = 0; c < kChains; ++c) acc[c] = seed + c;
#pragma unroll 1
  for (int it = 0; it < iterations; ++it) {
#pragma unroll
    for (int rep = 0; rep < 4; ++rep)
#pragma unroll
      for (int c = 0; c < kChains; ++c) asm volatile("fma.rn.f64 %0, %0, %1, %2;" : "+d"(acc[c]) : "d"(a), "d"(b));
  }
  double total = 0.0;
#pragma unroll
  for (int c = 0; c < kChains; ++c) total += acc[c];
  if (total == 123.456) sink[1 + (blockIdx.x * kThreads + threadIdx.x) % 1024] = total;
}

}  // namespace

extern "C" int luna_probe_fma(int kind, int iterations, void* sink, double* flops, void* stream_) {
  luna::clear_error();
  if (!sink || !flops || iterations <= 0 || (kind != 0 && kind != 1))
    return luna::fail(LUNA_ERR_INVALID_ARGUMENT, "luna_probe_fma: kind 0 (packed FP32) or 1 (FP64), a sink buffer of "
                                                 "at least 1025 doubles and a positive iteration count are required");
  int device = 0, sms = 0;
  LUNA_CUDA_CHECK(cudaGetDevice(&device));
  LUNA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  auto stream = static_cast<cudaStream_t>(stream_);
  const int blocks = sms * kCtasPerSm;
  const double fma_count = static_cast<double>(blocks) * kThreads * iterations * 4.0 * kChains;
  if (kind == 0) {
    probe_f32x2<<<blocks, kThreads, 0, stream>>>(iterations, static_cast<double*>(sink));
    *flops = fma_count * 4.0;  // two lanes per packed instruction, two FLOPs per multiply-add
  } else {
    probe_f64<<<blocks, kThreads, 0, stream>>>(iterations, static_cast<double*>(sink));
    *flops = fma_count * 2.0;
  }
  LUNA_LAUNCH_CHECK("arithmetic-peak probe");
  return LUNA_OK;
}
