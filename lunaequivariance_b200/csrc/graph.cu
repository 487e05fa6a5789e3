// Graph tables on the device: index bounds / sortedness scan, CSR row pointers by destination and by source, the
// stable permutation of edge ids grouped by source, and degree-descending node orders.  Everything runs on the
// caller's stream with caller-provided scratch; integer atomics only, so the tables are reproducible.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "common.h"

namespace luna {
namespace {

constexpr int kThreads = 256;

struct Bounds {
  long long min_index;
  long long max_src;
  long long max_dst;
  int unsorted;
  int pad;
};

template <typename Index>
__global__ void bounds_kernel(const Index* __restrict__ src, const Index* __restrict__ dst, int64_t edges,
                              Bounds* __restrict__ result) {
  long long lo = INT64_MAX, hi_s = INT64_MIN, hi_d = INT64_MIN;
  int unsorted = 0;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < edges;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const long long s = src[e], d = dst[e];
    lo = min(lo, min(s, d));
    hi_s = max(hi_s, s);
    hi_d = max(hi_d, d);
    if (e > 0 && dst[e - 1] > d) unsorted = 1;
  }
  for (int offset = 16; offset > 0; offset >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, offset));
    hi_s = max(hi_s, __shfl_xor_sync(0xffffffffu, hi_s, offset));
    hi_d = max(hi_d, __shfl_xor_sync(0xffffffffu, hi_d, offset));
    unsorted |= __shfl_xor_sync(0xffffffffu, unsorted, offset);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMin(&result->min_index, lo);
    atomicMax(&result->max_src, hi_s);
    atomicMax(&result->max_dst, hi_d);
    if (unsorted) atomicOr(&result->unsorted, 1);
  }
}

__global__ void init_bounds(Bounds* result) {
  result->min_index = INT64_MAX;
  result->max_src = INT64_MIN;
  result->max_dst = INT64_MIN;
  result->unsorted = 0;
}

template <typename Index>
__global__ void copy_and_count(const Index* __restrict__ src, const Index* __restrict__ dst, int64_t edges,
                               int32_t* __restrict__ src_out, int32_t* __restrict__ dst_out,
                               int32_t* __restrict__ src_rowptr, int32_t* __restrict__ dst_rowptr,
                               int32_t* __restrict__ iota) {
  const int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= edges) return;
  const int32_t s = static_cast<int32_t>(src[e]), d = static_cast<int32_t>(dst[e]);
  src_out[e] = s;
  dst_out[e] = d;
  iota[e] = static_cast<int32_t>(e);
  atomicAdd(&src_rowptr[s + 1], 1);
  atomicAdd(&dst_rowptr[d + 1], 1);
}

__global__ void degrees_and_iota(const int32_t* __restrict__ rowptr, int64_t nodes, int32_t* __restrict__ degree,
                                 int32_t* __restrict__ iota) {
  const int64_t n = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (n >= nodes) return;
  degree[n] = rowptr[n + 1] - rowptr[n];
  iota[n] = static_cast<int32_t>(n);
}

size_t align_up(size_t v) { return (v + 255) / 256 * 256; }

struct ScratchLayout {
  size_t bounds, keys_in, keys_out, values_in, cub_temp, cub_bytes, total;
};

ScratchLayout layout(int64_t nodes, int64_t edges) {
  ScratchLayout l{};
  const size_t items = static_cast<size_t>(std::max<int64_t>(std::max(nodes, edges), 1));
  size_t sort_bytes = 0, scan_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, static_cast<const int32_t*>(nullptr),
                                  static_cast<int32_t*>(nullptr), static_cast<const int32_t*>(nullptr),
                                  static_cast<int32_t*>(nullptr), static_cast<int64_t>(items));
  cub::DeviceScan::InclusiveSum(nullptr, scan_bytes, static_cast<int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
                                static_cast<int64_t>(items + 1));
  l.cub_bytes = std::max(sort_bytes, scan_bytes) + 256;
  size_t cursor = 0;
  l.bounds = cursor;
  cursor += align_up(sizeof(Bounds));
  l.keys_in = cursor;
  cursor += align_up(items * 4);
  l.keys_out = cursor;
  cursor += align_up(items * 4);
  l.values_in = cursor;
  cursor += align_up(items * 4);
  l.cub_temp = cursor;
  cursor += align_up(l.cub_bytes);
  l.total = cursor;
  return l;
}

int bits_for(int64_t max_value) {
  int bits = 1;
  while (bits < 32 && (1LL << bits) <= max_value) ++bits;
  return bits;
}

}  // namespace
}  // namespace luna

using namespace luna;

extern "C" int64_t luna_graph_scratch_bytes(int64_t num_nodes, int64_t num_edges) {
  if (num_nodes < 0 || num_edges < 0) return -1;
  return static_cast<int64_t>(layout(num_nodes, num_edges).total);
}

extern "C" int luna_graph_bounds(const void* src, const void* dst, int index_bits, int64_t num_edges,
                                 int64_t* min_index, int64_t* max_src, int64_t* max_dst, int* unsorted,
                                 void* scratch, int64_t scratch_bytes, void* stream_) {
  clear_error();
  if (!min_index || !max_src || !max_dst || !unsorted) return fail(LUNA_ERR_INVALID_ARGUMENT, "null result pointer");
  *min_index = 0;
  *max_src = *max_dst = -1;
  *unsorted = 0;
  if (num_edges == 0) return LUNA_OK;
  if (!src || !dst) return fail(LUNA_ERR_INVALID_ARGUMENT, "null edge list");
  if (index_bits != 32 && index_bits != 64) return fail(LUNA_ERR_INVALID_ARGUMENT, "index_bits must be 32 or 64");
  if (!scratch || scratch_bytes < static_cast<int64_t>(sizeof(Bounds)))
    return fail(LUNA_ERR_SCRATCH, "scratch too small for the bounds scan");
  auto stream = static_cast<cudaStream_t>(stream_);
  auto* result = static_cast<Bounds*>(scratch);
  init_bounds<<<1, 1, 0, stream>>>(result);
  const int blocks = static_cast<int>(std::min<int64_t>(ceil_div(num_edges, kThreads), 4096));
  if (index_bits == 64)
    bounds_kernel<int64_t><<<blocks, kThreads, 0, stream>>>(static_cast<const int64_t*>(src),
                                                            static_cast<const int64_t*>(dst), num_edges, result);
  else
    bounds_kernel<int32_t><<<blocks, kThreads, 0, stream>>>(static_cast<const int32_t*>(src),
                                                            static_cast<const int32_t*>(dst), num_edges, result);
  LUNA_LAUNCH_CHECK("graph bounds scan");
  Bounds host{};
  LUNA_CUDA_CHECK(cudaMemcpyAsync(&host, result, sizeof(Bounds), cudaMemcpyDeviceToHost, stream));
  LUNA_CUDA_CHECK(cudaStreamSynchronize(stream));
  *min_index = host.min_index;
  *max_src = host.max_src;
  *max_dst = host.max_dst;
  *unsorted = host.unsorted;
  return LUNA_OK;
}

extern "C" int luna_graph_build(const void* src, const void* dst, int index_bits, int64_t num_nodes,
                                int64_t num_src_nodes, int64_t num_edges, const luna_graph_out* out, void* scratch,
                                int64_t scratch_bytes, void* stream_) {
  clear_error();
  if (!out) return fail(LUNA_ERR_INVALID_ARGUMENT, "null output table set");
  if (num_src_nodes <= 0) num_src_nodes = num_nodes;
  if (num_nodes < 0 || num_edges < 0) return fail(LUNA_ERR_INVALID_ARGUMENT, "negative graph size");
  if (std::max(num_nodes, num_src_nodes) >= (1LL << 31) - 1024 || num_edges >= (1LL << 31) - 1024)
    return fail(LUNA_ERR_OVERFLOW, "graph exceeds the 32-bit index range of this build");
  if (index_bits != 32 && index_bits != 64) return fail(LUNA_ERR_INVALID_ARGUMENT, "index_bits must be 32 or 64");
  if (!out->dst_rowptr || !out->src_rowptr) return fail(LUNA_ERR_INVALID_ARGUMENT, "row pointer outputs missing");
  if (num_edges > 0 && (!src || !dst || !out->src || !out->dst || !out->edge_ids_by_src))
    return fail(LUNA_ERR_INVALID_ARGUMENT, "edge tables missing");
  if ((num_nodes > 0 && !out->node_order) || (num_src_nodes > 0 && !out->source_node_order))
    return fail(LUNA_ERR_INVALID_ARGUMENT, "node order outputs missing");
  const ScratchLayout l = layout(std::max(num_nodes, num_src_nodes), num_edges);
  if (!scratch || scratch_bytes < static_cast<int64_t>(l.total))
    return fail(LUNA_ERR_SCRATCH, "scratch too small: need %zu bytes", l.total);
  auto stream = static_cast<cudaStream_t>(stream_);
  auto* base = static_cast<unsigned char*>(scratch);
  auto* keys_in = reinterpret_cast<int32_t*>(base + l.keys_in);
  auto* keys_out = reinterpret_cast<int32_t*>(base + l.keys_out);
  auto* values_in = reinterpret_cast<int32_t*>(base + l.values_in);
  void* cub_temp = base + l.cub_temp;
  size_t cub_bytes = l.cub_bytes;

  LUNA_CUDA_CHECK(cudaMemsetAsync(out->src_rowptr, 0, (num_src_nodes + 1) * sizeof(int32_t), stream));
  LUNA_CUDA_CHECK(cudaMemsetAsync(out->dst_rowptr, 0, (num_nodes + 1) * sizeof(int32_t), stream));
  if (num_edges > 0) {
    const unsigned blocks = static_cast<unsigned>(ceil_div(num_edges, kThreads));
    if (index_bits == 64)
      copy_and_count<int64_t><<<blocks, kThreads, 0, stream>>>(static_cast<const int64_t*>(src),
                                                               static_cast<const int64_t*>(dst), num_edges, out->src,
                                                               out->dst, out->src_rowptr, out->dst_rowptr, values_in);
    else
      copy_and_count<int32_t><<<blocks, kThreads, 0, stream>>>(static_cast<const int32_t*>(src),
                                                               static_cast<const int32_t*>(dst), num_edges, out->src,
                                                               out->dst, out->src_rowptr, out->dst_rowptr, values_in);
    LUNA_LAUNCH_CHECK("graph copy and count");
    // stable grouping of edge ids by source
    LUNA_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(cub_temp, cub_bytes, static_cast<const int32_t*>(out->src),
                                                    keys_out, static_cast<const int32_t*>(values_in),
                                                    out->edge_ids_by_src, num_edges, 0,
                                                    bits_for(std::max<int64_t>(num_src_nodes - 1, 1)), stream));
  }
  const int degree_bits = bits_for(std::max<int64_t>(num_edges, 1));
  for (int pass = 0; pass < 2; ++pass) {
    const int64_t rows = pass == 0 ? num_nodes : num_src_nodes;
    int32_t* rowptr = pass == 0 ? out->dst_rowptr : out->src_rowptr;
    int32_t* order = pass == 0 ? out->node_order : out->source_node_order;
    if (rows == 0) continue;
    cub_bytes = l.cub_bytes;
    LUNA_CUDA_CHECK(cub::DeviceScan::InclusiveSum(cub_temp, cub_bytes, rowptr, rowptr, rows + 1, stream));
    degrees_and_iota<<<static_cast<unsigned>(ceil_div(rows, kThreads)), kThreads, 0, stream>>>(rowptr, rows, keys_in,
                                                                                              values_in);
    LUNA_LAUNCH_CHECK("graph degrees");
    cub_bytes = l.cub_bytes;
    LUNA_CUDA_CHECK(cub::DeviceRadixSort::SortPairsDescending(
        cub_temp, cub_bytes, static_cast<const int32_t*>(keys_in), keys_out, static_cast<const int32_t*>(values_in),
        order, rows, 0, degree_bits, stream));
  }
  return LUNA_OK;
}
