// luna_uvu_conv_bwd_noalloc: the first-derivative entry point for callers that must not allocate device memory.
//
// Who needs it.  luna_uvu_conv_bwd wants a caller-provided scratch buffer whenever a feature block is wider than
// one warp covers (for example 128 channels in FP64), because every channel chunk then writes its own partial
// edge-attribute gradient.  Some hosts of this library cannot hand one over: a plugin that runs inside another
// program's step and owns no allocator there, a real-time loop where cudaMalloc's implicit device synchronisation
// is not acceptable, or a process whose memory pool was sized up front and is closed.  For them the partial rows
// live in a fixed array that is part of the library image.
//
// What it costs.  The array below takes kFixedScratchBytes of device memory on every GPU that loads the library,
// from load until the process exits, whether or not this entry point is ever called.  Requests that need more are
// refused.  All calls on a device share the one array and it keeps whatever the previous call left in it: the
// backward kernel overwrites every partial row it later reads, so nothing has to be cleared, but two calls that
// run at the same time on one GPU (different streams, or different host threads) would overwrite each other's
// partial rows.  Keep calls to this entry point on one device in stream order.
#include <mutex>

#include "plan.h"

namespace {

constexpr int64_t kFixedScratchBytes = 8ll << 20;  // 8 MiB per GPU
constexpr int kMaxDevices = 64;

// Device storage.  In host code this name is only a handle for the runtime, never a device address: the address
// the kernels get comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_fixed_scratch[kFixedScratchBytes];

std::mutex g_setup_mutex;
void* g_device_address[kMaxDevices] = {};

// Resolves the array's address on the current device, once per device.  Allocates nothing, but the first call on a
// device may make the runtime load this module there, so it belongs before any stream capture.
int fixed_scratch_address(void** out) {
  int device = 0;
  LUNA_CUDA_CHECK(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices)
    return luna::fail(LUNA_ERR_UNSUPPORTED, "device ordinal %d is beyond the %d this entry point tracks", device,
                      kMaxDevices);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_device_address[device] == nullptr) {
    void* address = nullptr;
    LUNA_CUDA_CHECK(cudaGetSymbolAddress(&address, g_fixed_scratch));
    if (address == nullptr) return luna::fail(LUNA_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_device_address[device] = address;
  }
  *out = g_device_address[device];
  return LUNA_OK;
}

// Whether the plan's lookup tables are already on the current device.  They are uploaded (one cudaMalloc) by the
// first call of any other entry point with this plan on the device; this one must not do that itself.
int plan_is_resident(luna_uvu_plan* plan, bool* resident) {
  int device = 0;
  LUNA_CUDA_CHECK(cudaGetDevice(&device));
  std::lock_guard<std::mutex> lock(plan->mutex);
  *resident = plan->device_tables.find(device) != plan->device_tables.end();
  return LUNA_OK;
}

}  // namespace

extern "C" int64_t luna_uvu_conv_noalloc_max_scratch_bytes(void) { return kFixedScratchBytes; }

extern "C" int luna_uvu_conv_bwd_noalloc(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y,
                                         const void* w, const void* g, void* gx, void* gy, void* gw, void* stream) {
  luna::clear_error();
  if (!plan) return luna::fail(LUNA_ERR_INVALID_ARGUMENT, "null plan");
  if (!graph) return luna::fail(LUNA_ERR_INVALID_ARGUMENT, "null graph");
  const int64_t need = luna_uvu_conv_scratch_bytes(plan, graph->num_nodes, graph->num_edges);
  if (need < 0) return luna::fail(LUNA_ERR_INVALID_ARGUMENT, "negative graph size");
  if (need > kFixedScratchBytes)
    return luna::fail(LUNA_ERR_SCRATCH,
                      "this graph needs %lld bytes of scratch but the built-in array holds %lld: use "
                      "luna_uvu_conv_bwd with a caller-provided buffer",
                      static_cast<long long>(need), static_cast<long long>(kFixedScratchBytes));
  bool resident = false;
  int rc = plan_is_resident(plan, &resident);
  if (rc != LUNA_OK) return rc;
  if (!resident)
    return luna::fail(LUNA_ERR_INVALID_ARGUMENT,
                      "the plan's tables are not on this device yet and uploading them would allocate: call "
                      "luna_uvu_check_status (or any other entry point) with this plan on this device once, at "
                      "set-up time");
  void* scratch = nullptr;
  rc = fixed_scratch_address(&scratch);
  if (rc != LUNA_OK) return rc;
  return luna_uvu_conv_bwd(plan, graph, x, y, w, g, gx, gy, gw, scratch, kFixedScratchBytes, stream);
}
