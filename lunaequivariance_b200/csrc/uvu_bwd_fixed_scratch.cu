// luna_uvu_conv_bwd_noalloc: the first-derivative entry point for callers that must not allocate device memory.
//
// Who needs it.  luna_uvu_conv_bwd wants a caller-provided scratch buffer whenever a feature block is wider than
// one warp covers (for example 128 channels in FP64), because every channel chunk then writes its own partial
// edge-attribute gradient.  Some hosts of this library cannot hand one over: a plugin that runs inside another
// program's step and owns no allocator there, a real-time loop where cudaMalloc's implicit device synchronisation
// is not acceptable, or a process whose memory pool was sized up front and is closed.  For them the partial rows
// live in a fixed array that is part of the library image.
//
// What it costs.  The array below takes kFixedScratchBytes of device memory on a GPU from the moment this part of
// the library is loaded there until the process exits.  With the CUDA runtime's default lazy loading that moment
// is luna_uvu_conv_noalloc_prepare (the set-up call, which looks the array up); with eager loading it is the
// creation of the context.  Either way it is never the hot call: luna_uvu_conv_bwd_noalloc refuses to run on a
// device that has not been prepared.  Requests that need more than the array are refused.  All calls on a device
// share the one array and it keeps whatever the previous call left in it: the
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

int current_device(int* device) {
  LUNA_CUDA_CHECK(cudaGetDevice(device));
  if (*device < 0 || *device >= kMaxDevices)
    return luna::fail(LUNA_ERR_UNSUPPORTED, "device ordinal %d is beyond the %d this entry point tracks", *device,
                      kMaxDevices);
  return LUNA_OK;
}

// Set-up: resolves the array's address on the current device, once per device.  This is where the runtime may load
// this module onto the device (and the array starts to occupy memory), so it belongs before any stream capture and
// outside the part of the program that must not allocate.
int resolve_fixed_scratch() {
  int device = 0;
  int rc = current_device(&device);
  if (rc != LUNA_OK) return rc;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_device_address[device] == nullptr) {
    void* address = nullptr;
    LUNA_CUDA_CHECK(cudaGetSymbolAddress(&address, g_fixed_scratch));
    if (address == nullptr) return luna::fail(LUNA_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_device_address[device] = address;
  }
  return LUNA_OK;
}

// The address resolved by the set-up call, or null if this device has not been prepared.  Touches no CUDA state
// beyond asking which device is current.
int fixed_scratch_address(void** out) {
  int device = 0;
  int rc = current_device(&device);
  if (rc != LUNA_OK) return rc;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
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

extern "C" int luna_uvu_conv_noalloc_prepare(luna_uvu_plan* plan) {
  luna::clear_error();
  if (!plan) return luna::fail(LUNA_ERR_INVALID_ARGUMENT, "null plan");
  int rc = resolve_fixed_scratch();
  if (rc != LUNA_OK) return rc;
  const luna::DeviceTables* tables = nullptr;
  return luna::get_device_tables(plan, &tables);  // uploads the plan's lookup tables (one cudaMalloc) if needed
}

extern "C" int luna_uvu_conv_bwd_noalloc(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y,
                                         const void* w, const void* g, void* gx, void* gy, void* gw, void* stream) {
  luna::clear_error();
  if (!plan) return luna::fail(LUNA_ERR_INVALID_ARGUMENT, "null plan");
  if (!graph) return luna::fail(LUNA_ERR_INVALID_ARGUMENT, "null graph");
  if (graph->num_nodes < 0 || graph->num_edges < 0) return luna::fail(LUNA_ERR_INVALID_ARGUMENT, "negative graph size");
  // nothing to compute (only gx rows to clear): no scratch, no tables
  if (graph->num_nodes == 0 || graph->num_edges == 0)
    return luna_uvu_conv_bwd(plan, graph, x, y, w, g, gx, gy, gw, nullptr, 0, stream);
  // Only the edge-attribute gradient goes through partial rows; without it no scratch is used at all.
  const int64_t need = gy ? luna_uvu_conv_scratch_bytes(plan, graph->num_nodes, graph->num_edges) : 0;
  if (need > kFixedScratchBytes)
    return luna::fail(LUNA_ERR_SCRATCH,
                      "this graph needs %lld bytes of scratch but the built-in array holds %lld: use "
                      "luna_uvu_conv_bwd with a caller-provided buffer",
                      static_cast<long long>(need), static_cast<long long>(kFixedScratchBytes));
  bool resident = false;
  int rc = plan_is_resident(plan, &resident);
  if (rc != LUNA_OK) return rc;
  void* scratch = nullptr;
  rc = fixed_scratch_address(&scratch);
  if (rc != LUNA_OK) return rc;
  if (!resident || scratch == nullptr)
    return luna::fail(LUNA_ERR_INVALID_ARGUMENT,
                      "this plan and device have not been prepared: the plan's tables are not on this device yet or "
                      "the built-in array has not been looked up, and doing either here could allocate.  Call "
                      "luna_uvu_conv_noalloc_prepare(plan) once per plan and device at set-up time");
  return luna_uvu_conv_bwd(plan, graph, x, y, w, g, gx, gy, gw, scratch, kFixedScratchBytes, stream);
}
