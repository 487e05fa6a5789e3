// Placeholder until the staged kernels are linked in.
#include "plan.h"
namespace luna {
bool fast_available() { return false; }
int64_t fast_smem_bytes(const luna_uvu_plan*, int) { return 0; }
int64_t fast_scratch_bytes(const luna_uvu_plan*, int64_t, int64_t) { return 0; }
int fast_forward(luna_uvu_plan*, const luna_graph*, const void*, const void*, const void*, const void*, const void*,
                 const void*, void*, bool, cudaStream_t) { return fail(LUNA_ERR_UNSUPPORTED, "staged kernels not built"); }
int fast_backward(luna_uvu_plan*, const luna_graph*, const void*, const void*, const void*, const void*, void*, bool,
                  void*, bool, void*, bool, void*, int64_t, cudaStream_t) { return fail(LUNA_ERR_UNSUPPORTED, "staged kernels not built"); }
}
