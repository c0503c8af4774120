// Implementation of sb_grpo_group_adv_noalloc (see grpo_adv_noalloc.h for the contract).
// It forwards to the regular entry point sb_grpo_group_adv with scratch pointers that point into a file-scope
// device array instead of caller-provided buffers.
#include <stdio.h>

#include "grpo_adv_noalloc.h"
#include "launchers.h"

namespace {

// Scratch of the allocation-free entry point: [0, MaxRows) per-row score sums, then 3 * MaxGroups floats of
// per-group count / sum / squared deviation.  256-byte aligned so both parts are float4-aligned.
static __device__ __align__(256) float g_grpo_noalloc_scratch[kGrpoNoAllocMaxRows + 3 * kGrpoNoAllocMaxGroups];

constexpr int kMaxDevices = 64;
// Device address of the scratch array per device ordinal.  In host code the name of a __device__ array is only a
// handle for the runtime, not an address a kernel can use, so the address is asked for once per device.
float* g_scratch_addr[kMaxDevices] = {nullptr};

int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return kGrpoNoAllocBadArgument;
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_grpo_noalloc_scratch);
    if (e != cudaSuccess) {
      fprintf(stderr, "sb_grpo_group_adv_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return (int)e;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" int sb_grpo_group_adv_noalloc(const float* rewards, const float* mask, const int* gid, float* adv, int B,
                                         int R, int G, float eps, int norm_by_std, cudaStream_t stream) {
  if (B < 0 || R < 0 || G < 0) return kGrpoNoAllocBadArgument;
  if (B == 0 || R == 0) return 0;
  if (!rewards || !mask || !gid || !adv || G == 0) return kGrpoNoAllocBadArgument;
  if (B > kGrpoNoAllocMaxRows || G > kGrpoNoAllocMaxGroups) {
    fprintf(stderr,
            "sb_grpo_group_adv_noalloc: B=%d rows / G=%d groups exceed the built-in scratch (max %d rows, %d groups); "
            "use sb_grpo_group_adv with caller-provided scratch instead\n",
            B, G, kGrpoNoAllocMaxRows, kGrpoNoAllocMaxGroups);
    return kGrpoNoAllocTooLarge;
  }
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  float* scores_ws = scratch;                        // [B]
  float* group_ws = scratch + kGrpoNoAllocMaxRows;   // [3 * G], cleared by the callee at the start of every call
  return sb_grpo_group_adv(rewards, mask, gid, scores_ws, group_ws, adv, B, R, G, eps, norm_by_std, stream);
}
