// Allocation-free GRPO group advantage.  This entry point has no counterpart in the reference framework.
//
// Who it is for: code that must compute group-normalised advantages at a moment when it cannot obtain device
// memory.  Examples are a host program that links this library without PyTorch and runs under a fixed memory
// budget, a step that executes while the rollout engine's KV arena and the trainer's pools already hold all
// free HBM (so a fresh cudaMalloc would fail or force a cache flush), and latency-sensitive loops where a
// driver allocation call is not acceptable.  The regular entry point, sb_grpo_group_adv, expects the caller to
// bring two scratch buffers; this one brings its own.
//
// The scratch lives in a fixed array in device memory that is part of the library image: every GPU that loads
// the library holds kGrpoNoAllocScratchBytes of it until the process exits, whether or not this function is
// ever called.
//
//   rewards, mask : [B, R] fp32 row-major (token-level rewards and response mask)
//   gid           : [B] int32 dense group id in [0, G)
//   adv           : [B, R] fp32 output, adv[b,t] = (s_b - mean_g) / (std_g + eps) * mask[b,t]
//                   (s_b = sum_t rewards[b,t]; unbiased std; a group of one uses mean 0, std 1;
//                   norm_by_std == 0 leaves out the division)
//
// A row whose gid lies outside [0, G) belongs to no group: the kernels skip it when they accumulate the group
// statistics (nothing is read or written out of bounds) and its advantage row is written as zeros.
//
// Limits: B <= kGrpoNoAllocMaxRows and G <= kGrpoNoAllocMaxGroups.  Larger sizes are refused with
// kGrpoNoAllocTooLarge and a message on stderr; nothing is launched.
//
// Return value: 0 on success; kGrpoNoAllocTooLarge; kGrpoNoAllocBadArgument (null pointer, negative size);
// otherwise the cudaError_t of the failing runtime call.
//
// The function calls no cudaMalloc / cudaFree and no allocating library routine.  It only enqueues work on
// `stream` (one memset and four kernels).
//
// First call on a device: the first call made while a given device is current looks up the device address of the
// scratch array for that device (a synchronous runtime query).  Make that first call outside any stream capture.
//
// Host threads: the per-device address cache is filled without a lock.  Two host threads that make their first call
// on the same device at the same time both look the address up and both store the same value, which is harmless;
// the GPU-side sharing rule below applies to them like to any two calls.
//
// Sharing: all calls on one device use the same scratch, which keeps whatever the previous call left; the part
// that must start from zero is cleared at the beginning of every call.  Two calls whose work overlaps on the GPU
// (different streams without an ordering between them) race on the scratch and give wrong results; order them.
#pragma once
#include <cuda_runtime.h>

#define kGrpoNoAllocMaxRows 16384
#define kGrpoNoAllocMaxGroups 16384
#define kGrpoNoAllocScratchBytes ((kGrpoNoAllocMaxRows + 3 * kGrpoNoAllocMaxGroups) * 4)
#define kGrpoNoAllocTooLarge (-4)
#define kGrpoNoAllocBadArgument (-3)

#ifdef __cplusplus
extern "C" {
#endif
int sb_grpo_group_adv_noalloc(const float* rewards, const float* mask, const int* gid, float* adv, int B, int R,
                              int G, float eps, int norm_by_std, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
