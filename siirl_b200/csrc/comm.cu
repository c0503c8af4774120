// Peer-memory (NVLink 5 / NVSwitch) runtime and the fused collective kernels built on it.
//
// The reference moves every tensor between GPUs with NCCL through torch.distributed / FSDP / Megatron
// (siirl/dag_worker/dagworker.py:714-762, siirl/engine/fsdp_workers.py:897-1020) and every sample through the Ray
// object store (dagworker.py:1117-1239).  Here each rank maps its peers' buffers (CUDA IPC) and kernels read or
// write peer HBM directly with plain loads / stores, so the transfer is part of the kernel that does the math:
//
//   rs_reduce_kernel          gradient reduce-scatter: pulls this rank's shard of the fp32 gradient from every
//                             peer, sums, writes the reduced shard locally and accumulates ||g||^2
//   adamw_allgather_kernel    AdamW on the owned shard (clip factor from the global norm, read from device memory)
//                             and all-gather of the result: the new bf16 parameters are stored straight into every
//                             peer's replica
//   segment_pull_kernel       variable-length all-to-all-v / re-shard: copies a table of (peer, src offset,
//                             dst offset, bytes) segments from peer buffers into a local buffer in one launch
//                             (Data-Coordinator sample redistribution, train->rollout weight re-layout)
//   flag_barrier_kernel       cross-GPU barrier on epoch-tagged flags with a bounded wait (status word on timeout)
//
// No kernel here waits on another GPU except flag_barrier_kernel, and that wait is bounded.
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include "launchers.h"

namespace sb {

constexpr int kMaxRanks = 16;

struct PeerPtrs {
  void* p[kMaxRanks];
};

// ---------------------------------------------------------------------------------------
// reduce-scatter (pull) + squared norm
// ---------------------------------------------------------------------------------------
// `status` (optional): the device's status word.  When an earlier kernel of the stream gave up a bounded wait (the
// barrier in front of this reduction, for one) the peers' gradients may be incomplete: the squared norm is made
// infinite, which the ranks share through the norm all-reduce, so that every rank skips this optimizer step.
// `accumulate`: out_shard += sum instead of out_shard = sum (per-layer reductions of a sharded-parameter store, one per
// micro-batch); `sumsq` may be null then.
__global__ void rs_reduce_kernel(PeerPtrs grads, int world, int rank, long long lo, long long n,
                                 float* __restrict__ out_shard, float* __restrict__ sumsq, const int* status,
                                 int accumulate) {
  float ss = 0.f;
  if (sumsq && status && blockIdx.x == 0 && threadIdx.x == 0 &&
      *reinterpret_cast<const volatile int*>(status) != 0)
    atomicAdd(sumsq, __int_as_float(0x7f800000));
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < world; ++k) {
      const int r = (rank + 1 + k) % world;  // start at a different peer on every rank to spread the traffic
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + lo)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (accumulate) {
      const float4 o = reinterpret_cast<const float4*>(out_shard)[i];
      acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
    }
    reinterpret_cast<float4*>(out_shard)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  if (!sumsq) return;
  __shared__ float red[32];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) atomicAdd(sumsq, t);
  }
}

// ---------------------------------------------------------------------------------------
// AdamW on the shard + all-gather by peer stores
// ---------------------------------------------------------------------------------------
struct AdamAgParams {
  float *master, *m, *v;
  const float* grad;     // reduced shard
  PeerPtrs params;       // bf16 flat parameter buffer of every rank
  const float* sumsq;    // global sum of squares (already all-reduced)
  float* grad_norm_out;
  long long lo, n;
  int world;
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, max_norm, grad_scale;
};

__global__ void adamw_allgather_kernel(AdamAgParams p) {
  float clip = 1.f;
  bool skip = false;
  const float norm = sqrtf(*p.sumsq) * p.grad_scale;
  if (!isfinite(norm)) skip = true;
  else if (p.max_norm > 0.f) clip = fminf(1.f, p.max_norm / (norm + 1e-6f));
  if (p.grad_norm_out && blockIdx.x == 0 && threadIdx.x == 0) *p.grad_norm_out = norm;
  if (skip) return;
  const float gs = p.grad_scale * clip;
  const long long n8 = p.n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float w[8], g[8], m[8], v[8];
    *reinterpret_cast<float4*>(w) = reinterpret_cast<const float4*>(p.master)[2 * i];
    *reinterpret_cast<float4*>(w + 4) = reinterpret_cast<const float4*>(p.master)[2 * i + 1];
    *reinterpret_cast<float4*>(g) = reinterpret_cast<const float4*>(p.grad)[2 * i];
    *reinterpret_cast<float4*>(g + 4) = reinterpret_cast<const float4*>(p.grad)[2 * i + 1];
    *reinterpret_cast<float4*>(m) = reinterpret_cast<const float4*>(p.m)[2 * i];
    *reinterpret_cast<float4*>(m + 4) = reinterpret_cast<const float4*>(p.m)[2 * i + 1];
    *reinterpret_cast<float4*>(v) = reinterpret_cast<const float4*>(p.v)[2 * i];
    *reinterpret_cast<float4*>(v + 4) = reinterpret_cast<const float4*>(p.v)[2 * i + 1];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = g[k] * gs;
      m[k] = p.beta1 * m[k] + (1.f - p.beta1) * gk;
      v[k] = p.beta2 * v[k] + (1.f - p.beta2) * gk * gk;
      w[k] -= p.lr * p.weight_decay * w[k];
      w[k] -= p.lr * (m[k] / p.bc1) / (sqrtf(v[k] / p.bc2) + p.eps);
    }
    reinterpret_cast<float4*>(p.master)[2 * i] = *reinterpret_cast<float4*>(w);
    reinterpret_cast<float4*>(p.master)[2 * i + 1] = *reinterpret_cast<float4*>(w + 4);
    reinterpret_cast<float4*>(p.m)[2 * i] = *reinterpret_cast<float4*>(m);
    reinterpret_cast<float4*>(p.m)[2 * i + 1] = *reinterpret_cast<float4*>(m + 4);
    reinterpret_cast<float4*>(p.v)[2 * i] = *reinterpret_cast<float4*>(v);
    reinterpret_cast<float4*>(p.v)[2 * i + 1] = *reinterpret_cast<float4*>(v + 4);
    uint4 o;
    o.x = pack_bf16x2(w[0], w[1]);
    o.y = pack_bf16x2(w[2], w[3]);
    o.z = pack_bf16x2(w[4], w[5]);
    o.w = pack_bf16x2(w[6], w[7]);
    for (int r = 0; r < p.world; ++r)
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.params.p[r]) + p.lo)[i] = o;
  }
  __threadfence_system();
}

// ---------------------------------------------------------------------------------------
// segment pull: out[dst_off .. +bytes) = peer[src_rank][src_off .. +bytes); 16-byte granularity
// ---------------------------------------------------------------------------------------
struct Segment {
  long long src_off, dst_off, bytes;
  int src_rank, pad;
};

__global__ void segment_pull_kernel(PeerPtrs bases, const Segment* __restrict__ segs, int n_segs,
                                    unsigned char* __restrict__ out) {
  for (int s = blockIdx.y; s < n_segs; s += gridDim.y) {
    const Segment sg = segs[s];
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(bases.p[sg.src_rank]) + sg.src_off);
    uint4* dst = reinterpret_cast<uint4*>(out + sg.dst_off);
    const long long nv = sg.bytes / 16;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x)
      dst[i] = src[i];
  }
}

// ---------------------------------------------------------------------------------------
// flag barrier: flags[r] on every rank is an int slot per peer; epoch-tagged so a stale value never matches
// ---------------------------------------------------------------------------------------
// `limit_ns` bounds the wait: a barrier is where ranks absorb their skew (seconds after long independent phases),
// so its limit is a launch parameter instead of the short limit of waits inside compute kernels.
__global__ void flag_barrier_kernel(PeerPtrs flags, int world, int rank, int epoch, int* status,
                                    unsigned long long limit_ns) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    flag_store_release(reinterpret_cast<int*>(flags.p[t]) + rank, epoch);  // tell peer t that this rank arrived
    const int* mine = reinterpret_cast<int*>(flags.p[rank]) + t;
    const uint64_t t0 = global_timer_ns();
    bool ok = false;
    while (!ok) {
#pragma unroll 1
      for (int i = 0; i < 64 && !ok; ++i) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        ok = v >= epoch;
        if (!ok) __nanosleep(128);
      }
      if (!ok && global_timer_ns() - t0 > limit_ns) {
        if (status) atomicCAS(status, 0, (int)kStatusTimeoutFlag);
        break;
      }
    }
  }
  __syncthreads();
}

}  // namespace sb

using namespace sb;

static PeerPtrs to_peers(void* const* ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < kMaxRanks; ++i) pp.p[i] = i < world ? ptrs[i] : nullptr;
  return pp;
}

static int comm_grid(long long work, int threads, int per_sm) {
  long long b = (work + threads - 1) / threads;
  const long long cap = (long long)num_sms() * per_sm;
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

// ---- raw symmetric allocations and IPC handles -------------------------------------------------
extern "C" int sb_symm_alloc(void** out, long long bytes) { return (int)cudaMalloc(out, (size_t)bytes); }
extern "C" int sb_symm_free(void* p) { return (int)cudaFree(p); }
extern "C" int sb_ipc_get_handle(void* p, unsigned char* out64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(out64, &h, sizeof(h));
  return 0;
}
extern "C" int sb_ipc_open_handle(const unsigned char* in64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, in64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int sb_ipc_close_handle(void* p) { return (int)cudaIpcCloseMemHandle(p); }
extern "C" int sb_ipc_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }

// ---- fused collectives ---------------------------------------------------------------------------
extern "C" int sb_rs_reduce(void* const* grad_ptrs, int world, int rank, long long lo, long long n, float* out_shard,
                            float* sumsq, const int* status, cudaStream_t stream) {
  if (world > kMaxRanks || (n % 4) || (lo % 4)) return -3;
  if (n == 0) return 0;
  rs_reduce_kernel<<<comm_grid(n / 4, 256, 4), 256, 0, stream>>>(to_peers(grad_ptrs, world), world, rank, lo, n,
                                                                 out_shard, sumsq, status, 0);
  return (int)cudaGetLastError();
}

// out_shard[0, n) += sum over ranks of grads[r][lo, lo + n): the gradient reduce-scatter of one parameter unit
extern "C" int sb_rs_reduce_acc(void* const* grad_ptrs, int world, int rank, long long lo, long long n,
                                float* out_shard, cudaStream_t stream) {
  if (world > kMaxRanks || (n % 4) || (lo % 4)) return -3;
  if (n == 0) return 0;
  rs_reduce_kernel<<<comm_grid(n / 4, 256, 4), 256, 0, stream>>>(to_peers(grad_ptrs, world), world, rank, lo, n,
                                                                 out_shard, nullptr, nullptr, 1);
  return (int)cudaGetLastError();
}

extern "C" int sb_adamw_allgather(float* master, float* m, float* v, const float* grad, void* const* param_ptrs,
                                  int world, const float* sumsq, float* grad_norm_out, long long lo, long long n,
                                  float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                                  float max_norm, float grad_scale, cudaStream_t stream) {
  if (world > kMaxRanks || (n % 8) || (lo % 8)) return -3;
  if (n == 0) return 0;
  AdamAgParams p;
  p.master = master; p.m = m; p.v = v; p.grad = grad; p.params = to_peers(param_ptrs, world);
  p.sumsq = sumsq; p.grad_norm_out = grad_norm_out; p.lo = lo; p.n = n; p.world = world;
  p.lr = lr; p.beta1 = beta1; p.beta2 = beta2; p.eps = eps; p.weight_decay = weight_decay;
  p.bc1 = 1.f - powf(beta1, (float)step); p.bc2 = 1.f - powf(beta2, (float)step);
  p.max_norm = max_norm; p.grad_scale = grad_scale;
  adamw_allgather_kernel<<<comm_grid(n / 8, 256, 4), 256, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// strided block pull: the two all-to-alls of Ulysses sequence parallelism (sequence shard <-> head shard) as one
// launch each.  A block copies `rows` rows of `col_bytes` bytes from a peer's matrix into the local one; pitches
// and offsets are bytes, all multiples of 16.
// ---------------------------------------------------------------------------------------
struct PullBlock {
  long long src_off, dst_off;       // byte offset of the block's first element
  long long src_pitch, dst_pitch;   // row pitches in bytes
  int rows, col_bytes, src_rank, pad;
};
constexpr int kMaxPullBlocks = 64;
struct PullBlocks {
  PullBlock b[kMaxPullBlocks];
};

__global__ void block_pull_kernel(PeerPtrs bases, PullBlocks blocks, int n_blocks, unsigned char* __restrict__ out) {
  const PullBlock& blk = blocks.b[blockIdx.y];
  const unsigned char* src = reinterpret_cast<const unsigned char*>(bases.p[blk.src_rank]) + blk.src_off;
  unsigned char* dst = out + blk.dst_off;
  const int vec_per_row = blk.col_bytes / 16;
  const long long total = (long long)blk.rows * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int v = (int)(i % vec_per_row);
    *reinterpret_cast<uint4*>(dst + r * blk.dst_pitch + v * 16) =
        *reinterpret_cast<const uint4*>(src + r * blk.src_pitch + v * 16);
  }
}

// blocks: host array of n_blocks PullBlock (48 bytes each)
extern "C" int sb_block_pull(void* const* bases, int world, const void* blocks, int n_blocks, void* out,
                             cudaStream_t stream) {
  if (world > kMaxRanks || n_blocks > kMaxPullBlocks) return -3;
  if (n_blocks == 0) return 0;
  PullBlocks pb;
  memcpy(pb.b, blocks, sizeof(PullBlock) * n_blocks);
  dim3 grid(148 * 4 / n_blocks > 0 ? 148 * 4 / n_blocks : 1, n_blocks);
  block_pull_kernel<<<grid, 256, 0, stream>>>(to_peers(bases, world), pb, n_blocks, reinterpret_cast<unsigned char*>(out));
  return (int)cudaGetLastError();
}

// segs: device array of {src_off, dst_off, bytes, src_rank, pad} (32 bytes each); all offsets / sizes multiples of 16
extern "C" int sb_segment_pull(void* const* bases, int world, const void* segs, int n_segs, void* out,
                               cudaStream_t stream) {
  if (world > kMaxRanks) return -3;
  if (n_segs == 0) return 0;
  // enough CTAs to keep the NVLink loads of all SMs busy whether the table has two large segments (a parameter
  // gather) or thousands of small ones (sample redistribution)
  const int gy = n_segs < 2048 ? n_segs : 2048;
  int gx = (num_sms() * 8 + gy - 1) / gy;
  if (gx < 1) gx = 1;
  if (gx > 1024) gx = 1024;
  dim3 grid(gx, gy);
  segment_pull_kernel<<<grid, 256, 0, stream>>>(to_peers(bases, world), reinterpret_cast<const Segment*>(segs), n_segs,
                                                reinterpret_cast<unsigned char*>(out));
  return (int)cudaGetLastError();
}

extern "C" int sb_flag_barrier(void* const* flag_ptrs, int world, int rank, int epoch, int* status,
                               long long limit_ms, cudaStream_t stream) {
  if (world > kMaxRanks) return -3;
  if (limit_ms <= 0) limit_ms = 2000;
  flag_barrier_kernel<<<1, 32, 0, stream>>>(to_peers(flag_ptrs, world), world, rank, epoch, status,
                                            (unsigned long long)limit_ms * 1000000ull);
  return (int)cudaGetLastError();
}
