// Flat-buffer AdamW and gradient-norm kernels for the sharded optimizer.
// Replaces torch.optim.AdamW + clip_grad_norm_ of the reference (siirl/engine/fsdp_workers.py:1022-1088,
// siirl/engine/actor/dp_actor.py:265-283).  All parameters of a model live in one flat bf16 buffer with an fp32
// gradient buffer beside it; each rank owns a contiguous shard of fp32 master weights and Adam moments.
//   sumsq_kernel    partial sum of squares of an fp32 range -> one float (atomicAdd), for the global grad norm
//   adamw_kernel    p_master, m, v update on the owned shard with the clip factor read from device memory
//                   (no host sync), writes the bf16 working copy; a non-finite norm skips the update,
//                   as the reference does.
#include "common.cuh"
#include "launchers.h"

namespace sb {

__global__ void sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  float s = 0.f;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(g)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const float v = g[n4 * 4 + threadIdx.x];
    s += v * v;
  }
  __shared__ float red[32];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) atomicAdd(out, t);
  }
}

struct AdamParams {
  float* master;           // fp32 [n] owned shard
  float* m;
  float* v;
  const float* grad;       // fp32 [n] (already reduced over data-parallel ranks)
  __nv_bfloat16* param;    // bf16 [n] working copy of the shard
  const float* sumsq;      // device scalar: global sum of squared gradients (before grad_scale)
  float* grad_norm_out;    // optional device scalar receiving the norm
  long long n;
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, max_norm, grad_scale;
};

__global__ void adamw_kernel(AdamParams p) {
  float clip = 1.f;
  bool skip = false;
  if (p.sumsq) {
    const float norm = sqrtf(*p.sumsq) * p.grad_scale;
    if (!isfinite(norm)) skip = true;
    else if (p.max_norm > 0.f) clip = fminf(1.f, p.max_norm / (norm + 1e-6f));
    if (p.grad_norm_out && blockIdx.x == 0 && threadIdx.x == 0) *p.grad_norm_out = norm;
  }
  if (skip) return;
  const float gs = p.grad_scale * clip;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.n; i += (long long)gridDim.x * blockDim.x) {
    const float g = p.grad[i] * gs;
    float w = p.master[i];
    const float m = p.beta1 * p.m[i] + (1.f - p.beta1) * g;
    const float v = p.beta2 * p.v[i] + (1.f - p.beta2) * g * g;
    w -= p.lr * p.weight_decay * w;
    w -= p.lr * (m / p.bc1) / (sqrtf(v / p.bc2) + p.eps);
    p.m[i] = m;
    p.v[i] = v;
    p.master[i] = w;
    p.param[i] = __float2bfloat16(w);
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16(src[i]);
}

}  // namespace sb

using namespace sb;

static int grid_cap(long long work, int threads, int per_sm) {
  long long b = (work + threads - 1) / threads;
  const long long cap = (long long)num_sms() * per_sm;
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

extern "C" int sb_sumsq_accumulate(const float* g, long long n, float* out, cudaStream_t stream) {
  if (n == 0) return 0;
  sumsq_kernel<<<grid_cap(n / 4 + 1, 256, 8), 256, 0, stream>>>(g, n, out);
  return (int)cudaGetLastError();
}

extern "C" int sb_adamw_step(float* master, float* m, float* v, const float* grad, void* param_bf16,
                             const float* sumsq, float* grad_norm_out, long long n, float lr, float beta1,
                             float beta2, float eps, float weight_decay, int step, float max_norm, float grad_scale,
                             cudaStream_t stream) {
  if (n == 0) return 0;
  AdamParams p;
  p.master = master; p.m = m; p.v = v; p.grad = grad; p.param = (__nv_bfloat16*)param_bf16;
  p.sumsq = sumsq; p.grad_norm_out = grad_norm_out; p.n = n;
  p.lr = lr; p.beta1 = beta1; p.beta2 = beta2; p.eps = eps; p.weight_decay = weight_decay;
  p.bc1 = 1.f - powf(beta1, (float)step);
  p.bc2 = 1.f - powf(beta2, (float)step);
  p.max_norm = max_norm; p.grad_scale = grad_scale;
  adamw_kernel<<<grid_cap(n, 256, 8), 256, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

extern "C" int sb_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t stream) {
  if (n == 0) return 0;
  cast_f32_bf16_kernel<<<grid_cap(n, 256, 8), 256, 0, stream>>>(src, (__nv_bfloat16*)dst, n);
  return (int)cudaGetLastError();
}
