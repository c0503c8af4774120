// LM-head log-prob / entropy without keeping [tokens, vocab] probabilities around.
// Same contract as the reference's fused linear-cross-entropy family
// (siirl/utils/kernel/kernels.py:153-501 forward, :1124-1375 backward; wrapper
// siirl/utils/kernel/linear_cross_entropy.py:40-117): from hidden states and the vocabulary matrix
// produce, per token, log p(label) and the entropy of the tempered distribution.
//
// The vocabulary GEMM runs on the tcgen05 GEMM of gemm_tcgen05.cu over a chunk of tokens; the kernels here
// reduce a chunk of fp32 logits [rows, V] to the per-token statistics (one pass, online softmax) and, for
// backward, turn the same logits into bf16 d_logits in place of a second [rows, V] fp32 buffer:
//   z = logits / temperature,  p = softmax(z),  H = lse - sum p z
//   d z_j = g_logp * (1[j = y] - p_j) - g_H * p_j * (z_j - lse + H)
#include "common.cuh"
#include "launchers.h"

namespace sb {

constexpr int kLmThreads = 512;

struct OnlineStat {
  float m, s, t;  // running max, sum exp(z - m), sum exp(z - m) * z
};

__device__ __forceinline__ OnlineStat merge(const OnlineStat a, const OnlineStat b) {
  if (a.m == -INFINITY) return b;
  if (b.m == -INFINITY) return a;
  const float m = fmaxf(a.m, b.m);
  const float ea = __expf(a.m - m), eb = __expf(b.m - m);
  return {m, a.s * ea + b.s * eb, a.t * ea + b.t * eb};
}

__device__ __forceinline__ OnlineStat block_merge(OnlineStat v, OnlineStat* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    OnlineStat other;
    other.m = __shfl_xor_sync(0xffffffffu, v.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, v.s, o);
    other.t = __shfl_xor_sync(0xffffffffu, v.t, o);
    v = merge(v, other);
  }
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    OnlineStat w = lane < (blockDim.x >> 5) ? red[lane] : OnlineStat{-INFINITY, 0.f, 0.f};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      OnlineStat other;
      other.m = __shfl_xor_sync(0xffffffffu, w.m, o);
      other.s = __shfl_xor_sync(0xffffffffu, w.s, o);
      other.t = __shfl_xor_sync(0xffffffffu, w.t, o);
      w = merge(w, other);
    }
    if (lane == 0) red[0] = w;
  }
  __syncthreads();
  return red[0];
}

// One block per row.  labels < 0 produce logp = 0 (ignored token).
__global__ void __launch_bounds__(kLmThreads)
lmhead_stats_kernel(const float* __restrict__ logits, long long ld, const long long* __restrict__ labels,
                    float inv_temp, float* __restrict__ logp, float* __restrict__ entropy,
                    float* __restrict__ lse_out, int V) {
  __shared__ OnlineStat red[32];
  const int row = blockIdx.x;
  const float* z = logits + (size_t)row * ld;
  OnlineStat st = {-INFINITY, 0.f, 0.f};
  for (int i = threadIdx.x * 4; i < V; i += kLmThreads * 4) {
    float v[4];
    if (i + 4 <= V) {
      const float4 f = *reinterpret_cast<const float4*>(z + i);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = (i + u < V) ? z[i + u] : -INFINITY;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float x = v[u] * inv_temp;
      if (x == -INFINITY) continue;
      if (x > st.m) {
        const float e = __expf(st.m - x);
        st.s = st.s * e + 1.f;
        st.t = st.t * e + x;
        st.m = x;
      } else {
        const float e = __expf(x - st.m);
        st.s += e;
        st.t += e * x;
      }
    }
  }
  const OnlineStat tot = block_merge(st, red);
  if (threadIdx.x == 0) {
    const float lse = tot.m + __logf(tot.s);
    const long long y = labels[row];
    logp[row] = (y >= 0 && y < V) ? z[y] * inv_temp - lse : 0.f;
    if (entropy) entropy[row] = lse - tot.t / tot.s;
    if (lse_out) lse_out[row] = lse;
  }
}

// d_logits (bf16, row pitch ldd) from the recomputed logits of the same rows.
__global__ void __launch_bounds__(kLmThreads)
lmhead_dlogits_kernel(const float* __restrict__ logits, long long ld, const long long* __restrict__ labels,
                      const float* __restrict__ lse, const float* __restrict__ entropy,
                      const float* __restrict__ g_logp, const float* __restrict__ g_ent, float inv_temp,
                      __nv_bfloat16* __restrict__ dlogits, long long ldd, int V) {
  const int row = blockIdx.x;
  const float* z = logits + (size_t)row * ld;
  __nv_bfloat16* d = dlogits + (size_t)row * ldd;
  const long long y = labels[row];
  const float l = lse[row];
  const float glp = (y >= 0 && y < V) ? g_logp[row] : 0.f;
  const float ge = g_ent ? g_ent[row] : 0.f;
  const float H = entropy ? entropy[row] : 0.f;
  for (int i = threadIdx.x * 4; i < V; i += kLmThreads * 4) {
    float out[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = i + u;
      float g = 0.f;
      if (j < V) {
        const float x = z[j] * inv_temp;
        const float pj = __expf(x - l);
        g = glp * ((j == y ? 1.f : 0.f) - pj) - ge * pj * (x - l + H);
        g *= inv_temp;
      }
      out[u] = g;
    }
    if (i + 4 <= V) {
      uint2 o;
      o.x = pack_bf16x2(out[0], out[1]);
      o.y = pack_bf16x2(out[2], out[3]);
      *reinterpret_cast<uint2*>(d + i) = o;
    } else {
      for (int u = 0; u < 4 && i + u < V; ++u) d[i + u] = __float2bfloat16(out[u]);
    }
  }
}

// Folds the per-tile partial statistics written by the vocabulary GEMM's epilogue (EPI_LMSTAT in gemm_tcgen05.cu):
// partial[row, tile] = (max, sum exp(z - max), sum exp(z - max) * z, z[label] or -inf).  One warp per row.
__global__ void lmhead_merge_kernel(const float4* __restrict__ partial, int tiles, const long long* __restrict__ labels,
                                    float* __restrict__ logp, float* __restrict__ entropy, float* __restrict__ lse_out,
                                    int rows, int V) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  OnlineStat st = {-INFINITY, 0.f, 0.f};
  float zl = -INFINITY;
  for (int t = lane; t < tiles; t += 32) {
    const float4 q = partial[(size_t)row * tiles + t];
    st = merge(st, OnlineStat{q.x, q.y, q.z});
    zl = fmaxf(zl, q.w);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    OnlineStat other;
    other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, st.s, o);
    other.t = __shfl_xor_sync(0xffffffffu, st.t, o);
    st = merge(st, other);
    zl = fmaxf(zl, __shfl_xor_sync(0xffffffffu, zl, o));
  }
  if (lane == 0) {
    const float lse = st.m + __logf(st.s);
    const long long y = labels[row];
    logp[row] = (y >= 0 && y < V && zl != -INFINITY) ? zl - lse : 0.f;
    if (entropy) entropy[row] = lse - st.t / st.s;
    if (lse_out) lse_out[row] = lse;
  }
}

}  // namespace sb

using namespace sb;

extern "C" int sb_lmhead_merge(const void* partial, int tiles, const long long* labels, float* logp, float* entropy,
                               float* lse, int rows, int V, cudaStream_t stream) {
  if (rows == 0) return 0;
  lmhead_merge_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(reinterpret_cast<const float4*>(partial), tiles, labels, logp,
                                                         entropy, lse, rows, V);
  return (int)cudaGetLastError();
}

extern "C" int sb_lmhead_stats(const float* logits, long long ld, const long long* labels, float inv_temp,
                               float* logp, float* entropy, float* lse, int rows, int V, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (ld % 4) return -3;
  lmhead_stats_kernel<<<rows, kLmThreads, 0, stream>>>(logits, ld, labels, inv_temp, logp, entropy, lse, V);
  return (int)cudaGetLastError();
}

extern "C" int sb_lmhead_dlogits(const float* logits, long long ld, const long long* labels, const float* lse,
                                 const float* entropy, const float* g_logp, const float* g_ent, float inv_temp,
                                 void* dlogits, long long ldd, int rows, int V, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (ld % 4 || ldd % 4) return -3;
  lmhead_dlogits_kernel<<<rows, kLmThreads, 0, stream>>>(logits, ld, labels, lse, entropy, g_logp, g_ent, inv_temp,
                                                         (__nv_bfloat16*)dlogits, ldd, V);
  return (int)cudaGetLastError();
}
