// Token sampling for the rollout engine: temperature sampling by the Gumbel-max trick (exact sampling from
// softmax(z/T) in one pass, no sort, no cumulative sum), greedy argmax, and the log-probability of the chosen
// token under the full tempered distribution.  Replaces the sampler inside vLLM/SGLang that the reference calls
// (siirl/engine/rollout/vllm_rollout/vllm_rollout_spmd.py:261-416).  The random stream is counter-based
// (Philox4x32-10 keyed by seed, indexed by (step, row, column); the step is a host value plus an optional
// device counter so that a captured CUDA graph draws fresh numbers on every replay), so tensor-parallel ranks that hold the same
// logits draw the same token without exchanging RNG state.
#include "common.cuh"
#include "launchers.h"

namespace sb {

__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

__device__ __forceinline__ float u32_to_open_unit(uint32_t x) {
  return ((float)(x >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
}

struct ArgStat {
  float best;   // best perturbed score
  int idx;
  float m, s;   // online max / sum for the log-sum-exp of the statistic logits
};

__device__ __forceinline__ ArgStat merge(const ArgStat a, const ArgStat b) {
  ArgStat o;
  if (b.best > a.best || (b.best == a.best && b.idx < a.idx && b.idx >= 0)) {
    o.best = b.best;
    o.idx = b.idx;
  } else {
    o.best = a.best;
    o.idx = a.idx;
  }
  if (a.m == -INFINITY) {
    o.m = b.m;
    o.s = b.s;
  } else if (b.m == -INFINITY) {
    o.m = a.m;
    o.s = a.s;
  } else {
    o.m = fmaxf(a.m, b.m);
    o.s = a.s * __expf(a.m - o.m) + b.s * __expf(b.m - o.m);
  }
  return o;
}

constexpr int kSampleThreads = 512;

// sample_logits: logits the token is drawn from (possibly truncated with -inf by top-k / top-p);
// stat_logits: logits that define the reported log-probability (normally the untruncated ones).
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ sample_logits, const float* __restrict__ stat_logits, long long ld,
              float inv_temp, int greedy, unsigned long long seed, unsigned long long step_host,
              const long long* __restrict__ step_dev, long long* __restrict__ tokens, float* __restrict__ logp, int V,
              int chunk, ArgStat* __restrict__ partial) {
  __shared__ ArgStat red[32];
  const int row = blockIdx.x;
  const int v_begin = blockIdx.y * chunk, v_end = min(V, v_begin + chunk);
  const unsigned long long step = step_host + (step_dev ? (unsigned long long)*step_dev : 0ull);
  const float* zs = sample_logits + (size_t)row * ld;
  const float* zt = stat_logits + (size_t)row * ld;
  ArgStat st = {-INFINITY, -1, -INFINITY, 0.f};
  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  for (int i = v_begin + threadIdx.x * 4; i < v_end; i += kSampleThreads * 4) {
    uint4 rnd = make_uint4(0, 0, 0, 0);
    if (!greedy) rnd = philox4x32_10(make_uint4((uint32_t)i, (uint32_t)row, (uint32_t)step, (uint32_t)(step >> 32)), key);
    const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = i + u;
      if (j >= v_end) break;
      const float x = zt[j] * inv_temp;
      if (x != -INFINITY) {
        if (x > st.m) {
          st.s = st.s * __expf(st.m - x) + 1.f;
          st.m = x;
        } else {
          st.s += __expf(x - st.m);
        }
      }
      const float xs = zs[j] * (greedy ? 1.f : inv_temp);
      if (xs == -INFINITY) continue;
      float score = xs;
      if (!greedy) score += -__logf(-__logf(u32_to_open_unit(rr[u])));
      if (score > st.best) {
        st.best = score;
        st.idx = j;
      }
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgStat other;
    other.best = __shfl_xor_sync(0xffffffffu, st.best, o);
    other.idx = __shfl_xor_sync(0xffffffffu, st.idx, o);
    other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, st.s, o);
    st = merge(st, other);
  }
  if (lane == 0) red[warp] = st;
  __syncthreads();
  if (warp == 0) {
    ArgStat w = lane < (kSampleThreads >> 5) ? red[lane] : ArgStat{-INFINITY, -1, -INFINITY, 0.f};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgStat other;
      other.best = __shfl_xor_sync(0xffffffffu, w.best, o);
      other.idx = __shfl_xor_sync(0xffffffffu, w.idx, o);
      other.m = __shfl_xor_sync(0xffffffffu, w.m, o);
      other.s = __shfl_xor_sync(0xffffffffu, w.s, o);
      w = merge(w, other);
    }
    if (lane == 0) {
      if (partial) {
        partial[(size_t)row * gridDim.y + blockIdx.y] = w;
      } else {
        const int tok = w.idx < 0 ? 0 : w.idx;
        tokens[row] = tok;
        if (logp) logp[row] = zt[tok] * inv_temp - (w.m + __logf(w.s));
      }
    }
  }
}

// merges the per-chunk partial results of one row (one warp per row)
__global__ void sample_merge_kernel(const ArgStat* __restrict__ partial, int splits, const float* __restrict__ stat_logits,
                                    long long ld, float inv_temp, long long* __restrict__ tokens,
                                    float* __restrict__ logp, int rows) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  ArgStat w = {-INFINITY, -1, -INFINITY, 0.f};
  for (int s = lane; s < splits; s += 32) w = merge(w, partial[(size_t)row * splits + s]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgStat other;
    other.best = __shfl_xor_sync(0xffffffffu, w.best, o);
    other.idx = __shfl_xor_sync(0xffffffffu, w.idx, o);
    other.m = __shfl_xor_sync(0xffffffffu, w.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, w.s, o);
    w = merge(w, other);
  }
  if (lane == 0) {
    const int tok = w.idx < 0 ? 0 : w.idx;
    tokens[row] = tok;
    if (logp) logp[row] = stat_logits[(size_t)row * ld + tok] * inv_temp - (w.m + __logf(w.s));
  }
}

}  // namespace sb

using namespace sb;

extern "C" int sb_sample(const float* sample_logits, const float* stat_logits, long long ld, float temperature,
                         unsigned long long seed, unsigned long long step, const long long* step_dev,
                         long long* tokens, float* logp, int rows, int V, void* workspace, int splits,
                         cudaStream_t stream) {
  if (rows == 0) return 0;
  const int greedy = temperature <= 0.f;
  const float inv_temp = greedy ? 1.f : 1.f / temperature;
  const float* zt = stat_logits ? stat_logits : sample_logits;
  if (!workspace || splits <= 1) {
    sample_kernel<<<rows, kSampleThreads, 0, stream>>>(sample_logits, zt, ld, inv_temp, greedy, seed, step, step_dev,
                                                       tokens, logp, V, V, nullptr);
    return (int)cudaGetLastError();
  }
  // vocabulary split over `splits` blocks per row (workspace: rows * splits * 16 bytes), then one merge warp per row
  const int chunk = ((V + splits - 1) / splits + 3) / 4 * 4;
  dim3 grid(rows, splits);
  sample_kernel<<<grid, kSampleThreads, 0, stream>>>(sample_logits, zt, ld, inv_temp, greedy, seed, step, step_dev,
                                                     tokens, logp, V, chunk, reinterpret_cast<ArgStat*>(workspace));
  sample_merge_kernel<<<(rows + 3) / 4, 128, 0, stream>>>(reinterpret_cast<const ArgStat*>(workspace), splits, zt, ld,
                                                          inv_temp, tokens, logp, rows);
  return (int)cudaGetLastError();
}
