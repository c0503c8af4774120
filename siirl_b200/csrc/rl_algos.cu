// RL post-processing kernels over [B, R] response-token tensors:
//   gae_scan           reverse scan of generalised advantage estimation with carry-through on masked
//                      tokens (replaces the per-token Python loop of siirl/dag_worker/core_algos.py:229-276)
//   grpo_group_adv     group-normalised outcome advantage by prompt group
//                      (replaces the per-uid Python dict loop of core_algos.py:279-348)
//   ppo_token_loss     fused clipped-surrogate (+dual clip / GSPO / CPGD) + low-variance KL + entropy bonus:
//                      forward metrics and d(loss)/d(logp) in one pass (core_algos.py:710-862, dp_actor.py:468-501)
#include "common.cuh"
#include "launchers.h"

namespace sb {

// ---------------------------------------------------------------------------------------
// GAE.  One warp per row.  Both recurrences are affine maps composed right-to-left:
//   nv_t  = (1-m_t) * nv_{t+1} + m_t * V_t                      (value of the next valid token)
//   L_t   = (1-m_t + m_t*g*l) * L_{t+1} + m_t * delta_t,  delta_t = r_t + g*nv_{t+1} - V_t
// A chunk of 32 tokens is loaded coalesced, scanned with shuffles, and the carry moves to the next chunk.
// ---------------------------------------------------------------------------------------
struct Affine {
  float a, b;  // x -> a*x + b
};
// f after g  (apply g first, then f)
__device__ __forceinline__ Affine compose(const Affine f, const Affine g) { return {f.a * g.a, f.a * g.b + f.b}; }

// Inclusive scan from the right: lane i obtains the composition f_i o f_{i+1} o ... o f_31.
__device__ __forceinline__ Affine warp_scan_from_right(Affine f) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    Affine other;
    other.a = __shfl_down_sync(0xffffffffu, f.a, o);
    other.b = __shfl_down_sync(0xffffffffu, f.b, o);
    if (lane + o < 32) f = compose(f, other);
  }
  return f;
}

__global__ void gae_scan_kernel(const float* __restrict__ rewards, const float* __restrict__ values,
                                const float* __restrict__ mask, float* __restrict__ adv, float* __restrict__ ret,
                                int B, int R, float gamma, float lam) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= B) return;
  const size_t base = (size_t)warp * R;
  float nv_carry = 0.f, gae_carry = 0.f;
  const int nchunks = (R + 31) / 32;
  for (int c = nchunks - 1; c >= 0; --c) {
    const int t = c * 32 + lane;
    const bool in = t < R;
    const float m = in ? mask[base + t] : 0.f;
    const float v = in ? values[base + t] : 0.f;
    const float r = in ? rewards[base + t] : 0.f;
    // next-valid-value recurrence
    Affine fnv = {1.f - m, m * v};
    Affine snv = warp_scan_from_right(fnv);
    const float nv_incl = snv.a * nv_carry + snv.b;  // nv_t
    float nv_next = __shfl_down_sync(0xffffffffu, nv_incl, 1);
    if (lane == 31) nv_next = nv_carry;  // nv_{t+1}
    const float delta = r + gamma * nv_next - v;
    Affine fg = {1.f - m + m * gamma * lam, m * delta};
    Affine sg = warp_scan_from_right(fg);
    const float g = sg.a * gae_carry + sg.b;
    if (in) {
      adv[base + t] = g;
      ret[base + t] = g + v;
    }
    nv_carry = __shfl_sync(0xffffffffu, nv_incl, 0);
    gae_carry = __shfl_sync(0xffffffffu, g, 0);
  }
}

// ---------------------------------------------------------------------------------------
// GRPO group advantage
// ---------------------------------------------------------------------------------------
__global__ void row_sum_kernel(const float* __restrict__ x, float* __restrict__ out, int B, int R) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= B) return;
  float s = 0.f;
  for (int t = lane; t < R; t += 32) s += x[(size_t)warp * R + t];
  s = warp_sum(s);
  if (lane == 0) out[warp] = s;
}

// ws layout: [0,G) count, [G,2G) sum, [2G,3G) sum of squared deviations
__global__ void group_accum_kernel(const float* __restrict__ scores, const int* __restrict__ gid, float* ws, int B,
                                   int G, int pass) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B) return;
  const int g = gid[i];
  if (g < 0 || g >= G) return;
  if (pass == 0) {
    atomicAdd(&ws[g], 1.f);
    atomicAdd(&ws[G + g], scores[i]);
  } else {
    const float mean = ws[G + g] / fmaxf(ws[g], 1.f);
    const float d = scores[i] - mean;
    atomicAdd(&ws[2 * G + g], d * d);
  }
}

__global__ void grpo_apply_kernel(const float* __restrict__ scores, const int* __restrict__ gid,
                                  const float* __restrict__ ws, const float* __restrict__ mask,
                                  float* __restrict__ adv, int B, int R, int G, float eps, int norm_by_std) {
  const int row = blockIdx.y;
  const int g = gid[row];
  float a = 0.f;
  if (g >= 0 && g < G) {
    const float cnt = ws[g];
    float mean = ws[G + g] / fmaxf(cnt, 1.f);
    float sd = sqrtf(ws[2 * G + g] / fmaxf(cnt - 1.f, 1.f));
    if (cnt <= 1.f) {
      mean = 0.f;
      sd = 1.f;
    }
    a = norm_by_std ? (scores[row] - mean) / (sd + eps) : (scores[row] - mean);
  }
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < R; t += gridDim.x * blockDim.x)
    adv[(size_t)row * R + t] = a * mask[(size_t)row * R + t];
}

// ---------------------------------------------------------------------------------------
// Fused PPO token loss.
// mode: 0 vanilla (dual clip), 1 gspo (needs seq_logratio[B]), 2 cpgd.
// w_row[b] is the aggregation weight of every token of row b (e.g. 1/sum(mask) for token-mean), so that
// loss = sum_bt w_row[b] * m_bt * l_bt.  Outputs: dlogp[B,R] (gradient of the total scalar loss wrt logp,
// already multiplied by loss_scale) and stats[8] accumulated with atomics:
//   0 pg_loss  1 clipfrac_num  2 ppo_kl_num  3 clipfrac_lower_num  4 kl_loss  5 entropy_loss  6 mask_sum
// d(entropy term) is returned separately as dentropy[B,R] = -entropy_coeff * w * m * loss_scale.
// ---------------------------------------------------------------------------------------
struct PpoParams {
  const float *logp, *old_logp, *adv, *mask, *ref_logp, *entropy, *w_row, *seq_logratio;
  float *dlogp, *dentropy, *stats;
  int B, R, mode;
  float clip_lo, clip_hi, clip_c, kl_coef, entropy_coef, loss_scale;
  int use_kl;  // 0 none, 1 low_var_kl, 2 kl (k1), 3 abs, 4 mse
};

__global__ void ppo_token_loss_kernel(PpoParams p) {
  float acc[7] = {0, 0, 0, 0, 0, 0, 0};
  const long long total = (long long)p.B * p.R;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(idx / p.R);
    const float m = p.mask[idx];
    float dl = 0.f, de = 0.f;
    if (m != 0.f) {
      const float w = p.w_row[b] * m;
      const float lp = p.logp[idx], old = p.old_logp[idx], A = p.adv[idx];
      float loss = 0.f, g = 0.f;  // token loss and d loss / d logp
      const float raw = lp - old;
      if (p.mode == 0) {
        const float nk = fminf(fmaxf(raw, -20.f), 20.f);
        const float ratio = __expf(nk);
        const float dr = (raw > -20.f && raw < 20.f) ? ratio : 0.f;  // d ratio / d logp
        const float l1 = -A * ratio;
        const float rc = fminf(fmaxf(ratio, 1.f - p.clip_lo), 1.f + p.clip_hi);
        const float l2 = -A * rc;
        const bool rc_active = (ratio > 1.f - p.clip_lo) && (ratio < 1.f + p.clip_hi);
        float c1, g1;
        if (l2 > l1) {
          c1 = l2;
          g1 = rc_active ? -A * dr : 0.f;
          acc[1] += m;
        } else {
          c1 = l1;
          g1 = -A * dr;
        }
        if (A < 0.f) {
          const float l3 = -A * p.clip_c;
          if (c1 > l3) {
            acc[3] += m;
            loss = l3;
            g = 0.f;
          } else {
            loss = c1;
            g = g1;
          }
        } else {
          loss = c1;
          g = g1;
        }
        acc[2] += -nk * m;
      } else if (p.mode == 1) {
        // token ratio has the value of the sequence ratio s_b and the gradient s_b * dlogp (clamped at e^10)
        const float lsr = fminf(p.seq_logratio[b], 10.f);
        const float ratio = __expf(lsr);
        const float dr = p.seq_logratio[b] < 10.f ? ratio : 0.f;
        const float l1 = -A * ratio;
        const float rc = fminf(fmaxf(ratio, 1.f - p.clip_lo), 1.f + p.clip_hi);
        const float l2 = -A * rc;
        const bool rc_active = (ratio > 1.f - p.clip_lo) && (ratio < 1.f + p.clip_hi);
        if (l2 > l1) {
          loss = l2;
          g = rc_active ? -A * dr : 0.f;
          acc[1] += m;
        } else {
          loss = l1;
          g = -A * dr;
        }
        acc[2] += -raw * m;
      } else {
        const float up = old + log1pf(p.clip_hi), dn = old + log1pf(-p.clip_lo);
        float cl;
        bool active;
        if (A > 0.f) {
          active = lp <= up;
          cl = active ? lp : up;
          if (!active) acc[1] += m;
        } else {
          active = lp >= dn;
          cl = active ? lp : dn;
          if (!active) acc[3] += m;
        }
        loss = -cl * A;
        g = active ? -A : 0.f;
        acc[2] += -raw * m;
      }
      acc[0] += w * loss;
      dl = w * g;
      if (p.use_kl) {
        const float ref = p.ref_logp[idx];
        float kl = 0.f, gk = 0.f;
        if (p.use_kl == 1) {
          const float kraw = ref - lp;
          const float k = fminf(fmaxf(kraw, -20.f), 20.f);
          const float e = __expf(k);
          const float val = e - k - 1.f;
          kl = fminf(fmaxf(val, -10.f), 10.f);
          const bool inner = kraw > -20.f && kraw < 20.f;
          const bool outer = val > -10.f && val < 10.f;
          gk = (inner && outer) ? -(e - 1.f) : 0.f;
        } else if (p.use_kl == 2) {
          kl = lp - ref;
          gk = 1.f;
        } else if (p.use_kl == 3) {
          kl = fabsf(lp - ref);
          gk = lp > ref ? 1.f : (lp < ref ? -1.f : 0.f);
        } else {
          kl = 0.5f * (lp - ref) * (lp - ref);
          gk = lp - ref;
        }
        acc[4] += w * kl;
        dl += p.kl_coef * w * gk;
      }
      if (p.entropy) {
        acc[5] += w * p.entropy[idx];
        de = -p.entropy_coef * w;
      }
      acc[6] += m;
    }
    p.dlogp[idx] = dl * p.loss_scale;
    if (p.dentropy) p.dentropy[idx] = de * p.loss_scale;
  }
  __shared__ float red[7][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 7; ++i) {
    const float v = warp_sum(acc[i]);
    if (lane == 0) red[i][warp] = v;
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int i = 0; i < 7; ++i) {
      float v = lane < (blockDim.x >> 5) ? red[i][lane] : 0.f;
      v = warp_sum(v);
      if (lane == 0) atomicAdd(&p.stats[i], v);
    }
  }
}

}  // namespace sb

using namespace sb;

extern "C" int sb_gae_scan(const float* rewards, const float* values, const float* mask, float* adv, float* ret,
                           int B, int R, float gamma, float lam, cudaStream_t stream) {
  if (B == 0 || R == 0) return 0;
  const int threads = 128;
  const int blocks = (B * 32 + threads - 1) / threads;
  gae_scan_kernel<<<blocks, threads, 0, stream>>>(rewards, values, mask, adv, ret, B, R, gamma, lam);
  return (int)cudaGetLastError();
}

extern "C" int sb_grpo_group_adv(const float* rewards, const float* mask, const int* gid, float* scores_ws,
                                 float* group_ws, float* adv, int B, int R, int G, float eps, int norm_by_std,
                                 cudaStream_t stream) {
  if (B == 0 || R == 0) return 0;
  const cudaError_t me = cudaMemsetAsync(group_ws, 0, sizeof(float) * 3 * G, stream);
  if (me != cudaSuccess) return (int)me;
  row_sum_kernel<<<(B * 32 + 127) / 128, 128, 0, stream>>>(rewards, scores_ws, B, R);
  group_accum_kernel<<<(B + 127) / 128, 128, 0, stream>>>(scores_ws, gid, group_ws, B, G, 0);
  group_accum_kernel<<<(B + 127) / 128, 128, 0, stream>>>(scores_ws, gid, group_ws, B, G, 1);
  dim3 grid((R + 255) / 256 > 8 ? 8 : (R + 255) / 256, B);
  grpo_apply_kernel<<<grid, 256, 0, stream>>>(scores_ws, gid, group_ws, mask, adv, B, R, G, eps, norm_by_std);
  return (int)cudaGetLastError();
}

extern "C" int sb_ppo_token_loss(const float* logp, const float* old_logp, const float* adv, const float* mask,
                                 const float* ref_logp, const float* entropy, const float* w_row,
                                 const float* seq_logratio, float* dlogp, float* dentropy, float* stats, int B,
                                 int R, int mode, float clip_lo, float clip_hi, float clip_c, int use_kl,
                                 float kl_coef, float entropy_coef, float loss_scale, cudaStream_t stream) {
  if (B == 0 || R == 0) return 0;
  PpoParams p;
  p.logp = logp; p.old_logp = old_logp; p.adv = adv; p.mask = mask; p.ref_logp = ref_logp;
  p.entropy = entropy; p.w_row = w_row; p.seq_logratio = seq_logratio;
  p.dlogp = dlogp; p.dentropy = dentropy; p.stats = stats;
  p.B = B; p.R = R; p.mode = mode;
  p.clip_lo = clip_lo; p.clip_hi = clip_hi; p.clip_c = clip_c;
  p.kl_coef = kl_coef; p.entropy_coef = entropy_coef; p.loss_scale = loss_scale; p.use_kl = use_kl;
  cudaMemsetAsync(stats, 0, sizeof(float) * 8, stream);
  const long long total = (long long)B * R;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)num_sms() * 8;
  if (blocks > cap) blocks = cap;
  ppo_token_loss_kernel<<<(int)blocks, 256, 0, stream>>>(p);
  return (int)cudaGetLastError();
}
