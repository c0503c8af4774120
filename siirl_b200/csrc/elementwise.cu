// Memory-bound transformer ops for packed [tokens, hidden] bf16 activations:
// RMSNorm (+residual) fwd/bwd, RoPE / mrope, SwiGLU fwd/bwd, embedding gather / scatter-add,
// dtype casts.  They replace apex fused_rms_norm_affine, flash-attn's rotary and the eager HF
// activation code the reference runs (siirl/models/llama/megatron/layers/parallel_rmsnorm.py:18-48,
// siirl/models/transformers/qwen2.py).  All loads/stores are 16-byte vectors; fp32 math.
#include "common.cuh"
#include "launchers.h"

namespace sb {

__device__ __forceinline__ void bf16x8_to_float(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 float_to_bf16x8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  return o;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// ---------------------------------------------------------------------------------------
// RMSNorm forward:  h = x (+ residual);  y = h * rsqrt(mean(h^2) + eps) * w
// ---------------------------------------------------------------------------------------
constexpr int kNormThreads = 256;
constexpr int kNormMaxChunks = 4;  // hidden <= 256 * 8 * 4 = 8192

template <int CH>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int T, int H, float eps) {
  __shared__ float red[32];
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    float hv[CH][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int vi = threadIdx.x + c * kNormThreads;
      if (vi < nvec) {
        uint4 xv = reinterpret_cast<const uint4*>(x + (size_t)row * H)[vi];
        bf16x8_to_float(xv, hv[c]);
        if (residual) {
          float rv[8];
          uint4 r4 = reinterpret_cast<const uint4*>(residual + (size_t)row * H)[vi];
          bf16x8_to_float(r4, rv);
#pragma unroll
          for (int i = 0; i < 8; ++i) hv[c][i] += rv[i];
          if (h_out) {
            uint4 o = float_to_bf16x8(hv[c]);
            reinterpret_cast<uint4*>(h_out + (size_t)row * H)[vi] = o;
            // keep the math consistent with what backward will re-read
            bf16x8_to_float(o, hv[c]);
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += hv[c][i] * hv[c][i];
      }
    }
    const float tot = block_sum<kNormThreads>(ss, red);
    const float rstd = rsqrtf(tot / (float)H + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int vi = threadIdx.x + c * kNormThreads;
      if (vi < nvec) {
        float wv[8], o[8];
        bf16x8_to_float(reinterpret_cast<const uint4*>(w)[vi], wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = hv[c][i] * rstd * wv[i];
        reinterpret_cast<uint4*>(y + (size_t)row * H)[vi] = float_to_bf16x8(o);
      }
    }
  }
}

// RMSNorm backward.  dx = rstd * (g - xhat * mean(g * xhat)),  g = dy * w,  xhat = h * rstd.
// dx is optionally added to `dres` (gradient arriving through the residual branch).
// Per-block partial dw rows go to dw_partial[gridDim.x, H]; a second kernel folds them into fp32 dw.
template <int CH>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int T, int H) {
  __shared__ float red[32];
  const int nvec = H / 8;
  float dwacc[CH][8];
  float wv[CH][8];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int vi = threadIdx.x + c * kNormThreads;
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[c][i] = 0.f;
    if (vi < nvec) bf16x8_to_float(reinterpret_cast<const uint4*>(w)[vi], wv[c]);
  }
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const float rs = rstd[row];
    float g[CH][8], xh[CH][8];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int vi = threadIdx.x + c * kNormThreads;
      if (vi < nvec) {
        float dyv[8], hv[8];
        bf16x8_to_float(reinterpret_cast<const uint4*>(dy + (size_t)row * H)[vi], dyv);
        bf16x8_to_float(reinterpret_cast<const uint4*>(h + (size_t)row * H)[vi], hv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[c][i] = hv[i] * rs;
          g[c][i] = dyv[i] * wv[c][i];
          dot += g[c][i] * xh[c][i];
          dwacc[c][i] += dyv[i] * xh[c][i];
        }
      }
    }
    const float mean = block_sum<kNormThreads>(dot, red) / (float)H;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int vi = threadIdx.x + c * kNormThreads;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rs * (g[c][i] - xh[c][i] * mean);
        if (dres) {
          float rv[8];
          bf16x8_to_float(reinterpret_cast<const uint4*>(dres + (size_t)row * H)[vi], rv);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += rv[i];
        }
        reinterpret_cast<uint4*>(dx + (size_t)row * H)[vi] = float_to_bf16x8(o);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int vi = threadIdx.x + c * kNormThreads;
    if (vi < nvec) {
      float4* dst = reinterpret_cast<float4*>(dw_partial + (size_t)blockIdx.x * H + (size_t)vi * 8);
      dst[0] = make_float4(dwacc[c][0], dwacc[c][1], dwacc[c][2], dwacc[c][3]);
      dst[1] = make_float4(dwacc[c][4], dwacc[c][5], dwacc[c][6], dwacc[c][7]);
    }
  }
}

__global__ void colsum_accumulate_kernel(const float* __restrict__ partial, float* __restrict__ out, int rows,
                                         int H, int accumulate) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= H) return;
  float s = 0.f;
  for (int r = 0; r < rows; ++r) s += partial[(size_t)r * H + col];
  out[col] = accumulate ? out[col] + s : s;
}

// ---------------------------------------------------------------------------------------
// RoPE (rotate-half / "neox" layout) applied in place to the q and k parts of a packed qkv row.
// cos/sin come from a [max_pos, D/2] fp32 table.  `pos` is [rows_of_pos, T]; with 3 rows
// (t, h, w — Qwen2-VL mrope) frequency index i uses row 0 below sec0, row 1 below sec1, else row 2.
// `sign` = +1 forward, -1 backward (inverse rotation = gradient).
// ---------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                            const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int T,
                            int row_stride, int n_heads_rot, int D, int pos_rows, int sec0, int sec1,
                            float sign) {
  const int half = D / 2;
  const int pairs_per_tok = n_heads_rot * half;
  const long long total = (long long)T * pairs_per_tok;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / pairs_per_tok);
    const int r = (int)(idx % pairs_per_tok);
    const int head = r / half, i = r % half;
    int prow = 0;
    if (pos_rows == 3) prow = (i < sec0) ? 0 : (i < sec1 ? 1 : 2);
    const int pidx = pos[(size_t)prow * T + t];
    const float c = cos_tab[(size_t)pidx * half + i];
    const float s = sign * sin_tab[(size_t)pidx * half + i];
    __nv_bfloat16* base = qkv + (size_t)t * row_stride + (size_t)head * D;
    const float a = __bfloat162float(base[i]);
    const float b = __bfloat162float(base[i + half]);
    base[i] = __float2bfloat16(a * c - b * s);
    base[i + half] = __float2bfloat16(b * c + a * s);
  }
}

// ---------------------------------------------------------------------------------------
// SwiGLU on a fused gate|up projection: gu is [T, 2*I] with gate in columns [0,I), up in [I,2I).
// ---------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int T,
                                  int I) {
  const int nvec = I / 8;
  const long long total = (long long)T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / nvec), v = (int)(idx % nvec);
    float g[8], u[8], o[8];
    bf16x8_to_float(reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * I)[v], g);
    bf16x8_to_float(reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * I + I)[v], u);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
    reinterpret_cast<uint4*>(out + (size_t)t * I)[v] = float_to_bf16x8(o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgu, int T, int I) {
  const int nvec = I / 8;
  const long long total = (long long)T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / nvec), v = (int)(idx % nvec);
    float g[8], u[8], d[8], dg[8], du[8];
    bf16x8_to_float(reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * I)[v], g);
    bf16x8_to_float(reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * I + I)[v], u);
    bf16x8_to_float(reinterpret_cast<const uint4*>(dout + (size_t)t * I)[v], d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sig = 1.f / (1.f + __expf(-g[i]));
      const float silu = g[i] * sig;
      dg[i] = d[i] * u[i] * (sig + silu * (1.f - sig));
      du[i] = d[i] * silu;
    }
    reinterpret_cast<uint4*>(dgu + (size_t)t * 2 * I)[v] = float_to_bf16x8(dg);
    reinterpret_cast<uint4*>(dgu + (size_t)t * 2 * I + I)[v] = float_to_bf16x8(du);
  }
}

// ---------------------------------------------------------------------------------------
// Embedding gather and its gradient (fp32 scatter-add into the main-grad buffer).
// ---------------------------------------------------------------------------------------
SB_BOUNDS_WORD_DEFINE(elementwise)

__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int T, int H, int V) {
  const int nvec = H / 8;
  const long long total = (long long)T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / nvec), v = (int)(idx % nvec);
    long long id = ids[t];
    SB_CHECK_INDEX(id, V, 1);
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    reinterpret_cast<uint4*>(out + (size_t)t * H)[v] = reinterpret_cast<const uint4*>(table + (size_t)id * H)[v];
  }
}

__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dtable, int T, int H, int V) {
  const int nvec = H / 8;
  const long long total = (long long)T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / nvec), v = (int)(idx % nvec);
    long long id = ids[t];
    SB_CHECK_INDEX(id, V, 2);
    if (id < 0 || id >= V) continue;
    float d[8];
    bf16x8_to_float(reinterpret_cast<const uint4*>(dout + (size_t)t * H)[v], d);
    float* dst = dtable + (size_t)id * H + (size_t)v * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) atomicAdd(dst + i, d[i]);
  }
}

// out[i] = bf16(a[i] + b[i])  (residual adds outside the norm kernels)
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ out, long long nvec) {
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < nvec;
       idx += (long long)gridDim.x * blockDim.x) {
    float x[8], y[8];
    bf16x8_to_float(reinterpret_cast<const uint4*>(a)[idx], x);
    bf16x8_to_float(reinterpret_cast<const uint4*>(b)[idx], y);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] += y[i];
    reinterpret_cast<uint4*>(out)[idx] = float_to_bf16x8(x);
  }
}

static inline int grid_for(long long work, int threads, int per_sm = 8) {
  long long blocks = (work + threads - 1) / threads;
  long long cap = (long long)num_sms() * per_sm;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace sb

using namespace sb;

extern "C" int sb_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out,
                              float* rstd, int T, int H, float eps, cudaStream_t stream) {
  if (H % 8 || H > kNormThreads * 8 * kNormMaxChunks) return -3;
  if (T == 0) return 0;
  const int ch = (H / 8 + kNormThreads - 1) / kNormThreads;
  const int grid = T < num_sms() * 8 ? T : num_sms() * 8;
#define SB_LAUNCH(CH)                                                                                     \
  rmsnorm_fwd_kernel<CH><<<grid, kNormThreads, 0, stream>>>(                                              \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, \
      (__nv_bfloat16*)h_out, rstd, T, H, eps)
  switch (ch) {
    case 1: SB_LAUNCH(1); break;
    case 2: SB_LAUNCH(2); break;
    case 3: SB_LAUNCH(3); break;
    default: SB_LAUNCH(4); break;
  }
#undef SB_LAUNCH
  return (int)cudaGetLastError();
}

extern "C" int sb_rmsnorm_bwd_blocks(int T) {
  const int cap = num_sms() * 2;
  return T < cap ? (T > 0 ? T : 1) : cap;
}

extern "C" int sb_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres,
                              void* dx, float* dw_partial, float* dw, int dw_accumulate, int T, int H,
                              cudaStream_t stream) {
  if (H % 8 || H > kNormThreads * 8 * kNormMaxChunks) return -3;
  if (T == 0) return 0;
  const int ch = (H / 8 + kNormThreads - 1) / kNormThreads;
  const int grid = sb_rmsnorm_bwd_blocks(T);
#define SB_LAUNCH(CH)                                                                                       \
  rmsnorm_bwd_kernel<CH><<<grid, kNormThreads, 0, stream>>>(                                                \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, rstd,                      \
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, dw_partial, T, H)
  switch (ch) {
    case 1: SB_LAUNCH(1); break;
    case 2: SB_LAUNCH(2); break;
    case 3: SB_LAUNCH(3); break;
    default: SB_LAUNCH(4); break;
  }
#undef SB_LAUNCH
  colsum_accumulate_kernel<<<(H + 127) / 128, 128, 0, stream>>>(dw_partial, dw, grid, H, dw_accumulate);
  return (int)cudaGetLastError();
}

extern "C" int sb_rope(void* qkv, const int* pos, const float* cos_tab, const float* sin_tab, int T,
                       int row_stride, int n_heads_rot, int D, int pos_rows, int sec0, int sec1, float sign,
                       cudaStream_t stream) {
  if (T == 0) return 0;
  const long long total = (long long)T * n_heads_rot * (D / 2);
  rope_kernel<<<grid_for(total, 256), 256, 0, stream>>>((__nv_bfloat16*)qkv, pos, cos_tab, sin_tab, T, row_stride,
                                                        n_heads_rot, D, pos_rows, sec0, sec1, sign);
  return (int)cudaGetLastError();
}

extern "C" int sb_swiglu_fwd(const void* gu, void* out, int T, int I, cudaStream_t stream) {
  if (I % 8) return -3;
  if (T == 0) return 0;
  swiglu_fwd_kernel<<<grid_for((long long)T * (I / 8), 256), 256, 0, stream>>>((const __nv_bfloat16*)gu,
                                                                             (__nv_bfloat16*)out, T, I);
  return (int)cudaGetLastError();
}

extern "C" int sb_swiglu_bwd(const void* gu, const void* dout, void* dgu, int T, int I, cudaStream_t stream) {
  if (I % 8) return -3;
  if (T == 0) return 0;
  swiglu_bwd_kernel<<<grid_for((long long)T * (I / 8), 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgu, T, I);
  return (int)cudaGetLastError();
}

extern "C" int sb_embedding_fwd(const long long* ids, const void* table, void* out, int T, int H, int V,
                                cudaStream_t stream) {
  if (H % 8) return -3;
  if (T == 0) return 0;
  embedding_fwd_kernel<<<grid_for((long long)T * (H / 8), 256), 256, 0, stream>>>(
      ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, T, H, V);
  return (int)cudaGetLastError();
}

extern "C" int sb_embedding_bwd(const long long* ids, const void* dout, float* dtable, int T, int H, int V,
                                cudaStream_t stream) {
  if (H % 8) return -3;
  if (T == 0) return 0;
  embedding_bwd_kernel<<<grid_for((long long)T * (H / 8), 256), 256, 0, stream>>>(
      ids, (const __nv_bfloat16*)dout, dtable, T, H, V);
  return (int)cudaGetLastError();
}

extern "C" int sb_add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t stream) {
  if (n % 8) return -3;
  if (n == 0) return 0;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                           (__nv_bfloat16*)out, n / 8);
  return (int)cudaGetLastError();
}
