// Paged-KV cache kernels for the rollout engine: cache append and single-token (decode) attention.
// They replace the vLLM/SGLang paged-attention and cache ops the reference calls through
// `LLM.generate` (siirl/engine/rollout/vllm_rollout/vllm_rollout_spmd.py:261-416).
//
// Cache layout of one layer: [num_blocks, 2 (k|v), Hkv, 64 tokens, D] bf16.  A sequence owns a list of blocks
// (block_table[b, j]); token position p lives in block p/64 at row p%64.
//
// Decode attention: one CTA per (sequence, kv head).  The `rep` = Hq/Hkv query heads that share the kv head are
// the rows of one 128-row tcgen05 tile (rows >= rep are zero), so every K/V block is read from HBM exactly once
// per kv head and both GEMMs (S = Q K^T, O += P V) run on the tensor cores; the kernel is bound by the K/V stream.
// Context lengths and block ids are read from device memory, so a decode step can be replayed from a CUDA graph.
#include "common.cuh"
#include "launchers.h"

namespace sb {

constexpr int kBlk = 64;  // tokens per cache block = kv tile

// ---------------------------------------------------------------------------------------
// cache append: copies the k and v parts of packed qkv rows into their cache slots
// ---------------------------------------------------------------------------------------
SB_BOUNDS_WORD_DEFINE(kv_cache)

__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ qkv, int row_stride, const int* __restrict__ seq_ids,
                                 const int* __restrict__ positions, const int* __restrict__ block_table,
                                 int max_blocks, __nv_bfloat16* __restrict__ cache, int T, int Hq, int Hkv, int D) {
  const int vec_per_head = D / 8;
  const int per_tok = 2 * Hkv * vec_per_head;
  const long long total = (long long)T * per_tok;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / per_tok);
    int r = (int)(idx % per_tok);
    const int kv = r / (Hkv * vec_per_head);
    r -= kv * Hkv * vec_per_head;
    const int head = r / vec_per_head, v = r % vec_per_head;
    const int pos = positions[t];
    const int seq = seq_ids[t];
    if (pos < 0 || seq < 0) continue;
    SB_CHECK_INDEX(pos / kBlk, max_blocks, 3);
    if (pos / kBlk >= max_blocks) continue;
    const int blk = block_table[(size_t)seq * max_blocks + pos / kBlk];
    SB_CHECK_INDEX(blk, 0x7fffffff, 4);
    if (blk < 0) continue;
    const uint4 val = *reinterpret_cast<const uint4*>(qkv + (size_t)t * row_stride + (size_t)(Hq + kv * Hkv + head) * D + v * 8);
    __nv_bfloat16* dst = cache + ((((size_t)blk * 2 + kv) * Hkv + head) * kBlk + (pos % kBlk)) * D + v * 8;
    *reinterpret_cast<uint4*>(dst) = val;
  }
}

// copy whole blocks (src -> dst) inside one layer's cache: used when a shared prompt's last, partially
// filled block is forked for each of the n samples of the prompt
__global__ void kv_copy_blocks_kernel(__nv_bfloat16* __restrict__ cache, const int* __restrict__ src,
                                      const int* __restrict__ dst, int n_pairs, long long block_elems) {
  const long long vecs = block_elems / 8;
  for (int pair = blockIdx.y; pair < n_pairs; pair += gridDim.y) {
    const uint4* s = reinterpret_cast<const uint4*>(cache + (size_t)src[pair] * block_elems);
    uint4* d = reinterpret_cast<uint4*>(cache + (size_t)dst[pair] * block_elems);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < vecs; i += (long long)gridDim.x * blockDim.x)
      d[i] = s[i];
  }
}

// ---------------------------------------------------------------------------------------
// fused RoPE + cache append (rollout path): rotates the q and k heads of packed qkv rows in place and writes the
// rotated k and the v heads of every row to its cache slot -- one launch instead of clone + rope + append.
// One thread handles 8 rotation pairs (i, i + D/2) of one head, or 16 contiguous v elements.
// ---------------------------------------------------------------------------------------
__global__ void rope_kv_append_kernel(__nv_bfloat16* __restrict__ qkv, int row_stride, const int* __restrict__ rope_pos,
                                      int pos_rows, int sec0, int sec1, const float* __restrict__ cos_tab,
                                      const float* __restrict__ sin_tab, const int* __restrict__ seq_ids,
                                      const int* __restrict__ cache_pos, const int* __restrict__ block_table,
                                      int max_blocks, __nv_bfloat16* __restrict__ cache, int T, int Hq, int Hkv, int D) {
  const int half = D / 2;
  const int units_per_head = half / 8;                 // 8 pairs per thread
  const int heads = Hq + 2 * Hkv;
  const long long total = (long long)T * heads * units_per_head;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / (heads * units_per_head));
    int r = (int)(idx % (heads * units_per_head));
    const int head = r / units_per_head, u = r % units_per_head;
    const int i0 = u * 8;
    __nv_bfloat16* base = qkv + (size_t)t * row_stride + (size_t)head * D;
    uint4 lo = *reinterpret_cast<const uint4*>(base + i0);
    uint4 hi = *reinterpret_cast<const uint4*>(base + half + i0);
    const int seq = seq_ids[t], cp = cache_pos[t];
    const bool to_cache = head >= Hq && seq >= 0 && cp >= 0;
    if (head < Hq + Hkv) {
      __nv_bfloat16* a = reinterpret_cast<__nv_bfloat16*>(&lo);
      __nv_bfloat16* b = reinterpret_cast<__nv_bfloat16*>(&hi);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int i = i0 + k;
        int prow = 0;
        if (pos_rows == 3) prow = (i < sec0) ? 0 : (i < sec1 ? 1 : 2);
        const int p = rope_pos[(size_t)prow * T + t];
        const float c = cos_tab[(size_t)p * half + i], s = sin_tab[(size_t)p * half + i];
        const float x = __bfloat162float(a[k]), y = __bfloat162float(b[k]);
        a[k] = __float2bfloat16(x * c - y * s);
        b[k] = __float2bfloat16(y * c + x * s);
      }
      *reinterpret_cast<uint4*>(base + i0) = lo;
      *reinterpret_cast<uint4*>(base + half + i0) = hi;
    }
    if (to_cache) {
      const int kv = head >= Hq + Hkv ? 1 : 0;
      const int h = head - Hq - kv * Hkv;
      SB_CHECK_INDEX(cp / kBlk, max_blocks, 5);
      const int blk = cp / kBlk < max_blocks ? block_table[(size_t)seq * max_blocks + cp / kBlk] : -1;
      SB_CHECK_INDEX(blk, 0x7fffffff, 6);
      if (blk >= 0) {
        __nv_bfloat16* dst = cache + ((((size_t)blk * 2 + kv) * Hkv + h) * kBlk + (cp % kBlk)) * D;
        *reinterpret_cast<uint4*>(dst + i0) = lo;
        *reinterpret_cast<uint4*>(dst + half + i0) = hi;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// decode attention
// ---------------------------------------------------------------------------------------
struct DecodeParams {
  const __nv_bfloat16* q;  // packed rows [B, row_stride]; q heads first
  int row_stride;
  const int* seq_lens;     // [B] context length including the current token
  const int* block_table;  // [B, max_blocks]
  int max_blocks;
  __nv_bfloat16* out;      // [B, Hq*D]
  int B, Hq, Hkv;
  float scale_log2;
  int* status;
};

template <int D>
struct DecSmem {
  static constexpr int kQBytes = 128 * D * 2;
  static constexpr int kKBytes = kBlk * D * 2;
  static constexpr int kPBytes = 128 * kBlk * 2;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + kQBytes;
  static constexpr int kVOff = kKOff + 2 * kKBytes;
  static constexpr int kPOff = kVOff + 2 * kKBytes;
  static constexpr int kBarOff = kPOff + kPBytes;  // bar_kv[2], bar_s, bar_o
  static constexpr int kTotal = kBarOff + 4 * 8 + 32;
};

template <int D>
__global__ void __launch_bounds__(128, 2)
fmha_decode_kernel(const __grid_constant__ CUtensorMap map_cache, DecodeParams p) {
  using L = DecSmem<D>;
  constexpr int kDChunks = D / 64;
  constexpr uint32_t kTmemCols = (D == 128) ? 256 : 128;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, (int)kStatusBadArgument);
    return;
  }
  uint8_t* sQ = smem + L::kQOff;
  uint8_t* sK = smem + L::kKOff;
  uint8_t* sV = smem + L::kVOff;
  uint8_t* sP = smem + L::kPOff;
  uint64_t* bar_kv = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* bar_s = bar_kv + 2;
  uint64_t* bar_o = bar_kv + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_kv + 4);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int b = blockIdx.x, g = blockIdx.y;
  const int rep = p.Hq / p.Hkv;
  const int ctx = p.seq_lens[b];
  const int n_tiles = (ctx + kBlk - 1) / kBlk;
  const int* blocks = p.block_table + (size_t)b * p.max_blocks;

  if (tid == 0) {
    tma_prefetch_desc(&map_cache);
    mbar_init(&bar_kv[0], 1);
    mbar_init(&bar_kv[1], 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  // Q tile: row r < rep holds query head g*rep + r (swizzled K-major layout), other rows are zero
  {
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const __nv_bfloat16* qsrc = p.q + (size_t)b * p.row_stride + (size_t)(g * rep + tid) * D;
#pragma unroll
    for (int c = 0; c < kDChunks; ++c) {
#pragma unroll
      for (int piece = 0; piece < 8; ++piece) {
        uint4 v = zero;
        if (tid < rep) v = *reinterpret_cast<const uint4*>(qsrc + c * 64 + piece * 8);
        *reinterpret_cast<uint4*>(sQ + c * 16384 + tid * 128 + ((piece ^ (tid & 7)) << 4)) = v;
      }
    }
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 64;

  auto load_kv = [&](int j, int stage) {
    const int blk = blocks[j];
    mbar_arrive_expect_tx(&bar_kv[stage], 2 * L::kKBytes);
    const int krow = ((blk * 2 + 0) * p.Hkv + g) * kBlk;
    const int vrow = ((blk * 2 + 1) * p.Hkv + g) * kBlk;
#pragma unroll
    for (int c = 0; c < kDChunks; ++c) {
      tma_load_2d(sK + stage * L::kKBytes + c * 8192, &map_cache, &bar_kv[stage], c * 64, krow);
      tma_load_2d(sV + stage * L::kKBytes + c * 8192, &map_cache, &bar_kv[stage], c * 64, vrow);
    }
  };
  if (tid == 0 && n_tiles > 0) {
    load_kv(0, 0);
    if (n_tiles > 1) load_kv(1, 1);
  }

  constexpr uint32_t idesc_s = umma_idesc_bf16(128, kBlk, 0, 0);
  constexpr uint32_t idesc_o = umma_idesc_bf16(128, D, 0, 1);
  const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
  float m_run = -INFINITY, l_run = 0.f;
  bool ok = true;

  for (int j = 0; j < n_tiles && ok; ++j) {
    const int stage = j & 1;
    if (tid == 0) {
      if (mbar_wait(&bar_kv[stage], (j >> 1) & 1, p.status, kStatusTimeoutMma)) {
        tc_fence_after();
        const uint32_t aq = smem_u32(sQ), bk = smem_u32(sK + stage * L::kKBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t da = umma_smem_desc(aq + (kk / 4) * 16384 + (kk % 4) * 32, 16, 1024);
          const uint64_t db = umma_smem_desc(bk + (kk / 4) * 8192 + (kk % 4) * 32, 16, 1024);
          umma_bf16_ss(tmem_s, da, db, idesc_s, kk ? 1u : 0u);
        }
      }
      umma_commit(bar_s);
    }
    if (!__all_sync(0xffffffffu, mbar_wait(bar_s, j & 1, p.status, kStatusTimeoutEpilogue))) {
      ok = false;
      break;
    }
    tc_fence_after();
    const int kv0 = j * kBlk;
    float sv[kBlk];
    {
      uint32_t r0[32], r1[32];
      tmem_ld_32x32(tmem_s + lane_off, r0);
      tmem_ld_32x32(tmem_s + lane_off + 32, r1);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        sv[i] = __uint_as_float(r0[i]) * p.scale_log2;
        sv[32 + i] = __uint_as_float(r1[i]) * p.scale_log2;
      }
    }
    if (kv0 + kBlk > ctx) {
#pragma unroll
      for (int i = 0; i < kBlk; ++i)
        if (kv0 + i >= ctx) sv[i] = -INFINITY;
    }
    float m_new = m_run;
#pragma unroll
    for (int i = 0; i < kBlk; ++i) m_new = fmaxf(m_new, sv[i]);
    const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = exp2f(m_run - m_safe);
    float rsum = 0.f;
    uint32_t pk[kBlk / 2];
#pragma unroll
    for (int i = 0; i < kBlk; i += 2) {
      const float p0 = exp2f(sv[i] - m_safe), p1 = exp2f(sv[i + 1] - m_safe);
      rsum += p0 + p1;
      pk[i / 2] = pack_bf16x2(p0, p1);
    }
    l_run = l_run * alpha + rsum;
    m_run = m_new;
    // only the first warp holds meaningful rows (rep <= 32); the others skip the rescale
    if (j > 0 && __any_sync(0xffffffffu, tid < rep && alpha != 1.f)) {
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_o + lane_off + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
        tmem_st_32x32(tmem_o + lane_off + c * 32, r);
      }
      tmem_st_wait();
    }
    {
      uint8_t* prow = sP + tid * 128;
#pragma unroll
      for (int piece = 0; piece < 8; ++piece) {
        uint4 v = make_uint4(pk[piece * 4], pk[piece * 4 + 1], pk[piece * 4 + 2], pk[piece * 4 + 3]);
        if (tid >= rep) v = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(prow + ((piece ^ (tid & 7)) << 4)) = v;
      }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t ap = smem_u32(sP), bv = smem_u32(sV + stage * L::kKBytes);
#pragma unroll
      for (int kk = 0; kk < kBlk / 16; ++kk) {
        const uint64_t da = umma_smem_desc(ap + kk * 32, 16, 1024);
        const uint64_t db = umma_smem_desc(bv + kk * 2048, 8192, 1024);
        umma_bf16_ss(tmem_o, da, db, idesc_o, (j | kk) ? 1u : 0u);
      }
      umma_commit(bar_o);
    }
    if (!__all_sync(0xffffffffu, mbar_wait(bar_o, j & 1, p.status, kStatusTimeoutEpilogue))) {
      ok = false;
      break;
    }
    tc_fence_after();
    if (tid == 0 && j + 2 < n_tiles) load_kv(j + 2, stage);
  }

  ok = __all_sync(0xffffffffu, ok);
  if (ok && warp == 0) {
    const bool row_valid = tid < rep;
    const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
    __nv_bfloat16* orow = p.out + (size_t)b * (p.Hq * D) + (size_t)(g * rep + (row_valid ? tid : 0)) * D;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      if (n_tiles > 0) {
        tmem_ld_32x32(tmem_o + lane_off + c * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
      if (row_valid) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * inv_l, __uint_as_float(r[q * 8 + 1]) * inv_l);
          o.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * inv_l, __uint_as_float(r[q * 8 + 3]) * inv_l);
          o.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * inv_l, __uint_as_float(r[q * 8 + 5]) * inv_l);
          o.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * inv_l, __uint_as_float(r[q * 8 + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o;
        }
      }
    }
  }
  if (!ok && tid == 0) {
    mbar_wait(&bar_kv[0], 0, nullptr, 0);
    mbar_wait(&bar_kv[1], 0, nullptr, 0);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D>
static int launch_decode(const CUtensorMap& mc, const DecodeParams& p, cudaStream_t stream) {
  using L = DecSmem<D>;
  auto kernel = fmha_decode_kernel<D>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(p.B, p.Hkv);
  kernel<<<grid, 128, L::kTotal, stream>>>(mc, p);
  return (int)cudaGetLastError();
}

}  // namespace sb

using namespace sb;

extern "C" int sb_kv_append(const void* qkv, int row_stride, const int* seq_ids, const int* positions,
                            const int* block_table, int max_blocks, void* cache, int T, int Hq, int Hkv, int D,
                            cudaStream_t stream) {
  if (T == 0) return 0;
  if (D % 8) return -3;
  const long long total = (long long)T * 2 * Hkv * (D / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)num_sms() * 8;
  if (blocks > cap) blocks = cap;
  kv_append_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)qkv, row_stride, seq_ids, positions,
                                                    block_table, max_blocks, (__nv_bfloat16*)cache, T, Hq, Hkv, D);
  return (int)cudaGetLastError();
}

extern "C" int sb_rope_kv_append(void* qkv, int row_stride, const int* rope_pos, int pos_rows, int sec0, int sec1,
                                 const float* cos_tab, const float* sin_tab, const int* seq_ids, const int* cache_pos,
                                 const int* block_table, int max_blocks, void* cache, int T, int Hq, int Hkv, int D,
                                 cudaStream_t stream) {
  if (T == 0) return 0;
  if (D % 16) return -3;
  const long long total = (long long)T * (Hq + 2 * Hkv) * (D / 16);
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)num_sms() * 8;
  if (blocks > cap) blocks = cap;
  rope_kv_append_kernel<<<(int)blocks, 256, 0, stream>>>((__nv_bfloat16*)qkv, row_stride, rope_pos, pos_rows, sec0,
                                                         sec1, cos_tab, sin_tab, seq_ids, cache_pos, block_table,
                                                         max_blocks, (__nv_bfloat16*)cache, T, Hq, Hkv, D);
  return (int)cudaGetLastError();
}

extern "C" int sb_kv_copy_blocks(void* cache, const int* src, const int* dst, int n_pairs, long long block_elems,
                                 cudaStream_t stream) {
  if (n_pairs == 0) return 0;
  dim3 grid(8, n_pairs < 4096 ? n_pairs : 4096);
  kv_copy_blocks_kernel<<<grid, 256, 0, stream>>>((__nv_bfloat16*)cache, src, dst, n_pairs, block_elems);
  return (int)cudaGetLastError();
}

// cache: one layer [num_blocks, 2, Hkv, 64, D]; q: packed rows (q heads first) with `row_stride` elements per row.
extern "C" int sb_fmha_decode(const void* q, int row_stride, const void* cache, long long num_blocks,
                              const int* seq_lens, const int* block_table, int max_blocks, void* out, int B, int Hq,
                              int Hkv, int D, float scale, int* status, cudaStream_t stream) {
  if (B == 0) return 0;
  if (D != 64 && D != 128) return -2;
  if (Hq % Hkv || Hq / Hkv > 32) return -3;
  static thread_local bool tl_context_bound = false;
  if (!tl_context_bound) {
    cudaFree(0);
    tl_context_bound = true;
  }
  CUtensorMap mc;
  int r = make_tensor_map_bf16_2d(&mc, cache, D, num_blocks * 2 * Hkv * kBlk, D, 64, kBlk);
  if (r) return r;
  DecodeParams p;
  p.q = (const __nv_bfloat16*)q; p.row_stride = row_stride; p.seq_lens = seq_lens; p.block_table = block_table;
  p.max_blocks = max_blocks; p.out = (__nv_bfloat16*)out; p.B = B; p.Hq = Hq; p.Hkv = Hkv;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  return D == 128 ? launch_decode<128>(mc, p, stream) : launch_decode<64>(mc, p, stream);
}
