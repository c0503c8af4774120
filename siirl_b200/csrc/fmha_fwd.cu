// Packed variable-length attention forward (causal or full, GQA) on tcgen05 tensor cores.
// Replaces flash-attn's varlen forward that the reference reaches through HF
// `attn_implementation="flash_attention_2"` (siirl/engine/fsdp_workers.py:631-744,
// siirl/models/transformers/monkey_patch.py:51-109).
//
// Layout: one packed buffer qkv[T, (Hq + 2*Hkv) * D] (q heads, then k heads, then v heads per row);
// sequences are row ranges given by cu_seqlens.  One CTA = one 128-row query tile of one q head.
//   S  = Q K_j^T      tcgen05.mma 128 x 64 x D     -> TMEM (64 fp32 columns)
//   softmax on 128 threads (thread r owns query row r = TMEM lane r), online max / sum, P -> smem (bf16, swizzled)
//   O += P V_j        tcgen05.mma 128 x D x 64, V read through an MN-major descriptor (no transpose copy)
// K/V tiles are double-buffered with TMA; two CTAs fit per SM so one CTA's softmax overlaps the other's MMAs.
// Outputs: O[T, Hq*D] bf16 and LSE[Hq, T] fp32 (natural log) for the backward pass.
#include "common.cuh"
#include "launchers.h"

namespace sb {

constexpr int kQTile = 128;
constexpr int kKvTile = 64;

struct FmhaFwdParams {
  const int* tile_seq_start;  // [num_tiles] first token row of the tile's sequence
  const int* tile_seq_len;    // [num_tiles]
  const int* tile_q0;         // [num_tiles] first query position (within the sequence) of the tile
  __nv_bfloat16* out;         // [T, Hq*D]
  float* lse;                 // [Hq, T]
  int T, Hq, Hkv, causal;
  float scale_log2;  // softmax scale * log2(e)
  int* status;
};

template <int D>
struct FwdSmem {
  static constexpr int kQBytes = kQTile * D * 2;
  static constexpr int kKBytes = kKvTile * D * 2;
  static constexpr int kPBytes = kQTile * kKvTile * 2;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + kQBytes;             // 2 stages
  static constexpr int kVOff = kKOff + 2 * kKBytes;         // 2 stages
  static constexpr int kPOff = kVOff + 2 * kKBytes;
  static constexpr int kBarOff = kPOff + kPBytes;           // bar_q, bar_kv[2], bar_s, bar_o
  static constexpr int kTotal = kBarOff + 5 * 8 + 24;
};

template <int D>
__global__ void __launch_bounds__(128, 2)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                FmhaFwdParams p) {
  using L = FwdSmem<D>;
  constexpr int kDChunks = D / 64;
  constexpr uint32_t kTmemCols = (D == 128) ? 256 : 128;  // S: 64 columns, O: D columns
  // 1024-byte alignment is required by the 128-byte swizzle; no slack is reserved so that two CTAs fit per SM
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
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* bar_kv = bar_q + 1;
  uint64_t* bar_s = bar_q + 3;
  uint64_t* bar_o = bar_q + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_q + 5);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int tile = blockIdx.x, h = blockIdx.y;
  const int seq_start = p.tile_seq_start[tile], seq_len = p.tile_seq_len[tile], q0 = p.tile_q0[tile];
  const int rep = p.Hq / p.Hkv;
  const int kvh = h / rep;
  const int qcol = h * D, kcol = (p.Hq + kvh) * D, vcol = (p.Hq + p.Hkv + kvh) * D;
  const int q_hi = min(q0 + kQTile, seq_len);  // one past the last valid query position of this tile
  const int kv_end = p.causal ? q_hi : seq_len;
  const int n_tiles = (kv_end + kKvTile - 1) / kKvTile;

  if (tid == 0) {
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_kv);
    mbar_init(bar_q, 1);
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
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;        // 64 columns
  const uint32_t tmem_o = tmem_base + 64;   // D columns

  auto load_kv = [&](int j, int stage) {
    mbar_arrive_expect_tx(&bar_kv[stage], 2 * L::kKBytes);
    const int row = seq_start + j * kKvTile;
#pragma unroll
    for (int c = 0; c < kDChunks; ++c) {
      tma_load_2d(sK + stage * L::kKBytes + c * 8192, &map_kv, &bar_kv[stage], kcol + c * 64, row);
      tma_load_2d(sV + stage * L::kKBytes + c * 8192, &map_kv, &bar_kv[stage], vcol + c * 64, row);
    }
  };

  if (tid == 0) {
    mbar_arrive_expect_tx(bar_q, L::kQBytes);
#pragma unroll
    for (int c = 0; c < kDChunks; ++c)
      tma_load_2d(sQ + c * 16384, &map_q, bar_q, qcol + c * 64, seq_start + q0);
    load_kv(0, 0);
    if (n_tiles > 1) load_kv(1, 1);
  }

  constexpr uint32_t idesc_s = umma_idesc_bf16(128, kKvTile, 0, 0);
  constexpr uint32_t idesc_o = umma_idesc_bf16(128, D, 0, 1);
  const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
  const int qpos = q0 + tid;  // this thread's query position within the sequence
  float m_run = -INFINITY, l_run = 0.f;
  bool ok = true;

  for (int j = 0; j < n_tiles && ok; ++j) {
    const int stage = j & 1;
    // ---- S = Q K_j^T ----
    if (tid == 0) {
      bool w = true;
      if (j == 0) w = mbar_wait(bar_q, 0, p.status, kStatusTimeoutMma);
      w = w && mbar_wait(&bar_kv[stage], (j >> 1) & 1, p.status, kStatusTimeoutMma);
      if (w) {
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

    // ---- online softmax on this thread's row ----
    const int kv0 = j * kKvTile;
    const bool need_mask = (kv0 + kKvTile > seq_len) || (p.causal && kv0 + kKvTile - 1 > q0);
    float sv[kKvTile];
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
    if (need_mask) {
#pragma unroll
      for (int i = 0; i < kKvTile; ++i) {
        const int kp = kv0 + i;
        const bool valid = kp < seq_len && (!p.causal || kp <= qpos);
        if (!valid) sv[i] = -INFINITY;
      }
    }
    float m_new = m_run;
#pragma unroll
    for (int i = 0; i < kKvTile; ++i) m_new = fmaxf(m_new, sv[i]);
    const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = exp2f(m_run - m_safe);  // m_run = -inf -> 0
    float rsum = 0.f;
    uint32_t pk[kKvTile / 2];
#pragma unroll
    for (int i = 0; i < kKvTile; i += 2) {
      const float p0 = exp2f(sv[i] - m_safe), p1 = exp2f(sv[i + 1] - m_safe);
      rsum += p0 + p1;
      pk[i / 2] = pack_bf16x2(p0, p1);
    }
    l_run = l_run * alpha + rsum;
    m_run = m_new;

    // ---- rescale the running O in TMEM when some row of this warp raised its maximum ----
    if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
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
    // ---- P (bf16) -> smem, 128-byte swizzled K-major tile [128 rows x 64 cols] ----
    {
      uint8_t* prow = sP + tid * 128;
#pragma unroll
      for (int piece = 0; piece < 8; ++piece) {
        uint4 v = make_uint4(pk[piece * 4], pk[piece * 4 + 1], pk[piece * 4 + 2], pk[piece * 4 + 3]);
        *reinterpret_cast<uint4*>(prow + ((piece ^ (tid & 7)) << 4)) = v;
      }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- O += P V_j ----
    if (tid == 0) {
      tc_fence_after();
      const uint32_t ap = smem_u32(sP), bv = smem_u32(sV + stage * L::kKBytes);
#pragma unroll
      for (int kk = 0; kk < kKvTile / 16; ++kk) {
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

  // ---- epilogue: O / l -> bf16, LSE (TMEM loads are warp-collective; only the stores are predicated) ----
  ok = __all_sync(0xffffffffu, ok);
  if (ok) {
    const bool row_valid = qpos < seq_len;
    const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
    const size_t row = (size_t)(seq_start + (row_valid ? qpos : 0));
    __nv_bfloat16* orow = p.out + row * (size_t)(p.Hq * D) + (size_t)h * D;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(tmem_o + lane_off + c * 32, r);
      tmem_ld_wait();
      if (row_valid) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(r[g * 8 + 0]) * inv_l, __uint_as_float(r[g * 8 + 1]) * inv_l);
          o.y = pack_bf16x2(__uint_as_float(r[g * 8 + 2]) * inv_l, __uint_as_float(r[g * 8 + 3]) * inv_l);
          o.z = pack_bf16x2(__uint_as_float(r[g * 8 + 4]) * inv_l, __uint_as_float(r[g * 8 + 5]) * inv_l);
          o.w = pack_bf16x2(__uint_as_float(r[g * 8 + 6]) * inv_l, __uint_as_float(r[g * 8 + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = o;
        }
      }
    }
    if (row_valid)
      p.lse[(size_t)h * p.T + row] =
          (m_run == -INFINITY) ? -INFINITY : (m_run + log2f(l_run)) * 0.6931471805599453f;
  }
  if (!ok && tid == 0) {
    // let outstanding bulk copies land before shared memory is released
    mbar_wait(&bar_kv[0], 0, nullptr, 0);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D>
static int launch_fwd(const CUtensorMap& mq, const CUtensorMap& mkv, const FmhaFwdParams& p, int num_tiles,
                      cudaStream_t stream) {
  using L = FwdSmem<D>;
  auto kernel = fmha_fwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(num_tiles, p.Hq);
  kernel<<<grid, 128, L::kTotal, stream>>>(mq, mkv, p);
  return (int)cudaGetLastError();
}

}  // namespace sb

using namespace sb;

extern "C" int sb_fmha_fwd(const void* qkv, void* out, float* lse, const int* tile_seq_start,
                           const int* tile_seq_len, const int* tile_q0, int num_tiles, int T, int Hq, int Hkv,
                           int D, int causal, float scale, int* status, cudaStream_t stream) {
  if (num_tiles == 0 || T == 0) return 0;
  if (D != 64 && D != 128) return -2;
  static thread_local bool tl_context_bound = false;
  if (!tl_context_bound) {
    cudaFree(0);
    tl_context_bound = true;
  }
  const long long width = (long long)(Hq + 2 * Hkv) * D;
  CUtensorMap mq, mkv;
  int r = make_tensor_map_bf16_2d(&mq, qkv, width, T, width, 64, kQTile);
  if (r) return r;
  r = make_tensor_map_bf16_2d(&mkv, qkv, width, T, width, 64, kKvTile);
  if (r) return r;
  FmhaFwdParams p;
  p.tile_seq_start = tile_seq_start; p.tile_seq_len = tile_seq_len; p.tile_q0 = tile_q0;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.lse = lse;
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  return D == 128 ? launch_fwd<128>(mq, mkv, p, num_tiles, stream) : launch_fwd<64>(mq, mkv, p, num_tiles, stream);
}
