// Packed variable-length attention backward (causal or full, GQA) on tcgen05 tensor cores.
// Counterpart of fmha_fwd.cu; replaces flash-attn's varlen backward used by the reference's training path
// (siirl/engine/actor/dp_actor.py:87-263 through HF flash_attention_2).
//
// One CTA owns one 128-row K/V tile of one kv head and walks over the q heads of its GQA group and the
// query tiles that can attend to it.  Per step (TMEM lane r = query row r of the current query tile):
//   S  = Q K^T,  dP = dO V^T                          two 128x128xD MMAs into TMEM
//   P  = exp2(S*c - LSE),  dS = P (dP - Delta) * scale            -> bf16, swizzled smem ([q][kv])
//   dV += P^T dO        dK += dS^T Q                  accumulate in TMEM over all steps (no atomics);
//                                                      P^T / dS^T are P / dS read through MN-major descriptors
//   dQ_i = dS K                                        read back, turned through smem and added to an fp32
//                                                      buffer one whole row per warp instruction
// Q, dO and K tiles are read by the second group of MMAs through MN-major descriptors of the same shared
// memory that the first group read K-major, so nothing is transposed in memory.
#include "common.cuh"
#include "launchers.h"

namespace sb {

struct FmhaBwdParams {
  const int* tile_seq_start;  // per kv tile
  const int* tile_seq_len;
  const int* tile_k0;         // first kv position of the tile inside its sequence
  const float* lse;           // [Hq, T]
  const float* delta;         // [Hq, T]  rowsum(dO * O)
  float* dq_accum;            // [T, Hq*D] fp32, zero-initialised
  __nv_bfloat16* dqkv;        // [T, (Hq+2Hkv)*D]; this kernel writes the k and v parts
  int T, Hq, Hkv, causal;
  float scale, scale_log2;
  int* status;
};

template <int D>
struct BwdSmem {
  static constexpr int kTile = 128 * D * 2;      // K, V, Q, dO tiles
  static constexpr int kSq = 128 * 128 * 2;      // P^T, dS^T
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kKOff + kTile;
  static constexpr int kQOff = kVOff + kTile;
  static constexpr int kDoOff = kQOff + kTile;
  static constexpr int kPtOff = kDoOff + kTile;
  static constexpr int kDstOff = kPtOff + kSq;
  static constexpr int kLseOff = kDstOff + kSq;   // 128 floats lse*log2e, 128 floats delta
  static constexpr int kBarOff = kLseOff + 1024;  // bar_kv, bar_ld, bar_mma, bar_mma2
  static constexpr int kTotal = kBarOff + 4 * 8 + 32;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr int kBwdThreads = 256;

// 256 threads = 8 warps.  Warp w works on TMEM lanes 32 * (w % 4) .. +31 (the hardware's lane quarter of a warp) and
// on column half w / 4 of every tile it reads, so two warps share each scheduler and cover each other's latencies.
// Thread <-> query row: lane r of the S / dP / dQ tiles is query row r, so the row's log-sum-exp and delta are two
// registers; dV / dK tiles have lane = kv row.
template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
fmha_bwd_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do,
                FmhaBwdParams p) {
  using L = BwdSmem<D>;
  constexpr int kDChunks = D / 64;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, (int)kStatusBadArgument);
    return;
  }
  uint8_t* sK = smem + L::kKOff;
  uint8_t* sV = smem + L::kVOff;
  uint8_t* sQ = smem + L::kQOff;
  uint8_t* sDo = smem + L::kDoOff;
  uint8_t* sP = smem + L::kPtOff;    // P  [q rows][kv cols], bf16, 128-byte swizzle, two 64-column chunks
  uint8_t* sDs = smem + L::kDstOff;  // dS, same layout
  uint64_t* bar_kv = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* bar_ld = bar_kv + 1;
  uint64_t* bar_mma = bar_kv + 2;
  uint64_t* bar_mma2 = bar_kv + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_kv + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quarter = warp & 3, half = warp >> 2;
  const int r = quarter * 32 + lane;  // row of the tile this thread owns (query row, or kv row for dK / dV)
  const int tile = blockIdx.x, kvh = blockIdx.y;
  const int seq_start = p.tile_seq_start[tile], seq_len = p.tile_seq_len[tile], k0 = p.tile_k0[tile];
  const int rep = p.Hq / p.Hkv;
  const int n_q_tiles = (seq_len + 127) / 128;
  const int i_start = p.causal ? (k0 / 128) : 0;
  const int steps_per_head = n_q_tiles - i_start;
  const int total_steps = steps_per_head * rep;
  const int kcol = (p.Hq + kvh) * D, vcol = (p.Hq + p.Hkv + kvh) * D;

  if (tid == 0) {
    tma_prefetch_desc(&map_qkv);
    tma_prefetch_desc(&map_do);
    mbar_init(bar_kv, 1);
    mbar_init(bar_ld, 1);
    mbar_init(bar_mma, 1);
    mbar_init(bar_mma2, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_dv = tmem_base + 256, tm_dk = tmem_base + 384;
  const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;

  auto issue_loads = [&](int step) {
    const int h = kvh * rep + step / steps_per_head;
    const int qi = i_start + step % steps_per_head;
    const int row = seq_start + qi * 128;
    mbar_arrive_expect_tx(bar_ld, 2 * L::kTile);
#pragma unroll
    for (int c = 0; c < kDChunks; ++c) {
      tma_load_2d(sQ + c * 16384, &map_qkv, bar_ld, h * D + c * 64, row);
      tma_load_2d(sDo + c * 16384, &map_do, bar_ld, h * D + c * 64, row);
    }
  };

  if (tid == 0 && total_steps > 0) {
    mbar_arrive_expect_tx(bar_kv, 2 * L::kTile);
#pragma unroll
    for (int c = 0; c < kDChunks; ++c) {
      tma_load_2d(sK + c * 16384, &map_qkv, bar_kv, kcol + c * 64, seq_start + k0);
      tma_load_2d(sV + c * 16384, &map_qkv, bar_kv, vcol + c * 64, seq_start + k0);
    }
    issue_loads(0);
  }

  constexpr uint32_t idesc_kk = umma_idesc_bf16(128, 128, 0, 0);    // both operands K-major, N = 128
  constexpr uint32_t idesc_kmn = umma_idesc_bf16(128, D, 0, 1);     // A K-major, B MN-major, N = D
  constexpr uint32_t idesc_mnmn = umma_idesc_bf16(128, D, 1, 1);    // both MN-major, N = D
  bool ok = true;

  for (int step = 0; step < total_steps && ok; ++step) {
    const int h = kvh * rep + step / steps_per_head;
    const int qi = i_start + step % steps_per_head;
    const int q0 = qi * 128;
    // ---- S = Q K^T and dP = dO V^T (lane = query row, column = kv position) ----
    if (tid == 0) {
      bool w = true;
      if (step == 0) w = mbar_wait(bar_kv, 0, p.status, kStatusTimeoutMma);
      w = w && mbar_wait(bar_ld, step & 1, p.status, kStatusTimeoutMma);
      if (w) {
        tc_fence_after();
        const uint32_t ak = smem_u32(sK), av = smem_u32(sV), aq = smem_u32(sQ), ado = smem_u32(sDo);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          umma_bf16_ss(tm_s, umma_smem_desc(aq + off, 16, 1024), umma_smem_desc(ak + off, 16, 1024), idesc_kk,
                       kk ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          umma_bf16_ss(tm_dp, umma_smem_desc(ado + off, 16, 1024), umma_smem_desc(av + off, 16, 1024), idesc_kk,
                       kk ? 1u : 0u);
        }
      }
      umma_commit(bar_mma);
    }
    // this row's statistics travel while the MMAs run
    const int qp = q0 + r;
    float lse2 = 0.f, dlt = 0.f;
    if (qp < seq_len) {
      lse2 = p.lse[(size_t)h * p.T + seq_start + qp] * 1.4426950408889634f;
      dlt = p.delta[(size_t)h * p.T + seq_start + qp];
    }
    if (!__all_sync(0xffffffffu, mbar_wait(bar_mma, step & 1, p.status, kStatusTimeoutEpilogue))) {
      ok = false;
      break;
    }
    tc_fence_after();

    // ---- P and dS for this thread's query row, its half of the kv columns ----
    // masks are only needed on the diagonal tile (causal) and on tiles that stick out of the sequence
    const bool need_mask = (p.causal && q0 < k0 + 128) || q0 + 128 > seq_len || k0 + 128 > seq_len;
#pragma unroll 1
    for (int cc = 0; cc < 2; ++cc) {
      const int c = half * 2 + cc;  // 32-column chunk of the 128 kv columns
      uint32_t rs[32], rd[32];
      tmem_ld_32x32(tm_s + lane_off + c * 32, rs);
      tmem_ld_32x32(tm_dp + lane_off + c * 32, rd);
      tmem_ld_wait();
      uint32_t pp[16], dd[16];
      if (!need_mask) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse2));
          const float p1 = ex2_approx(fmaf(__uint_as_float(rs[i + 1]), p.scale_log2, -lse2));
          const float d0 = p0 * (__uint_as_float(rd[i]) - dlt) * p.scale;
          const float d1 = p1 * (__uint_as_float(rd[i + 1]) - dlt) * p.scale;
          pp[i / 2] = pack_bf16x2(p0, p1);
          dd[i / 2] = pack_bf16x2(d0, d1);
        }
      } else {
        const bool row_ok = qp < seq_len;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int kp = k0 + c * 32 + i + u;
            const bool valid = row_ok && kp < seq_len && (!p.causal || qp >= kp);
            const float prob = valid ? ex2_approx(fmaf(__uint_as_float(rs[i + u]), p.scale_log2, -lse2)) : 0.f;
            pv[u] = prob;
            dv[u] = prob * (__uint_as_float(rd[i + u]) - dlt) * p.scale;
          }
          pp[i / 2] = pack_bf16x2(pv[0], pv[1]);
          dd[i / 2] = pack_bf16x2(dv[0], dv[1]);
        }
      }
      // columns [c*32, c*32+32) of row r: 64-column chunk c/2, 16-byte pieces (c%2)*4 .. +3, swizzled by the row
      uint8_t* prow = sP + (c >> 1) * 16384 + r * 128;
      uint8_t* drow = sDs + (c >> 1) * 16384 + r * 128;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int piece = ((c & 1) * 4 + q) ^ (r & 7);
        *reinterpret_cast<uint4*>(prow + (piece << 4)) = make_uint4(pp[q * 4], pp[q * 4 + 1], pp[q * 4 + 2], pp[q * 4 + 3]);
        *reinterpret_cast<uint4*>(drow + (piece << 4)) = make_uint4(dd[q * 4], dd[q * 4 + 1], dd[q * 4 + 2], dd[q * 4 + 3]);
      }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();

    // ---- dV += P^T dO,  dK += dS^T Q,  dQ = dS K ----
    if (tid == 0) {
      tc_fence_after();
      const uint32_t ap = smem_u32(sP), ads = smem_u32(sDs);
      const uint32_t bdo = smem_u32(sDo), bq = smem_u32(sQ), bk = smem_u32(sK);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {  // contraction over 128 query rows; A = P^T read MN-major from P
        umma_bf16_ss(tm_dv, umma_smem_desc(ap + kk * 2048, 16384, 1024), umma_smem_desc(bdo + kk * 2048, 16384, 1024),
                     idesc_mnmn, (step | kk) ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        umma_bf16_ss(tm_dk, umma_smem_desc(ads + kk * 2048, 16384, 1024), umma_smem_desc(bq + kk * 2048, 16384, 1024),
                     idesc_mnmn, (step | kk) ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {  // contraction over 128 kv rows; A = dS K-major, B = K read MN-major
        const uint32_t aoff = (kk / 4) * 16384 + (kk % 4) * 32;
        umma_bf16_ss(tm_s, umma_smem_desc(ads + aoff, 16, 1024), umma_smem_desc(bk + kk * 2048, 16384, 1024), idesc_kmn,
                     kk ? 1u : 0u);
      }
      umma_commit(bar_mma2);
    }
    if (!__all_sync(0xffffffffu, mbar_wait(bar_mma2, step & 1, p.status, kStatusTimeoutEpilogue))) {
      ok = false;
      break;
    }
    tc_fence_after();
    // Q / dO of the next step stream in while dQ is written out
    if (step + 1 < total_steps && tid == 0) issue_loads(step + 1);

    // ---- dQ tile -> fp32 reduction buffer ----
    // TMEM hands every thread one query row.  Adding a row to global memory from its own thread would make each warp
    // instruction touch 32 rows, 16 bytes each.  The tile is turned through shared memory instead (the P / dS
    // buffers, which the MMAs above have finished reading): 16-byte pieces at slot (piece ^ (row & 31)), read back
    // with lane = piece, so that each warp instruction adds one whole row of D floats.
    {
      float4* stage = reinterpret_cast<float4*>(sP);  // [128 rows][D / 4 pieces] fp32 = 64 KB at D = 128
      static_assert(L::kDstOff == L::kPtOff + L::kSq, "the dQ staging tile spans the P and dS buffers");
      constexpr int kPieces = D / 4;
#pragma unroll 1
      for (int cc = 0; cc < D / 64; ++cc) {
        const int c = half * (D / 64) + cc;  // 32-column chunk of the D columns
        uint32_t rq[32];
        tmem_ld_32x32(tm_s + lane_off + c * 32, rq);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const int piece = c * 8 + g;
          stage[r * kPieces + (piece ^ (r & (kPieces - 1)))] =
              make_float4(__uint_as_float(rq[g * 4]), __uint_as_float(rq[g * 4 + 1]), __uint_as_float(rq[g * 4 + 2]),
                          __uint_as_float(rq[g * 4 + 3]));
        }
      }
      tc_fence_before();
      __syncthreads();
      if (lane < kPieces) {
#pragma unroll 4
        for (int rr = 0; rr < 16; ++rr) {
          const int row = warp * 16 + rr;
          const int qrow = q0 + row;
          if (qrow >= seq_len) break;
          const float4 v = stage[row * kPieces + (lane ^ (row & (kPieces - 1)))];
          float* dst = p.dq_accum + (size_t)(seq_start + qrow) * (size_t)(p.Hq * D) + (size_t)h * D + lane * 4;
          red_add_v4(dst, v.x, v.y, v.z, v.w);
        }
      }
    }
    __syncthreads();  // the staging tile is free again before the next step's P / dS are written
  }

  // ---- dK, dV tiles (lane = kv row) -> bf16 into the packed gradient buffer ----
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  if (ok) {
    const int kp = k0 + r;
    const bool row_valid = kp < seq_len;
    const size_t width = (size_t)(p.Hq + 2 * p.Hkv) * D;
    __nv_bfloat16* krow = p.dqkv + (size_t)(seq_start + (row_valid ? kp : 0)) * width + kcol;
    __nv_bfloat16* vrow = p.dqkv + (size_t)(seq_start + (row_valid ? kp : 0)) * width + vcol;
#pragma unroll 1
    for (int cc = 0; cc < D / 64; ++cc) {
      const int c = half * (D / 64) + cc;
      uint32_t rk[32], rv[32];
      if (total_steps > 0) {
        tmem_ld_32x32(tm_dk + lane_off + c * 32, rk);
        tmem_ld_32x32(tm_dv + lane_off + c * 32, rv);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) rk[i] = rv[i] = 0u;
      }
      if (row_valid) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 a, b;
          a.x = pack_bf16x2(__uint_as_float(rk[g * 8 + 0]), __uint_as_float(rk[g * 8 + 1]));
          a.y = pack_bf16x2(__uint_as_float(rk[g * 8 + 2]), __uint_as_float(rk[g * 8 + 3]));
          a.z = pack_bf16x2(__uint_as_float(rk[g * 8 + 4]), __uint_as_float(rk[g * 8 + 5]));
          a.w = pack_bf16x2(__uint_as_float(rk[g * 8 + 6]), __uint_as_float(rk[g * 8 + 7]));
          b.x = pack_bf16x2(__uint_as_float(rv[g * 8 + 0]), __uint_as_float(rv[g * 8 + 1]));
          b.y = pack_bf16x2(__uint_as_float(rv[g * 8 + 2]), __uint_as_float(rv[g * 8 + 3]));
          b.z = pack_bf16x2(__uint_as_float(rv[g * 8 + 4]), __uint_as_float(rv[g * 8 + 5]));
          b.w = pack_bf16x2(__uint_as_float(rv[g * 8 + 6]), __uint_as_float(rv[g * 8 + 7]));
          *reinterpret_cast<uint4*>(krow + c * 32 + g * 8) = a;
          *reinterpret_cast<uint4*>(vrow + c * 32 + g * 8) = b;
        }
      }
    }
  }
  if (!ok && tid == 0) {
    mbar_wait(bar_ld, 0, nullptr, 0);
    mbar_wait(bar_ld, 1, nullptr, 0);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h)
__global__ void fmha_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int T, int Hq, int D) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)T * Hq) return;
  const int t = (int)(w / Hq), h = (int)(w % Hq);
  const __nv_bfloat16* a = o + ((size_t)t * Hq + h) * D;
  const __nv_bfloat16* b = d_o + ((size_t)t * Hq + h) * D;
  float s = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + i));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(b + i));
    s += x.x * y.x + x.y * y.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[(size_t)h * T + t] = s;
}

// dqkv[t, h*D + d] = bf16(dq_accum[t, h*D + d]) for the q part of the packed gradient
__global__ void fmha_dq_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dqkv, int T,
                                    int qwidth, int width) {
  const long long total = (long long)T * (qwidth / 4);
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / (qwidth / 4)), c = (int)(idx % (qwidth / 4)) * 4;
    const float4 v = *reinterpret_cast<const float4*>(acc + (size_t)t * qwidth + c);
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dqkv + (size_t)t * width + c) = o;
  }
}

template <int D>
static int launch_bwd(const CUtensorMap& mqkv, const CUtensorMap& mdo, const FmhaBwdParams& p, int num_tiles,
                      cudaStream_t stream) {
  using L = BwdSmem<D>;
  auto kernel = fmha_bwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(num_tiles, p.Hkv);
  kernel<<<grid, kBwdThreads, L::kTotal, stream>>>(mqkv, mdo, p);
  return (int)cudaGetLastError();
}

}  // namespace sb

using namespace sb;

// qkv: packed forward input; out/d_out: [T, Hq*D]; dq_accum: fp32 scratch [T, Hq*D] (zeroed here);
// delta: fp32 scratch [Hq, T]; dqkv: packed gradient output.
extern "C" int sb_fmha_bwd(const void* qkv, const void* out, const void* d_out, const float* lse, float* delta,
                           float* dq_accum, void* dqkv, const int* tile_seq_start, const int* tile_seq_len,
                           const int* tile_k0, int num_tiles, int T, int Hq, int Hkv, int D, int causal,
                           float scale, int* status, cudaStream_t stream) {
  if (num_tiles == 0 || T == 0) return 0;
  if (D != 64 && D != 128) return -2;
  static thread_local bool tl_context_bound = false;
  if (!tl_context_bound) {
    cudaFree(0);
    tl_context_bound = true;
  }
  const long long width = (long long)(Hq + 2 * Hkv) * D;
  const long long qwidth = (long long)Hq * D;
  CUtensorMap mqkv, mdo;
  int r = make_tensor_map_bf16_2d(&mqkv, qkv, width, T, width, 64, 128);
  if (r) return r;
  r = make_tensor_map_bf16_2d(&mdo, d_out, qwidth, T, qwidth, 64, 128);
  if (r) return r;
  cudaMemsetAsync(dq_accum, 0, sizeof(float) * (size_t)T * qwidth, stream);
  {
    const long long warps = (long long)T * Hq;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    fmha_delta_kernel<<<(unsigned)blocks, threads, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)d_out,
                                                                delta, T, Hq, D);
  }
  FmhaBwdParams p;
  p.tile_seq_start = tile_seq_start; p.tile_seq_len = tile_seq_len; p.tile_k0 = tile_k0;
  p.lse = lse; p.delta = delta; p.dq_accum = dq_accum; p.dqkv = reinterpret_cast<__nv_bfloat16*>(dqkv);
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  r = (D == 128) ? launch_bwd<128>(mqkv, mdo, p, num_tiles, stream) : launch_bwd<64>(mqkv, mdo, p, num_tiles, stream);
  if (r) return r;
  {
    const long long total = (long long)T * (qwidth / 4);
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)num_sms() * 8;
    if (blocks > cap) blocks = cap;
    fmha_dq_cast_kernel<<<(unsigned)blocks, 256, 0, stream>>>(dq_accum, (__nv_bfloat16*)dqkv, T, (int)qwidth, (int)width);
  }
  return (int)cudaGetLastError();
}
