// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, operands
// staged by TMA into 128-byte-swizzled shared memory).  Replaces the cuBLAS calls behind every
// nn.Linear of the reference (its models are HF/Megatron modules: siirl/engine/fsdp_workers.py:631-744).
//
//   C[M,N] (+)= sum_k A[m,k] * B[n,k]
//
// Operand storage ("major"):
//   A K-major : global [M, K] row-major (K contiguous)          -- activations in forward/dgrad
//   A MN-major: global [K, M] row-major (M contiguous)          -- dy^T in wgrad
//   B K-major : global [N, K] row-major                          -- nn.Linear weight in forward
//   B MN-major: global [K, N] row-major                          -- weight in dgrad, x in wgrad
//
// Kernel shape: persistent, one CTA per SM, 6 warps:
//   warp 0      TMA producer (one lane)          smem ring of STAGES x (A 128x64 + B BNx64)
//   warp 1      TMEM allocator + MMA issuer      tcgen05.mma 128xBNx16, two TMEM accumulators
//   warps 2..5  epilogue                         tcgen05.ld -> (+bias) -> bf16/fp32 -> global
// The epilogue of tile i overlaps the main loop of tile i+1 through the two accumulators.
#include "common.cuh"
#include "launchers.h"

namespace sb {

constexpr int kBM = 128;
constexpr int kBK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;  // optional, length N (EPI_BF16 only)
  int* status;
  int num_m_blocks, num_n_blocks, num_k_blocks;
  // split-K: tile t covers k-blocks [ks*kb_per_split, (ks+1)*kb_per_split) and writes slab ks of C
  // (C + ks * slab_stride elements); a separate kernel sums the slabs.  k_splits == 1 is the normal GEMM.
  int k_splits, kb_per_split;
  long long slab_stride;
  const struct ArParams* ar;  // EPI_F32_AR only (device memory)
  // grouped GEMM (mixture-of-experts), both optional:
  //  * tile_group[mb] >= 0 selects the group (expert) whose B matrix m-block mb multiplies; B holds the groups
  //    stacked along its outer dimension, b_group_rows rows each; -1 skips the m-block (padding past the last
  //    routed row, known only on the device).
  //  * group_rows[g], group_rows[g+1] (multiples of 64) bound the contraction rows of group g; tiles are
  //    (g, mb, nb) and C advances by c_group_stride elements per group (per-expert weight gradients).
  const int* tile_group;
  long long b_group_rows;
  const int* group_rows;
  long long c_group_stride;
  const struct AgParams* ag;  // all-gather of B fused into the GEMM (device memory), or nullptr
  int ag_copiers;             // number of copier CTAs (== ag->copiers), 0 without ag
  // vocabulary GEMM epilogues (EPI_LMSTAT / EPI_DLOGITS): rows are tokens, columns vocabulary entries
  const long long* labels;    // [M] target id per row (< 0 or >= N: no target)
  float inv_temp;             // logits are multiplied by this before the softmax
  float4* lm_partial;         // EPI_LMSTAT out: [M, num_n_blocks] (max, sum exp(z - max), sum exp(z - max) * z, z[label] or -inf)
  const float* lm_lse;        // EPI_DLOGITS in: [M] log-sum-exp, entropy (or null), d loss / d logp, d loss / d entropy (or null)
  const float* lm_ent;
  const float* lm_glogp;
  const float* lm_gent;
};

// all-gather -> GEMM in one launch: B [N, K] is sharded by rows over the ranks (rows_per_rank each, in symmetric
// memory).  The first `copiers` CTAs pull the shards chunk by chunk (one chunk = one BN-row n-block) from the peers
// into the local `staging` copy of B with plain peer loads and count each finished chunk in flags[chunk]; the other
// CTAs run the tcgen05 GEMM on `staging`, their TMA producers waiting (bounded) for a chunk's count before its
// first load.  Tiles and chunks start at this rank's own shard, so the math on local rows hides the first transfers.
constexpr int kAgMaxRanks = 16;
struct AgParams {
  const __nv_bfloat16* shard[kAgMaxRanks];  // every rank's shard [rows_per_rank, K], row pitch ld
  __nv_bfloat16* staging;                   // local [N, K], row pitch ld
  int* flags;                               // [num_n_blocks] arrival counters (monotonic over launches)
  int* local;                               // [0] epoch, [1] exit counter
  long long ld;
  int world, rank, rows_per_rank, copiers;
};

struct TileInfo {
  int m0, n0, kb0, kb1, b_off;
  long long c_off;
  bool skip;
};

// EPI_BF16_T / EPI_F32_T store the tile TRANSPOSED (C[col * ldc + row]): the "swap A and B" form of a GEMM with few
// tokens, where the weight matrix rides in the 128-row A operand (every weight byte is fetched once) and all tokens
// sit in the B operand.  EPI_LMSTAT reduces each row of a vocabulary tile to online-softmax partial statistics and
// EPI_DLOGITS turns the tile into the gradient of the logits; neither writes fp32 logits to memory.
enum { EPI_BF16 = 0, EPI_F32_ACC = 1, EPI_F32 = 2, EPI_F32_AR = 3, EPI_BF16_T = 4, EPI_F32_T = 5, EPI_LMSTAT = 6,
       EPI_DLOGITS = 7 };

// Row-parallel GEMM fused with its all-reduce over peer memory (EPI_F32_AR).  Every rank of a tensor-parallel
// group runs the same launch on its K-shard.  Per output tile: the fp32 partial goes to this rank's symmetric
// `partial` buffer (after a local split-K reduction when k_splits > 1) and a ready flag is raised at the tile's
// owner (tile % world); the owner's epilogue warps wait for the flags (bounded), pull the tile from every peer
// with plain peer loads, add the bias, convert to bf16 and store the result into every rank's `out`, then raise
// done flags.  A rank leaves the kernel only when all its tiles are done, so at kernel end `out` is complete
// locally and `partial` may be overwritten by the next launch.  Flags carry a launch epoch that lives in device
// memory (`local[0]`, advanced by the last CTA to exit), so replaying the launch from a CUDA graph works.
constexpr int kArMaxRanks = 16;
struct ArParams {
  float* partial[kArMaxRanks];          // fp32 [M, N] per rank
  __nv_bfloat16* out[kArMaxRanks];      // bf16 [M, ldo] per rank
  int* ready[kArMaxRanks];              // ready[tile * kArMaxRanks + src] on each rank
  int* done[kArMaxRanks];               // done[tile] on each rank
  int* local;                           // [0] epoch, [1] exit counter, [2 + tile] split arrival counters
  long long ldo;
  int world, rank;
  float* recv[kArMaxRanks];             // one-shot: fp32 [2 (epoch parity)][world (source)][recv_slab] per rank
  long long recv_slab;                  // floats per (parity, source) slab: >= rows of the largest one-shot call * N
  int one_shot;                         // 1: push protocol, 0: owner pull protocol
};

__device__ __forceinline__ float4 ld_volatile_f4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierOffset = STAGES * kStageBytes;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem slot, abort flag
  static constexpr int kTotalBytes = kBarrierOffset + (2 * STAGES + 4) * 8 + 16 + 1024 /*align slack*/;
};

__device__ __forceinline__ void tile_coords(int tile, int num_m_blocks, int num_n_blocks, int& mb,
                                            int& nb, int kGroupM = 8) {
  const int tiles_per_group = kGroupM * num_n_blocks;
  const int group = tile / tiles_per_group;
  const int first_m = group * kGroupM;
  const int gm = min(kGroupM, num_m_blocks - first_m);
  const int t = tile - group * tiles_per_group;
  mb = first_m + t % gm;
  nb = t / gm;
}

template <int BN>
__device__ __forceinline__ TileInfo tile_info(const GemmParams& p, int tile, int tiles_mn) {
  TileInfo t;
  int mb, nb;
  const int outer = tile / tiles_mn;  // k-split index, or group index when group_rows is set
  // all-gather mode sweeps more m-blocks per n-block, so that later chunks of B are needed later
  tile_coords(tile - outer * tiles_mn, p.num_m_blocks, p.num_n_blocks, mb, nb, p.ag ? 32 : 8);
  if (p.ag) {  // start at the n-blocks of this rank's own shard
    const int first = (p.ag->rank * p.ag->rows_per_rank) / BN;
    nb = (nb + first) % p.num_n_blocks;
  }
  t.m0 = mb * kBM;
  t.n0 = nb * BN;
  t.b_off = 0;
  t.skip = false;
  if (p.group_rows) {
    t.kb0 = p.group_rows[outer] / kBK;
    t.kb1 = p.group_rows[outer + 1] / kBK;
    t.c_off = outer * p.c_group_stride;
    t.skip = t.kb1 <= t.kb0;
  } else {
    t.kb0 = outer * p.kb_per_split;
    t.kb1 = min(t.kb0 + p.kb_per_split, p.num_k_blocks);
    t.c_off = outer * p.slab_stride;
    if (p.tile_group) {
      const int g = p.tile_group[mb];
      t.skip = g < 0;
      t.b_off = g < 0 ? 0 : (int)(g * p.b_group_rows);
    }
  }
  return t;
}

// Copier CTA of the all-gather -> GEMM kernel.  One thread drives bulk asynchronous copies (the TMA engine, without
// multicast): each n-block chunk of B is one contiguous byte range (row pitch == K) in the owner's shard and in the
// local staging matrix; pieces of kAgPiece bytes bounce through a ring of shared-memory stages, so a CTA keeps
// (stages - 1) * kAgPiece bytes in flight over NVLink with no registers involved.  Chunk c belongs to copier
// c % copiers.  After a chunk's stores have completed the chunk is counted in flags[c].
constexpr int kAgPiece = 32768;

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}

template <int BN, int STAGES_BYTES>
__device__ __forceinline__ void ag_copier(const GemmParams& p, uint8_t* smem, uint64_t* bars, int nbars) {
  if (threadIdx.x != 0) return;
  const AgParams& ag = *p.ag;
  const int nblk = p.num_n_blocks;
  const int first = (ag.rank * ag.rows_per_rank) / BN;
  constexpr int kStages = STAGES_BYTES / kAgPiece < 6 ? STAGES_BYTES / kAgPiece : 6;
  const int S = kStages < nbars ? kStages : nbars;
  uint32_t phase_bits = 0;  // parity of each stage's barrier
  bool ok = true;
  for (int i = blockIdx.x; i < nblk && ok; i += ag.copiers) {
    const int nb = (first + i) % nblk;
    const int r0 = nb * BN;
    const int rows = min(BN, p.N - r0);
    const int owner = r0 / ag.rows_per_rank;  // rows_per_rank is a multiple of BN: one owner per chunk
    const uint8_t* src = reinterpret_cast<const uint8_t*>(ag.shard[owner] + (long long)(r0 - owner * ag.rows_per_rank) * ag.ld);
    uint8_t* dst = reinterpret_cast<uint8_t*>(ag.staging + (long long)r0 * ag.ld);
    const long long bytes = (long long)rows * ag.ld * 2;
    const int pieces = (int)((bytes + kAgPiece - 1) / kAgPiece);
    // software pipeline: loads run S-1 pieces ahead of the stores
    for (int j = 0; j < pieces + S - 1 && ok; ++j) {
      if (j < pieces) {
        const int st = j % S;
        if (j >= S) tma_store_wait_read<0>();  // the store that last used this stage has read it
        const uint32_t n = (uint32_t)min((long long)kAgPiece, bytes - (long long)j * kAgPiece);
        mbar_arrive_expect_tx(&bars[st], n);
        bulk_g2s(smem + st * kAgPiece, src + (long long)j * kAgPiece, n, &bars[st]);
      }
      const int k = j - (S - 1);
      if (k >= 0 && k < pieces) {
        const int st = k % S;
        if (!mbar_wait(&bars[st], (phase_bits >> st) & 1u, p.status, kStatusTimeoutProducer)) {
          ok = false;
          break;
        }
        phase_bits ^= 1u << st;
        const uint32_t n = (uint32_t)min((long long)kAgPiece, bytes - (long long)k * kAgPiece);
        bulk_s2g(dst + (long long)k * kAgPiece, smem + st * kAgPiece, n);
        tma_store_commit();
      }
    }
    tma_store_wait<0>();  // all stores of the chunk have completed
    asm volatile("fence.proxy.async;" ::: "memory");
    __threadfence();
    if (ok) flag_add_release(ag.flags + nb, 1);
  }
  tma_store_wait<0>();
}

// Epilogue of one output tile: this thread owns row `row` of the tile (TMEM lane) and sweeps the BN accumulator
// columns starting at TMEM address `taddr` in chunks of 32.  Shared by the one-CTA and the CTA-pair kernels.
template <int BN, int EPI>
__device__ __forceinline__ void gemm_epilogue_tile(const GemmParams& p, const TileInfo& ti, uint32_t taddr, int row) {
  const int n0 = ti.n0;
  if constexpr (EPI == EPI_BF16_T || EPI == EPI_F32_T) {
    // lane = output column (weight row), register = output row (token): 32 lanes store 32 neighbouring elements
    float bv = 0.f;
    if constexpr (EPI == EPI_BF16_T) {
      if (p.bias && row < p.M) bv = __bfloat162float(p.bias[row]);
    }
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      const int col0 = n0 + c * 32;
      if (col0 >= p.N) break;  // uniform over the CTA: the remaining columns are tokens that do not exist
      uint32_t r[32];
      tmem_ld_32x32(taddr + c * 32, r);
      tmem_ld_wait();
      if (row < p.M) {
        if constexpr (EPI == EPI_BF16_T) {
          __nv_bfloat16* cb = reinterpret_cast<__nv_bfloat16*>(p.C) + ti.c_off + row;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + i < p.N) cb[(long long)(col0 + i) * p.ldc] = __float2bfloat16(__uint_as_float(r[i]) + bv);
        } else {
          float* cf = reinterpret_cast<float*>(p.C) + ti.c_off + row;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + i < p.N) cf[(long long)(col0 + i) * p.ldc] = __uint_as_float(r[i]);
        }
      }
    }
  } else if constexpr (EPI == EPI_LMSTAT) {
    // two sweeps over this thread's row of the tile in TMEM: row maximum, then the sums relative to it
    constexpr float kLog2e = 1.4426950408889634f;
    const float sc2 = p.inv_temp * kLog2e;
    const long long y = row < p.M ? p.labels[row] : -1;
    float m2 = -INFINITY;  // maximum of z * log2(e)
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      const int col0 = n0 + c * 32;
      if (col0 >= p.N) break;
      uint32_t r[32];
      tmem_ld_32x32(taddr + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) m2 = fmaxf(m2, __uint_as_float(r[i]) * sc2);
    }
    float ssum = 0.f, tsum = 0.f, zl = -INFINITY;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      const int col0 = n0 + c * 32;
      if (col0 >= p.N) break;
      uint32_t r[32];
      tmem_ld_32x32(taddr + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (col0 + i < p.N) {
          const float v = __uint_as_float(r[i]);
          const float e = exp2f(v * sc2 - m2);
          ssum += e;
          tsum += e * (v * p.inv_temp);
          if ((long long)(col0 + i) == y) zl = v * p.inv_temp;
        }
      }
    }
    if (row < p.M)
      p.lm_partial[(long long)row * p.num_n_blocks + n0 / BN] = make_float4(m2 * (1.f / kLog2e), ssum, tsum, zl);
  } else if constexpr (EPI == EPI_DLOGITS) {
    // d z_j = g_logp * (1[j = y] - p_j) - g_H * p_j * (z_j - lse + H), times 1/temperature for d logits_j
    const bool rv = row < p.M;
    const long long y = rv ? p.labels[row] : -1;
    const float l = rv ? p.lm_lse[row] : 0.f;
    // y == -2: the target exists but in another rank's vocabulary slice (vocabulary-parallel LM head): the
    // softmax term of its gradient still applies here, the one-hot term never matches
    const float glp = (rv && ((y >= 0 && y < p.N) || y == -2)) ? p.lm_glogp[row] : 0.f;
    const float ge = (rv && p.lm_gent) ? p.lm_gent[row] : 0.f;
    const float H = (rv && p.lm_ent) ? p.lm_ent[row] : 0.f;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      const int col0 = n0 + c * 32;
      if (col0 >= p.N) break;
      uint32_t r[32];
      tmem_ld_32x32(taddr + c * 32, r);
      tmem_ld_wait();
      if (rv) {
        __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (col0 + g * 8 + 8 <= p.N) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float x = __uint_as_float(r[g * 8 + i]) * p.inv_temp;
              const float pj = __expf(x - l);
              const float onehot = ((long long)(col0 + g * 8 + i) == y) ? 1.f : 0.f;
              v[i] = (glp * (onehot - pj) - ge * pj * (x - l + H)) * p.inv_temp;
            }
            uint4 o;
            o.x = pack_bf16x2(v[0], v[1]);
            o.y = pack_bf16x2(v[2], v[3]);
            o.z = pack_bf16x2(v[4], v[5]);
            o.w = pack_bf16x2(v[6], v[7]);
            *reinterpret_cast<uint4*>(crow + g * 8) = o;
          }
        }
      }
    }
  } else {
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(taddr + c * 32, r);
    tmem_ld_wait();
    const int col0 = n0 + c * 32;
    if (row < p.M && col0 < p.N) {
      if constexpr (EPI == EPI_BF16) {
        __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + ti.c_off + (long long)row * p.ldc + col0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (col0 + g * 8 + 8 <= p.N) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]);
            if (p.bias) {
              uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col0 + g * 8);
              const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                float2 f = __bfloat1622float2(b2[i]);
                v[2 * i] += f.x;
                v[2 * i + 1] += f.y;
              }
            }
            uint4 o;
            o.x = pack_bf16x2(v[0], v[1]);
            o.y = pack_bf16x2(v[2], v[3]);
            o.z = pack_bf16x2(v[4], v[5]);
            o.w = pack_bf16x2(v[6], v[7]);
            *reinterpret_cast<uint4*>(crow + g * 8) = o;
          }
        }
      } else {
        float* crow = reinterpret_cast<float*>(p.C) + ti.c_off + (long long)row * p.ldc + col0;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          if (col0 + g * 4 + 4 <= p.N) {
            float4 o = make_float4(__uint_as_float(r[g * 4]), __uint_as_float(r[g * 4 + 1]),
                                   __uint_as_float(r[g * 4 + 2]), __uint_as_float(r[g * 4 + 3]));
            if constexpr (EPI == EPI_F32_ACC) {
              const float4 old = *reinterpret_cast<const float4*>(crow + g * 4);
              o.x += old.x;
              o.y += old.y;
              o.z += old.z;
              o.w += old.w;
            }
            *reinterpret_cast<float4*>(crow + g * 4) = o;
          }
        }
      }
    }
  }
  }
}

#include "gemm_ar.cuh"

template <int BN, int STAGES, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                         const __grid_constant__ CUtensorMap map_b, GemmParams p) {
  using L = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarrierOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_mn = p.num_m_blocks * p.num_n_blocks;
  const int copiers = p.ag_copiers;
  const bool is_copier = (int)blockIdx.x < copiers;
  const int cta0 = (int)blockIdx.x - copiers;       // index among the GEMM CTAs
  const int nctas = (int)gridDim.x - copiers;
  const int ag_epoch = p.ag ? p.ag->local[0] + 1 : 0;
  const int num_tiles = tiles_mn * p.k_splits;  // k_splits holds the group count when group_rows is set
  constexpr uint32_t kTmemCols = 2 * BN;  // 256 or 512 (power of two)

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 128);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (is_copier) {
    ag_copier<BN, L::kBarrierOffset>(p, smem, full_bar, STAGES);
  } else if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int last_armed[STAGES];
#pragma unroll
      for (int s = 0; s < STAGES; ++s) last_armed[s] = -1;
      bool ok = true;
      for (int tile = cta0; tile < num_tiles && ok; tile += nctas) {
        const TileInfo ti = tile_info<BN>(p, tile, tiles_mn);
        if (ti.skip) continue;
        const int m0 = ti.m0, n0 = ti.n0, kb0 = ti.kb0, kb1 = ti.kb1;
        if (p.ag) {
          // the n-block's rows must have landed in the staging copy (written by copier CTAs through the generic
          // proxy, read below by TMA through the async proxy)
          if (!flag_wait_ge(p.ag->flags + n0 / BN, ag_epoch, p.status)) {
            ok = false;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kStatusTimeoutProducer)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb_ = sa + L::kABytes;
          mbar_arrive_expect_tx(&full_bar[stage], L::kStageBytes);
          last_armed[stage] = (int)phase;
          const int k0 = kb * kBK;
          if constexpr (!A_MN) {
            tma_load_2d(sa, &map_a, &full_bar[stage], k0, m0);
          } else {
            tma_load_2d(sa, &map_a, &full_bar[stage], m0, k0);
            tma_load_2d(sa + 8192, &map_a, &full_bar[stage], m0 + 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb_, &map_b, &full_bar[stage], k0, n0 + ti.b_off);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb_ + c * 8192, &map_b, &full_bar[stage], n0 + c * 64, k0 + ti.b_off);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // leave no bulk copy in flight into shared memory that is about to be released
        for (int s = 0; s < STAGES; ++s)
          if (last_armed[s] >= 0) mbar_wait(&full_bar[s], (uint32_t)last_armed[s], nullptr, 0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    constexpr uint32_t idesc = umma_idesc_bf16(kBM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = cta0; tile < num_tiles && ok; tile += nctas) {
      const TileInfo ti = tile_info<BN>(p, tile, tiles_mn);
      if (ti.skip) continue;
      if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, kStatusTimeoutMma)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + acc * BN;
      const int kb0 = ti.kb0, kb1 = ti.kb1;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, p.status, kStatusTimeoutMma)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb_ = sa + L::kABytes;
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            const uint64_t da = A_MN ? umma_smem_desc(sa + kk * 2048, 8192, 1024)
                                     : umma_smem_desc(sa + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc(sb_ + kk * 2048, 8192, 1024)
                                     : umma_smem_desc(sb_ + kk * 32, 16, 1024);
            umma_bf16_ss(tmem_d, da, db, idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs have read it
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok && lane == 0) umma_commit(&tmem_full[acc]);
      __syncwarp();
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5) ------------------------------
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    const int row_in_tile = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    // all-reduce state (EPI_F32_AR): tiles whose done flag this CTA still has to see, by loop iteration
    const int epi_tid = (int)threadIdx.x - 64;
    volatile uint32_t* ar_smem = tmem_slot + 1;  // [0] "this CTA finishes the tile", [1] abort
    unsigned long long ar_pending = 0ull;
    int ar_iter = 0;
    int ar_epoch = 0;
    bool ar_ok = true;
    if constexpr (EPI == EPI_F32_AR) {
      ar_epoch = p.ar->local[0] + 1;
      if (epi_tid == 0) ar_smem[1] = 0;
      epi_bar();
    }
    for (int tile = cta0; tile < num_tiles; tile += nctas) {
      const TileInfo ti = tile_info<BN>(p, tile, tiles_mn);
      if (ti.skip) continue;
      const int ks = tile / tiles_mn;
      const int row = ti.m0 + row_in_tile;
      const int n0 = ti.n0;
      if constexpr (EPI == EPI_F32_AR) {
        // the 128 epilogue threads meet at named barriers below: leave the loop together or not at all
        if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, kStatusTimeoutEpilogue)) ar_smem[1] = 1;
        epi_bar();
        if (ar_smem[1] != 0) break;
      } else {
        if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, kStatusTimeoutEpilogue)) break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      gemm_epilogue_tile<BN, EPI>(p, ti, taddr, row);
      tc_fence_before();
      mbar_arrive(&tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
      if constexpr (EPI == EPI_F32_AR) {
        ar_tile_phase<BN>(p, tile - ks * tiles_mn, ti.m0, n0, quarter, lane, epi_tid, ar_smem, ar_epoch, ar_ok,
                          ar_pending, ar_iter);
        ++ar_iter;
      }
    }
    if constexpr (EPI == EPI_F32_AR) {
      // every tile this CTA handed to a remote owner must be finished before `out` is used and before the
      // next launch may overwrite `partial`
      if (epi_tid == 0) {
        int it = 0;
        for (int tile = cta0; tile < num_tiles && it < 64; tile += nctas, ++it) {
          if (!((ar_pending >> it) & 1ull) || !ar_ok) continue;
          const int tile_mn = tile % tiles_mn;
          if (!flag_wait_ge(p.ar->done[p.ar->rank] + tile_mn, ar_epoch, p.status)) ar_ok = false;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (p.ag && threadIdx.x == 0) {
    __threadfence();
    const int prev = atomicAdd(&p.ag->local[1], 1);
    if (prev == (int)gridDim.x - 1) {
      p.ag->local[1] = 0;
      p.ag->local[0] = ag_epoch;
    }
  }
  if constexpr (EPI == EPI_F32_AR) {
    if (threadIdx.x == 64) {  // an epilogue thread: it knows the epoch
      __threadfence();
      const int prev = atomicAdd(&p.ar->local[1], 1);
      if (prev == (int)gridDim.x - 1) {
        p.ar->local[1] = 0;
        p.ar->local[0] = p.ar->local[0] + 1;
      }
    }
  }
}


// ---------------------------------------------------------------------------------------
// CTA-pair variant: clusters of two CTAs share one 256 x 256 output tile through tcgen05 cta_group::2.
// Each CTA stages its own 128 rows of A and its own 128 of the tile's 256 B rows (its TMA loads count on the leader's
// mbarrier; nothing is broadcast between the CTAs), the leader's MMA thread issues one 256 x 256 x 16 instruction per
// k-step that reads both CTAs' shared memory, and each CTA's TMEM receives the accumulator rows of its own 128 A
// rows.  Per SM and k-block this moves 32 KB through shared memory for 2 x 128 x 256 x 64 multiply-adds where the
// one-CTA kernel moves 48 KB, and the freed shared memory makes the pipeline six stages deep instead of four.
// Tiles are (k-split, m-pair-block, n-block); split-K writes fp32 slabs like the one-CTA kernel.
// ---------------------------------------------------------------------------------------
constexpr int kPairBN = 256;
constexpr int kPairStages = 6;
constexpr int kPairHalfBytes = 128 * kBK * 2;            // one operand half of one stage: 16 KB
constexpr int kPairStageBytes = 2 * kPairHalfBytes;      // A half + B half per CTA
constexpr int kPairBarrierOffset = kPairStages * kPairStageBytes;
constexpr int kPairSmemBytes = kPairBarrierOffset + (2 * kPairStages + 4) * 8 + 16 + 1024;

template <bool A_MN, bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kPairBarrierOffset);   // used in the leader CTA only
  uint64_t* empty_bar = full_bar + kPairStages;                                  // one copy per CTA
  uint64_t* tmem_full = empty_bar + kPairStages;                                 // one copy per CTA
  uint64_t* tmem_empty = tmem_full + 2;                                          // used in the leader CTA only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = (int)blockIdx.x >> 1;
  const int npairs = (int)gridDim.x >> 1;
  const int num_m2 = (p.M + 255) / 256;
  const int num_n = (p.N + kPairBN - 1) / kPairBN;
  const int tiles_mn = num_m2 * num_n;
  const int num_tiles = tiles_mn * p.k_splits;
  constexpr uint32_t kTmemCols = 2 * kPairBN;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 256);  // the epilogue threads of both CTAs
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // the partner's barriers are initialised before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_of = [&](int tile, int& m0, int& n0, int& kb0, int& kb1, long long& c_off) {
    const int ks = tile / tiles_mn;
    int mb, nb;
    tile_coords(tile - ks * tiles_mn, num_m2, num_n, mb, nb, 4);
    m0 = mb * 256;
    n0 = nb * kPairBN;
    kb0 = ks * p.kb_per_split;
    kb1 = min(kb0 + p.kb_per_split, p.num_k_blocks);
    c_off = ks * p.slab_stride;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int armed = 0;  // stages this CTA has ever issued loads into (for the abort path)
      for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
        int m0, n0, kb0, kb1;
        long long c_off;
        tile_of(tile, m0, n0, kb0, kb1, c_off);
        const int my_m0 = m0 + (int)rank * 128;   // this CTA's 128 rows of A
        const int my_n0 = n0 + (int)rank * 128;   // this CTA's 128 of the tile's 256 B rows
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kStatusTimeoutProducer)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kPairStageBytes;
          uint8_t* sb_ = sa + kPairHalfBytes;
          const uint32_t bar = mapa_shared(smem_u32(&full_bar[stage]), 0);  // the leader's barrier counts all bytes
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * kPairStageBytes);
          const int k0 = kb * kBK;
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, &map_a, bar, k0, my_m0);
          } else {
            tma_load_2d_pair(sa, &map_a, bar, my_m0, k0);
            tma_load_2d_pair(sa + 8192, &map_a, bar, my_m0 + 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb_, &map_b, bar, k0, my_n0);
          } else {
            tma_load_2d_pair(sb_, &map_b, bar, my_n0, k0);
            tma_load_2d_pair(sb_ + 8192, &map_b, bar, my_n0 + 64, k0);
          }
          if (armed < kPairStages) ++armed;
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      (void)armed;
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (leader) {
      constexpr uint32_t idesc = umma_idesc_bf16(256, kPairBN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // cluster addresses of the barriers this thread signals in both CTAs
      for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
        int m0, n0, kb0, kb1;
        long long c_off;
        tile_of(tile, m0, n0, kb0, kb1, c_off);
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, kStatusTimeoutMma)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kPairBN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, kStatusTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (lane == 0) {
            const uint32_t sa = smem_u32(smem + stage * kPairStageBytes);
            const uint32_t sb_ = sa + kPairHalfBytes;
#pragma unroll
            for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
              const uint64_t da = A_MN ? umma_smem_desc(sa + kk * 2048, 8192, 1024)
                                       : umma_smem_desc(sa + kk * 32, 16, 1024);
              const uint64_t db = B_MN ? umma_smem_desc(sb_ + kk * 2048, 8192, 1024)
                                       : umma_smem_desc(sb_ + kk * 32, 16, 1024);
              umma_bf16_ss_pair(tmem_d, da, db, idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
            }
            // free the stage in both CTAs once these MMAs have read it
            const uint32_t eb = smem_u32(&empty_bar[stage]);
            umma_commit_pair(mapa_shared(eb, 0));
            umma_commit_pair(mapa_shared(eb, 1));
          }
          __syncwarp();
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && lane == 0) {
          const uint32_t fb = smem_u32(&tmem_full[acc]);
          umma_commit_pair(mapa_shared(fb, 0));
          umma_commit_pair(mapa_shared(fb, 1));
        }
        __syncwarp();
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5 of both CTAs) ------------------------------
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = pair; tile < num_tiles; tile += npairs) {
      TileInfo ti;
      tile_of(tile, ti.m0, ti.n0, ti.kb0, ti.kb1, ti.c_off);
      ti.m0 += (int)rank * 128;
      ti.b_off = 0;
      ti.skip = false;
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, kStatusTimeoutEpilogue)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kPairBN;
      gemm_epilogue_tile<kPairBN, EPI>(p, ti, taddr, ti.m0 + row_in_tile);
      tc_fence_before();
      mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[acc]), 0));  // the accumulator is free: tell the leader
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();  // neither CTA releases shared memory or TMEM while the other may still touch it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

static bool g_pair_enabled = true;
static int g_pair_max_clusters[8] = {0};

template <bool A_MN, bool B_MN, int EPI>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t stream) {
  auto kernel = gemm_bf16_pair_kernel<A_MN, B_MN, EPI>;
  static bool configured = false;
  static int max_clusters = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * num_sms(), 1, 1);
    cfg.blockDim = dim3(192, 1, 1);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg);
    if (e != cudaSuccess || max_clusters < 1) {
      cudaGetLastError();
      max_clusters = num_sms() / 2;
    }
    configured = true;
  }
  const int tiles = ((p.M + 255) / 256) * ((p.N + kPairBN - 1) / kPairBN) * p.k_splits;
  const int clusters = tiles < max_clusters ? tiles : max_clusters;
  kernel<<<2 * clusters, 192, kPairSmemBytes, stream>>>(ma, mb, p);
  return (int)cudaGetLastError();
}

static int dispatch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int a_mn, int b_mn, int epi,
                         cudaStream_t stream) {
#define SB_PAIR(AM, BM_, E)                  \
  if (a_mn == AM && b_mn == BM_ && epi == E) \
    return launch_pair<AM != 0, BM_ != 0, E>(ma, mb, p, stream);
  SB_PAIR(0, 0, EPI_BF16)
  SB_PAIR(0, 1, EPI_BF16)
  SB_PAIR(1, 1, EPI_F32_ACC)
  SB_PAIR(1, 1, EPI_F32)
  SB_PAIR(0, 0, EPI_F32)
  SB_PAIR(0, 0, EPI_BF16_T)
  SB_PAIR(0, 0, EPI_F32_T)
  SB_PAIR(0, 0, EPI_LMSTAT)
  SB_PAIR(0, 0, EPI_DLOGITS)
#undef SB_PAIR
  return -2;
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor map: inner extent `inner` (contiguous), outer extent `outer` with row pitch
// `pitch_elems`; box = box_inner x box_outer, 128-byte swizzle, zero fill out of bounds.
int make_tensor_map_bf16_2d(CUtensorMap* map, const void* base, long long inner, long long outer,
                            long long pitch_elems, int box_inner, int box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)pitch_elems * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

static int g_num_sms = 0;
int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int EPI>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int max_ctas,
                       cudaStream_t stream) {
  using L = GemmSmem<BN, STAGES>;
  auto kernel = gemm_bf16_tcgen05_kernel<BN, STAGES, A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotalBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = p.num_m_blocks * p.num_n_blocks * p.k_splits;
  const int avail = num_sms() - p.ag_copiers;
  int grid = tiles < avail ? tiles : avail;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  grid += p.ag_copiers;
  kernel<<<grid, 192, L::kTotalBytes, stream>>>(ma, mb, p);
  return (int)cudaGetLastError();
}

template <int BN, int STAGES>
static int dispatch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int a_mn, int b_mn,
                         int epi, int max_ctas, cudaStream_t stream) {
#define SB_CASE(AM, BM_, E)                                    \
  if (a_mn == AM && b_mn == BM_ && epi == E)                   \
    return launch_gemm<BN, STAGES, AM != 0, BM_ != 0, E>(ma, mb, p, max_ctas, stream);
  SB_CASE(0, 0, EPI_BF16)
  SB_CASE(0, 1, EPI_BF16)
  SB_CASE(1, 1, EPI_BF16)
  SB_CASE(1, 1, EPI_F32_ACC)
  SB_CASE(1, 1, EPI_F32)
  SB_CASE(0, 0, EPI_F32)
  SB_CASE(0, 1, EPI_F32)
  SB_CASE(0, 0, EPI_F32_AR)
  SB_CASE(0, 0, EPI_BF16_T)
  SB_CASE(0, 0, EPI_F32_T)
  SB_CASE(0, 0, EPI_LMSTAT)
  SB_CASE(0, 0, EPI_DLOGITS)
#undef SB_CASE
  return -2;
}

}  // namespace sb

namespace sb {
// out[m, n] = bf16(sum_s slabs[s, m, n] + bias[n]); one thread per 8 columns
__global__ void splitk_reduce_kernel(const float* __restrict__ slabs, long long slab_stride, int splits,
                                     const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                     long long ldo, int M, int N) {
  const int nvec = N / 8;
  const long long total = (long long)M * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(idx / nvec), v = (int)(idx % nvec);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < splits; ++s) {
      const float4* src = reinterpret_cast<const float4*>(slabs + s * slab_stride + (long long)m * N + v * 8);
      const float4 a = src[0], b = src[1];
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    if (bias) {
      const uint4 bv = *reinterpret_cast<const uint4*>(bias + v * 8);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(b2[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + (long long)m * ldo + v * 8) = o;
  }
}
}  // namespace sb

using namespace sb;

extern "C" int sb_splitk_reduce(const float* slabs, long long slab_stride, int splits, const void* bias, void* out,
                                long long ldo, int M, int N, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (N % 8 || ldo % 8) return -3;
  const long long total = (long long)M * (N / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)num_sms() * 8;
  if (blocks > cap) blocks = cap;
  splitk_reduce_kernel<<<(int)blocks, 256, 0, stream>>>(slabs, slab_stride, splits, (const __nv_bfloat16*)bias,
                                                       (__nv_bfloat16*)out, ldo, M, N);
  return (int)cudaGetLastError();
}

struct GroupArgs {
  const int* tile_group;   // per m-block group id (grouped along M), or nullptr
  long long b_group_rows;  // rows of B's outer dimension per group
  const int* group_rows;   // num_groups + 1 contraction-row offsets (grouped along K), or nullptr
  int num_groups;
  long long c_group_stride;
};

struct LmArgs {
  const long long* labels;
  float inv_temp;
  void* partial;
  const float *lse, *ent, *glogp, *gent;
};

static int gemm_impl(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                     long long ldb, long long ldc, int a_mn, int b_mn, int epi, int tile_n, int max_ctas,
                     int k_splits, long long slab_stride, const ArParams* ar, int* status, cudaStream_t stream,
                     const GroupArgs* grp = nullptr, const AgParams* ag = nullptr, int ag_copiers = 0,
                     const LmArgs* lm = nullptr) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // TMA needs 16-byte aligned bases and row pitches; the epilogue stores whole 16-byte groups of a row
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -3;
  if (epi == EPI_BF16_T || epi == EPI_F32_T || epi == EPI_LMSTAT) {
    // element-wise (transposed) stores or no matrix output at all
  } else if (epi == EPI_BF16 || epi == EPI_DLOGITS) {
    if (((uintptr_t)C & 15) || (ldc % 8) || (N % 8)) return -3;
  } else {
    if (((uintptr_t)C & 15) || (ldc % 4) || (N % 4)) return -3;
  }
  if ((epi == EPI_LMSTAT || epi == EPI_DLOGITS) && !lm) return -3;
  // The driver-API tensor-map encoder needs a current context on the calling thread; threads
  // that only ever launched through torch (autograd workers) may not have one bound yet.
  static thread_local bool tl_context_bound = false;
  if (!tl_context_bound) {
    cudaFree(0);
    tl_context_bound = true;
  }
  int BN = tile_n;
  if (BN != 128 && BN != 256) {
    // 256-wide tiles halve the A traffic per FLOP and measured 1.5x faster than 128-wide ones on
    // B200 for every large shape; the narrow tile only wins when it removes a mostly empty wave.
    const int sms = num_sms();
    const long long mbk = (M + kBM - 1) / kBM;
    auto waves_cost = [&](int bn, double per_tile) {
      long long tiles = mbk * ((N + bn - 1) / bn);
      long long waves = (tiles + sms - 1) / sms;
      return (double)waves * per_tile;
    };
    BN = (N > 128 && waves_cost(256, 1.0) <= waves_cost(128, 0.75)) ? 256 : 128;
  }
  CUtensorMap ma, mb;
  int r;
  if (!a_mn) r = make_tensor_map_bf16_2d(&ma, A, K, M, lda, kBK, kBM);
  else r = make_tensor_map_bf16_2d(&ma, A, M, K, lda, 64, kBK);
  if (r) return r;
  const bool by_m = grp && grp->tile_group;
  const long long b_groups = by_m ? grp->num_groups : 1;
  if (!b_mn) r = make_tensor_map_bf16_2d(&mb, B, K, by_m ? b_groups * grp->b_group_rows : N, ldb, kBK, BN);
  else r = make_tensor_map_bf16_2d(&mb, B, N, by_m ? b_groups * grp->b_group_rows : K, ldb, 64, kBK);
  if (r) return r;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.status = status;
  p.num_m_blocks = (M + kBM - 1) / kBM;
  p.num_n_blocks = (N + BN - 1) / BN;
  p.num_k_blocks = (K + kBK - 1) / kBK;
  if (k_splits < 1) k_splits = 1;
  if (k_splits > 1 && epi != EPI_F32 && epi != EPI_F32_AR && epi != EPI_F32_T) return -2;  // split-K writes fp32 slabs
  if (k_splits > p.num_k_blocks) k_splits = p.num_k_blocks;
  p.ar = ar;
  p.labels = nullptr; p.inv_temp = 1.f; p.lm_partial = nullptr;
  p.lm_lse = p.lm_ent = p.lm_glogp = p.lm_gent = nullptr;
  if (lm) {
    p.labels = lm->labels; p.inv_temp = lm->inv_temp; p.lm_partial = reinterpret_cast<float4*>(lm->partial);
    p.lm_lse = lm->lse; p.lm_ent = lm->ent; p.lm_glogp = lm->glogp; p.lm_gent = lm->gent;
  }
  p.ag = ag;
  p.ag_copiers = ag ? ag_copiers : 0;
  p.tile_group = nullptr;
  p.group_rows = nullptr;
  p.b_group_rows = 0;
  p.c_group_stride = 0;
  if (grp) {
    if (k_splits != 1 || epi == EPI_F32_AR) return -2;
    p.tile_group = grp->tile_group;
    p.b_group_rows = grp->b_group_rows;
    p.group_rows = grp->group_rows;
    p.c_group_stride = grp->c_group_stride;
    if (grp->group_rows) k_splits = grp->num_groups;  // one "split" per group; the kernel reads its row range
  }
  if (epi == EPI_F32_AR && k_splits > 1) {
    // the tile finisher waits for peers inside the kernel: with split-K every CTA must own exactly one tile, so
    // that no wait can sit in front of work another rank is waiting for
    const int per_tile = num_sms() / (p.num_m_blocks * p.num_n_blocks);
    if (per_tile < 2) return -5;
    if (k_splits > per_tile) k_splits = per_tile;
    max_ctas = 0;
  }
  p.kb_per_split = (p.num_k_blocks + k_splits - 1) / k_splits;
  p.k_splits = (p.num_k_blocks + p.kb_per_split - 1) / p.kb_per_split;
  if (grp && grp->group_rows) p.k_splits = grp->num_groups;
  p.slab_stride = slab_stride;
  // one 256 x 256 tile per CTA pair: worth it when the output has at least two 128-row blocks and the caller did
  // not pin the tile width or the grid (tensor-parallel all-reduce, all-gather and grouped modes keep the one-CTA kernel)
  const bool pair_ok = !grp && !ag && !ar && epi != EPI_F32_AR && M > 128 && N >= 128 && tile_n != 128 && max_ctas == 0;
  if (g_pair_enabled && pair_ok) {
    // CTA-pair kernel: its operand boxes are 128 rows wide whatever the one-CTA kernel would have chosen
    CUtensorMap pa, pb;
    if (!a_mn) r = make_tensor_map_bf16_2d(&pa, A, K, M, lda, kBK, 128);
    else r = make_tensor_map_bf16_2d(&pa, A, M, K, lda, 64, kBK);
    if (r) return r;
    if (!b_mn) r = make_tensor_map_bf16_2d(&pb, B, K, N, ldb, kBK, 128);
    else r = make_tensor_map_bf16_2d(&pb, B, N, K, ldb, 64, kBK);
    if (r) return r;
    const int rc = dispatch_pair(pa, pb, p, a_mn, b_mn, epi, stream);
    if (rc != -2) return rc;
  }
  if (BN == 256) return dispatch_gemm<256, 4>(ma, mb, p, a_mn, b_mn, epi, max_ctas, stream);
  return dispatch_gemm<128, 6>(ma, mb, p, a_mn, b_mn, epi, max_ctas, stream);
}

// 0 routes every GEMM through the one-CTA kernel (benchmarks compare the two; a fallback switch)
extern "C" int sb_gemm_set_pair_kernel(int enabled) {
  const int old = g_pair_enabled ? 1 : 0;
  g_pair_enabled = enabled != 0;
  return old;
}

extern "C" int sb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                            long long lda, long long ldb, long long ldc, int a_mn, int b_mn, int epi,
                            int tile_n, int max_ctas, int k_splits, long long slab_stride, int* status,
                            cudaStream_t stream) {
  if (epi == EPI_F32_AR) return -2;
  return gemm_impl(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, epi, tile_n, max_ctas, k_splits, slab_stride,
                   nullptr, status, stream);
}

// Vocabulary GEMM fused with the softmax statistics: logits[M, N] = A[M, K] * B[N, K]^T are reduced tile by tile in
// the epilogue, `partial` receives [M, ceil(N / 256)] float4 (max, sum exp, sum exp * z, z[label]) of z = logits *
// inv_temp; sb_lmhead_merge (lm_head.cu) folds them into log p(label), entropy and log-sum-exp per row.
extern "C" int sb_gemm_lmstat_bf16(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                                   const long long* labels, float inv_temp, void* partial, int* status,
                                   cudaStream_t stream) {
  LmArgs lm{labels, inv_temp, partial, nullptr, nullptr, nullptr, nullptr};
  return gemm_impl(A, B, partial, nullptr, M, N, K, lda, ldb, 0, 0, 0, EPI_LMSTAT, 256, 0, 1, 0, nullptr, status, stream,
                   nullptr, nullptr, 0, &lm);
}

// The same GEMM recomputed for backward: the epilogue writes bf16 d_logits[M, ldd] from the per-row log-sum-exp,
// entropy (optional), d loss / d logp and d loss / d entropy (optional).
extern "C" int sb_gemm_dlogits_bf16(const void* A, const void* B, void* dlogits, int M, int N, int K, long long lda,
                                    long long ldb, long long ldd, const long long* labels, float inv_temp,
                                    const float* lse, const float* ent, const float* g_logp, const float* g_ent,
                                    int* status, cudaStream_t stream) {
  LmArgs lm{labels, inv_temp, nullptr, lse, ent, g_logp, g_ent};
  return gemm_impl(A, B, dlogits, nullptr, M, N, K, lda, ldb, ldd, 0, 0, EPI_DLOGITS, 256, 0, 1, 0, nullptr, status, stream,
                   nullptr, nullptr, 0, &lm);
}

// Grouped GEMM for mixture-of-experts layers, one launch for all experts.
//  tile_group != null (forward / dgrad): rows of A are sorted by expert and padded so that every 128-row block
//    belongs to one expert; tile_group[mb] names it (-1: block unused).  B stacks the experts' matrices along its
//    outer dimension (b_group_rows rows each): [E*N, K] for K-major B, [E*Kc, N] for MN-major B.
//  group_rows != null (wgrad): C_g[M, N] (+)= sum over rows [group_rows[g], group_rows[g+1]) of A^T B with A
//    [rows, M] and B [rows, N] MN-major; C advances c_group_stride elements per group.
extern "C" int sb_gemm_grouped_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                    long long ldb, long long ldc, int a_mn, int b_mn, int epi, int tile_n,
                                    const int* tile_group, long long b_group_rows, const int* group_rows,
                                    int num_groups, long long c_group_stride, int* status, cudaStream_t stream) {
  GroupArgs g{tile_group, b_group_rows, group_rows, num_groups, c_group_stride};
  if ((!tile_group) == (!group_rows) || num_groups < 1) return -3;
  return gemm_impl(A, B, C, nullptr, M, N, K, lda, ldb, ldc, a_mn, b_mn, epi, tile_n, 0, 1, 0, nullptr, status, stream,
                   &g);
}

// C[M, N] = A[M, K] * B[N, K]^T (+ bias) where B is sharded by rows over the ranks: the launch gathers B into
// `staging` (local [N, K], row pitch ld) while it multiplies.  `ag_params` is an AgParams struct in device memory.
// a_mn/b_mn = 0 (forward layout); with b_mn = 1 the staging matrix is read as [N (contraction), K] (dgrad layout:
// C[M, K] = A[M, N] * B[N, K], chunks along the contraction) -- not offered: the forward layout is the only user.
extern "C" int sb_ag_gemm_bf16(const void* A, const void* staging, void* C, const void* bias, int M, int N, int K,
                               long long lda, long long ld, long long ldc, const void* ag_params, int copiers,
                               int tile_n, int* status, cudaStream_t stream) {
  if (copiers < 1 || copiers > 64 || (K % 8)) return -3;
  return gemm_impl(A, staging, C, bias, M, N, K, lda, ld, ldc, 0, 0, EPI_BF16, tile_n == 256 ? 256 : 128, 0, 1, 0,
                   nullptr, status, stream, nullptr, reinterpret_cast<const AgParams*>(ag_params), copiers);
}

// out[q] = bf16(sum_r A_r[M, K_r] * B_r[N, K_r]^T + bias) on every rank q of the tensor-parallel group, one launch
// per rank.  `ar_params` is an ArParams struct in device memory (same buffers on every call of a group);
// `c_local` receives this rank's fp32 partial: the rank's own `partial` buffer when k_splits == 1, else a local
// slab buffer of k_splits * slab_stride floats.  N must be a multiple of 8.
extern "C" int sb_gemm_ar_bf16(const void* A, const void* B, const void* bias, int M, int N, int K, long long lda,
                               long long ldb, const void* ar_params, void* c_local, int tile_n, int k_splits,
                               long long slab_stride, int max_tiles, int* status, cudaStream_t stream) {
  if (N % 8) return -3;
  int BN = (tile_n == 256) ? 256 : 128;
  const int tiles_mn = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
  if (tiles_mn > max_tiles) return -4;  // flag arrays too small
  return gemm_impl(A, B, c_local, bias, M, N, K, lda, ldb, (long long)N, 0, 0, EPI_F32_AR, BN, 0, k_splits, slab_stride,
                   reinterpret_cast<const ArParams*>(ar_params), status, stream);
}
