// Persistent, warp-specialised decode attention with split K/V (flash-decoding) for the rollout engine.
//
// The simple kernel in fmha_decode.cu runs one CTA per (sequence, kv head) and walks the serial chain
// wait(K) -> S MMA -> softmax -> P -> PV MMA -> issue the next load; it is bound by that chain's latency (about one
// 32 KB stage in flight per CTA) and by the tail wave of a grid that is not a multiple of the resident slots.  Here:
//   * one CTA per SM walks a list of work items (chunk, sequence, kv head); a sequence is cut into chunks of
//     kChunkTiles cache blocks, so items are of similar size whatever the batch and the context lengths;
//   * four working warps: warp 0 soft-max, warp 1 TMA producer, warp 2 MMA issuer, warp 4 output (warp 3 only makes
//     warp 4 exist: rows 0..31 of TMEM belong to the warps whose index is a multiple of four).  The producer keeps a
//     ring of K/V stages full across item boundaries (128 KB in flight per SM at d = 128) and fetches the NEXT item's
//     query rows while the current item runs; S is double-buffered in TMEM so the scores of tile t+1 are computed while
//     tile t is in the soft-max, P is double-buffered in shared memory, and the output accumulator is double-buffered
//     in TMEM so that an item's normalisation and store overlap the next item's tiles: an item boundary costs no
//     pipeline drain;
//   * the running maximum is only raised when it grows by more than 2^8 (the accumulator is rescaled rarely);
//   * chunks of one sequence leave (normalised partial output, log-sum-exp) in a workspace and a small kernel merges
//     them; a sequence that fits one chunk is written directly.
// The `rep` = Hq / Hkv (<= 32) query heads sharing a kv head are rows 0..rep-1 of the 128-row MMA tile; the other
// rows are never read.  The reference reaches paged decode attention through vLLM
// (siirl/engine/rollout/vllm_rollout/vllm_rollout_spmd.py:261-416).
#include "common.cuh"
#include "launchers.h"

namespace sb {

constexpr int kSBlk = 64;          // tokens per cache block = kv tile
constexpr int kChunkTiles = 16;    // cache blocks per work item (1024 tokens)

struct SplitParams {
  const int* seq_lens;     // [B] context length including the current token
  const int* block_table;  // [B, max_blocks]
  int max_blocks;
  int max_chunks;          // ceil(max_blocks / kChunkTiles)
  __nv_bfloat16* out;      // [B, Hq*D]
  float* ws_o;             // [B, Hq, max_chunks, D] normalised partial outputs
  float* ws_lse;           // [B, Hq, max_chunks] log2-sum-exp of the chunk (scaled scores)
  int B, Hq, Hkv;
  int q_rows_per_seq;      // rows of width D per sequence in the q tensor map (row_stride / D)
  float scale_log2;
  int* status;
};

template <int D>
struct SplitSmem {
  static constexpr int kStages = (D == 128) ? 4 : 8;
  static constexpr int kQBytes = 128 * D * 2;          // one query tile; there are two
  static constexpr int kKBytes = kSBlk * D * 2;        // one K (or V) tile
  static constexpr int kPBytes = 128 * kSBlk * 2;
  static constexpr int kQOff = 0;
  static constexpr int kPOff = kQOff + 2 * kQBytes;
  static constexpr int kKVOff = kPOff + 2 * kPBytes;   // stage s: K at kKVOff + s * 2 * kKBytes, V right after
  static constexpr int kBarOff = kKVOff + kStages * 2 * kKBytes;
  // kv_full[S], kv_empty[S], then pairs: q_full, q_empty, s_full, s_empty, p_full, p_empty, o_full, o_empty,
  // stat_full, stat_empty
  static constexpr int kNumBars = 2 * kStages + 20;
  static constexpr int kStatOff = kBarOff + kNumBars * 8 + 16;   // [2][32] reference maxima, [2][32] row sums
  static constexpr int kTotal = kStatOff + 4 * 32 * 4;
};

// work item `idx` -> (chunk, sequence, kv head); chunk-major so that the valid items of equal-length sequences form a
// prefix of the list and the round-robin over CTAs stays balanced
__device__ __forceinline__ void split_item(int idx, int B, int Hkv, int& c, int& b, int& g) {
  const int per = B * Hkv;
  c = idx / per;
  const int r = idx - c * per;
  b = r / Hkv;
  g = r - b * Hkv;
}

template <int D>
__global__ void __launch_bounds__(160, 1)
fmha_decode_split_kernel(const __grid_constant__ CUtensorMap map_cache, const __grid_constant__ CUtensorMap map_q,
                         SplitParams p) {
  using L = SplitSmem<D>;
  constexpr int NS = L::kStages;
  constexpr int kDChunks = D / 64;
  constexpr uint32_t kTmemCols = 512;   // S: 2 x 64 columns, O: 2 x 128 columns
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, (int)kStatusBadArgument);
    return;
  }
  uint8_t* sQ = smem + L::kQOff;
  uint8_t* sP = smem + L::kPOff;
  uint8_t* sKV = smem + L::kKVOff;
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_empty = kv_full + NS;
  uint64_t* q_full = kv_empty + NS;
  uint64_t* q_empty = q_full + 2;
  uint64_t* s_full = q_empty + 2;
  uint64_t* s_empty = s_full + 2;
  uint64_t* p_full = s_empty + 2;
  uint64_t* p_empty = p_full + 2;
  uint64_t* o_full = p_empty + 2;
  uint64_t* o_empty = o_full + 2;
  uint64_t* stat_full = o_empty + 2;
  uint64_t* stat_empty = stat_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stat_empty + 2);
  float* s_mref = reinterpret_cast<float*>(smem + L::kStatOff);      // [2][32]
  float* s_lrun = s_mref + 64;                                       // [2][32]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rep = p.Hq / p.Hkv;
  const int q_box_rows = (rep + 7) & ~7;
  const int total_items = p.max_chunks * p.B * p.Hkv;

  if (tid == 0) {
    tma_prefetch_desc(&map_cache);
    tma_prefetch_desc(&map_q);
    for (int i = 0; i < L::kNumBars; ++i) mbar_init(&kv_full[i], 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  // rows the MMAs read but nobody writes start as zeros (Q rows >= the TMA box, P rows >= 32)
  for (int i = tid; i < (2 * L::kQBytes + 2 * L::kPBytes) / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;      // output accumulator b at tmem_o + b * 128

  // (chunk, sequence, kv head, first tile, tile count) of the first valid work item at or after `idx`; false at the end
  auto find_item = [&](int& idx, int& c, int& b, int& g, int& t0, int& n, int& seq_tiles) -> bool {
    for (; idx < total_items; idx += gridDim.x) {
      split_item(idx, p.B, p.Hkv, c, b, g);
      const int ctx = p.seq_lens[b];
      seq_tiles = (ctx + kSBlk - 1) / kSBlk;
      t0 = c * kChunkTiles;
      const int t1 = min(seq_tiles, t0 + kChunkTiles);
      if (t1 > t0) {
        n = t1 - t0;
        return true;
      }
    }
    return false;
  };

  if (warp == 1) {
    // ------------------------------ producer: K/V ring and query rows ------------------------------
    if (lane == 0) {
      uint32_t tile_no = 0, item_no = 0;   // tiles / items issued so far by this CTA (ring position and phases)
      bool ok = true;
      auto load_q = [&](uint32_t item, int b, int g) -> bool {
        const int qb = item & 1;
        if (!mbar_wait(&q_empty[qb], ((item >> 1) & 1) ^ 1, p.status, kStatusTimeoutProducer)) return false;
        mbar_arrive_expect_tx(&q_full[qb], (uint32_t)(kDChunks * q_box_rows * 128));
#pragma unroll
        for (int cc = 0; cc < kDChunks; ++cc)
          tma_load_2d(sQ + qb * L::kQBytes + cc * 16384, &map_q, &q_full[qb], cc * 64,
                      b * p.q_rows_per_seq + g * rep);
        return true;
      };
      int idx = blockIdx.x, c, b, g, t0, n, st;
      bool have = find_item(idx, c, b, g, t0, n, st);
      if (have) ok = load_q(0, b, g);
      while (have && ok) {
        // the item after this one (its query rows are fetched a few tiles into the current item, when the score
        // MMAs of the item before have long completed and their query buffer is free)
        int idx2 = idx + gridDim.x, c2, b2, g2, t02, n2, st2;
        const bool have2 = find_item(idx2, c2, b2, g2, t02, n2, st2);
        const int q_at = min(n - 1, 3);
        const int* blocks = p.block_table + (size_t)b * p.max_blocks;
        for (int t = 0; t < n && ok; ++t, ++tile_no) {
          const int stage = tile_no % NS;
          const uint32_t round = tile_no / NS;
          if (!mbar_wait(&kv_empty[stage], (round & 1) ^ 1, p.status, kStatusTimeoutProducer)) {
            ok = false;
            break;
          }
          const int blk = blocks[t0 + t];
          uint8_t* sk = sKV + stage * 2 * L::kKBytes;
          uint8_t* sv = sk + L::kKBytes;
          mbar_arrive_expect_tx(&kv_full[stage], 2 * L::kKBytes);
          const int krow = ((blk * 2 + 0) * p.Hkv + g) * kSBlk;
          const int vrow = ((blk * 2 + 1) * p.Hkv + g) * kSBlk;
#pragma unroll
          for (int cc = 0; cc < kDChunks; ++cc) {
            tma_load_2d(sk + cc * 8192, &map_cache, &kv_full[stage], cc * 64, krow);
            tma_load_2d(sv + cc * 8192, &map_cache, &kv_full[stage], cc * 64, vrow);
          }
          if (t == q_at && have2) ok = load_q(item_no + 1, b2, g2);
        }
        ++item_no;
        idx = idx2; c = c2; b = b2; g = g2; t0 = t02; n = n2; st = st2;
        have = have2;
      }
    }
  } else if (warp == 2) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, kSBlk, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, D, 0, 1);
      uint32_t tile_no = 0, item_no = 0;
      bool ok = true;
      int idx = blockIdx.x, c, b, g, t0, n, st;
      for (; ok && find_item(idx, c, b, g, t0, n, st); idx += gridDim.x) {
        const int ib = item_no & 1;                   // query buffer and output accumulator of this item
        const uint32_t aq = smem_u32(sQ + ib * L::kQBytes);
        const uint32_t tmem_oi = tmem_o + ib * 128;
        if (!mbar_wait(&q_full[ib], (item_no >> 1) & 1, p.status, kStatusTimeoutMma)) break;
        tc_fence_after();
        const uint32_t first_tile = tile_no;
        for (int t = 0; t <= n && ok; ++t) {
          if (t < n) {
            // S(t) = Q K(t)^T into S buffer (tile_no & 1)
            const uint32_t tn = first_tile + t;
            const int stage = tn % NS;
            const int sb_ = tn & 1;
            if (!mbar_wait(&kv_full[stage], (tn / NS) & 1, p.status, kStatusTimeoutMma) ||
                !mbar_wait(&s_empty[sb_], ((tn >> 1) & 1) ^ 1, p.status, kStatusTimeoutMma)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t bk = smem_u32(sKV + stage * 2 * L::kKBytes);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint64_t da = umma_smem_desc(aq + (kk / 4) * 16384 + (kk % 4) * 32, 16, 1024);
              const uint64_t db = umma_smem_desc(bk + (kk / 4) * 8192 + (kk % 4) * 32, 16, 1024);
              umma_bf16_ss(tmem_s + sb_ * 64, da, db, idesc_s, kk ? 1u : 0u);
            }
            umma_commit(&s_full[sb_]);
            if (t == n - 1) umma_commit(&q_empty[ib]);
          }
          if (t > 0) {
            // O += P(t-1) V(t-1)
            const uint32_t tn = first_tile + t - 1;
            const int stage = tn % NS;
            const int pb = tn & 1;
            // (first PV of the item: the output warp has read this accumulator's previous item)
            if (!mbar_wait(&p_full[pb], (tn >> 1) & 1, p.status, kStatusTimeoutMma) ||
                (t == 1 && !mbar_wait(&o_empty[ib], ((item_no >> 1) & 1) ^ 1, p.status, kStatusTimeoutMma))) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t ap = smem_u32(sP + pb * L::kPBytes);
            const uint32_t bv = smem_u32(sKV + stage * 2 * L::kKBytes + L::kKBytes);
#pragma unroll
            for (int kk = 0; kk < kSBlk / 16; ++kk) {
              const uint64_t da = umma_smem_desc(ap + kk * 32, 16, 1024);
              const uint64_t db = umma_smem_desc(bv + kk * 2048, 8192, 1024);
              umma_bf16_ss(tmem_oi, da, db, idesc_o, (t > 1 || kk) ? 1u : 0u);
            }
            umma_commit(&kv_empty[stage]);
            umma_commit(&p_empty[pb]);
            if (t == n) umma_commit(&o_full[ib]);
          }
        }
        tile_no += n;
        ++item_no;
      }
    }
  } else if (warp == 0) {
    // ------------------------------ soft-max (warp 0: TMEM lanes 0..31) ------------------------------
    uint32_t tile_no = 0, item_no = 0;
    bool ok = true;
    const bool row_valid = lane < rep;
    int idx = blockIdx.x, c, b, g, t0, n, n_seq_tiles;
    for (; ok && find_item(idx, c, b, g, t0, n, n_seq_tiles); idx += gridDim.x) {
      const int ctx = p.seq_lens[b];
      const uint32_t tmem_oi = tmem_o + (item_no & 1) * 128;
      float m_ref = -INFINITY, l_run = 0.f;
      if (rep <= 8) {
        // Narrow groups (at most 8 query heads per kv head): the scores are read in the accumulator-fragment layout,
        // where the 4 threads 4r .. 4r+3 share row r and hold 16 of its 64 columns each, so the exponentials of a
        // tile are spread over the whole warp instead of sitting in `rep` lanes.  m_ref is kept per row (equal in
        // the 4 threads), l_run is a per-thread partial sum that is reduced at the end of the item.
        const int frow = lane >> 2, fq = lane & 3;
        const bool fvalid = frow < rep;
        for (int t = 0; t < n; ++t) {
          const uint32_t tn = tile_no + t;
          const int sb_ = tn & 1;
          if (!__all_sync(0xffffffffu, mbar_wait(&s_full[sb_], (tn >> 1) & 1, p.status, kStatusTimeoutEpilogue))) {
            ok = false;
            break;
          }
          tc_fence_after();
          float sv[16];
          {
            uint32_t r[32];
            tmem_ld_16x256_x8(tmem_s + sb_ * 64, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              sv[2 * i] = __uint_as_float(r[4 * i]) * p.scale_log2;
              sv[2 * i + 1] = __uint_as_float(r[4 * i + 1]) * p.scale_log2;
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_empty[sb_]);
          const int kv0 = (t0 + t) * kSBlk;
          if (kv0 + kSBlk > ctx) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int col = kv0 + 8 * i + 2 * fq;
              if (col >= ctx) sv[2 * i] = -INFINITY;
              if (col + 1 >= ctx) sv[2 * i + 1] = -INFINITY;
            }
          }
          float m_tile = -INFINITY;
#pragma unroll
          for (int i = 0; i < 16; ++i) m_tile = fmaxf(m_tile, sv[i]);
          m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
          m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 2));
          if (t == 0) {
            m_ref = (m_tile == -INFINITY) ? 0.f : m_tile;
          } else if (__any_sync(0xffffffffu, fvalid && m_tile > m_ref + 8.f)) {
            const uint32_t tp = tn - 1;
            if (!__all_sync(0xffffffffu, mbar_wait(&p_empty[tp & 1], (tp >> 1) & 1, p.status, kStatusTimeoutEpilogue))) {
              ok = false;
              break;
            }
            tc_fence_after();
            const float m_new = fmaxf(m_ref, m_tile);
            const float alpha_f = exp2f(m_ref - m_new);
            l_run *= alpha_f;
            m_ref = m_new;
            // the accumulator is addressed one row per lane: lane r takes the factor of row r from thread 4r
            float alpha = __shfl_sync(0xffffffffu, alpha_f, (lane * 4) & 31);
            if (lane >= 8) alpha = 1.f;
#pragma unroll 1
            for (int cc = 0; cc < D / 32; ++cc) {
              uint32_t r[32];
              tmem_ld_32x32(tmem_oi + cc * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x32(tmem_oi + cc * 32, r);
            }
            tmem_st_wait();
            tc_fence_before();
          }
          uint32_t pk[8];
          float rsum = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float p0 = exp2f(sv[2 * i] - m_ref), p1 = exp2f(sv[2 * i + 1] - m_ref);
            rsum += p0 + p1;
            pk[i] = fvalid ? pack_bf16x2(p0, p1) : 0u;
          }
          l_run += rsum;
          if (!__all_sync(0xffffffffu, mbar_wait(&p_empty[sb_], ((tn >> 1) & 1) ^ 1, p.status, kStatusTimeoutEpilogue))) {
            ok = false;
            break;
          }
          {
            uint8_t* prow = sP + sb_ * L::kPBytes + frow * 128 + fq * 4;
#pragma unroll
            for (int i = 0; i < 8; ++i) *reinterpret_cast<uint32_t*>(prow + ((i ^ frow) << 4)) = pk[i];
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_full[sb_]);
        }
        // row totals, then hand row r's statistics to lane r (the output below is addressed one row per lane)
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
        l_run = __shfl_sync(0xffffffffu, l_run, (lane * 4) & 31);
        m_ref = __shfl_sync(0xffffffffu, m_ref, (lane * 4) & 31);
      } else {
        for (int t = 0; t < n; ++t) {
          const uint32_t tn = tile_no + t;
          const int sb_ = tn & 1;
          if (!__all_sync(0xffffffffu, mbar_wait(&s_full[sb_], (tn >> 1) & 1, p.status, kStatusTimeoutEpilogue))) {
            ok = false;
            break;
          }
          tc_fence_after();
          float sv[kSBlk];
          {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(tmem_s + sb_ * 64, r0);
            tmem_ld_32x32(tmem_s + sb_ * 64 + 32, r1);
            tmem_ld_wait();
  #pragma unroll
            for (int i = 0; i < 32; ++i) {
              sv[i] = __uint_as_float(r0[i]) * p.scale_log2;
              sv[32 + i] = __uint_as_float(r1[i]) * p.scale_log2;
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_empty[sb_]);   // the MMA warp may overwrite this S buffer
          const int kv0 = (t0 + t) * kSBlk;
          if (kv0 + kSBlk > ctx) {
  #pragma unroll
            for (int i = 0; i < kSBlk; ++i)
              if (kv0 + i >= ctx) sv[i] = -INFINITY;
          }
          float m_tile = -INFINITY;
  #pragma unroll
          for (int i = 0; i < kSBlk; ++i) m_tile = fmaxf(m_tile, sv[i]);
          if (t == 0) {
            m_ref = (m_tile == -INFINITY) ? 0.f : m_tile;
          } else if (__any_sync(0xffffffffu, row_valid && m_tile > m_ref + 8.f)) {
            // rare: raise the reference maximum and rescale the accumulator; PV(t-1) must have finished
            const uint32_t tp = tn - 1;
            if (!__all_sync(0xffffffffu, mbar_wait(&p_empty[tp & 1], (tp >> 1) & 1, p.status, kStatusTimeoutEpilogue))) {
              ok = false;
              break;
            }
            tc_fence_after();
            const float m_new = fmaxf(m_ref, m_tile);
            const float alpha = exp2f(m_ref - m_new);
            l_run *= alpha;
            m_ref = m_new;
  #pragma unroll 1
            for (int cc = 0; cc < D / 32; ++cc) {
              uint32_t r[32];
              tmem_ld_32x32(tmem_oi + cc * 32, r);
              tmem_ld_wait();
  #pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x32(tmem_oi + cc * 32, r);
            }
            tmem_st_wait();
            tc_fence_before();
          }
          float rsum = 0.f;
          uint32_t pk[kSBlk / 2];
  #pragma unroll
          for (int i = 0; i < kSBlk; i += 2) {
            const float p0 = exp2f(sv[i] - m_ref), p1 = exp2f(sv[i + 1] - m_ref);
            rsum += p0 + p1;
            pk[i / 2] = pack_bf16x2(p0, p1);
          }
          l_run += rsum;
          // P buffer (tn & 1) was read by PV(tn - 2)
          if (!__all_sync(0xffffffffu, mbar_wait(&p_empty[sb_], ((tn >> 1) & 1) ^ 1, p.status, kStatusTimeoutEpilogue))) {
            ok = false;
            break;
          }
          {
            uint8_t* prow = sP + sb_ * L::kPBytes + lane * 128;
  #pragma unroll
            for (int piece = 0; piece < 8; ++piece) {
              uint4 v = make_uint4(pk[piece * 4], pk[piece * 4 + 1], pk[piece * 4 + 2], pk[piece * 4 + 3]);
              if (!row_valid) v = make_uint4(0, 0, 0, 0);
              *reinterpret_cast<uint4*>(prow + ((piece ^ (lane & 7)) << 4)) = v;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_full[sb_]);
        }
      }
      if (!ok) break;
      tile_no += n;
      // hand the row statistics to the output warp (lane r holds row r's values in both paths) and go on with the
      // next item: normalisation and store of this item's accumulator overlap its tiles
      {
        const int ib = item_no & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&stat_empty[ib], ((item_no >> 1) & 1) ^ 1, p.status,
                                               kStatusTimeoutEpilogue))) {
          ok = false;
          break;
        }
        s_mref[ib * 32 + lane] = m_ref;
        s_lrun[ib * 32 + lane] = l_run;
        __syncwarp();
        if (lane == 0) mbar_arrive(&stat_full[ib]);
      }
      ++item_no;
    }
  } else if (warp == 4) {
    // ------------------------------ output (warp 4: TMEM lanes 0..31) ------------------------------
    uint32_t item_no = 0;
    bool ok = true;
    const bool row_valid = lane < rep;
    int idx = blockIdx.x, c, b, g, t0, n, n_seq_tiles;
    for (; ok && find_item(idx, c, b, g, t0, n, n_seq_tiles); idx += gridDim.x) {
      const int ib = item_no & 1;
      const uint32_t par = (item_no >> 1) & 1;
      const uint32_t tmem_oi = tmem_o + ib * 128;
      // the item's statistics are in shared memory and all its PV MMAs have completed
      if (!__all_sync(0xffffffffu, mbar_wait(&stat_full[ib], par, p.status, kStatusTimeoutEpilogue)) ||
          !__all_sync(0xffffffffu, mbar_wait(&o_full[ib], par, p.status, kStatusTimeoutEpilogue))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const float m_ref = s_mref[ib * 32 + lane], l_run = s_lrun[ib * 32 + lane];
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      const int head = g * rep + (row_valid ? lane : 0);
      const bool single = n_seq_tiles <= kChunkTiles;
      __nv_bfloat16* orow = p.out + (size_t)b * (p.Hq * D) + (size_t)head * D;
      float* wrow = p.ws_o + (((size_t)b * p.Hq + head) * p.max_chunks + c) * D;
#pragma unroll 1
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_oi + cc * 32, r);
        tmem_ld_wait();
        if (row_valid) {
          if (single) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * inv_l, __uint_as_float(r[q * 8 + 1]) * inv_l);
              o.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * inv_l, __uint_as_float(r[q * 8 + 3]) * inv_l);
              o.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * inv_l, __uint_as_float(r[q * 8 + 5]) * inv_l);
              o.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * inv_l, __uint_as_float(r[q * 8 + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + cc * 32 + q * 8) = o;
            }
          } else {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 o = make_float4(__uint_as_float(r[q * 4 + 0]) * inv_l, __uint_as_float(r[q * 4 + 1]) * inv_l,
                                     __uint_as_float(r[q * 4 + 2]) * inv_l, __uint_as_float(r[q * 4 + 3]) * inv_l);
              *reinterpret_cast<float4*>(wrow + cc * 32 + q * 4) = o;
            }
          }
        }
      }
      if (row_valid && !single)
        p.ws_lse[((size_t)b * p.Hq + head) * p.max_chunks + c] = l_run > 0.f ? m_ref + log2f(l_run) : -INFINITY;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&o_empty[ib]);
        mbar_arrive(&stat_empty[ib]);
      }
      ++item_no;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// merges the chunk partials of sequences longer than one chunk; zero rows for empty slots
template <int D>
__global__ void fmha_decode_merge_kernel(SplitParams p) {
  const int b = blockIdx.x, h = blockIdx.y;
  const int ctx = p.seq_lens[b];
  const int n_tiles = (ctx + kSBlk - 1) / kSBlk;
  __nv_bfloat16* orow = p.out + (size_t)b * (p.Hq * D) + (size_t)h * D;
  const int d = threadIdx.x;   // blockDim.x == D
  if (ctx <= 0) {
    orow[d] = __float2bfloat16(0.f);
    return;
  }
  if (n_tiles <= kChunkTiles) return;   // written by the attention kernel
  const int nc = (n_tiles + kChunkTiles - 1) / kChunkTiles;
  const float* lse = p.ws_lse + ((size_t)b * p.Hq + h) * p.max_chunks;
  const float* wo = p.ws_o + ((size_t)b * p.Hq + h) * p.max_chunks * D;
  float m = -INFINITY;
  for (int c = 0; c < nc; ++c) m = fmaxf(m, lse[c]);
  float acc = 0.f, wsum = 0.f;
  for (int c = 0; c < nc; ++c) {
    const float w = exp2f(lse[c] - m);
    wsum += w;
    acc += w * wo[(size_t)c * D + d];
  }
  orow[d] = __float2bfloat16(wsum > 0.f ? acc / wsum : 0.f);
}

template <int D>
static int launch_decode_split(const CUtensorMap& mc, const CUtensorMap& mq, const SplitParams& p, cudaStream_t stream) {
  using L = SplitSmem<D>;
  auto kernel = fmha_decode_split_kernel<D>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int items = p.max_chunks * p.B * p.Hkv;
  const int grid = items < num_sms() ? items : num_sms();
  kernel<<<grid, 160, L::kTotal, stream>>>(mc, mq, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  fmha_decode_merge_kernel<D><<<dim3(p.B, p.Hq), D, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace sb

using namespace sb;

// workspace sizes in floats for `sb_fmha_decode_split`: ws_o = B * Hq * max_chunks * D, ws_lse = B * Hq * max_chunks
// with max_chunks = ceil(max_blocks / 16).
extern "C" int sb_fmha_decode_chunk_tiles() { return kChunkTiles; }

// Same contract as sb_fmha_decode plus the workspace.  q rows must be `row_stride` elements apart with
// row_stride % D == 0; Hq / Hkv <= 32.
extern "C" int sb_fmha_decode_split(const void* q, int row_stride, const void* cache, long long num_blocks,
                                    const int* seq_lens, const int* block_table, int max_blocks, void* out,
                                    float* ws_o, float* ws_lse, int B, int Hq, int Hkv, int D, float scale,
                                    int* status, cudaStream_t stream) {
  if (B == 0) return 0;
  if (D != 64 && D != 128) return -2;
  if (Hq % Hkv || Hq / Hkv > 32 || row_stride % D) return -3;
  static thread_local bool tl_context_bound = false;
  if (!tl_context_bound) {
    cudaFree(0);
    tl_context_bound = true;
  }
  const int rep = Hq / Hkv;
  CUtensorMap mc, mq;
  int r = make_tensor_map_bf16_2d(&mc, cache, D, num_blocks * 2 * Hkv * kSBlk, D, 64, kSBlk);
  if (r) return r;
  r = make_tensor_map_bf16_2d(&mq, q, D, (long long)B * (row_stride / D), D, 64, (rep + 7) & ~7);
  if (r) return r;
  SplitParams p;
  p.seq_lens = seq_lens; p.block_table = block_table; p.max_blocks = max_blocks;
  p.max_chunks = (max_blocks + kChunkTiles - 1) / kChunkTiles;
  p.out = (__nv_bfloat16*)out; p.ws_o = ws_o; p.ws_lse = ws_lse;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.q_rows_per_seq = row_stride / D;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  return D == 128 ? launch_decode_split<128>(mc, mq, p, stream) : launch_decode_split<64>(mc, mq, p, stream);
}
