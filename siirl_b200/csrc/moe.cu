// Mixture-of-experts token movement, local or expert-parallel over peer memory (NVLink 5 / NVSwitch).
//
// The reference reaches MoE through Megatron-core's token dispatcher (NCCL all-to-all, then a permutation kernel, then
// grouped GEMM; siirl/models/mcore/config_converter.py, qwen3moe branch).  Here the all-to-all IS the permutation
// kernel: rows are read straight from the peer that holds them (plain peer loads) and land in the expert-sorted,
// 128-row-padded layout the grouped tcgen05 GEMM consumes; the way back sums a token's top-k expert outputs while it
// pulls them.  With one rank the peer table has a single entry and the same kernels do the local permutation.
//
//   moe_gather_rows   out[slot] = scale[slot] * src[src_rank[slot]][src_row[slot]]   (zero row when src_row < 0)
//                     dispatch (forward), and the backward of combine (scale = routing weight)
//   moe_combine       out[t] = sum_k w[t,k] * y[pair_rank[t,k]][pair_slot[t,k]]
//                     combine (forward), and the backward of dispatch (w = 1)
//   moe_pair_dot      dots[t,k] = <dout[t], y[pair_rank[t,k]][pair_slot[t,k]]>         (gradient of the routing weights)
//
// One warp per row, 16-byte accesses; H must be a multiple of 8.  No kernel here waits on another GPU: the caller
// orders producers and consumers with the communicator's barrier.
#include "common.cuh"
#include "launchers.h"

namespace sb {

constexpr int kMoeMaxRanks = 16;
struct MoePeers {
  const __nv_bfloat16* p[kMoeMaxRanks];
};

__global__ void moe_gather_rows_kernel(MoePeers src, const int* __restrict__ src_rank, const int* __restrict__ src_row,
                                       const float* __restrict__ scale, __nv_bfloat16* __restrict__ out, int M, int H) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = H / 8;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < M; row += gridDim.x * warps_per_block) {
    const int sr = src_row[row];
    uint4* dst = reinterpret_cast<uint4*>(out + (long long)row * H);
    if (sr < 0) {
      for (int v = lane; v < nvec; v += 32) dst[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const uint4* s = reinterpret_cast<const uint4*>(src.p[src_rank ? src_rank[row] : 0] + (long long)sr * H);
    if (!scale) {
      for (int v = lane; v < nvec; v += 32) dst[v] = s[v];
    } else {
      const float a = scale[row];
      for (int v = lane; v < nvec; v += 32) {
        uint4 x = s[v];
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(h2[i]);
          h2[i] = __floats2bfloat162_rn(f.x * a, f.y * a);
        }
        dst[v] = x;
      }
    }
  }
}

__global__ void moe_combine_kernel(MoePeers y, const int* __restrict__ pair_rank, const int* __restrict__ pair_slot,
                                   const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int T, int k, int H) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = H / 8;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < T; t += gridDim.x * warps_per_block) {
    uint4* dst = reinterpret_cast<uint4*>(out + (long long)t * H);
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
        const int slot = pair_slot[t * k + j];
        if (slot < 0) continue;
        const float a = w ? w[t * k + j] : 1.f;
        const uint4 x = reinterpret_cast<const uint4*>(y.p[pair_rank ? pair_rank[t * k + j] : 0] + (long long)slot * H)[v];
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h2[i]);
          acc[2 * i] += a * f.x;
          acc[2 * i + 1] += a * f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      dst[v] = o;
    }
  }
}

__global__ void moe_pair_dot_kernel(MoePeers y, const int* __restrict__ pair_rank, const int* __restrict__ pair_slot,
                                    const __nv_bfloat16* __restrict__ dout, float* __restrict__ dots, int T, int k,
                                    int H) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = H / 8;
  const int P = T * k;
  for (int pr = blockIdx.x * warps_per_block + (threadIdx.x >> 5); pr < P; pr += gridDim.x * warps_per_block) {
    const int slot = pair_slot[pr];
    float acc = 0.f;
    if (slot >= 0) {
      const uint4* a = reinterpret_cast<const uint4*>(dout + (long long)(pr / k) * H);
      const uint4* b = reinterpret_cast<const uint4*>(y.p[pair_rank ? pair_rank[pr] : 0] + (long long)slot * H);
      for (int v = lane; v < nvec; v += 32) {
        const uint4 xa = a[v], xb = b[v];
        const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&xa);
        const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&xb);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 fa = __bfloat1622float2(ha[i]), fb = __bfloat1622float2(hb[i]);
          acc += fa.x * fb.x + fa.y * fb.y;
        }
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) dots[pr] = acc;
  }
}

static int moe_grid(int rows) {
  int blocks = (rows + 7) / 8;
  const int cap = 148 * 8;
  return blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
}

static bool fill_peers(MoePeers& mp, const void* const* ptrs, int world) {
  if (world < 1 || world > kMoeMaxRanks) return false;
  for (int r = 0; r < kMoeMaxRanks; ++r) mp.p[r] = r < world ? reinterpret_cast<const __nv_bfloat16*>(ptrs[r]) : nullptr;
  return true;
}

}  // namespace sb

using namespace sb;

extern "C" int sb_moe_gather_rows(const void* const* src_ptrs, int world, const int* src_rank, const int* src_row,
                                  const float* scale, void* out, int M, int H, cudaStream_t stream) {
  if (M <= 0) return 0;
  MoePeers mp;
  if (H % 8 || !fill_peers(mp, src_ptrs, world)) return -3;
  moe_gather_rows_kernel<<<moe_grid(M), 256, 0, stream>>>(mp, src_rank, src_row, scale, (__nv_bfloat16*)out, M, H);
  return (int)cudaGetLastError();
}

extern "C" int sb_moe_combine(const void* const* y_ptrs, int world, const int* pair_rank, const int* pair_slot,
                              const float* w, void* out, int T, int k, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  MoePeers mp;
  if (H % 8 || !fill_peers(mp, y_ptrs, world)) return -3;
  moe_combine_kernel<<<moe_grid(T), 256, 0, stream>>>(mp, pair_rank, pair_slot, w, (__nv_bfloat16*)out, T, k, H);
  return (int)cudaGetLastError();
}

extern "C" int sb_moe_pair_dot(const void* const* y_ptrs, int world, const int* pair_rank, const int* pair_slot,
                               const void* dout, float* dots, int T, int k, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  MoePeers mp;
  if (H % 8 || !fill_peers(mp, y_ptrs, world)) return -3;
  moe_pair_dot_kernel<<<moe_grid(T * k), 256, 0, stream>>>(mp, pair_rank, pair_slot, (const __nv_bfloat16*)dout, dots,
                                                          T, k, H);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// router: softmax over experts + top-k (+ renormalisation) in one pass, and its backward
// ---------------------------------------------------------------------------------------
// One warp per token; lane l holds experts l, l+32, ... (E <= 32 * kRouteMaxPerLane).  Ties go to the lower
// expert id.  Forward keeps nothing but (weights, ids): the backward recomputes the softmax from the logits.
constexpr int kRouteMaxPerLane = 8;

template <typename T>
__device__ __forceinline__ float route_load(const T* p);
template <>
__device__ __forceinline__ float route_load<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float route_load<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__device__ __forceinline__ float route_softmax(const T* row, int E, int lane, float (&p)[kRouteMaxPerLane]) {
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kRouteMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? route_load(row + e) : -INFINITY;
    mx = fmaxf(mx, p[i]);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kRouteMaxPerLane; ++i) {
    p[i] = (lane + 32 * i < E) ? __expf(p[i] - mx) : 0.f;
    sum += p[i];
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
#pragma unroll
  for (int i = 0; i < kRouteMaxPerLane; ++i) p[i] *= inv;
  return inv;
}

template <typename T>
__global__ void __launch_bounds__(256) moe_route_topk_kernel(const T* __restrict__ logits, int ld, float* __restrict__ w,
                                                             int* __restrict__ idx, int Tn, int E, int k, int norm) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < Tn; t += warps) {
    float p[kRouteMaxPerLane];
    route_softmax(logits + (size_t)t * ld, E, lane, p);
    float sel_sum = 0.f, my_w = 0.f;
    int my_id = -1;
    for (int j = 0; j < k; ++j) {
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kRouteMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        if (e < E && p[i] > best) { best = p[i]; best_e = e; }   // ascending e in a lane: the first maximum wins
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
      if ((best_e & 31) == lane) {                        // taken: never selected again (probabilities are >= 0)
#pragma unroll
        for (int i = 0; i < kRouteMaxPerLane; ++i)
          if (i == (best_e >> 5)) p[i] = -1.f;
      }
      sel_sum += best;
      if (lane == j) { my_w = best; my_id = best_e; }
    }
    if (lane < k) {
      w[(size_t)t * k + lane] = norm ? my_w / sel_sum : my_w;
      idx[(size_t)t * k + lane] = my_id;
    }
  }
}

// dlogits = p * (dp - sum_e dp_e p_e), with dp_e = (dw_e - sum_j dw_j w_j) / S for selected e (S = sum of the
// selected probabilities; without renormalisation dp_e = dw_e), 0 elsewhere.
template <typename T>
__global__ void __launch_bounds__(256) moe_route_topk_bwd_kernel(const T* __restrict__ logits, int ld,
                                                                 const int* __restrict__ idx, const float* __restrict__ dw,
                                                                 float* __restrict__ dlogits, int Tn, int E, int k, int norm) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < Tn; t += warps) {
    float p[kRouteMaxPerLane], dp[kRouteMaxPerLane];
    route_softmax(logits + (size_t)t * ld, E, lane, p);
#pragma unroll
    for (int i = 0; i < kRouteMaxPerLane; ++i) dp[i] = 0.f;
    // lanes < k hold one selected expert each
    const int my_e = lane < k ? idx[(size_t)t * k + lane] : -1;
    const float my_dw = lane < k ? dw[(size_t)t * k + lane] : 0.f;
    float S = 0.f, dot = 0.f;
    for (int j = 0; j < k; ++j) {
      const int e = __shfl_sync(0xffffffffu, my_e, j);
      const float g = __shfl_sync(0xffffffffu, my_dw, j);
      float mine = 0.f;
#pragma unroll
      for (int i = 0; i < kRouteMaxPerLane; ++i)
        if (i == (e >> 5)) mine = p[i];
      const float pe = __shfl_sync(0xffffffffu, mine, e & 31);
      S += pe;
      dot += g * pe;
    }
    float acc = 0.f;
    // with renormalisation: w_j = p_j / S  =>  dp_e = (dw_e - sum_j dw_j p_j / S) / S on the selected set
    const float mean = norm ? dot / S : 0.f;
    const float invS = norm ? 1.f / S : 1.f;
    for (int j = 0; j < k; ++j) {
      const int e = __shfl_sync(0xffffffffu, my_e, j);
      const float g = __shfl_sync(0xffffffffu, my_dw, j);
      if ((e & 31) == lane) {
#pragma unroll
        for (int i = 0; i < kRouteMaxPerLane; ++i)
          if (i == (e >> 5)) dp[i] = (g - mean) * invS;
      }
    }
#pragma unroll
    for (int i = 0; i < kRouteMaxPerLane; ++i) acc += dp[i] * p[i];
#pragma unroll
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
#pragma unroll
    for (int i = 0; i < kRouteMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      if (e < E) dlogits[(size_t)t * E + e] = p[i] * (dp[i] - acc);
    }
  }
}

extern "C" int sb_moe_route_topk(const void* logits, int is_bf16, int ld, float* w, int* idx, int T, int E, int k,
                                 int norm, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > 32 * kRouteMaxPerLane || k < 1 || k > 32 || k > E) return -3;
  const int grid = moe_grid(T);
  if (is_bf16)
    moe_route_topk_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)logits, ld, w, idx, T, E, k, norm);
  else
    moe_route_topk_kernel<<<grid, 256, 0, stream>>>((const float*)logits, ld, w, idx, T, E, k, norm);
  return (int)cudaGetLastError();
}

extern "C" int sb_moe_route_topk_bwd(const void* logits, int is_bf16, int ld, const int* idx, const float* dw,
                                     float* dlogits, int T, int E, int k, int norm, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > 32 * kRouteMaxPerLane || k < 1 || k > 32 || k > E) return -3;
  const int grid = moe_grid(T);
  if (is_bf16)
    moe_route_topk_bwd_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)logits, ld, idx, dw, dlogits, T, E, k, norm);
  else
    moe_route_topk_bwd_kernel<<<grid, 256, 0, stream>>>((const float*)logits, ld, idx, dw, dlogits, T, E, k, norm);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// expert-sorted, 128-padded slot layout from the routing table: three launches
// ---------------------------------------------------------------------------------------
// Pair p = (src_rank * T + t) * k + j routes token t of src_rank to expert idx[p] (negative: padding token, gets
// no slot).  Experts are laid out in id order, each padded to a multiple of 128 rows; inside an expert the pairs
// keep ascending p (what a stable sort by expert gives), so the layout is deterministic.
//   count:  per-chunk histograms (chunk = 1024 consecutive pairs) + initial values of the slot arrays
//   scan:   per-expert exclusive scan over chunks, padded expert starts, per-rank bases, block -> expert table
//   place:  stable rank inside the chunk (warp match + per-warp counts), slot of every pair, owner's slot arrays
constexpr int kLayoutChunk = 1024;
constexpr int kLayoutMaxE = 256;   // real experts; one dummy expert for padding tokens is appended

__global__ void __launch_bounds__(kLayoutChunk) moe_layout_count_kernel(
    const int* __restrict__ idx, int P, int E, int* __restrict__ chunk_counts, long long* __restrict__ slot_pair,
    int* __restrict__ slot_src_rank, int* __restrict__ slot_src_row, int capacity) {
  __shared__ int hist[kLayoutMaxE + 1];
  for (int e = threadIdx.x; e <= E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int p = blockIdx.x * kLayoutChunk + threadIdx.x;
  if (p < P) {
    int e = idx[p];
    if (e < 0 || e >= E) e = E;
    atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) chunk_counts[(size_t)blockIdx.x * (E + 1) + e] = hist[e];
  for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < capacity; s += gridDim.x * blockDim.x) {
    slot_pair[s] = -1;
    slot_src_rank[s] = 0;
    slot_src_row[s] = -1;
  }
}

__global__ void __launch_bounds__(1024) moe_layout_scan_kernel(int* __restrict__ chunk_counts, int n_chunks, int E,
                                                               int world, int rank, int capacity,
                                                               int* __restrict__ starts, int* __restrict__ rank_base,
                                                               int* __restrict__ tile_group,
                                                               int* __restrict__ group_rows) {
  __shared__ int counts[kLayoutMaxE + 1];
  __shared__ int s_starts[kLayoutMaxE + 2];
  const int El = E / world;
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    int running = 0;
    for (int c = 0; c < n_chunks; ++c) {
      const int v = chunk_counts[(size_t)c * (E + 1) + e];
      chunk_counts[(size_t)c * (E + 1) + e] = running;
      running += v;
    }
    counts[e] = running;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e <= E; ++e) {
      s_starts[e] = acc;
      acc += (counts[e] + 127) / 128 * 128;
    }
    s_starts[E + 1] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E + 1; e += blockDim.x) starts[e] = s_starts[e];
  for (int r = threadIdx.x; r <= world; r += blockDim.x) rank_base[r] = s_starts[r * El];
  const int base = s_starts[rank * El];
  // padded end of my local experts in local coordinates: s_starts[rank*El + i + 1] - base
  for (int i = threadIdx.x; i <= El; i += blockDim.x) {
    const int v = i == 0 ? 0 : s_starts[rank * El + i] - base;
    group_rows[i] = v < capacity ? v : capacity;
  }
  for (int b = threadIdx.x; b < capacity / 128; b += blockDim.x) {
    const int row = b * 128;
    int g = 0;   // number of local experts whose padded end is <= row
    while (g < El && s_starts[rank * El + g + 1] - base <= row) ++g;
    tile_group[b] = g < El ? g : -1;
  }
}

__global__ void __launch_bounds__(kLayoutChunk) moe_layout_place_kernel(
    const int* __restrict__ idx, int P, int E, int world, int rank, int T, int k, int capacity,
    const int* __restrict__ chunk_offsets, const int* __restrict__ starts, const int* __restrict__ rank_base,
    int* __restrict__ pair_rank, int* __restrict__ pair_slot, long long* __restrict__ slot_pair,
    int* __restrict__ slot_src_rank, int* __restrict__ slot_src_row) {
  __shared__ int wc[kLayoutChunk / 32][kLayoutMaxE + 2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (kLayoutChunk / 32) * (kLayoutMaxE + 2); i += blockDim.x) (&wc[0][0])[i] = 0;
  __syncthreads();
  const int p = blockIdx.x * kLayoutChunk + threadIdx.x;
  int e = E + 1;                                    // lanes past the end: a key of their own, never placed
  if (p < P) {
    e = idx[p];
    if (e < 0 || e >= E) e = E;
  }
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (rank_in_warp == 0) wc[warp][e] = __popc(peers);
  __syncthreads();
  for (int x = threadIdx.x; x <= E; x += blockDim.x) {
    int running = 0;
    for (int w = 0; w < kLayoutChunk / 32; ++w) {
      const int v = wc[w][x];
      wc[w][x] = running;
      running += v;
    }
  }
  __syncthreads();
  if (p >= P) return;
  const int El = E / world;
  const int rank_in_e = chunk_offsets[(size_t)blockIdx.x * (E + 1) + e] + wc[warp][e] + rank_in_warp;
  const int host = e / El;                          // == world for padding pairs
  if (host >= world) {
    pair_rank[p] = world - 1;
    pair_slot[p] = -1;
    return;
  }
  const int lslot = starts[e] + rank_in_e - rank_base[host];
  pair_rank[p] = host;
  pair_slot[p] = lslot < capacity ? lslot : -1;
  if (host == rank && lslot < capacity) {
    slot_pair[lslot] = p;
    slot_src_rank[lslot] = p / (T * k);
    slot_src_row[lslot] = (p / k) % T;
  }
}

// scratch: chunk_counts [n_chunks * (E + 1)], starts [E + 2], rank_base [world + 1] (all int32)
extern "C" int sb_moe_build_layout(const int* idx, int P, int E, int world, int rank, int T, int k, int capacity,
                                   int* chunk_counts, int* starts, int* rank_base, int* pair_rank, int* pair_slot,
                                   long long* slot_pair, int* slot_src_rank, int* slot_src_row, int* tile_group,
                                   int* group_rows, cudaStream_t stream) {
  if (P <= 0 || E < 1 || E > kLayoutMaxE || world < 1 || E % world || rank < 0 || rank >= world || capacity % 128 ||
      capacity <= 0 || T <= 0 || k <= 0)
    return -3;
  const int n_chunks = (P + kLayoutChunk - 1) / kLayoutChunk;
  moe_layout_count_kernel<<<n_chunks, kLayoutChunk, 0, stream>>>(idx, P, E, chunk_counts, slot_pair, slot_src_rank,
                                                                slot_src_row, capacity);
  moe_layout_scan_kernel<<<1, 1024, 0, stream>>>(chunk_counts, n_chunks, E, world, rank, capacity, starts, rank_base,
                                                 tile_group, group_rows);
  moe_layout_place_kernel<<<n_chunks, kLayoutChunk, 0, stream>>>(idx, P, E, world, rank, T, k, capacity, chunk_counts,
                                                                starts, rank_base, pair_rank, pair_slot, slot_pair,
                                                                slot_src_rank, slot_src_row);
  return (int)cudaGetLastError();
}
