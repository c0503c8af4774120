// Cross-rank phase of the row-parallel GEMM fused with its all-reduce (included by gemm_tcgen05.cu inside namespace
// sb; runs in the 128 epilogue threads of the CTA that completed an output tile).  Two protocols:
//
//  one-shot (ar.one_shot; decode batches, and every size in a group of two): the finisher adds the local split-K slabs and PUSHES the fp32 tile
//    into every rank's receive slab (remote stores do not stall), raises the tile's flag on every rank, waits for the
//    flags of all ranks in its own array and sums the received tiles from LOCAL memory into the bf16 output.  Receive
//    slabs alternate with the launch epoch, so a rank one launch ahead never overwrites data still being read; it
//    cannot be two launches ahead because each launch needs every rank's flags.
//  two-shot (larger M): tile owner = tile % world pulls the partial tile from every rank, reduces, stores bf16 to every
//    rank and raises done flags; the non-owners wait for them before the kernel ends.
//
// All peer waits are bounded (flag_wait_ge); on a timeout the status word is set and the CTA stops waiting.
#pragma once

__device__ __forceinline__ void add8(float* acc, const float4& x, const float4& y) {
  acc[0] += x.x; acc[1] += x.y; acc[2] += x.z; acc[3] += x.w;
  acc[4] += y.x; acc[5] += y.y; acc[6] += y.z; acc[7] += y.w;
}

__device__ __forceinline__ uint4 bias_pack8(float* v, const __nv_bfloat16* bias, int c) {
  if (bias) {
    const uint4 bv = *reinterpret_cast<const uint4*>(bias + c);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(b2[i]);
      v[2 * i] += f.x;
      v[2 * i + 1] += f.y;
    }
  }
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]);
  o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]);
  o.w = pack_bf16x2(v[6], v[7]);
  return o;
}

// Sums `nsrc` fp32 tiles (source s at base[s], row pitch `pitch` floats) over this warp's 32 rows of the tile, with
// the loads of kU row-chunks in flight together, and hands each 8-column group to `sink(r, c, acc)`.
template <int BN, typename BaseFn, typename Sink>
__device__ __forceinline__ void ar_sum_tile(int nsrc, BaseFn base, long long pitch, int m0, int n0, int quarter,
                                            int lane, int M, int N, Sink sink) {
  constexpr int kVecRow = BN / 8;
  constexpr int kItems = 32 * kVecRow;
  constexpr int kU = 4;
  for (int it0 = lane; it0 < kItems; it0 += 32 * kU) {
    float acc[kU][8];
    int rr[kU], cc[kU];
    bool ok[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int it = it0 + 32 * u;
      rr[u] = m0 + quarter * 32 + it / kVecRow;
      cc[u] = n0 + (it % kVecRow) * 8;
      ok[u] = it < kItems && rr[u] < M && cc[u] + 8 <= N;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[u][i] = 0.f;
    }
    for (int s = 0; s < nsrc; ++s) {
      const float* b = base(s);
      float4 x[kU], y[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        if (ok[u]) {
          const float* src = b + (long long)rr[u] * pitch + cc[u];
          x[u] = ld_volatile_f4(src);
          y[u] = ld_volatile_f4(src + 4);
        }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u)
        if (ok[u]) add8(acc[u], x[u], y[u]);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u)
      if (ok[u]) sink(rr[u], cc[u], acc[u]);
  }
}

template <int BN>
__device__ __forceinline__ void ar_tile_phase(const GemmParams& p, int tile_mn, int m0, int n0, int quarter, int lane,
                                              int epi_tid, volatile uint32_t* ar_smem, int ar_epoch, bool& ar_ok,
                                              unsigned long long& ar_pending, int ar_iter) {
  const ArParams& ar = *p.ar;
  __threadfence();  // this thread's slab stores, device-wide
  epi_bar();
  if (epi_tid == 0) {
    uint32_t last = 1;
    if (p.k_splits > 1) {
      const int prev = atomicAdd(&ar.local[2 + tile_mn], 1);
      last = (prev == p.k_splits - 1) ? 1u : 0u;
      if (last) ar.local[2 + tile_mn] = 0;
    }
    ar_smem[0] = last;
  }
  epi_bar();
  const bool finisher = ar_smem[0] != 0;
  epi_bar();  // ar_smem[0] may be rewritten for the next tile
  if (!finisher || !ar_ok) return;
  __threadfence();
  const float* slabs = reinterpret_cast<const float*>(p.C);
  const int world = ar.world, rank = ar.rank;

  if (ar.one_shot) {
    // ---- push the locally reduced tile to every rank ----
    const long long slot = (long long)((ar_epoch & 1) * world + rank) * ar.recv_slab;
    ar_sum_tile<BN>(
        p.k_splits, [&](int s) { return slabs + s * p.slab_stride; }, p.ldc, m0, n0, quarter, lane, p.M, p.N,
        [&](int r, int c, float* a) {
          const float4 lo = make_float4(a[0], a[1], a[2], a[3]), hi = make_float4(a[4], a[5], a[6], a[7]);
          for (int k = 0; k < world; ++k) {
            float* dst = ar.recv[(rank + k) % world] + slot + (long long)r * p.N + c;
            *reinterpret_cast<float4*>(dst) = lo;
            *reinterpret_cast<float4*>(dst + 4) = hi;
          }
        });
    __threadfence_system();
    epi_bar();
    if (epi_tid < world) flag_store_release(ar.ready[epi_tid] + tile_mn * kArMaxRanks + rank, ar_epoch);
    if (epi_tid < world && !flag_wait_ge(ar.ready[rank] + tile_mn * kArMaxRanks + epi_tid, ar_epoch, p.status))
      ar_smem[1] = 1;
    epi_bar();
    ar_ok = ar_smem[1] == 0;
    if (!ar_ok) return;
    const float* mine = ar.recv[rank] + (long long)((ar_epoch & 1) * world) * ar.recv_slab;
    __nv_bfloat16* out = ar.out[rank];
    ar_sum_tile<BN>(
        world, [&](int s) { return mine + s * ar.recv_slab; }, p.N, m0, n0, quarter, lane, p.M, p.N,
        [&](int r, int c, float* a) {
          *reinterpret_cast<uint4*>(out + (long long)r * ar.ldo + c) = bias_pack8(a, p.bias, c);
        });
    return;
  }

  // ---- two-shot: publish the partial tile, owner reduces and broadcasts ----
  if (p.k_splits > 1) {
    float* my_partial = ar.partial[rank];
    ar_sum_tile<BN>(
        p.k_splits, [&](int s) { return slabs + s * p.slab_stride; }, p.ldc, m0, n0, quarter, lane, p.M, p.N,
        [&](int r, int c, float* a) {
          float* dst = my_partial + (long long)r * p.N + c;
          *reinterpret_cast<float4*>(dst) = make_float4(a[0], a[1], a[2], a[3]);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(a[4], a[5], a[6], a[7]);
        });
  }
  __threadfence_system();
  epi_bar();
  const int owner = tile_mn % world;
  if (epi_tid == 0) flag_store_release(ar.ready[owner] + tile_mn * kArMaxRanks + rank, ar_epoch);
  if (owner == rank) {
    if (epi_tid < world && !flag_wait_ge(ar.ready[rank] + tile_mn * kArMaxRanks + epi_tid, ar_epoch, p.status))
      ar_smem[1] = 1;
    epi_bar();
    ar_ok = ar_smem[1] == 0;
    if (!ar_ok) return;
    ar_sum_tile<BN>(
        world, [&](int s) { return (const float*)ar.partial[(rank + s) % world]; }, p.N, m0, n0, quarter, lane, p.M,
        p.N, [&](int r, int c, float* a) {
          const uint4 o = bias_pack8(a, p.bias, c);
          for (int q = 0; q < world; ++q) *reinterpret_cast<uint4*>(ar.out[q] + (long long)r * ar.ldo + c) = o;
        });
    __threadfence_system();
    epi_bar();
    if (epi_tid < world) flag_store_release(ar.done[epi_tid] + tile_mn, ar_epoch);
  } else if (ar_iter < 64) {
    ar_pending |= 1ull << ar_iter;
  } else {
    if (epi_tid == 0 && !flag_wait_ge(ar.done[rank] + tile_mn, ar_epoch, p.status)) ar_smem[1] = 1;
    epi_bar();
    ar_ok = ar_smem[1] == 0;
  }
}
