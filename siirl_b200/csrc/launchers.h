// Plain-C launch entry points of the sm_100a kernels.  The .cu files include no torch header
// (fast to compile, callable from C, ctypes or the torch bindings in bindings.cpp).
// Every function returns 0 on success, a cudaError_t / CUresult value, or a negative code:
//   -1 driver entry point unavailable, -2 unsupported variant, -3 bad shape or alignment.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>

namespace sb {
int num_sms();
int make_tensor_map_bf16_2d(CUtensorMap* map, const void* base, long long inner, long long outer,
                            long long pitch_elems, int box_inner, int box_outer);
}  // namespace sb

extern "C" {

// ---- gemm_tcgen05.cu ----
// C[M,N] (+)= A * B^T.  a_mn/b_mn: operand stored with the contraction index strided
// (A as [K,M], B as [K,N]).  epi: 0 bf16 store (+bias), 1 fp32 accumulate, 2 fp32 store.
// tile_n: 128, 256 or 0 (auto).  max_ctas: 0 = one CTA per SM.
int sb_gemm_ar_bf16(const void* A, const void* B, const void* bias, int M, int N, int K, long long lda, long long ldb,
                    const void* ar_params, void* c_local, int tile_n, int k_splits, long long slab_stride,
                    int max_tiles, int* status, cudaStream_t stream);
int sb_moe_gather_rows(const void* const* src_ptrs, int world, const int* src_rank, const int* src_row,
                       const float* scale, void* out, int M, int H, cudaStream_t stream);
int sb_moe_combine(const void* const* y_ptrs, int world, const int* pair_rank, const int* pair_slot, const float* w,
                   void* out, int T, int k, int H, cudaStream_t stream);
int sb_moe_pair_dot(const void* const* y_ptrs, int world, const int* pair_rank, const int* pair_slot, const void* dout,
                    float* dots, int T, int k, int H, cudaStream_t stream);
int sb_moe_route_topk(const void* logits, int is_bf16, int ld, float* w, int* idx, int T, int E, int k, int norm,
                      cudaStream_t stream);
int sb_moe_route_topk_bwd(const void* logits, int is_bf16, int ld, const int* idx, const float* dw, float* dlogits,
                          int T, int E, int k, int norm, cudaStream_t stream);
int sb_moe_build_layout(const int* idx, int P, int E, int world, int rank, int T, int k, int capacity,
                        int* chunk_counts, int* starts, int* rank_base, int* pair_rank, int* pair_slot,
                        long long* slot_pair, int* slot_src_rank, int* slot_src_row, int* tile_group, int* group_rows,
                        cudaStream_t stream);
int sb_ag_gemm_bf16(const void* A, const void* staging, void* C, const void* bias, int M, int N, int K, long long lda,
                    long long ld, long long ldc, const void* ag_params, int copiers, int tile_n, int* status,
                    cudaStream_t stream);
int sb_block_pull(void* const* bases, int world, const void* blocks, int n_blocks, void* out, cudaStream_t stream);
int sb_gemm_grouped_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, int a_mn, int b_mn, int epi, int tile_n, const int* tile_group,
                         long long b_group_rows, const int* group_rows, int num_groups, long long c_group_stride,
                         int* status, cudaStream_t stream);
int sb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                 long long ldb, long long ldc, int a_mn, int b_mn, int epi, int tile_n, int max_ctas,
                 int k_splits, long long slab_stride, int* status, cudaStream_t stream);
int sb_gemm_lmstat_bf16(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                        const long long* labels, float inv_temp, void* partial, int* status, cudaStream_t stream);
int sb_gemm_dlogits_bf16(const void* A, const void* B, void* dlogits, int M, int N, int K, long long lda, long long ldb,
                         long long ldd, const long long* labels, float inv_temp, const float* lse, const float* ent,
                         const float* g_logp, const float* g_ent, int* status, cudaStream_t stream);
// out = bf16(sum over `splits` fp32 slabs [M, N] + bias)
int sb_splitk_reduce(const float* slabs, long long slab_stride, int splits, const void* bias, void* out,
                     long long ldo, int M, int N, cudaStream_t stream);

// ---- elementwise.cu ----
int sb_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out, float* rstd,
                   int T, int H, float eps, cudaStream_t stream);
int sb_rmsnorm_bwd_blocks(int T);
int sb_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres, void* dx,
                   float* dw_partial, float* dw, int dw_accumulate, int T, int H, cudaStream_t stream);
int sb_rope(void* qkv, const int* pos, const float* cos_tab, const float* sin_tab, int T, int row_stride,
            int n_heads_rot, int D, int pos_rows, int sec0, int sec1, float sign, cudaStream_t stream);
int sb_swiglu_fwd(const void* gu, void* out, int T, int I, cudaStream_t stream);
int sb_swiglu_bwd(const void* gu, const void* dout, void* dgu, int T, int I, cudaStream_t stream);
int sb_embedding_fwd(const long long* ids, const void* table, void* out, int T, int H, int V,
                     cudaStream_t stream);
int sb_embedding_bwd(const long long* ids, const void* dout, float* dtable, int T, int H, int V,
                     cudaStream_t stream);
int sb_add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t stream);

}  // extern "C"

extern "C" {
// ---- rl_algos.cu ----
int sb_gae_scan(const float* rewards, const float* values, const float* mask, float* adv, float* ret, int B,
                int R, float gamma, float lam, cudaStream_t stream);
int sb_grpo_group_adv(const float* rewards, const float* mask, const int* gid, float* scores_ws, float* group_ws,
                      float* adv, int B, int R, int G, float eps, int norm_by_std, cudaStream_t stream);
int sb_ppo_token_loss(const float* logp, const float* old_logp, const float* adv, const float* mask,
                      const float* ref_logp, const float* entropy, const float* w_row, const float* seq_logratio,
                      float* dlogp, float* dentropy, float* stats, int B, int R, int mode, float clip_lo,
                      float clip_hi, float clip_c, int use_kl, float kl_coef, float entropy_coef,
                      float loss_scale, cudaStream_t stream);
}

extern "C" {
// ---- fmha_fwd.cu / fmha_bwd.cu ----
int sb_fmha_fwd(const void* qkv, void* out, float* lse, const int* tile_seq_start, const int* tile_seq_len,
                const int* tile_q0, int num_tiles, int T, int Hq, int Hkv, int D, int causal, float scale,
                int* status, cudaStream_t stream);
int sb_fmha_bwd(const void* qkv, const void* out, const void* d_out, const float* lse, float* delta,
                float* dq_accum, void* dqkv, const int* tile_seq_start, const int* tile_seq_len,
                const int* tile_k0, int num_tiles, int T, int Hq, int Hkv, int D, int causal, float scale,
                int* status, cudaStream_t stream);
}

extern "C" {
// ---- lm_head.cu ----
int sb_lmhead_merge(const void* partial, int tiles, const long long* labels, float* logp, float* entropy, float* lse,
                    int rows, int V, cudaStream_t stream);
int sb_lmhead_stats(const float* logits, long long ld, const long long* labels, float inv_temp, float* logp,
                    float* entropy, float* lse, int rows, int V, cudaStream_t stream);
int sb_lmhead_dlogits(const float* logits, long long ld, const long long* labels, const float* lse,
                      const float* entropy, const float* g_logp, const float* g_ent, float inv_temp, void* dlogits,
                      long long ldd, int rows, int V, cudaStream_t stream);
// ---- sampling.cu ----
int sb_sample(const float* sample_logits, const float* stat_logits, long long ld, float temperature,
              unsigned long long seed, unsigned long long step, const long long* step_dev, long long* tokens,
              float* logp, int rows, int V, void* workspace, int splits, cudaStream_t stream);
// ---- optimizer.cu ----
int sb_sumsq_accumulate(const float* g, long long n, float* out, cudaStream_t stream);
int sb_adamw_step(float* master, float* m, float* v, const float* grad, void* param_bf16, const float* sumsq,
                  float* grad_norm_out, long long n, float lr, float beta1, float beta2, float eps,
                  float weight_decay, int step, float max_norm, float grad_scale, cudaStream_t stream);
int sb_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t stream);
}

extern "C" {
// ---- fmha_decode.cu ----
int sb_kv_append(const void* qkv, int row_stride, const int* seq_ids, const int* positions, const int* block_table,
                 int max_blocks, void* cache, int T, int Hq, int Hkv, int D, cudaStream_t stream);
int sb_rope_kv_append(void* qkv, int row_stride, const int* rope_pos, int pos_rows, int sec0, int sec1,
                      const float* cos_tab, const float* sin_tab, const int* seq_ids, const int* cache_pos,
                      const int* block_table, int max_blocks, void* cache, int T, int Hq, int Hkv, int D,
                      cudaStream_t stream);
int sb_kv_copy_blocks(void* cache, const int* src, const int* dst, int n_pairs, long long block_elems,
                      cudaStream_t stream);
int sb_fmha_decode(const void* q, int row_stride, const void* cache, long long num_blocks, const int* seq_lens,
                   const int* block_table, int max_blocks, void* out, int B, int Hq, int Hkv, int D, float scale,
                   int* status, cudaStream_t stream);
// ---- fmha_decode_split.cu ----
// Persistent split-K/V variant of sb_fmha_decode.  Workspaces in floats: ws_o = B * Hq * chunks * D and
// ws_lse = B * Hq * chunks with chunks = ceil(max_blocks / sb_fmha_decode_chunk_tiles()).
int sb_fmha_decode_chunk_tiles();
int sb_fmha_decode_split(const void* q, int row_stride, const void* cache, long long num_blocks, const int* seq_lens,
                         const int* block_table, int max_blocks, void* out, float* ws_o, float* ws_lse, int B, int Hq,
                         int Hkv, int D, float scale, int* status, cudaStream_t stream);
}

extern "C" {
// ---- host/kk_partition.cpp ----
int sb_kk_partition(const long long* workloads, int n, int k, int equal_size, int* out_part);
}

extern "C" {
// ---- comm.cu ----
int sb_symm_alloc(void** out, long long bytes);
int sb_symm_free(void* p);
int sb_ipc_get_handle(void* p, unsigned char* out64);
int sb_ipc_open_handle(const unsigned char* in64, void** out);
int sb_ipc_close_handle(void* p);
int sb_ipc_handle_bytes();
int sb_rs_reduce(void* const* grad_ptrs, int world, int rank, long long lo, long long n, float* out_shard,
                 float* sumsq, const int* status, cudaStream_t stream);
int sb_rs_reduce_acc(void* const* grad_ptrs, int world, int rank, long long lo, long long n, float* out_shard,
                     cudaStream_t stream);
int sb_adamw_allgather(float* master, float* m, float* v, const float* grad, void* const* param_ptrs, int world,
                       const float* sumsq, float* grad_norm_out, long long lo, long long n, float lr, float beta1,
                       float beta2, float eps, float weight_decay, int step, float max_norm, float grad_scale,
                       cudaStream_t stream);
int sb_segment_pull(void* const* bases, int world, const void* segs, int n_segs, void* out, cudaStream_t stream);
int sb_flag_barrier(void* const* flag_ptrs, int world, int rank, int epoch, int* status, long long limit_ms,
                    cudaStream_t stream);
}

extern "C" {
// ---- decode_state.cu ----
int sb_decode_prepare(const void* finished, const int* ctx_len, const int* rope_delta, int* pos, int* seq_ids,
                      int* seq_lens, int* rope_pos, int S, cudaStream_t stream);
int sb_decode_commit(const long long* tok, const float* lp, void* finished, void* hit_eos, int* ctx_len,
                     int* remaining, int* gen_index, long long* last_token, long long* tokens_out, float* logp_out,
                     long long* step_counter, int S, int R, long long eos, cudaStream_t stream);
}

extern "C" {
// ---- image_ops.cu ----
int sb_resize_bilinear_u8(const void* src, void* dst, int N, int H, int W, int C, int OH, int OW, float crop_y0,
                          float crop_x0, float crop_h, float crop_w, cudaStream_t stream);
int sb_raster_synth_env(const float* state, void* out, int N, int H, int W, cudaStream_t stream);
}
