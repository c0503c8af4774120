// Per-step bookkeeping of the rollout engine's lock-step decode, two launches per step instead of some thirty
// element-wise ones: everything a decode step reads and updates (context lengths, last tokens, finished flags,
// token and log-prob output rows, the sampler's step counter) lives in device memory so that the step replays from a
// CUDA graph.  The reference gets this bookkeeping from vLLM's scheduler and sampler output processing
// (siirl/engine/rollout/vllm_rollout/vllm_rollout_spmd.py:261-416).
//
//   decode_prepare_kernel   slot state -> inputs of the forward pass (cache position, sequence id or -1 for an idle
//                           slot, context length including the new token, rope position)
//   decode_commit_kernel    sampled token + log-prob -> output rows, counters, finished / hit-EOS flags
#include "common.cuh"
#include "launchers.h"

namespace sb {

__global__ void decode_prepare_kernel(const unsigned char* __restrict__ finished, const int* __restrict__ ctx_len,
                                      const int* __restrict__ rope_delta, int* __restrict__ pos,
                                      int* __restrict__ seq_ids, int* __restrict__ seq_lens,
                                      int* __restrict__ rope_pos, int S) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= S) return;
  const bool active = finished[i] == 0;
  const int c = ctx_len[i];
  pos[i] = active ? max(c, 0) : 0;
  seq_ids[i] = active ? i : -1;
  seq_lens[i] = active ? c + 1 : 0;
  rope_pos[i] = active ? max(c - rope_delta[i], 0) : 0;
}

__global__ void decode_commit_kernel(const long long* __restrict__ tok, const float* __restrict__ lp,
                                     unsigned char* __restrict__ finished, unsigned char* __restrict__ hit_eos,
                                     int* __restrict__ ctx_len, int* __restrict__ remaining,
                                     int* __restrict__ gen_index, long long* __restrict__ last_token,
                                     long long* __restrict__ tokens_out, float* __restrict__ logp_out,
                                     long long* __restrict__ step_counter, int S, int R, long long eos) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) *step_counter += 1;     // the sampler of this step has run already (same stream)
  if (i >= S) return;
  if (finished[i]) return;
  const long long t = tok[i];
  const int col = min(gen_index[i], R - 1);
  tokens_out[(size_t)i * R + col] = t;
  logp_out[(size_t)i * R + col] = lp[i];
  gen_index[i] += 1;
  ctx_len[i] += 1;
  const int rem = remaining[i] - 1;
  remaining[i] = rem;
  last_token[i] = t;
  bool done = rem <= 0;
  if (eos >= 0 && t == eos) {
    done = true;
    hit_eos[i] = 1;
  }
  if (done) finished[i] = 1;
}

}  // namespace sb

using namespace sb;

extern "C" int sb_decode_prepare(const void* finished, const int* ctx_len, const int* rope_delta, int* pos,
                                 int* seq_ids, int* seq_lens, int* rope_pos, int S, cudaStream_t stream) {
  if (S <= 0) return 0;
  decode_prepare_kernel<<<(S + 127) / 128, 128, 0, stream>>>(reinterpret_cast<const unsigned char*>(finished),
                                                             ctx_len, rope_delta, pos, seq_ids, seq_lens, rope_pos, S);
  return (int)cudaGetLastError();
}

// eos < 0: no end-of-sequence token (or it is ignored)
extern "C" int sb_decode_commit(const long long* tok, const float* lp, void* finished, void* hit_eos, int* ctx_len,
                                int* remaining, int* gen_index, long long* last_token, long long* tokens_out,
                                float* logp_out, long long* step_counter, int S, int R, long long eos,
                                cudaStream_t stream) {
  if (S <= 0) return 0;
  decode_commit_kernel<<<(S + 127) / 128, 128, 0, stream>>>(
      tok, lp, reinterpret_cast<unsigned char*>(finished), reinterpret_cast<unsigned char*>(hit_eos), ctx_len,
      remaining, gen_index, last_token, tokens_out, logp_out, step_counter, S, R, eos);
  return (int)cudaGetLastError();
}
