// Between the query/key projection and attention, for mixers whose queries and keys are normalised over the whole
// projected row and whose values are the keys as projected.
//
// Per token, from the float32 sums of the projection (row = [q: n_heads * dim | k: n_kv * dim]):
//   values   the key columns as projected, rounded once to the cache's dtype, appended to the value cache;
//   q, k     divided by the root mean square of the whole stretch (all heads together, eps inside the root), times a
//            gain per column; then in every head the first 2 * rot_pairs dimensions are turned, pair (2i, 2i + 1) by
//            the angle pos * inv_freq[i] (float32): (u, v) -> (u cos - v sin, v cos + u sin);
//   q goes to q_out [tokens][ldq] in the compute dtype, k is appended to the key cache.
// Everything between the projection's sums and the rounding of the results is float32.  Tokens of no sequence
// (sequence index -1) write nothing to the caches.  One block per token; the block's shape is fixed, so a row's sums
// do not depend on the step.
#include <math.h>

#include "common.cuh"

struct QKNormRope {
  const float* proj;        // [tokens][ld]
  const int* token_pos;
  const int* token_seq;
  const int* block_table;   // [seqs][bt_stride]
  const float* q_gain;      // [n_heads * dim]
  const float* k_gain;      // [n_kv * dim]
  const float* inv_freq;    // [rot_pairs]
  void* q_out;              // [tokens][ldq]
  void* k_cache;            // [pages][n_kv][page_tokens][dim]
  void* v_cache;            // the same shape
  int ld, ldq, bt_stride, n_tokens;
  int n_heads, n_kv, dim, rot_pairs;
  int page_tokens, write_cache;
  float eps, reserved;
};

#define QK_THREADS 256

template <typename T>
__global__ void __launch_bounds__(QK_THREADS) qk_norm_rope_kernel(const QKNormRope P) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();                                        // the projection is the work of the kernel before: ld_fresh
  const int t = blockIdx.x;
  const float* row = P.proj + (size_t)t * P.ld;
  const int D = P.dim, nq = P.n_heads * D, nk = P.n_kv * D;
  float ssq = 0.f, ssk = 0.f;
  for (int c = threadIdx.x; c < nq; c += QK_THREADS) {
    const float v = ld_fresh(row + c);
    ssq = fmaf(v, v, ssq);
  }
  for (int c = threadIdx.x; c < nk; c += QK_THREADS) {
    const float v = ld_fresh(row + nq + c);
    ssk = fmaf(v, v, ssk);
  }
  ssq = block_sum(ssq, scratch);
  ssk = block_sum(ssk, scratch);
  const float sq = 1.0f / sqrtf(ssq / (float)nq + P.eps), sk = 1.0f / sqrtf(ssk / (float)nk + P.eps);
  const int pos = P.token_pos[t], seq = P.token_seq[t];
  const int rot = 2 * P.rot_pairs;

  T* qo = (T*)P.q_out + (size_t)t * P.ldq;
  for (int c = threadIdx.x; c < nq; c += QK_THREADS) {
    const int d = c % D;
    float v = ld_fresh(row + c) * sq * P.q_gain[c];
    if (d < rot) {
      const int mate = (d & 1) ? c - 1 : c + 1;
      const float w = ld_fresh(row + mate) * sq * P.q_gain[mate];
      float sn, cs;
      sincosf((float)pos * P.inv_freq[d >> 1], &sn, &cs);
      v = (d & 1) ? v * cs + w * sn : v * cs - w * sn;
    }
    qo[c] = from_float<T>(v);
  }
  if (!P.write_cache || seq < 0) return;
  const int page = P.block_table[(size_t)seq * P.bt_stride + pos / P.page_tokens];
  if (page < 0) return;
  const int in_page = pos % P.page_tokens;
  for (int c = threadIdx.x; c < nk; c += QK_THREADS) {
    const int h = c / D, d = c - h * D;
    const size_t at = (((size_t)page * P.n_kv + h) * P.page_tokens + in_page) * D + d;
    const float raw = ld_fresh(row + nq + c);
    ((T*)P.v_cache)[at] = from_float<T>(raw);
    float v = raw * sk * P.k_gain[c];
    if (d < rot) {
      const int mate = (d & 1) ? c - 1 : c + 1;
      const float w = ld_fresh(row + nq + mate) * sk * P.k_gain[mate];
      float sn, cs;
      sincosf((float)pos * P.inv_freq[d >> 1], &sn, &cs);
      v = (d & 1) ? v * cs + w * sn : v * cs - w * sn;
    }
    ((T*)P.k_cache)[at] = from_float<T>(v);
  }
}

STRATUM_EXPORT int stratum_qk_norm_rope(const QKNormRope* params, int dtype, cudaStream_t stream) {
  const QKNormRope& P = *params;
  if (P.n_tokens <= 0) return 0;
  if (P.n_heads < 1 || P.n_kv < 1 || P.dim < 1 || P.rot_pairs < 0 || 2 * P.rot_pairs > P.dim || P.page_tokens < 1)
    return STRATUM_ERR_SHAPE;
  if (P.ld < (P.n_heads + P.n_kv) * P.dim || P.ldq < P.n_heads * P.dim) return STRATUM_ERR_SHAPE;
  if (dtype == STRATUM_DT_F32) launch_pdl(qk_norm_rope_kernel<float>, P.n_tokens, QK_THREADS, 0, stream, P);
  else if (dtype == STRATUM_DT_BF16) launch_pdl(qk_norm_rope_kernel<bf16>, P.n_tokens, QK_THREADS, 0, stream, P);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}
