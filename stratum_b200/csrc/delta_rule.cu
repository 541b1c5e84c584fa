// The gated delta rule: a recurrent mixer whose state is one matrix S [dim][vdim] per head, in float32.
//
// Per token, from the float32 sums of the fused input projection (row = [q | k | v | b | a | g]: n_kv * dim,
// n_kv * dim, n_heads * vdim conv channels, then n_heads, n_heads, n_heads * vdim):
//   prep      the conv channels pass a short causal convolution over time (taps per channel, the last tap is the
//             current token's; the taps - 1 inputs before a step's first token come from the sequence's state, zeros
//             before the sequence's start) and silu; q and k become unit vectors per head (x / sqrt(sum x^2 + 1e-6)),
//             q times dim^(-1/2); beta = sigmoid(b); decay = exp(-exp(A_log) * softplus(a + dt_bias)).
//   recur     per head, token after token:  S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//             (head h reads the q and k of head h / (n_heads / n_kv)).  The convolution's tail is moved on as well.
//   finish    o / sqrt(mean_vdim(o^2) + eps) * gain * silu(g), rounded to the compute dtype for the output product.
// All of it is float32 whatever the compute dtype.
//
// The recurrence is sequential in the tokens of a sequence and independent across sequences, heads and columns of S:
// a block owns (sequence, head, a tile of columns), a thread 16 rows of one column, so a column's sums are split over
// dim / 16 neighbouring lanes and added by shuffles in a fixed order; the tokens' k, q, v, beta and decay come through
// a double buffer in shared memory that the next tokens fill (cp.async) while the current ones are worked on.  Nothing depends on how a sequence's tokens are
// cut into steps or on the other sequences of a step.
#include <math.h>

#include "common.cuh"

struct DeltaRule {
  const float* proj;        // [tokens][ld]
  const float* conv_w;      // [channels][taps]
  const float* a_log;       // [n_heads]
  const float* dt_bias;     // [n_heads]
  const float* gain;        // [vdim]
  float* act;               // [tokens][lda]: q | k | v (after prep) | beta | decay
  float* o_raw;             // [tokens][n_heads * vdim]
  void* out;                // [tokens][ldo] compute dtype
  float* state;             // [slots][state_stride]: S^T [n_heads][vdim][dim], then the tail [taps - 1][channels]
  const int* token_pos;
  const int* token_seq;
  const int* seq_start;     // [seqs + 1]
  const int* seq_slot;      // [seqs]
  int ld, lda, ldo, n_tokens, n_seqs;
  int n_heads, n_kv, dim, vdim, taps;
  int state_stride, write_state;
  float eps, reserved;
};

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// ---------------------------------------------------------------- prep: one block per token
#define DR_PREP_THREADS 256
__global__ void __launch_bounds__(DR_PREP_THREADS) delta_prep_kernel(const DeltaRule P) {
  extern __shared__ float dr_act[];                  // [channels]
  const int t = blockIdx.x;
  const int D = P.dim, V = P.vdim, nqk = P.n_kv * D, C = 2 * nqk + P.n_heads * V;
  const int seq = P.token_seq[t];
  const int pos = P.token_pos[t];
  int in_step = 0;                                   // tokens of this sequence that the step brought before this one
  const float* tail = nullptr;
  if (seq >= 0) {
    in_step = t - P.seq_start[seq];
    tail = P.state + (size_t)P.seq_slot[seq] * P.state_stride + (size_t)P.n_heads * D * V;
  }
  const int n = P.taps;
  for (int c = threadIdx.x; c < C; c += DR_PREP_THREADS) {
    const float* w = P.conv_w + (size_t)c * n;
    float acc = 0.f;
    for (int i = n - 1; i >= 0; i--) {               // oldest input first: one fixed order
      float x = 0.f;
      if (i <= in_step) x = P.proj[(size_t)(t - i) * P.ld + c];
      else if (tail && pos - i >= 0) x = tail[(size_t)(n - 1 - (i - in_step)) * C + c];
      acc = fmaf(w[n - 1 - i], x, acc);
    }
    dr_act[c] = silu_f(acc);
  }
  __syncthreads();
  float* out = P.act + (size_t)t * P.lda;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int hd = warp; hd < 2 * P.n_kv; hd += DR_PREP_THREADS / 32) {       // q heads, then k heads
    const float* x = dr_act + (size_t)hd * D;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) ss = fmaf(x[d], x[d], ss);
    ss = warp_sum(ss);
    float mul = 1.0f / sqrtf(ss + 1e-6f);
    if (hd < P.n_kv) mul *= 1.0f / sqrtf((float)D);
    for (int d = lane; d < D; d += 32) out[(size_t)hd * D + d] = x[d] * mul;
  }
  for (int c = 2 * nqk + threadIdx.x; c < C; c += DR_PREP_THREADS) out[c] = dr_act[c];
  if (threadIdx.x < P.n_heads) {
    const int h = threadIdx.x;
    const float* row = P.proj + (size_t)t * P.ld;
    out[C + h] = 1.0f / (1.0f + expf(-row[C + h]));
    const float z = row[C + P.n_heads + h] + P.dt_bias[h];
    const float sp = z > 20.f ? z : log1pf(expf(z));
    out[C + P.n_heads + h] = expf(-expf(P.a_log[h]) * sp);
  }
}

// ---------------------------------------------------------------- the recurrence
#define DR_THREADS 128
#define DR_ROWS 16            // rows of S a thread holds
#define DR_PITCH 20           // floats between two lanes' stretches of k and q in shared memory: 16-byte aligned, and
                              // eight neighbouring lanes' float4 reads fall on different banks
#define DR_MAX_CHUNK 16       // tokens staged in shared memory at a time, at most

__device__ __forceinline__ void dr_copy4(float* dst_shared, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void dr_copy16(float* dst_shared, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void dr_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void dr_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// The state of a head lies in memory column by column (S^T: [vdim][dim]), so the 16 rows a thread holds are 64
// contiguous bytes and neighbouring lanes read neighbouring stretches.
template <int L>              // lanes per column: dim <= 16 * L
__global__ void __launch_bounds__(DR_THREADS) delta_recur_kernel(const DeltaRule P) {
  constexpr int COLS = DR_THREADS / L;
  constexpr int CHUNK = (64 / L) < DR_MAX_CHUNK ? ((64 / L) < 2 ? 2 : (64 / L)) : DR_MAX_CHUNK;
  constexpr int KQ = L * DR_PITCH;
  __shared__ __align__(16) float kq_s[2][CHUNK][2][KQ];
  __shared__ float v_s[2][CHUNK][COLS];
  __shared__ float bg_s[2][CHUNK][2];
  const int seq = blockIdx.z, h = blockIdx.y, tile = blockIdx.x;
  const int r0 = P.seq_start[seq], r1 = P.seq_start[seq + 1];
  if (r0 >= r1) return;
  const int D = P.dim, V = P.vdim, nqk = P.n_kv * D, C = 2 * nqk + P.n_heads * V;
  const int part = threadIdx.x % L, col = threadIdx.x / L;
  const int j = tile * COLS + col;
  const bool live = j < V;
  if (P.token_seq[r0] < 0) {                         // rows of no sequence: nothing is kept, the output is zero
    if (part == 0 && live)
      for (int r = r0; r < r1; r++) P.o_raw[(size_t)r * P.n_heads * V + (size_t)h * V + j] = 0.f;
    return;
  }
  float* slot = P.state + (size_t)P.seq_slot[seq] * P.state_stride;

  // the convolution's tail moves on by this step's tokens: the blocks of a sequence share the channels, a thread
  // takes a channel through time in order, so that an entry is read before it is overwritten
  if (P.write_state && P.taps > 1) {
    float* tail = slot + (size_t)P.n_heads * D * V;
    const int keep = P.taps - 1, n_new = r1 - r0;
    const int n_blocks = gridDim.x * gridDim.y, me = blockIdx.y * gridDim.x + blockIdx.x;
    const int per = (C + n_blocks - 1) / n_blocks;
    const int c_end = min(C, (me + 1) * per);
    for (int c = me * per + threadIdx.x; c < c_end; c += DR_THREADS)
      for (int i = 0; i < keep; i++) {
        const int back = keep - i;                   // this entry is the input `back` tokens before the next one
        tail[(size_t)i * C + c] = back <= n_new ? P.proj[(size_t)(r1 - back) * P.ld + c]
                                                : tail[(size_t)(i + n_new) * C + c];
      }
  }

  const int kv = h / (P.n_heads / P.n_kv);
  float* Sg = slot + ((size_t)h * V + (live ? j : 0)) * D + part * DR_ROWS;
  const bool vec = D % 4 == 0 && (P.state_stride % 4) == 0 && (((uintptr_t)P.state) & 15) == 0;
  float S[DR_ROWS];
#pragma unroll
  for (int i = 0; i < DR_ROWS; i += 4) {
    const int d = part * DR_ROWS + i;
    if (live && vec && d + 3 < D) {
      const float4 v4 = *reinterpret_cast<const float4*>(Sg + i);
      S[i] = v4.x; S[i + 1] = v4.y; S[i + 2] = v4.z; S[i + 3] = v4.w;
    } else {
#pragma unroll
      for (int u = 0; u < 4; u++) S[i + u] = (live && d + u < D) ? Sg[i + u] : 0.f;
    }
  }
  // the dimensions beyond dim in the staging buffers stay zero: nothing below writes them
  for (int i = threadIdx.x; i < 2 * CHUNK * 2 * KQ; i += DR_THREADS) (&kq_s[0][0][0][0])[i] = 0.f;
  __syncthreads();

  const bool vec_act = D % 4 == 0 && P.lda % 4 == 0 && (((uintptr_t)P.act) & 15) == 0;
  auto stage = [&](int buf, int c0) {                // ask for the tokens c0 .. of this sequence
    const int n_here = min(CHUNK, r1 - c0);
    for (int tok = 0; tok < n_here; tok++) {
      const float* a = P.act + (size_t)(c0 + tok) * P.lda + (size_t)kv * D;
      if (vec_act) {
        for (int d = 4 * threadIdx.x; d < 2 * D; d += 4 * DR_THREADS) {          // k, then q
          const int which = d >= D, dd = d - which * D;
          dr_copy16(&kq_s[buf][tok][which][(dd / DR_ROWS) * DR_PITCH + dd % DR_ROWS], a + (which ? 0 : nqk) + dd);
        }
      } else {
        for (int d = threadIdx.x; d < 2 * D; d += DR_THREADS) {
          const int which = d >= D, dd = d - which * D;
          dr_copy4(&kq_s[buf][tok][which][(dd / DR_ROWS) * DR_PITCH + dd % DR_ROWS], a + (which ? 0 : nqk) + dd);
        }
      }
    }
    for (int i = threadIdx.x; i < n_here * COLS; i += DR_THREADS) {
      const int tok = i / COLS, cc = i - tok * COLS, jj = tile * COLS + cc;
      if (jj < V) dr_copy4(&v_s[buf][tok][cc], P.act + (size_t)(c0 + tok) * P.lda + 2 * nqk + (size_t)h * V + jj);
    }
    if (threadIdx.x < n_here * 2) {
      const int tok = threadIdx.x >> 1, which = threadIdx.x & 1;                 // 0 = beta, 1 = decay
      dr_copy4(&bg_s[buf][tok][which], P.act + (size_t)(c0 + tok) * P.lda + C + which * P.n_heads + h);
    }
    dr_commit();
  };

  // Per token the two sums over a column, S^T k and S^T q, are taken from the state as the token finds it, together
  // and with one round of shuffles; the read-out after the token's own write follows from them:
  //   S' = decay S + k u^T,  u = beta (v - decay S^T k)   =>   S'^T q = decay S^T q + (k . q) u.
  stage(0, r0);
  int buf = 0;
  for (int c0 = r0; c0 < r1; c0 += CHUNK, buf ^= 1) {
    dr_wait_all();
    __syncthreads();                                 // this chunk has landed, and the other buffer is free again
    if (c0 + CHUNK < r1) stage(buf ^ 1, c0 + CHUNK);
    const int n_here = min(CHUNK, r1 - c0);
    for (int tok = 0; tok < n_here; tok++) {
      const float4* kk = reinterpret_cast<const float4*>(&kq_s[buf][tok][0][part * DR_PITCH]);
      const float4* qq = reinterpret_cast<const float4*>(&kq_s[buf][tok][1][part * DR_PITCH]);
      const float beta = bg_s[buf][tok][0], decay = bg_s[buf][tok][1], vj = v_s[buf][tok][col];
      float4 k4[DR_ROWS / 4];
      float sk[4] = {0.f, 0.f, 0.f, 0.f}, sq[4] = {0.f, 0.f, 0.f, 0.f}, kq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < DR_ROWS / 4; i++) {
        k4[i] = kk[i];
        const float4 q4 = qq[i];
        sk[0] = fmaf(S[4 * i], k4[i].x, sk[0]); sk[1] = fmaf(S[4 * i + 1], k4[i].y, sk[1]);
        sk[2] = fmaf(S[4 * i + 2], k4[i].z, sk[2]); sk[3] = fmaf(S[4 * i + 3], k4[i].w, sk[3]);
        sq[0] = fmaf(S[4 * i], q4.x, sq[0]); sq[1] = fmaf(S[4 * i + 1], q4.y, sq[1]);
        sq[2] = fmaf(S[4 * i + 2], q4.z, sq[2]); sq[3] = fmaf(S[4 * i + 3], q4.w, sq[3]);
        kq[0] = fmaf(k4[i].x, q4.x, kq[0]); kq[1] = fmaf(k4[i].y, q4.y, kq[1]);
        kq[2] = fmaf(k4[i].z, q4.z, kq[2]); kq[3] = fmaf(k4[i].w, q4.w, kq[3]);
      }
      float a = (sk[0] + sk[1]) + (sk[2] + sk[3]), b = (sq[0] + sq[1]) + (sq[2] + sq[3]);
      float c = (kq[0] + kq[1]) + (kq[2] + kq[3]);
#pragma unroll
      for (int o = 1; o < L; o <<= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
        c += __shfl_xor_sync(0xffffffffu, c, o);
      }
      const float u = beta * (vj - decay * a);
#pragma unroll
      for (int i = 0; i < DR_ROWS / 4; i++) {
        S[4 * i] = fmaf(k4[i].x, u, decay * S[4 * i]);
        S[4 * i + 1] = fmaf(k4[i].y, u, decay * S[4 * i + 1]);
        S[4 * i + 2] = fmaf(k4[i].z, u, decay * S[4 * i + 2]);
        S[4 * i + 3] = fmaf(k4[i].w, u, decay * S[4 * i + 3]);
      }
      if (part == 0 && live) P.o_raw[(size_t)(c0 + tok) * P.n_heads * V + (size_t)h * V + j] = fmaf(c, u, decay * b);
    }
  }
  if (P.write_state && live) {
#pragma unroll
    for (int i = 0; i < DR_ROWS; i += 4) {
      const int d = part * DR_ROWS + i;
      if (vec && d + 3 < D) {
        *reinterpret_cast<float4*>(Sg + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
      } else {
#pragma unroll
        for (int u = 0; u < 4; u++)
          if (d + u < D) Sg[i + u] = S[i + u];
      }
    }
  }
}

// ---------------------------------------------------------------- finish: one warp per (token, head)
template <typename T>
__global__ void __launch_bounds__(128) delta_finish_kernel(const DeltaRule P) {
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long long)P.n_tokens * P.n_heads) return;
  const int t = (int)(item / P.n_heads), h = (int)(item - (long long)t * P.n_heads);
  const int V = P.vdim, C = 2 * P.n_kv * P.dim + P.n_heads * V;
  const float* o = P.o_raw + (size_t)t * P.n_heads * V + (size_t)h * V;
  const float* g = P.proj + (size_t)t * P.ld + C + 2 * P.n_heads + (size_t)h * V;
  float ss = 0.f;
  for (int d = lane; d < V; d += 32) ss = fmaf(o[d], o[d], ss);
  ss = warp_sum(ss);
  const float mul = 1.0f / sqrtf(ss / (float)V + P.eps);
  T* out = (T*)P.out + (size_t)t * P.ldo + (size_t)h * V;
  for (int d = lane; d < V; d += 32) out[d] = from_float<T>(o[d] * mul * P.gain[d] * silu_f(g[d]));
}

static int delta_check(const DeltaRule& P) {
  if (P.n_heads < 1 || P.n_kv < 1 || P.n_heads % P.n_kv != 0 || P.dim < 1 || P.vdim < 1 || P.taps < 1)
    return STRATUM_ERR_SHAPE;
  const int C = 2 * P.n_kv * P.dim + P.n_heads * P.vdim;
  if (P.ld < C + 2 * P.n_heads + P.n_heads * P.vdim || P.lda < C + 2 * P.n_heads) return STRATUM_ERR_SHAPE;
  if (P.state_stride < P.n_heads * P.dim * P.vdim + (P.taps - 1) * C) return STRATUM_ERR_SHAPE;
  if (P.n_heads > DR_PREP_THREADS || P.dim > 32 * 16) return STRATUM_ERR_LIMIT;
  return 0;
}

// Everything of a step: prep, recurrence, finish (three launches).  out_dtype: the compute dtype of `out`.
STRATUM_EXPORT int stratum_delta_rule(const DeltaRule* params, int out_dtype, cudaStream_t stream) {
  const DeltaRule& P = *params;
  if (P.n_tokens <= 0 || P.n_seqs <= 0) return 0;
  const int bad = delta_check(P);
  if (bad) return bad;
  const int C = 2 * P.n_kv * P.dim + P.n_heads * P.vdim;
  const size_t smem = (size_t)C * sizeof(float);
  if (smem > 200 * 1024) return STRATUM_ERR_LIMIT;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  delta_prep_kernel<<<P.n_tokens, DR_PREP_THREADS, smem, stream>>>(P);
  int st = launch_status();
  if (st) return st;
  int L = 1;
  while (DR_ROWS * L < P.dim) L <<= 1;
  const int cols = DR_THREADS / L;
  if (P.n_heads > 65535 || P.n_seqs > 65535) return STRATUM_ERR_LIMIT;
  const dim3 grid((P.vdim + cols - 1) / cols, P.n_heads, P.n_seqs);
  switch (L) {
    case 1: delta_recur_kernel<1><<<grid, DR_THREADS, 0, stream>>>(P); break;
    case 2: delta_recur_kernel<2><<<grid, DR_THREADS, 0, stream>>>(P); break;
    case 4: delta_recur_kernel<4><<<grid, DR_THREADS, 0, stream>>>(P); break;
    case 8: delta_recur_kernel<8><<<grid, DR_THREADS, 0, stream>>>(P); break;
    case 16: delta_recur_kernel<16><<<grid, DR_THREADS, 0, stream>>>(P); break;
    default: delta_recur_kernel<32><<<grid, DR_THREADS, 0, stream>>>(P); break;
  }
  st = launch_status();
  if (st) return st;
  const long long items = (long long)P.n_tokens * P.n_heads;
  const long long blocks = (items + 3) / 4;
  if (blocks > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  if (out_dtype == STRATUM_DT_F32) delta_finish_kernel<float><<<(unsigned)blocks, 128, 0, stream>>>(P);
  else if (out_dtype == STRATUM_DT_BF16) delta_finish_kernel<bf16><<<(unsigned)blocks, 128, 0, stream>>>(P);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}
