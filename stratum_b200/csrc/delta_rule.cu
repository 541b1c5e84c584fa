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
// a block owns (sequence, head, a tile of columns), a thread 4, 8 or 16 rows of one column, so a column's sums are
// split over neighbouring lanes and added by shuffles in a fixed order; the tokens' k, q, v, beta, decay and k . q
// come through a double buffer in shared memory that the next tokens fill (cp.async) while the current ones are
// worked on.  Nothing depends on how a sequence's tokens are cut into steps; the other sequences of a step decide
// at most how many rows a lane holds, that is, the order in which a column's sums are added.
#include <math.h>

#include "common.cuh"

struct DeltaRule {
  const float* proj;        // [tokens][ld]
  const float* conv_w;      // [channels][taps]
  const float* a_log;       // [n_heads]
  const float* dt_bias;     // [n_heads]
  const float* gain;        // [vdim]
  float* act;               // [tokens][lda]: q | k | v (after prep) | beta | decay [n_heads each] | k . q [n_kv]
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

// ---------------------------------------------------------------- prep: one block per (token, unit)
// Units: the n_kv pairs of a q head and its k head (convolution, silu, two unit norms, and the pair's k . q, which
// the recurrence needs once per token and not once per column), then the n_heads value heads (convolution, silu, and
// the head's beta and decay).
#define DR_PREP_THREADS 128
__device__ __forceinline__ float dr_conv(const DeltaRule& P, const float* tail, int t, int in_step, int pos, int C,
                                         int c) {
  const int n = P.taps;
  const float* w = P.conv_w + (size_t)c * n;
  float acc = 0.f;
  for (int i = n - 1; i >= 0; i--) {                 // oldest input first: one fixed order
    float x = 0.f;
    if (i <= in_step) x = ld_fresh(P.proj + (size_t)(t - i) * P.ld + c);
    else if (tail && pos - i >= 0) x = ld_fresh(tail + (size_t)(n - 1 - (i - in_step)) * C + c);
    acc = fmaf(w[n - 1 - i], x, acc);
  }
  return silu_f(acc);
}

__device__ __forceinline__ float dr_block_sum(float x, float* red) {         // every thread gets the sum
  x = warp_sum(x);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                                   // red may still be read from the call before
  if (lane == 0) red[warp] = x;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < DR_PREP_THREADS / 32; w++) total += red[w];
  return total;
}

__global__ void __launch_bounds__(DR_PREP_THREADS) delta_prep_kernel(const DeltaRule P) {
  extern __shared__ float dr_act[];                  // [2 * dim] for a q/k pair, [vdim] for a value head
  __shared__ float red[DR_PREP_THREADS / 32];
  pdl_trigger();
  pdl_wait();                // the projection and the state are the work of kernels before this one: ld_fresh
  const int t = blockIdx.x, unit = blockIdx.y;
  const int D = P.dim, V = P.vdim, nqk = P.n_kv * D, C = 2 * nqk + P.n_heads * V;
  const int seq = P.token_seq[t];
  const int pos = P.token_pos[t];
  int in_step = 0;                                   // tokens of this sequence that the step brought before this one
  const float* tail = nullptr;
  if (seq >= 0) {
    in_step = t - P.seq_start[seq];
    tail = P.state + (size_t)P.seq_slot[seq] * P.state_stride + (size_t)P.n_heads * D * V;
  }
  float* out = P.act + (size_t)t * P.lda;
  if (unit < P.n_kv) {
    const int cq = unit * D, ck = nqk + unit * D;
    float sq = 0.f, sk = 0.f;
    for (int d = threadIdx.x; d < D; d += DR_PREP_THREADS) {
      const float q = dr_conv(P, tail, t, in_step, pos, C, cq + d), k = dr_conv(P, tail, t, in_step, pos, C, ck + d);
      dr_act[d] = q; dr_act[D + d] = k;
      sq = fmaf(q, q, sq); sk = fmaf(k, k, sk);
    }
    sq = dr_block_sum(sq, red);
    sk = dr_block_sum(sk, red);
    const float mq = 1.0f / sqrtf(sq + 1e-6f) * (1.0f / sqrtf((float)D)), mk = 1.0f / sqrtf(sk + 1e-6f);
    float kq = 0.f;
    for (int d = threadIdx.x; d < D; d += DR_PREP_THREADS) {               // a thread reads what it wrote itself
      const float q = dr_act[d] * mq, k = dr_act[D + d] * mk;
      out[cq + d] = q; out[ck + d] = k;
      kq = fmaf(k, q, kq);
    }
    kq = dr_block_sum(kq, red);
    if (threadIdx.x == 0) out[C + 2 * P.n_heads + unit] = kq;
    return;
  }
  const int h = unit - P.n_kv, cv = 2 * nqk + h * V;
  for (int d = threadIdx.x; d < V; d += DR_PREP_THREADS) out[cv + d] = dr_conv(P, tail, t, in_step, pos, C, cv + d);
  if (threadIdx.x == 0) {
    const float* row = P.proj + (size_t)t * P.ld;
    out[C + h] = 1.0f / (1.0f + expf(-ld_fresh(row + C + h)));
    const float z = ld_fresh(row + C + P.n_heads + h) + P.dt_bias[h];
    const float sp = z > 20.f ? z : log1pf(expf(z));
    out[C + P.n_heads + h] = expf(-expf(P.a_log[h]) * sp);
  }
}

// ---------------------------------------------------------------- the recurrence
#define DR_THREADS 128
#define DR_ROWS 16            // rows of a column of S that a lane holds
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

// The state of a head lies in memory column by column (S^T: [vdim][dim]), so the ROWS rows a thread holds are
// contiguous and neighbouring lanes read neighbouring stretches.  A column is spread over L lanes of ROWS rows each
// (dim <= ROWS * L).  A token's step is one chain of dependent instructions (sums, shuffles, the update) that a
// warp issues at one instruction in two to four cycles; measured at dim = vdim = 128, 16 heads, one sequence of
// 2,048 tokens: 16 rows a lane 0.60 ms, 8 rows 0.72, 4 rows 0.77 (more warps, but two to three times the
// instructions), and four tokens at a time with their mutual dot products formed once per group 0.76: what counts
// is the number of instructions per token, which 16 rows a lane keep smallest.
template <int ROWS, int L>
__global__ void __launch_bounds__(DR_THREADS) delta_recur_kernel(const DeltaRule P) {
  constexpr int COLS = DR_THREADS / L;
  // floats between two lanes' stretches of k and q in shared memory: 16-byte aligned, and the float4 reads of eight
  // neighbouring lanes fall on different banks
  constexpr int PITCH = ROWS == 16 ? 20 : (ROWS == 8 ? 12 : ROWS);
  constexpr int KQ = L * PITCH;
  constexpr int FIT = 2048 / KQ;
  constexpr int CHUNK = FIT < 4 ? 4 : (FIT > DR_MAX_CHUNK ? DR_MAX_CHUNK : (FIT & ~3));   // a multiple of four
  __shared__ __align__(16) float kq_s[2][CHUNK][2][KQ];
  __shared__ float v_s[2][CHUNK][COLS];
  __shared__ float bg_s[2][CHUNK][4];                // beta, decay, k . q
  pdl_trigger();             // (launched the ordinary way itself: it starts when prep is done; its loads need no care)
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
  float* Sg = slot + ((size_t)h * V + (live ? j : 0)) * D + part * ROWS;
  const bool vec = D % 4 == 0 && (P.state_stride % 4) == 0 && (((uintptr_t)P.state) & 15) == 0;
  float2 S[ROWS / 2];        // pairs of rows: the sums and the update run on packed pairs of floats (fma.f32x2)
#pragma unroll
  for (int i = 0; i < ROWS; i += 4) {
    const int d = part * ROWS + i;
    if (live && vec && d + 3 < D) {
      const float4 v4 = *reinterpret_cast<const float4*>(Sg + i);
      S[i / 2] = make_float2(v4.x, v4.y); S[i / 2 + 1] = make_float2(v4.z, v4.w);
    } else {
      float e[4];
#pragma unroll
      for (int u = 0; u < 4; u++) e[u] = (live && d + u < D) ? Sg[i + u] : 0.f;
      S[i / 2] = make_float2(e[0], e[1]); S[i / 2 + 1] = make_float2(e[2], e[3]);
    }
  }
  if (D != ROWS * L) {       // the dimensions beyond dim in the staging buffers stay zero: nothing below writes them
    for (int i = threadIdx.x; i < 2 * CHUNK * 2 * KQ; i += DR_THREADS) (&kq_s[0][0][0][0])[i] = 0.f;
    __syncthreads();
  }

  const bool vec_act = D % 4 == 0 && P.lda % 4 == 0 && (((uintptr_t)P.act) & 15) == 0;
  auto stage = [&](int buf, int c0) {                // ask for the tokens c0 .. of this sequence
    const int n_here = min(CHUNK, r1 - c0);
    for (int tok = 0; tok < n_here; tok++) {
      const float* a = P.act + (size_t)(c0 + tok) * P.lda + (size_t)kv * D;
      if (vec_act) {
        for (int d = 4 * threadIdx.x; d < 2 * D; d += 4 * DR_THREADS) {          // k, then q
          const int which = d >= D, dd = d - which * D;
          dr_copy16(&kq_s[buf][tok][which][(dd / ROWS) * PITCH + dd % ROWS], a + (which ? 0 : nqk) + dd);
        }
      } else {
        for (int d = threadIdx.x; d < 2 * D; d += DR_THREADS) {
          const int which = d >= D, dd = d - which * D;
          dr_copy4(&kq_s[buf][tok][which][(dd / ROWS) * PITCH + dd % ROWS], a + (which ? 0 : nqk) + dd);
        }
      }
    }
    for (int i = threadIdx.x; i < n_here * COLS; i += DR_THREADS) {
      const int tok = i / COLS, cc = i - tok * COLS, jj = tile * COLS + cc;
      if (jj < V) dr_copy4(&v_s[buf][tok][cc], P.act + (size_t)(c0 + tok) * P.lda + 2 * nqk + (size_t)h * V + jj);
    }
    if (threadIdx.x < n_here * 4) {
      const int tok = threadIdx.x >> 2, which = threadIdx.x & 3;                 // 0 = beta, 1 = decay, 2 = k . q
      const float* a = P.act + (size_t)(c0 + tok) * P.lda + C;
      if (which < 2) dr_copy4(&bg_s[buf][tok][which], a + which * P.n_heads + h);
      else if (which == 2) dr_copy4(&bg_s[buf][tok][2], a + 2 * P.n_heads + kv);
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
    float* o_row = P.o_raw + (size_t)c0 * P.n_heads * V + (size_t)h * V + (live ? j : 0);
#pragma unroll 2
    for (int tok = 0; tok < n_here; tok++, o_row += (size_t)P.n_heads * V) {
      const float4* kk = reinterpret_cast<const float4*>(&kq_s[buf][tok][0][part * PITCH]);
      const float4* qq = reinterpret_cast<const float4*>(&kq_s[buf][tok][1][part * PITCH]);
      const float beta = bg_s[buf][tok][0], decay = bg_s[buf][tok][1], kq = bg_s[buf][tok][2];
      const float vj = v_s[buf][tok][col];
      float2 k2[ROWS / 2];
      float2 sk0 = make_float2(0.f, 0.f), sk1 = sk0, sq0 = sk0, sq1 = sk0;
#pragma unroll
      for (int i = 0; i < ROWS / 4; i++) {
        const float4 k4 = kk[i], q4 = qq[i];
        k2[2 * i] = make_float2(k4.x, k4.y); k2[2 * i + 1] = make_float2(k4.z, k4.w);
        sk0 = __ffma2_rn(S[2 * i], k2[2 * i], sk0); sk1 = __ffma2_rn(S[2 * i + 1], k2[2 * i + 1], sk1);
        sq0 = __ffma2_rn(S[2 * i], make_float2(q4.x, q4.y), sq0);
        sq1 = __ffma2_rn(S[2 * i + 1], make_float2(q4.z, q4.w), sq1);
      }
      const float2 sk = __fadd2_rn(sk0, sk1), sq = __fadd2_rn(sq0, sq1);
      float a = sk.x + sk.y, b = sq.x + sq.y;
#pragma unroll
      for (int o = 1; o < L; o <<= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
      }
      const float u = beta * (vj - decay * a);
      const float2 uu = make_float2(u, u), dd = make_float2(decay, decay);
#pragma unroll
      for (int i = 0; i < ROWS / 2; i++) S[i] = __ffma2_rn(k2[i], uu, __fmul2_rn(dd, S[i]));
      if (part == 0 && live) *o_row = fmaf(kq, u, decay * b);
    }
  }
  if (P.write_state && live) {
#pragma unroll
    for (int i = 0; i < ROWS; i += 4) {
      const int d = part * ROWS + i;
      const float e[4] = {S[i / 2].x, S[i / 2].y, S[i / 2 + 1].x, S[i / 2 + 1].y};
      if (vec && d + 3 < D) {
        *reinterpret_cast<float4*>(Sg + i) = make_float4(e[0], e[1], e[2], e[3]);
      } else {
#pragma unroll
        for (int u = 0; u < 4; u++)
          if (d + u < D) Sg[i + u] = e[u];
      }
    }
  }
}

// ---------------------------------------------------------------- finish: one warp per (token, head)
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16* p, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<const uint32_t*>(&lo); v.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = v;
}
template <typename T>
__global__ void __launch_bounds__(128) delta_finish_kernel(const DeltaRule P) {
  const int lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();                // o_raw and the projection are the work of kernels before this one: ld_fresh
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long long)P.n_tokens * P.n_heads) return;
  const int t = (int)(item / P.n_heads), h = (int)(item - (long long)t * P.n_heads);
  const int V = P.vdim, C = 2 * P.n_kv * P.dim + P.n_heads * V;
  const float* o = P.o_raw + (size_t)t * P.n_heads * V + (size_t)h * V;
  const float* g = P.proj + (size_t)t * P.ld + C + 2 * P.n_heads + (size_t)h * V;
  T* out = (T*)P.out + (size_t)t * P.ldo + (size_t)h * V;
  const bool vec = V % 4 == 0 && P.ld % 4 == 0 && (C + 2 * P.n_heads) % 4 == 0 && P.ldo % 4 == 0 &&
                   ((((uintptr_t)P.o_raw) | ((uintptr_t)P.proj) | ((uintptr_t)P.gain)) & 15) == 0 &&
                   (((uintptr_t)P.out) & (4 * sizeof(T) - 1)) == 0;
  float ss = 0.f;
  if (vec) {
    for (int d = 4 * lane; d < V; d += 128) {
      const float4 x = ld_fresh(reinterpret_cast<const float4*>(o + d));
      ss = fmaf(x.x, x.x, ss); ss = fmaf(x.y, x.y, ss); ss = fmaf(x.z, x.z, ss); ss = fmaf(x.w, x.w, ss);
    }
  } else {
    for (int d = lane; d < V; d += 32) {
      const float x = ld_fresh(o + d);
      ss = fmaf(x, x, ss);
    }
  }
  ss = warp_sum(ss);
  const float mul = 1.0f / sqrtf(ss / (float)V + P.eps);
  if (vec) {
    for (int d = 4 * lane; d < V; d += 128) {
      const float4 x = ld_fresh(reinterpret_cast<const float4*>(o + d));
      const float4 gg = ld_fresh(reinterpret_cast<const float4*>(g + d));
      const float4 w = *reinterpret_cast<const float4*>(P.gain + d);
      store4(out + d, x.x * mul * w.x * silu_f(gg.x), x.y * mul * w.y * silu_f(gg.y), x.z * mul * w.z * silu_f(gg.z),
             x.w * mul * w.w * silu_f(gg.w));
    }
  } else {
    for (int d = lane; d < V; d += 32)
      out[d] = from_float<T>(ld_fresh(o + d) * mul * P.gain[d] * silu_f(ld_fresh(g + d)));
  }
}

static int delta_check(const DeltaRule& P) {
  if (P.n_heads < 1 || P.n_kv < 1 || P.n_heads % P.n_kv != 0 || P.dim < 1 || P.vdim < 1 || P.taps < 1)
    return STRATUM_ERR_SHAPE;
  const int C = 2 * P.n_kv * P.dim + P.n_heads * P.vdim;
  if (P.ld < C + 2 * P.n_heads + P.n_heads * P.vdim || P.lda < C + 2 * P.n_heads + P.n_kv) return STRATUM_ERR_SHAPE;
  if (P.state_stride < P.n_heads * P.dim * P.vdim + (P.taps - 1) * C) return STRATUM_ERR_SHAPE;
  if (P.dim > 32 * DR_ROWS) return STRATUM_ERR_LIMIT;
  if (P.n_heads > 65535 || P.n_heads + P.n_kv > 65535 || P.n_seqs > 65535) return STRATUM_ERR_LIMIT;
  return 0;
}

static int lanes_for(int rows, int dim) {
  int L = 1;
  while (rows * L < dim) L <<= 1;
  return L;
}

template <int L>
static void recur_launch(const DeltaRule& P, cudaStream_t stream) {
  const int cols = DR_THREADS / L;
  const dim3 grid((P.vdim + cols - 1) / cols, P.n_heads, P.n_seqs);
  delta_recur_kernel<DR_ROWS, L><<<grid, DR_THREADS, 0, stream>>>(P);
}

// Everything of a step: prep, recurrence, finish (three launches).  out_dtype: the compute dtype of `out`.
STRATUM_EXPORT int stratum_delta_rule(const DeltaRule* params, int out_dtype, cudaStream_t stream) {
  const DeltaRule& P = *params;
  if (P.n_tokens <= 0 || P.n_seqs <= 0) return 0;
  const int bad = delta_check(P);
  if (bad) return bad;
  const dim3 prep_grid(P.n_tokens, P.n_kv + P.n_heads);
  launch_pdl(delta_prep_kernel, prep_grid, DR_PREP_THREADS, 2 * (size_t)P.dim * sizeof(float), stream, P);
  int st = launch_status();
  if (st) return st;
  switch (lanes_for(DR_ROWS, P.dim)) {
    case 1: recur_launch<1>(P, stream); break;
    case 2: recur_launch<2>(P, stream); break;
    case 4: recur_launch<4>(P, stream); break;
    case 8: recur_launch<8>(P, stream); break;
    case 16: recur_launch<16>(P, stream); break;
    default: recur_launch<32>(P, stream); break;
  }
  st = launch_status();
  if (st) return st;
  const long long items = (long long)P.n_tokens * P.n_heads;
  const long long blocks = (items + 3) / 4;
  if (blocks > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  if (out_dtype == STRATUM_DT_F32) launch_pdl(delta_finish_kernel<float>, (unsigned)blocks, 128, 0, stream, P);
  else if (out_dtype == STRATUM_DT_BF16) launch_pdl(delta_finish_kernel<bf16>, (unsigned)blocks, 128, 0, stream, P);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}
