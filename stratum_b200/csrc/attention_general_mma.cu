// The general attention (attention_general.cu) in bfloat16 on tensor cores, for prompts and for decode steps.
//
// A CTA of four warps owns one work item: up to 16 query rows that share their keys (consecutive new tokens of a
// sequence x the heads of one key/value group, for one score map) and one contiguous range of that sequence's
// keys.  Keys are visited in tiles of 64 (one page).  Per tile:
//   scores   warp w computes the 16 x 16 block of rows x keys 16w..16w+15: mma.sync.m16n8k16 over the key
//            dimension, Q fragments from shared memory, K fragments straight from the cache rows (a dot product
//            may visit the dimension in any order as long as Q and K agree: lane t of a row takes the 8
//            contiguous values 8t..8t+7 of every 32, as attention_mma.cu does);
//   softmax  scale, query factor, tanh cap and mask in float32; the row maximum of the tile goes through shared
//            memory; every warp rescales by the same running maximum and keeps the sum of its own keys;
//   values   the probabilities are float32; the tensor core takes bfloat16, so each is split into a high and a low
//            bfloat16 part (p = hi + lo to 16 bits of mantissa) that go through shared memory, and warp w adds
//            hi V + lo V for the chunks of 32 value dimensions c = w, w + 4, ...  (V fragments straight from the
//            cache rows, transposed by movmatrix as in attention_mma.cu).
// With one key range and one map the normalised result is written directly.  Otherwise every item leaves its
// unnormalised value sum, its maximum and its denominator in scratch, and the finishing kernel merges the
// ranges in order and combines the maps (see attention_general.cu for the formulas).
#include <math.h>

#include "attention_general.h"
#include "common.cuh"
#include "mma_common.cuh"

#define GM_WARPS 4
#define GM_TILE 64
#define GM_PSTRIDE 72          // bf16 per row of the probability tiles: 64 keys + 8 of padding (no bank conflicts)

__device__ __forceinline__ uint4 gm_ldg16(const void* p) { return ld_fresh((const uint4*)p); }

__host__ __device__ __forceinline__ int gm_q_stride(int D) {       // bytes per row of Q in shared memory: = 64 mod 128
  int s = ((D * 2 + 15) / 16) * 16;
  while (s % 128 != 64) s += 16;
  return s;
}

template <int CPW>
__global__ void __launch_bounds__(GM_WARPS * 32)
attention_general_mma_kernel(const GeneralAttention P) {
  extern __shared__ __align__(16) unsigned char gm_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int D = P.qk_dim, Dv = P.v_dim;
  const int qstride = gm_q_stride(D);
  unsigned char* q_s = gm_smem;                                                  // [16][qstride bytes]
  bf16* p_hi = reinterpret_cast<bf16*>(gm_smem + 16 * qstride);                  // [16][GM_PSTRIDE]
  bf16* p_lo = p_hi + 16 * GM_PSTRIDE;
  float* max_s = reinterpret_cast<float*>(p_lo + 16 * GM_PSTRIDE);               // [GM_WARPS][16]
  float* sum_s = max_s + GM_WARPS * 16;                                          // [GM_WARPS][16]

  const int rows_per_token = P.group < 16 ? P.group : 16;
  const int head_groups = (P.group + 15) / 16;
  const int n_kv = P.n_heads / P.group;
  int item = blockIdx.x;
  const int split = item % P.n_splits; item /= P.n_splits;
  const int map = item % P.maps; item /= P.maps;
  const int hg = item % head_groups; item /= head_groups;
  const int kv = item % n_kv; item /= n_kv;
  const int qb = item;
  const int seq = P.qb_seq ? P.qb_seq[qb] : P.token_seq[qb];
  if (seq < 0) return;                                                           // padding
  const int tok0 = P.qb_tok0 ? P.qb_tok0[qb] : qb;
  const int ntok = P.qb_ntok ? P.qb_ntok[qb] : 1;

  // the two rows of this lane: r = g and g + 8;  row -> (token of the block, head of the group)
  int row_tok[2], row_head[2], row_pos[2];
  bool row_ok[2];
  float row_factor[2];
#pragma unroll
  for (int e = 0; e < 2; e++) {
    const int r = g + 8 * e;
    const int tr = r / rows_per_token, hr = r % rows_per_token;
    const int hq = hg * 16 + hr;
    row_ok[e] = tr < ntok && tr < P.tokens_per_block && hq < P.group;
    row_tok[e] = tok0 + (row_ok[e] ? tr : 0);
    row_head[e] = kv * P.group + (row_ok[e] ? hq : 0);
    row_pos[e] = P.token_pos[row_tok[e]];
    float temp = 1.f;
    if (P.temp_coef != 0.f) temp = 1.f + P.temp_coef * logf((float)((row_pos[e] + 1) / P.temp_every) + 1.f);
    row_factor[e] = P.scale * temp;
  }
  const int first_pos = P.token_pos[tok0];
  const int last_pos = first_pos + ntok - 1;
  const int lo_block = (P.window > 0 && first_pos - P.window + 1 > 0) ? first_pos - P.window + 1 : 0;
  int k_begin = split * P.chunk;
  const int k_end = min((split + 1) * P.chunk, last_pos + 1);
  if (k_begin < (lo_block / GM_TILE) * GM_TILE) k_begin = (lo_block / GM_TILE) * GM_TILE;
  const int* bt = P.block_table + (size_t)seq * P.bt_stride;

  // Q rows of this item into shared memory (16 bytes per thread and turn; rows that do not exist are zero)
  {
    const int pieces = D / 8;
    for (int i = threadIdx.x; i < 16 * pieces; i += blockDim.x) {
      const int r = i / pieces, c = i - r * pieces;
      const int tr = r / rows_per_token, hr = r % rows_per_token;
      const int hq = hg * 16 + hr;
      const bool ok = tr < ntok && tr < P.tokens_per_block && hq < P.group;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (ok)
        v = gm_ldg16((const bf16*)P.q + (size_t)(tok0 + tr) * P.ldq +
                     ((size_t)(kv * P.group + hq) * P.maps + map) * D + 8 * c);
      *reinterpret_cast<uint4*>(q_s + (size_t)r * qstride + 16 * c) = v;
    }
  }
  __syncthreads();

  const size_t k_page = (size_t)P.n_k_heads * P.page_tokens * D;
  const size_t k_head = (size_t)(kv * P.maps + map) * P.page_tokens * D;
  const bf16* v_base = P.v_in_k ? (const bf16*)P.k_cache : (const bf16*)P.v_cache;
  const int v_row = P.v_in_k ? D : Dv;
  const size_t v_page = P.v_in_k ? k_page : (size_t)P.n_v_heads * P.page_tokens * Dv;
  const size_t v_head = P.v_in_k ? (size_t)(kv * P.maps) * P.page_tokens * D : (size_t)kv * P.page_tokens * Dv;
  const int n_kc = (D + 31) / 32;                 // chunks of the key dimension
  const int n_vc = (Dv + 31) / 32;                // chunks of the value dimension

  float o[CPW * 4][4];
#pragma unroll
  for (int i = 0; i < CPW * 4; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const uint4 zero4 = make_uint4(0, 0, 0, 0);

  for (int key0 = (k_begin / GM_TILE) * GM_TILE; key0 < k_end; key0 += GM_TILE) {
    const int page = bt[key0 / P.page_tokens];
    const int in_page = key0 % P.page_tokens;
    // ---- scores of keys key0 + 16 warp + [0, 16)
    const int kw = key0 + 16 * warp;
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; i++) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
    const bool any = kw < k_end && kw + 15 >= k_begin;
    if (any) {
      const bf16* kr = (const bf16*)P.k_cache + (size_t)page * k_page + k_head + (size_t)(in_page + 16 * warp) * D;
#pragma unroll 4
      for (int c = 0; c < n_kc; c++) {
        const int d = 32 * c + 8 * t;
        const bool d_ok = d < D;
        const uint4 ka = d_ok ? gm_ldg16(kr + (size_t)g * D + d) : zero4;
        const uint4 kb = d_ok ? gm_ldg16(kr + (size_t)(g + 8) * D + d) : zero4;
        const uint4 qa = d_ok ? *reinterpret_cast<const uint4*>(q_s + (size_t)g * qstride + 2 * d) : zero4;
        const uint4 qc = d_ok ? *reinterpret_cast<const uint4*>(q_s + (size_t)(g + 8) * qstride + 2 * d) : zero4;
        mma16816(s[0], qa.x, qc.x, qa.y, qc.y, ka.x, ka.y);
        mma16816(s[0], qa.z, qc.z, qa.w, qc.w, ka.z, ka.w);
        mma16816(s[1], qa.x, qc.x, qa.y, qc.y, kb.x, kb.y);
        mma16816(s[1], qa.z, qc.z, qa.w, qc.w, kb.z, kb.w);
      }
    }
    float bm[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 2; i++) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int e = j >> 1;
        const int key = kw + 8 * i + 2 * t + (j & 1);
        const int lo = (P.window > 0 && row_pos[e] - P.window + 1 > 0) ? row_pos[e] - P.window + 1 : 0;
        const bool ok = any && row_ok[e] && key <= row_pos[e] && key >= lo && key < k_end && key >= k_begin;
        float v = s[i][j] * row_factor[e];
        if (P.softcap > 0.f) v = P.softcap * tanhf(v / P.softcap);
        s[i][j] = ok ? v : -INFINITY;
        bm[e] = fmaxf(bm[e], s[i][j]);
      }
    }
#pragma unroll
    for (int e = 0; e < 2; e++) {
      bm[e] = fmaxf(bm[e], __shfl_xor_sync(0xffffffffu, bm[e], 1));
      bm[e] = fmaxf(bm[e], __shfl_xor_sync(0xffffffffu, bm[e], 2));
      if (t == 0) max_s[warp * 16 + g + 8 * e] = bm[e];
    }
    __syncthreads();
    float corr[2], m_use[2];
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const int r = g + 8 * e;
      const float tile_max = fmaxf(fmaxf(max_s[r], max_s[16 + r]), fmaxf(max_s[32 + r], max_s[48 + r]));
      const float m_new = fmaxf(m_run[e], tile_max);
      m_use[e] = (m_new == -INFINITY) ? 0.f : m_new;      // a row with no key yet: exponents of -inf give 0
      corr[e] = expf(m_run[e] - m_use[e]);                // first keys: exp(-inf) = 0
      m_run[e] = m_new;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; i++) {
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const float p0 = expf(s[i][2 * e] - m_use[e]), p1 = expf(s[i][2 * e + 1] - m_use[e]);
        psum[e] += p0 + p1;
        const __nv_bfloat162 hi = __floats2bfloat162_rn(p0, p1);
        const __nv_bfloat162 lo = __floats2bfloat162_rn(p0 - __bfloat162float(hi.x), p1 - __bfloat162float(hi.y));
        const int at = (g + 8 * e) * GM_PSTRIDE + 16 * warp + 8 * i + 2 * t;
        *reinterpret_cast<__nv_bfloat162*>(p_hi + at) = hi;
        *reinterpret_cast<__nv_bfloat162*>(p_lo + at) = lo;
      }
    }
#pragma unroll
    for (int e = 0; e < 2; e++) l_run[e] = l_run[e] * corr[e] + psum[e];
    __syncthreads();
    // ---- values: chunks of 32 dimensions c = warp, warp + 4, ...
#pragma unroll
    for (int i = 0; i < CPW * 4; i++) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    const bf16* vr = v_base + (size_t)page * v_page + v_head + (size_t)in_page * v_row;
    const int blocks = min(GM_TILE, k_end - key0 + 15) / 16;          // blocks of 16 keys that hold a key
#pragma unroll
    for (int cc = 0; cc < CPW; cc++) {
      const int c = warp + GM_WARPS * cc;
      const int d = 32 * c + 8 * t;
      if (c >= n_vc) break;
      for (int kb = 0; kb < blocks; kb++) {
        const uint4 va = d < Dv ? gm_ldg16(vr + (size_t)(16 * kb + g) * v_row + d) : zero4;
        const uint4 vb = d < Dv ? gm_ldg16(vr + (size_t)(16 * kb + 8 + g) * v_row + d) : zero4;
        const int a_at = g * GM_PSTRIDE + 16 * kb + 2 * t;
        const uint32_t h0 = *reinterpret_cast<const uint32_t*>(p_hi + a_at);
        const uint32_t h1 = *reinterpret_cast<const uint32_t*>(p_hi + a_at + 8 * GM_PSTRIDE);
        const uint32_t h2 = *reinterpret_cast<const uint32_t*>(p_hi + a_at + 8);
        const uint32_t h3 = *reinterpret_cast<const uint32_t*>(p_hi + a_at + 8 * GM_PSTRIDE + 8);
        const uint32_t l0 = *reinterpret_cast<const uint32_t*>(p_lo + a_at);
        const uint32_t l1 = *reinterpret_cast<const uint32_t*>(p_lo + a_at + 8 * GM_PSTRIDE);
        const uint32_t l2 = *reinterpret_cast<const uint32_t*>(p_lo + a_at + 8);
        const uint32_t l3 = *reinterpret_cast<const uint32_t*>(p_lo + a_at + 8 * GM_PSTRIDE + 8);
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const uint32_t b0 = transpose8x8(reg_of(va, i));
          const uint32_t b1 = transpose8x8(reg_of(vb, i));
          mma16816(o[4 * cc + i], h0, h1, h2, h3, b0, b1);
          mma16816(o[4 * cc + i], l0, l1, l2, l3, b0, b1);
        }
      }
    }
    __syncthreads();                               // the tiles of probabilities and the maxima are written again
  }

  // denominators: across the four lanes of a row, then across the warps
#pragma unroll
  for (int e = 0; e < 2; e++) {
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 1);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 2);
    if (t == 0) sum_s[warp * 16 + g + 8 * e] = l_run[e];
  }
  __syncthreads();
#pragma unroll
  for (int e = 0; e < 2; e++) {
    const int r = g + 8 * e;
    l_run[e] = (sum_s[r] + sum_s[16 + r]) + (sum_s[32 + r] + sum_s[48 + r]);
  }
  const bool direct = P.n_splits == 1 && P.combine == 0;
#pragma unroll
  for (int e = 0; e < 2; e++) {
    if (!row_ok[e]) continue;
    if (direct) {
      const float inv = 1.0f / l_run[e];
      bf16* op = (bf16*)P.out + (size_t)row_tok[e] * P.ldo + (size_t)row_head[e] * Dv;
#pragma unroll
      for (int cc = 0; cc < CPW; cc++) {
        const int d = 32 * (warp + GM_WARPS * cc) + 8 * t;
        if (d >= Dv) continue;
        uint4 v;
        v.x = pack_bf16(o[4 * cc + 0][2 * e] * inv, o[4 * cc + 0][2 * e + 1] * inv);
        v.y = pack_bf16(o[4 * cc + 1][2 * e] * inv, o[4 * cc + 1][2 * e + 1] * inv);
        v.z = pack_bf16(o[4 * cc + 2][2 * e] * inv, o[4 * cc + 2][2 * e + 1] * inv);
        v.w = pack_bf16(o[4 * cc + 3][2 * e] * inv, o[4 * cc + 3][2 * e + 1] * inv);
        *reinterpret_cast<uint4*>(op + d) = v;
      }
    } else {
      const size_t slot = (((size_t)row_tok[e] * P.n_heads + row_head[e]) * P.maps + map) * P.n_splits + split;
      float* po = P.part_o + slot * Dv;
#pragma unroll
      for (int cc = 0; cc < CPW; cc++) {
        const int d = 32 * (warp + GM_WARPS * cc) + 8 * t;
        if (d >= Dv) continue;
        *reinterpret_cast<float4*>(po + d) = make_float4(o[4 * cc + 0][2 * e], o[4 * cc + 0][2 * e + 1],
                                                         o[4 * cc + 1][2 * e], o[4 * cc + 1][2 * e + 1]);
        *reinterpret_cast<float4*>(po + d + 4) = make_float4(o[4 * cc + 2][2 * e], o[4 * cc + 2][2 * e + 1],
                                                             o[4 * cc + 3][2 * e], o[4 * cc + 3][2 * e + 1]);
      }
      if (warp == 0 && t == 0) {
        P.part_ml[slot * 2] = m_run[e];
        P.part_ml[slot * 2 + 1] = l_run[e];
      }
    }
  }
}

// Merge the key ranges of every (token, head, map) in range order, then combine the maps; one warp per
// (token, head).  A range that held no key of a row left maximum -inf and sum 0 and drops out.
template <int MAPS>
__global__ void __launch_bounds__(128) attention_general_finish_kernel(const GeneralAttention P) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + warp;
  if (item >= (long long)P.n_tokens * P.n_heads) return;
  const int tok = (int)(item / P.n_heads), h = (int)(item - (long long)tok * P.n_heads);
  if (P.token_seq[tok] < 0) return;
  const int Dv = P.v_dim;
  bf16* op = (bf16*)P.out + (size_t)tok * P.ldo + (size_t)h * Dv;
  float ss = 0.f;
  for (int d0 = 0; d0 < Dv; d0 += 32) {
    const int d = d0 + lane;
    float a[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      const size_t slot0 = ((size_t)item * MAPS + m) * P.n_splits;
      float mx = -INFINITY;
      for (int s = 0; s < P.n_splits; s++) mx = fmaxf(mx, P.part_ml[(slot0 + s) * 2]);
      float l = 0.f, acc = 0.f;
      for (int s = 0; s < P.n_splits; s++) {
        const float ms = P.part_ml[(slot0 + s) * 2];
        if (ms == -INFINITY) continue;
        const float w = expf(ms - mx);
        l += P.part_ml[(slot0 + s) * 2 + 1] * w;
        if (d < Dv) acc += P.part_o[(slot0 + s) * Dv + d] * w;
      }
      a[m] = acc / l;
    }
    if (MAPS == 1) {
      if (d < Dv) op[d] = __float2bfloat16_rn(a[0]);
    } else {
      const float o = d < Dv ? a[0] - P.lambda * a[MAPS - 1] : 0.f;
      ss = fmaf(o, o, ss);
      if (d < Dv) P.part_o[(size_t)item * MAPS * P.n_splits * Dv + d] = o;     // this row's own scratch, read below
    }
  }
  if (MAPS == 1) return;
  ss = warp_sum(ss);
  float mul = P.out_scale / sqrtf(ss / (float)Dv + P.eps);
  if (P.gate_col >= 0) {
    const float z = ld_fresh((const bf16*)P.q + (size_t)tok * P.ldq + P.gate_col + h);
    mul *= 1.0f / (1.0f + expf(-z));
  }
  __syncwarp();
  for (int d = lane; d < Dv; d += 32)
    op[d] = __float2bfloat16_rn(P.part_o[(size_t)item * MAPS * P.n_splits * Dv + d] * mul);
}

STRATUM_EXPORT long long stratum_attention_general_mma_smem(int qk_dim) {
  return 16LL * gm_q_stride(qk_dim) + 2LL * 16 * GM_PSTRIDE * sizeof(bf16) + 2LL * GM_WARPS * 16 * sizeof(float);
}

// q, the caches and out bfloat16.  Needs qk_dim % 8 == 0, v_dim % 8 == 0 (v_dim % 32 == 0 when results go through
// scratch is not needed: rows of scratch are v_dim floats and v_dim % 8 == 0 keeps them 16-byte aligned), rows of
// q and out 16-byte aligned, pages of 64 tokens.
STRATUM_EXPORT int stratum_attention_general_mma(const GeneralAttention* params, cudaStream_t stream) {
  const GeneralAttention& P = *params;
  if (P.n_tokens <= 0 || P.n_qblocks <= 0) return 0;
  const int bad = general_attention_check(P);
  if (bad) return bad;
  if (P.qk_dim % 8 != 0 || P.v_dim % 8 != 0 || P.ldq % 8 != 0 || P.ldo % 8 != 0 || P.page_tokens != GM_TILE)
    return STRATUM_ERR_SHAPE;
  if ((((uintptr_t)P.q | (uintptr_t)P.out | (uintptr_t)P.k_cache | (uintptr_t)P.v_cache) & 15) != 0)
    return STRATUM_ERR_ALIGN;
  if (P.n_splits < 1 || P.chunk < GM_TILE || P.chunk % GM_TILE != 0 || P.tokens_per_block < 1) return STRATUM_ERR_SHAPE;
  const bool direct = P.n_splits == 1 && P.combine == 0;
  if (!direct && (!P.part_o || !P.part_ml)) return STRATUM_ERR_SHAPE;
  const int n_vc = (P.v_dim + 31) / 32;
  const int cpw = (n_vc + GM_WARPS - 1) / GM_WARPS;
  const size_t smem = (size_t)stratum_attention_general_mma_smem(P.qk_dim);
  if (smem > 200 * 1024) return STRATUM_ERR_LIMIT;
  const int head_groups = (P.group + 15) / 16;
  const long long items = (long long)P.n_qblocks * (P.n_heads / P.group) * head_groups * P.maps * P.n_splits;
  if (items > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  void (*kern)(const GeneralAttention) = nullptr;
  if (cpw <= 1) kern = attention_general_mma_kernel<1>;
  else if (cpw <= 2) kern = attention_general_mma_kernel<2>;
  else if (cpw <= 4) kern = attention_general_mma_kernel<4>;
  else return STRATUM_ERR_LIMIT;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  kern<<<(unsigned)items, GM_WARPS * 32, smem, stream>>>(P);
  int st = launch_status();
  if (st || direct) return st;
  const long long rows = (long long)P.n_tokens * P.n_heads;
  if (P.maps == 1) attention_general_finish_kernel<1><<<(unsigned)((rows + 3) / 4), 128, 0, stream>>>(P);
  else attention_general_finish_kernel<2><<<(unsigned)((rows + 3) / 4), 128, 0, stream>>>(P);
  return launch_status();
}
