// Routing of a mixture of experts, in float32, and the weighting of the experts' activations.
//
// route: per token, z = W_r h (h in the compute dtype, W_r and the sums float32); s = sigmoid(z); the choice score of
//   expert e is c_e = s_e + correction_e.  The experts form `n_groups` equal groups of neighbours; a group's score is
//   the sum of its two largest c (of its only c when a group is one expert); only the `keep` best groups stay (the
//   others' c count as -inf).  The `top` experts with the largest c are chosen (among equals the lowest index), and
//   their weights are s_e / (sum of the chosen s + 1e-20) * scale.  Written: the chosen experts and their weights
//   [tokens][top], and the same as a row of n_experts weights with zeros for the others.
//   One warp per token; a sum's order depends on the row's length alone.
// scale_column_blocks: a[t][e * block + j] *= w[t][e] for e < n_blocks (columns beyond n_blocks * block are left
//   alone): the activations of every expert, side by side in one row, times the token's weight for that expert, so
//   that one product with the experts' stacked down matrices sums the weighted expert outputs.
#include <math.h>

#include "common.cuh"

struct MoeRoute {
  const void* x;            // [tokens][ldx]
  const float* w_router;    // [n_experts][width]
  const float* correction;  // [n_experts]
  float* dense;             // [tokens][ldd] weights, zeros for experts not chosen
  int* chosen;              // [tokens][top]
  float* weights;           // [tokens][top]
  int ldx, ldd, n_tokens, width;
  int n_experts, top, n_groups, keep;
  float scale, reserved;
};

#define MR_WARPS 4

template <typename T>
__global__ void __launch_bounds__(MR_WARPS * 32) moe_route_kernel(const MoeRoute P) {
  extern __shared__ float mr_s[];                    // per warp: s [E], c [E], group score [n_groups]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * MR_WARPS + warp;
  if (t >= P.n_tokens) return;
  const int E = P.n_experts, G = P.n_groups, per = E / G;
  float* s = mr_s + (size_t)warp * (2 * E + G);
  float* c = s + E;
  float* gs = c + E;
  const T* x = (const T*)P.x + (size_t)t * P.ldx;
  for (int e = 0; e < E; e++) {
    const float* w = P.w_router + (size_t)e * P.width;
    float acc = 0.f;
    for (int i = lane; i < P.width; i += 32) acc = fmaf(to_float(x[i]), w[i], acc);
    acc = warp_sum(acc);
    if (lane == 0) {
      const float sg = 1.0f / (1.0f + expf(-acc));
      s[e] = sg;
      c[e] = sg + P.correction[e];
    }
  }
  __syncwarp();
  // group scores, then all but the `keep` best groups are closed
  for (int g = lane; g < G; g += 32) {
    float a = -INFINITY, b = -INFINITY;              // the two largest
    for (int i = 0; i < per; i++) {
      const float v = c[g * per + i];
      if (v > a) { b = a; a = v; } else if (v > b) b = v;
    }
    gs[g] = per > 1 ? a + b : a;
  }
  __syncwarp();
  if (P.keep < G) {
    for (int g = lane; g < G; g += 32) {
      int better = 0;                                // groups ahead of g: a larger score, or the same and a lower index
      for (int o = 0; o < G; o++) better += (gs[o] > gs[g]) || (gs[o] == gs[g] && o < g);
      if (better >= P.keep)
        for (int i = 0; i < per; i++) c[g * per + i] = -INFINITY;
    }
    __syncwarp();
  }
  float* dense = P.dense + (size_t)t * P.ldd;
  for (int e = lane; e < E; e += 32) dense[e] = 0.f;
  __syncwarp();
  float total = 0.f;
  for (int k = 0; k < P.top; k++) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (c[e] > best || (c[e] == best && e < at && c[e] != -INFINITY)) { best = c[e]; at = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = 0;                    // fewer open experts than `top` (refused by the host)
    total += s[at];
    if (lane == 0) {
      P.chosen[(size_t)t * P.top + k] = at;
      c[at] = -INFINITY;
    }
    __syncwarp();
  }
  const float mul = P.scale / (total + 1e-20f);
  for (int k = lane; k < P.top; k += 32) {
    const int e = P.chosen[(size_t)t * P.top + k];
    const float w = s[e] * mul;
    P.weights[(size_t)t * P.top + k] = w;
    dense[e] = w;
  }
}

STRATUM_EXPORT int stratum_moe_route(const MoeRoute* params, int dtype, cudaStream_t stream) {
  const MoeRoute& P = *params;
  if (P.n_tokens <= 0) return 0;
  if (P.n_experts < 1 || P.n_groups < 1 || P.n_experts % P.n_groups != 0 || P.keep < 1 || P.keep > P.n_groups ||
      P.top < 1 || P.top > (P.n_experts / P.n_groups) * P.keep || P.ldd < P.n_experts || P.ldx < P.width)
    return STRATUM_ERR_SHAPE;
  const size_t smem = (size_t)MR_WARPS * (2 * P.n_experts + P.n_groups) * sizeof(float);
  if (smem > 48 * 1024) return STRATUM_ERR_LIMIT;
  const int blocks = (P.n_tokens + MR_WARPS - 1) / MR_WARPS;
  if (dtype == STRATUM_DT_F32) moe_route_kernel<float><<<blocks, MR_WARPS * 32, smem, stream>>>(P);
  else if (dtype == STRATUM_DT_BF16) moe_route_kernel<bf16><<<blocks, MR_WARPS * 32, smem, stream>>>(P);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}

template <typename T>
__global__ void scale_column_blocks_kernel(T* a, int lda, const float* __restrict__ w, int ldw, int n_rows, int block,
                                           int n_blocks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cols = block * n_blocks;
  if (i >= (long long)n_rows * cols) return;
  const int r = (int)(i / cols), col = (int)(i - (long long)r * cols);
  T* p = a + (size_t)r * lda + col;
  *p = from_float<T>(to_float(*p) * w[(size_t)r * ldw + col / block]);
}

STRATUM_EXPORT int stratum_scale_column_blocks(void* a, int dtype, int lda, const float* w, int ldw, int n_rows,
                                               int block, int n_blocks, cudaStream_t stream) {
  if (n_rows <= 0 || n_blocks <= 0) return 0;
  if (block < 1 || lda < block * n_blocks || ldw < n_blocks) return STRATUM_ERR_SHAPE;
  const long long n = (long long)n_rows * block * n_blocks;
  const long long blocks = (n + 255) / 256;
  if (blocks > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  if (dtype == STRATUM_DT_F32)
    scale_column_blocks_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((float*)a, lda, w, ldw, n_rows, block, n_blocks);
  else if (dtype == STRATUM_DT_BF16)
    scale_column_blocks_kernel<bf16><<<(unsigned)blocks, 256, 0, stream>>>((bf16*)a, lda, w, ldw, n_rows, block, n_blocks);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}
