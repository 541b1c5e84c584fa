// One small matrix product per head, in one launch, in bfloat16 on tensor cores:
//   out[m][j * o_step + n] = sum_k x[m][j * x_step + k] * w[j][n][k]        (head j; w [heads][N][K])
// which is how a mixer carries per-head vectors from one space into another (queries into a latent space, mixed
// latents into value heads).  The matrices are small (tens to hundreds of rows and columns), so a launch per head
// would cost more than the work; here the heads are the grid's third dimension.
//
// A warp owns MT x 16 rows of x and 64 columns of one head: mma.sync.m16n8k16 with the rows of x as the A operand
// and 8 weight rows per B operand, both straight from global memory (lane t of a row takes the 8 contiguous values
// 8t..8t+7 of every 32 of k, for x and for w alike, so the products pair up as in the definition).  With few rows
// (decode steps) the four warps of a CTA take four column tiles and the kernel streams the weights once; with many
// (prompts) they take four row tiles and share the weight rows through L1.  float32 accumulation over k in order.
#include "common.cuh"
#include "mma_common.cuh"

#define HG_WARPS 4
#define HG_COLS 64

template <int MT>
__global__ void __launch_bounds__(HG_WARPS * 32)
head_gemm_kernel(const bf16* x, const bf16* __restrict__ w, bf16* out, int M, int N, int K, int ldx, int ldo,
                 int x_step, int o_step, int warps_split_columns) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int head = blockIdx.z;
  pdl_trigger();
  int row0, n0;
  if (warps_split_columns) {
    row0 = blockIdx.x * 16 * MT;
    n0 = (blockIdx.y * HG_WARPS + warp) * HG_COLS;
  } else {
    row0 = (blockIdx.x * HG_WARPS + warp) * 16 * MT;
    n0 = blockIdx.y * HG_COLS;
  }
  if (row0 >= M || n0 >= N) return;
  const bf16* xh = x + (size_t)head * x_step;
  const bf16* wh = w + (size_t)head * N * K;
  float acc[MT][8][4];
#pragma unroll
  for (int a = 0; a < MT; a++)
#pragma unroll
    for (int j = 0; j < 8; j++) { acc[a][j][0] = acc[a][j][1] = acc[a][j][2] = acc[a][j][3] = 0.f; }
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  pdl_wait();                                   // x comes from the kernel before this one
#pragma unroll 2
  for (int k0 = 0; k0 < K; k0 += 32) {
    const int k = k0 + 8 * t;
    const bool k_ok = k < K;
    uint4 xa[MT], xc[MT];
#pragma unroll
    for (int a = 0; a < MT; a++) {
      const int r = row0 + 16 * a + g;
      xa[a] = (k_ok && r < M) ? ld_fresh((const uint4*)(xh + (size_t)r * ldx + k)) : zero4;
      xc[a] = (k_ok && r + 8 < M) ? ld_fresh((const uint4*)(xh + (size_t)(r + 8) * ldx + k)) : zero4;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int n = n0 + 8 * j + g;
      const uint4 wb = (k_ok && n < N) ? __ldg((const uint4*)(wh + (size_t)n * K + k)) : zero4;
#pragma unroll
      for (int a = 0; a < MT; a++) {
        mma16816(acc[a][j], xa[a].x, xc[a].x, xa[a].y, xc[a].y, wb.x, wb.y);
        mma16816(acc[a][j], xa[a].z, xc[a].z, xa[a].w, xc[a].w, wb.z, wb.w);
      }
    }
  }
  bf16* oh = out + (size_t)head * o_step;
#pragma unroll
  for (int a = 0; a < MT; a++) {
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int n = n0 + 8 * j + 2 * t;
      if (n >= N) continue;                     // N % 8 == 0: a pair of columns is inside or outside together
      const int r = row0 + 16 * a + g;
      if (r < M) *reinterpret_cast<uint32_t*>(oh + (size_t)r * ldo + n) = pack_bf16(acc[a][j][0], acc[a][j][1]);
      if (r + 8 < M) *reinterpret_cast<uint32_t*>(oh + (size_t)(r + 8) * ldo + n) = pack_bf16(acc[a][j][2], acc[a][j][3]);
    }
  }
}

// x bf16 [M][ldx], w bf16 [heads][N][K], out bf16 [M][ldo].  Needs K % 8 == 0, N % 8 == 0, x_step % 8 == 0,
// ldx % 8 == 0, o_step and ldo even, x and w 16-byte aligned, out 4-byte aligned.
STRATUM_EXPORT int stratum_head_gemm(const void* x, const void* w, void* out, int heads, int M, int N, int K, int ldx,
                                     int ldo, int x_step, int o_step, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || heads <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || N % 8 != 0 || x_step % 8 != 0 || ldx % 8 != 0 || o_step % 2 != 0 || ldo % 2 != 0)
    return STRATUM_ERR_SHAPE;
  if ((long long)(heads - 1) * x_step + K > ldx || (long long)(heads - 1) * o_step + N > ldo) return STRATUM_ERR_SHAPE;
  if ((((uintptr_t)x | (uintptr_t)w) & 15) != 0 || ((uintptr_t)out & 3) != 0) return STRATUM_ERR_ALIGN;
  if (heads > 65535) return STRATUM_ERR_LIMIT;
  const int col_tiles = (N + HG_COLS - 1) / HG_COLS;
  if (M <= 16) {
    dim3 grid(1, (col_tiles + HG_WARPS - 1) / HG_WARPS, heads);
    return launch_pdl(head_gemm_kernel<1>, grid, HG_WARPS * 32, 0, stream, (const bf16*)x, (const bf16*)w, (bf16*)out,
                      M, N, K, ldx, ldo, x_step, o_step, 1);
  }
  if (M <= 32) {
    dim3 grid(1, (col_tiles + HG_WARPS - 1) / HG_WARPS, heads);
    return launch_pdl(head_gemm_kernel<2>, grid, HG_WARPS * 32, 0, stream, (const bf16*)x, (const bf16*)w, (bf16*)out,
                      M, N, K, ldx, ldo, x_step, o_step, 1);
  }
  const long long row_groups = ((long long)M + 32 * HG_WARPS - 1) / (32 * HG_WARPS);
  if (row_groups > 0x7fffffffLL || col_tiles > 65535) return STRATUM_ERR_LIMIT;
  dim3 grid((unsigned)row_groups, col_tiles, heads);
  return launch_pdl(head_gemm_kernel<2>, grid, HG_WARPS * 32, 0, stream, (const bf16*)x, (const bf16*)w, (bf16*)out, M,
                    N, K, ldx, ldo, x_step, o_step, 0);
}
