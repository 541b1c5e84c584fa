// y = x W^T (+ bias) for any sizes, on CUDA cores, float32 accumulation in a fixed order.
//
// This is the whole linear layer of the true 32-bit path (no tensor-core mode of reduced
// precision anywhere), and the fallback of the bfloat16 path for shapes the tensor-core
// kernels refuse.  W is row-major [N][K] as stored in the file: y[m][n] = sum_k x[m][k] W[n][k]
// (stratum/native/stratum_linear.h:491-507).  Each output element is one chain of fused
// multiply-adds over k = 0..K-1, so its value does not depend on M, on the tile it falls in,
// or on what else is in the step.
//
// Epilogues: 0 store as T; 1 add into a float32 tensor in place (the residual stream);
//            2 store as float32 (logits).
#include "common.cuh"

#define LS_BM 64
#define LS_BN 64
#define LS_BK 16
#define LS_TM 4
#define LS_TN 4

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
linear_simple_kernel(const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ bias,
                     void* __restrict__ out, int M, int N, int K, int ldx, int ldo, int x_step, long long w_step,
                     int o_step, int act) {
  __shared__ float xs[LS_BK][LS_BM + 1];
  __shared__ float ws[LS_BK][LS_BN + 1];
  const int tid = threadIdx.x;
  // one product per blockIdx.z (the heads of linear_heads): operands and result move on by their steps
  x += (size_t)blockIdx.z * x_step;
  w += (size_t)blockIdx.z * w_step;
  const size_t o_shift = (size_t)blockIdx.z * o_step;
  const int m0 = blockIdx.y * LS_BM, n0 = blockIdx.x * LS_BN;
  const int tm = (tid / 16) * LS_TM, tn = (tid % 16) * LS_TN;
  float acc[LS_TM][LS_TN];
#pragma unroll
  for (int i = 0; i < LS_TM; i++)
#pragma unroll
    for (int j = 0; j < LS_TN; j++) acc[i][j] = 0.f;

  // each thread loads 4 elements of each tile per step: row = tid / 4, k = (tid % 4) * 4 .. +3
  const int lr = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += LS_BK) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int k = k0 + lk + j;
      const int m = m0 + lr, n = n0 + lr;
      xs[lk + j][lr] = (m < M && k < K) ? to_float(x[(size_t)m * ldx + k]) : 0.f;
      ws[lk + j][lr] = (n < N && k < K) ? to_float(w[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < LS_BK; kk++) {
      float a[LS_TM], b[LS_TN];
#pragma unroll
      for (int i = 0; i < LS_TM; i++) a[i] = xs[kk][tm + i];
#pragma unroll
      for (int j = 0; j < LS_TN; j++) b[j] = ws[kk][tn + j];
#pragma unroll
      for (int i = 0; i < LS_TM; i++)
#pragma unroll
        for (int j = 0; j < LS_TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < LS_TM; i++) {
    const int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < LS_TN; j++) {
      const int n = n0 + tn + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      const size_t o = (size_t)m * ldo + n + o_shift;
      if (EPI == 0) ((T*)out)[o] = from_float<T>(activate(v, act));
      else if (EPI == 1) ((float*)out)[o] += v;
      else ((float*)out)[o] = v;
    }
  }
}

template <typename T>
static int launch_linear_simple(const void* x, const void* w, const float* bias, void* out, int epilogue,
                                int M, int N, int K, int ldx, int ldo, cudaStream_t stream, int heads = 1,
                                int x_step = 0, long long w_step = 0, int o_step = 0, int act = 0) {
  dim3 grid((N + LS_BN - 1) / LS_BN, (M + LS_BM - 1) / LS_BM, heads);
  if (epilogue == 0)
    linear_simple_kernel<T, 0><<<grid, 256, 0, stream>>>((const T*)x, (const T*)w, bias, out, M, N, K, ldx, ldo,
                                                      x_step, w_step, o_step, act);
  else if (epilogue == 1)
    linear_simple_kernel<T, 1><<<grid, 256, 0, stream>>>((const T*)x, (const T*)w, bias, out, M, N, K, ldx, ldo,
                                                      x_step, w_step, o_step, act);
  else if (epilogue == 2)
    linear_simple_kernel<T, 2><<<grid, 256, 0, stream>>>((const T*)x, (const T*)w, bias, out, M, N, K, ldx, ldo,
                                                      x_step, w_step, o_step, act);
  else
    return STRATUM_ERR_SHAPE;
  return launch_status();
}

// x: [M][ldx] T (first K columns used); w: [N][K] T; bias: float32 [N] or null; out: [M][ldo].
// act (epilogue 0 only): an activation applied to what is stored, see common.cuh.
STRATUM_EXPORT int stratum_linear_simple(const void* x, const void* w, const float* bias, void* out, int dtype,
                                         int epilogue, int M, int N, int K, int ldx, int ldo, int act,
                                         cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || ldx < K || ldo < N) return STRATUM_ERR_SHAPE;
  if (act != 0 && epilogue != 0) return STRATUM_ERR_SHAPE;
  if ((M + LS_BM - 1) / LS_BM > 65535) return STRATUM_ERR_LIMIT;
  if (dtype == STRATUM_DT_F32)
    return launch_linear_simple<float>(x, w, bias, out, epilogue, M, N, K, ldx, ldo, stream, 1, 0, 0, 0, act);
  if (dtype == STRATUM_DT_BF16)
    return launch_linear_simple<bf16>(x, w, bias, out, epilogue, M, N, K, ldx, ldo, stream, 1, 0, 0, 0, act);
  return STRATUM_ERR_DTYPE;
}

// The same product once per head: head j multiplies columns [j * x_step, j * x_step + K) of x by the matrix
// w[j] ([heads][N][K]) into columns [j * o_step, j * o_step + N) of out.  No bias.
STRATUM_EXPORT int stratum_linear_heads(const void* x, const void* w, void* out, int dtype, int epilogue, int heads,
                                        int M, int N, int K, int ldx, int ldo, int x_step, int o_step,
                                        cudaStream_t stream) {
  if (M <= 0 || N <= 0 || heads <= 0) return 0;
  if (K <= 0 || x_step < 0 || o_step < 0 || (long long)(heads - 1) * x_step + K > ldx ||
      (long long)(heads - 1) * o_step + N > ldo)
    return STRATUM_ERR_SHAPE;
  if ((M + LS_BM - 1) / LS_BM > 65535 || heads > 65535) return STRATUM_ERR_LIMIT;
  const long long w_step = (long long)N * K;
  if (dtype == STRATUM_DT_F32)
    return launch_linear_simple<float>(x, w, nullptr, out, epilogue, M, N, K, ldx, ldo, stream, heads, x_step, w_step,
                                       o_step);
  if (dtype == STRATUM_DT_BF16)
    return launch_linear_simple<bf16>(x, w, nullptr, out, epilogue, M, N, K, ldx, ldo, stream, heads, x_step, w_step,
                                      o_step);
  return STRATUM_ERR_DTYPE;
}
