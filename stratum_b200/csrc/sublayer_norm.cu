// Norms that stand behind a sublayer instead of in front of it, and the rounding of the residual stream for the
// sublayer that reads it.
//
//   norm_into_residual   x[r] (+)= y[r] / sqrt(mean(y[r]^2) + eps) * gain,  float32 in, float32 out (the residual
//                        stream); optionally the new row is also written in bfloat16, which is what the next
//                        sublayer's matrix products read.  y may be x itself when nothing is accumulated (a norm in
//                        place, e.g. on freshly embedded tokens).
//   cast_rows            out = bfloat16(x), row by row.
//
// One block per row; the block's shape follows from the row's length alone, so the order of a row's sum of squares
// (and with it every bit of the result) does not depend on how many rows the step has.
#include "common.cuh"

template <bool COPY>
__global__ void norm_into_residual_kernel(const float* y, const float* __restrict__ gain, float* x, bf16* copy,
                                          int hidden, float eps, int accumulate) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();                                        // y and x are the work of kernels before this one: ld_fresh
  const size_t row = (size_t)blockIdx.x * hidden;
  const float* yr = y + row;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = ld_fresh(yr + i);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
  float* xr = x + row;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float r = ld_fresh(yr + i) * scale * gain[i];
    if (accumulate) r += ld_fresh(xr + i);
    xr[i] = r;
    if (COPY) copy[row + i] = __float2bfloat16_rn(r);
  }
}

// The same with four values per thread and turn (rows of a multiple of four values, 16-byte aligned).
template <bool COPY>
__global__ void norm_into_residual_vec_kernel(const float* y, const float* __restrict__ gain, float* x, bf16* copy,
                                              int hidden, float eps, int accumulate) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * hidden;
  const float4* yr = reinterpret_cast<const float4*>(y + row);
  const int n4 = hidden >> 2;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 v = ld_fresh(yr + i);
    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
  float4* xr = reinterpret_cast<float4*>(x + row);
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 v = ld_fresh(yr + i), g = reinterpret_cast<const float4*>(gain)[i];
    float4 r = make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
    if (accumulate) {
      const float4 o = ld_fresh(xr + i);
      r.x += o.x; r.y += o.y; r.z += o.z; r.w += o.w;
    }
    xr[i] = r;
    if (COPY) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(r.x, r.y), hi = __floats2bfloat162_rn(r.z, r.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(copy + row)[i] = pk;
    }
  }
}

static inline int row_threads(int hidden) { return hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128); }

STRATUM_EXPORT int stratum_norm_into_residual(const float* y, const float* gain, float* x, void* copy, int n_rows,
                                              int hidden, float eps, int accumulate, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden < 1) return STRATUM_ERR_SHAPE;
  const bool vec = hidden % 4 == 0 && ((((uintptr_t)y | (uintptr_t)gain | (uintptr_t)x | (uintptr_t)copy) & 15) == 0);
  if (vec) {
    // (the choice depends on the row's length and on alignment alone, which a model's buffers share from step to step)
    if (copy)
      launch_pdl(norm_into_residual_vec_kernel<true>, n_rows, row_threads(hidden / 4), 0, stream, y, gain, x,
                 (bf16*)copy, hidden, eps, accumulate);
    else
      launch_pdl(norm_into_residual_vec_kernel<false>, n_rows, row_threads(hidden / 4), 0, stream, y, gain, x,
                 (bf16*)nullptr, hidden, eps, accumulate);
    return launch_status();
  }
  if (copy)
    launch_pdl(norm_into_residual_kernel<true>, n_rows, row_threads(hidden), 0, stream, y, gain, x, (bf16*)copy, hidden,
               eps, accumulate);
  else
    launch_pdl(norm_into_residual_kernel<false>, n_rows, row_threads(hidden), 0, stream, y, gain, x, (bf16*)nullptr,
               hidden, eps, accumulate);
  return launch_status();
}

__global__ void cast_rows_kernel(const float* x, bf16* out, size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16_rn(ld_fresh(x + i));
}

STRATUM_EXPORT int stratum_cast_rows(const float* x, void* out, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long long blocks = (n + 255) / 256;
  if (blocks > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  launch_pdl(cast_rows_kernel, (unsigned)blocks, 256, 0, stream, x, (bf16*)out, (size_t)n);
  return launch_status();
}
