// Layer norm over the float32 residual stream, fused with the adds that complete the stream:
//
//   v   = x [+ d0] [+ d1] [+ c]          d0, d1: sublayer results [T, H] in the activation dtype,
//                                         c: a vector [H] added to every row (an output bias)
//   x  <- v                               (writeback, when the stream is to be completed in place)
//   out = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w + b
//
// All arithmetic is float32; the row waits in shared memory between the passes (sum, sum of
// squared deviations, output), so the variance is taken from the deviations themselves and not
// from a difference of large sums.  One block a row; the order of a row's additions depends on
// its width only.  `rows`: out[r] is made from row rows[r] (the rows whose logits are wanted).
//
//   add_rows   x += d0 [+ d1] [+ c]        for a stream that no such norm reads next
#include "common.cuh"
#include <math.h>

template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
layernorm_kernel(float* x, const TD* d0, const TD* d1, const float* __restrict__ c, const int* rows,
                 const float* __restrict__ w, const float* __restrict__ b, TO* out, int H, float eps, int writeback) {
  extern __shared__ float row[];
  __shared__ float red[32];
  pdl_wait_on(x, d0, d1, rows);
  pdl_launch();
  const int r = blockIdx.x;
  const size_t src = (size_t)(rows ? rows[r] : r) * H;
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = x[src + i];
    if (d0 || d1 || c) {
      float a = 0.f;                                   // the sublayers' sum first, then into the stream
      if (d0) a = to_f32(d0[src + i]);
      if (d1) a += to_f32(d1[src + i]);
      if (c) a += c[i];
      v += a;
      if (writeback) x[src + i] = v;
    }
    row[i] = v;
    s += v;
  }
  const float mean = block_sum(s, red) / (float)H;
  float q = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) { const float dlt = row[i] - mean; q = fmaf(dlt, dlt, q); }
  const float inv = 1.0f / sqrtf(block_sum(q, red) / (float)H + eps);
  TO* o = out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TO>((row[i] - mean) * inv * w[i] + b[i]);
}

RLLM_EXPORT int rllm_layernorm(float* x, const void* d0, const void* d1, const float* c, const int* rows,
                               const float* w, const float* b, void* out, int act_dtype, int R, int H, float eps,
                               int writeback, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (H <= 0 || !(eps >= 0.f) || !w || !b) return RLLM_E_BADARG;
  if (rows && writeback) return RLLM_E_BADARG;
  if (d1 && !d0) return RLLM_E_BADARG;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return RLLM_E_UNSUPPORTED;
  const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
  RLLM_DISPATCH_DTYPE(act_dtype, TD, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(layernorm_kernel<TD, TD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e = rllm_launch_pdl(layernorm_kernel<TD, TD>, dim3(R), dim3(threads), smem, stream, x, (const TD*)d0,
                                    (const TD*)d1, c, rows, w, b, (TD*)out, H, eps, writeback);
    if (e != cudaSuccess) return (int)e;
  });
  return 0;
}

template <typename TD>
__global__ void add_rows_kernel(float* x, const TD* d0, const TD* d1, const float* __restrict__ c, size_t n, int H) {
  pdl_wait_on(x, d0, d1);
  pdl_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float a = to_f32(d0[i]);
  if (d1) a += to_f32(d1[i]);
  if (c) a += c[i % H];
  x[i] += a;
}

RLLM_EXPORT int rllm_add_rows(float* x, const void* d0, const void* d1, const float* c, int act_dtype, int R, int H,
                              cudaStream_t stream) {
  if (R <= 0) return 0;
  if (H <= 0 || !d0) return RLLM_E_BADARG;
  const size_t n = (size_t)R * H;
  RLLM_DISPATCH_DTYPE(act_dtype, TD, {
    cudaError_t e = rllm_launch_pdl(add_rows_kernel<TD>, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)0, stream,
                                    x, (const TD*)d0, (const TD*)d1, c, n, H);
    if (e != cudaSuccess) return (int)e;
  });
  return 0;
}

// y[T, N] (activation dtype) += c[N] (float32) on every row: a projection's bias where no later kernel takes it
template <typename TD>
__global__ void add_row_bias_kernel(TD* y, const float* __restrict__ c, size_t n, int N) {
  pdl_wait_on(y);
  pdl_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  y[i] = from_f32<TD>(to_f32(y[i]) + c[i % N]);
}

RLLM_EXPORT int rllm_add_row_bias(void* y, const float* c, int act_dtype, int R, int N, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (N <= 0 || !c) return RLLM_E_BADARG;
  const size_t n = (size_t)R * N;
  RLLM_DISPATCH_DTYPE(act_dtype, TD, {
    cudaError_t e = rllm_launch_pdl(add_row_bias_kernel<TD>, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)0,
                                    stream, (TD*)y, c, n, N);
    if (e != cudaSuccess) return (int)e;
  });
  return 0;
}
