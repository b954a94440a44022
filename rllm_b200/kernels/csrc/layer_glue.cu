// What stands between the sublayers of a layer whose sublayer results are gated
// and normalised before they join the residual stream, and whose stream is a
// weighted sum of the results of all layers so far.  All arithmetic is float32;
// the stream and the layer results are float32 in memory.
//
//   gated_postnorm_add:  v = (sum_k c[t, k] y[t, k, :]) * sigmoid(g[t, :] + b)      (g absent: no gate)
//                        x_out[t, :] = x_in[t, :] + v / sqrt(mean(v^2) + eps) * w
//                        and, if asked, next[t, :] = x_out / sqrt(mean(x_out^2) + eps2) * w2
//                        (the norm that reads the stream next).  With a history of layer results
//                        (x_out being its last level) the depth average follows in the same kernel:
//                        s = sum_j a[j] X[j, t, :] is written as the stream and the next norm reads s.
//   depth_average:       s[r, :] = sum_j a[j] X[j, row(r), :], the stream itself and/or
//                        its RMS norm in the activation dtype; row(r) = rows[r] or r.
// One block per row; the order of a row's additions depends on H and the block
// size only.
#include "common.cuh"

#define GLUE_THREADS 256

template <typename TA, typename TW>
__global__ void __launch_bounds__(GLUE_THREADS)
gated_postnorm_add_kernel(const float* x_in, float* x_out, const TA* y,
                          int slots, const float* slot_w, const TA* g, int g_stride,
                          const TW* gb, const TW* nw, float eps,
                          const TW* next_w, TA* next_out, float next_eps, const float* hist,
                          long long level_stride, int levels, const TW* coeff, float* stream_out, int H) {
  // (Every kernel of this file starts with the wait for the kernel ahead of it in the stream and lets the
  // next one in right after: launches overlap the tails of their predecessors.  The pointer parameters
  // carry no __restrict__, so that no load is proved independent of that wait and moved above it.)
  pdl_wait();
  pdl_launch();
  extern __shared__ float row[];
  __shared__ float red[32];
  const int t = blockIdx.x;
  const TA* gr = g + (size_t)t * g_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v;
    if (slot_w == nullptr) {
      v = to_f32(y[(size_t)t * H + i]);
    } else {
      v = 0.f;
      for (int k = 0; k < slots; ++k)
        v = fmaf(slot_w[(size_t)t * slots + k], to_f32(y[((size_t)t * slots + k) * H + i]), v);
    }
    if (g != nullptr) {                                  // no gate: the sublayer's result as it is
      const float a = to_f32(gr[i]) + (gb ? to_f32(gb[i]) : 0.f);
      v *= 1.0f / (1.0f + expf(-a));
    }
    row[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  float ss2 = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float xn = x_in[(size_t)t * H + i] + row[i] * inv * to_f32(nw[i]);
    x_out[(size_t)t * H + i] = xn;
    if (hist != nullptr) {
      // the depth average in the order of depth_average_kernel; x_out is the history's last level
      float s = 0.f;
      for (int j = 0; j + 1 < levels; ++j) s = fmaf(to_f32(coeff[j]), hist[(size_t)j * level_stride + (size_t)t * H + i], s);
      xn = fmaf(to_f32(coeff[levels - 1]), xn, s);
      stream_out[(size_t)t * H + i] = xn;
    }
    row[i] = xn;
    ss2 += xn * xn;
  }
  if (next_w == nullptr) return;
  ss2 = block_sum(ss2, red);
  const float inv2 = 1.0f / sqrtf(ss2 / (float)H + next_eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    next_out[(size_t)t * H + i] = from_f32<TA>(row[i] * inv2 * to_f32(next_w[i]));
}

RLLM_EXPORT int rllm_gated_postnorm_add(const float* x_in, float* x_out, const void* y, int slots,
                                        const float* slot_w, const void* g, int g_stride, const void* gb,
                                        const void* nw, float eps, const void* next_w, void* next_out,
                                        float next_eps, const float* hist, long long level_stride, int levels,
                                        const void* coeff, float* stream_out, int T, int H, int act_dtype,
                                        int w_dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || slots < 1 || (g != nullptr && g_stride < H)) return RLLM_E_BADARG;
  if (hist != nullptr && (levels < 1 || coeff == nullptr || stream_out == nullptr)) return RLLM_E_BADARG;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return RLLM_E_UNSUPPORTED;
#define GLUE_LAUNCH(TA, TW)                                                                              \
  do {                                                                                                   \
    if (smem > 48 * 1024)                                                                                \
      cudaFuncSetAttribute(gated_postnorm_add_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)smem);                                                                   \
    rllm_launch_pdl(gated_postnorm_add_kernel<TA, TW>, dim3(T), dim3(GLUE_THREADS), (size_t)(smem), stream,                                 \
        x_in, x_out, (const TA*)y, slots, slot_w, (const TA*)g, g_stride, (const TW*)gb, (const TW*)nw,  \
        eps, (const TW*)next_w, (TA*)next_out, next_eps, hist, level_stride, levels, (const TW*)coeff, stream_out, H);                                             \
  } while (0)
  RLLM_DISPATCH_DTYPE(act_dtype, TA_, RLLM_DISPATCH_DTYPE(w_dtype, TW_, GLUE_LAUNCH(TA_, TW_)));
#undef GLUE_LAUNCH
  RLLM_LAUNCH_CHECK();
  return 0;
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(GLUE_THREADS)
depth_average_kernel(const float* hist, long long level_stride, int levels,
                     const TW* a, const int* rows, float* stream_out,
                     const TW* nw, TA* norm_out, float eps, int H) {
  pdl_wait();
  pdl_launch();
  extern __shared__ float row[];
  __shared__ float red[32];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float s = 0.f;
    for (int j = 0; j < levels; ++j) s = fmaf(to_f32(a[j]), hist[(size_t)j * level_stride + (size_t)src * H + i], s);
    if (stream_out) stream_out[(size_t)r * H + i] = s;
    row[i] = s;
    ss += s * s;
  }
  if (nw == nullptr) return;
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    norm_out[(size_t)r * H + i] = from_f32<TA>(row[i] * inv * to_f32(nw[i]));
}

RLLM_EXPORT int rllm_depth_average(const float* hist, long long level_stride, int levels, const void* a,
                                   const int* rows, float* stream_out, const void* nw, void* norm_out,
                                   float eps, int R, int H, int act_dtype, int w_dtype, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (H <= 0 || levels < 1) return RLLM_E_BADARG;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return RLLM_E_UNSUPPORTED;
#define GLUE_LAUNCH(TA, TW)                                                                            \
  do {                                                                                                 \
    if (smem > 48 * 1024)                                                                              \
      cudaFuncSetAttribute(depth_average_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                           (int)smem);                                                                 \
    rllm_launch_pdl(depth_average_kernel<TA, TW>, dim3(R), dim3(GLUE_THREADS), (size_t)(smem), stream,                                    \
        hist, level_stride, levels, (const TW*)a, rows, stream_out, (const TW*)nw, (TA*)norm_out, eps, H); \
  } while (0)
  RLLM_DISPATCH_DTYPE(act_dtype, TA_, RLLM_DISPATCH_DTYPE(w_dtype, TW_, GLUE_LAUNCH(TA_, TW_)));
#undef GLUE_LAUNCH
  RLLM_LAUNCH_CHECK();
  return 0;
}
