// The matrix memory of an mLSTM layer (xLSTM's matrix LSTM), with its gates' soft cap
// and the running maximum that keeps the exponentials in range.  Per head, with q, k of
// size d and v of size dv, log input gate a_t and log forget gate b_t:
//
//   a_t = cap * tanh((zi_t + bi) / cap),   b_t = logsigmoid(cap * tanh((zf_t + bf) / cap))
//   m_t = max(b_t + m_(t-1), a_t)
//   S_t = exp(b_t + m_(t-1) - m_t) S_(t-1) + exp(a_t - m_t) k_t v_t^T        [d, dv]
//   n_t = exp(b_t + m_(t-1) - m_t) n_(t-1) + exp(a_t - m_t) k_t              [d]
//   o_t = S_t^T (q_t * qscale) / (max(|n_t . (q_t * qscale)|, exp(-m_t)) + 1e-6)
//
// S, n and m start at zero (m too: not at minus infinity), live in float32 in the
// request's state slot [heads][d * dv + d + 1] and are carried from step to step.
// Everything but the loads of q, k and v (which may be bfloat16) is float32 arithmetic;
// the gates' pre-activations zi, zf arrive as float32.
//
//   mlstm_scan           one warp per (sequence, head, 32 value columns): it walks the
//                        sequence's tokens of this step in order with its slice of S in
//                        shared memory and n in registers (every warp of a head carries n;
//                        the first writes it back).  A token's arithmetic does not depend
//                        on how the sequence was cut into steps or on the batch around it.
//   head_gated_rmsnorm   out = o / sqrt(mean_head(o^2) + eps) * w * sigmoid(g): the norm runs
//                        over each head's dv values, w is [heads * dv]; one warp a (token, head).
#include "common.cuh"
#include <math.h>

#define ML_MAX_D 256

__device__ __forceinline__ float ml_soft_cap(float z, float cap) { return cap > 0.f ? cap * tanhf(z / cap) : z; }
__device__ __forceinline__ float ml_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename T>
__global__ void __launch_bounds__(32)
mlstm_scan_kernel(const T* q, const T* k, const T* v, int stride, const float* gates, const float* bias_i,
                  const float* bias_f, float cap, float qscale, float* state, const int* q_start, const int* slots,
                  float* out, int heads, int d, int dv, int num_slots, int* err) {
  pdl_wait();
  pdl_launch();
  extern __shared__ float sm[];          // S slice [d][32], then k [d], then q [d]
  float* S = sm;
  float* ks = sm + (size_t)d * 32;
  float* qs = ks + d;
  const int lane = threadIdx.x;
  const int j = blockIdx.x * 32 + lane;  // value column
  const int h = blockIdx.y, s = blockIdx.z;
  const int t0 = q_start[s], t1 = q_start[s + 1];
  const int slot = slots[s];
  if (slot < 0 || slot >= num_slots) {
    if (lane == 0) atomicOr(err, 8);
    return;
  }
  const size_t per_head = (size_t)d * dv + d + 1;
  float* st = state + ((size_t)slot * heads + h) * per_head;
  const bool live = j < dv;
  for (int i = 0; i < d; ++i) S[i * 32 + lane] = live ? st[(size_t)i * dv + j] : 0.f;
  float n[ML_MAX_D / 32];
#pragma unroll
  for (int r = 0; r < ML_MAX_D / 32; ++r) {
    const int i = lane + 32 * r;
    n[r] = i < d ? st[(size_t)d * dv + i] : 0.f;
  }
  float m = st[(size_t)d * dv + d];
  const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;
  for (int t = t0; t < t1; ++t) {
    const float a = ml_soft_cap(gates[(size_t)t * 2 * heads + h] + bi, cap);
    const float b = ml_logsigmoid(ml_soft_cap(gates[(size_t)t * 2 * heads + heads + h] + bf, cap));
    const float m_new = fmaxf(b + m, a);
    const float keep = expf(b + m - m_new), take = expf(a - m_new);
    m = m_new;
    const T* qr = q + (size_t)t * stride + (size_t)h * d;
    const T* kr = k + (size_t)t * stride + (size_t)h * d;
    __syncwarp();
    for (int i = lane; i < d; i += 32) { ks[i] = take * to_f32(kr[i]); qs[i] = to_f32(qr[i]) * qscale; }
    const float vj = live ? to_f32(v[(size_t)t * stride + (size_t)h * dv + j]) : 0.f;
    __syncwarp();
    float part = 0.f;
#pragma unroll
    for (int r = 0; r < ML_MAX_D / 32; ++r) {
      const int i = lane + 32 * r;
      if (i < d) { n[r] = fmaf(keep, n[r], ks[i]); part = fmaf(n[r], qs[i], part); }
    }
    const float dot = warp_sum(part);
    float num = 0.f;
#pragma unroll 4
    for (int i = 0; i < d; ++i) {
      const float sij = fmaf(keep, S[i * 32 + lane], ks[i] * vj);
      S[i * 32 + lane] = sij;
      num = fmaf(sij, qs[i], num);
    }
    const float den = fmaxf(fabsf(dot), expf(-m)) + 1e-6f;
    if (live) out[(size_t)t * heads * dv + (size_t)h * dv + j] = num / den;
  }
  if (t1 > t0) {
    if (live) for (int i = 0; i < d; ++i) st[(size_t)i * dv + j] = S[i * 32 + lane];
    if (blockIdx.x == 0) {
#pragma unroll
      for (int r = 0; r < ML_MAX_D / 32; ++r) {
        const int i = lane + 32 * r;
        if (i < d) st[(size_t)d * dv + i] = n[r];
      }
      if (lane == 0) st[(size_t)d * dv + d] = m;
    }
  }
}

// q, k: rows of heads * d; v: rows of heads * dv; all three with the row stride `stride` (views into one
// product's result).  gates float32 [T, 2 heads]: the input gates' pre-activations, then the forget gates'.
// state float32 [slots, heads, d * dv + d + 1]; out float32 [T, heads * dv].
RLLM_EXPORT int rllm_mlstm_scan(const void* q, const void* k, const void* v, int stride, int dtype, const float* gates,
                                const float* bias_i, const float* bias_f, float cap, float qscale, float* state,
                                const int* q_start, const int* slots, float* out, int num_seqs, int heads, int d,
                                int dv, int num_slots, int* err, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (heads <= 0 || d <= 0 || dv <= 0 || num_slots <= 0 || !(cap >= 0.f)) return RLLM_E_BADARG;
  if (d > ML_MAX_D || heads > 65535 || num_seqs > 65535) return RLLM_E_UNSUPPORTED;
  const size_t smem = ((size_t)d * 32 + 2 * (size_t)d) * sizeof(float);
  const dim3 grid((dv + 31) / 32, heads, num_seqs);
#define ML_GO(T_)                                                                                             \
  do {                                                                                                        \
    if (smem > 48 * 1024)                                                                                     \
      cudaFuncSetAttribute(mlstm_scan_kernel<T_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    rllm_launch_pdl(mlstm_scan_kernel<T_>, grid, dim3(32), smem, stream, (const T_*)q, (const T_*)k,          \
                    (const T_*)v, stride, gates, bias_i, bias_f, cap, qscale, state, q_start, slots, out,     \
                    heads, d, dv, num_slots, err);                                                            \
  } while (0)
  RLLM_DISPATCH_DTYPE(dtype, TT, ML_GO(TT));
#undef ML_GO
  RLLM_LAUNCH_CHECK();
  return 0;
}

template <typename T, typename TW>
__global__ void __launch_bounds__(128)
head_gated_rmsnorm_kernel(const float* x, const T* g, int g_stride, const TW* w, T* out, long long rows, int heads,
                          int dv, float eps) {
  pdl_wait();
  pdl_launch();
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= rows) return;
  const long long t = r / heads;
  const int h = (int)(r - t * heads);
  const float* xr = x + (size_t)r * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss = fmaf(xr[i], xr[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  const T* gr = g + (size_t)t * g_stride + (size_t)h * dv;
  for (int i = lane; i < dv; i += 32) {
    const float gate = 1.0f / (1.0f + expf(-to_f32(gr[i])));
    out[(size_t)r * dv + i] = from_f32<T>(xr[i] * inv * to_f32(w[(size_t)h * dv + i]) * gate);
  }
}

RLLM_EXPORT int rllm_head_gated_rmsnorm(const float* x, const void* g, int g_stride, const void* w, int w_dtype,
                                        void* out, int dtype, int T, int heads, int dv, float eps,
                                        cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads <= 0 || dv <= 0 || g_stride < heads * dv) return RLLM_E_BADARG;
  const long long rows = (long long)T * heads;
  const unsigned blocks = (unsigned)((rows + 3) / 4);
  RLLM_DISPATCH_DTYPE(dtype, TT, RLLM_DISPATCH_DTYPE(w_dtype, TW,
    (rllm_launch_pdl(head_gated_rmsnorm_kernel<TT, TW>, dim3(blocks), dim3(128), (size_t)0, stream, x, (const TT*)g,
                     g_stride, (const TW*)w, (TT*)out, rows, heads, dv, eps))));
  RLLM_LAUNCH_CHECK();
  return 0;
}
