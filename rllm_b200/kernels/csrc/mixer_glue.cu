// Small steps around mixers, each one pass over its rows, float32 arithmetic:
//
//   head_norm_kv_write   per-head RMS norm of queries (in place) and keys, and the write of
//                        a token's keys and values into its cache pages; keys and values may
//                        have different sizes per head; without norm weights it is the bare write.
//                        The cache rows may be wider than the heads (dkp >= dk, dvp >= dv): the
//                        rest of a row is written as zeros, and the queries then go, padded with
//                        zeros to dkp a head, into a buffer of their own.  (Zeros change no score
//                        and add columns of zeros to the result: keys and values of two sizes
//                        can so be served by kernels that want one.)  Optional steps on the way, in this
//                        order: a bias on every element of the row (float32 [nq dk + nkv dk + nkv dv]), the
//                        norm, and a rotation of queries and keys by position over the first rd dims of a
//                        head (dimension i with i + rd / 2, angle position * inv_freq[i], cosine and sine
//                        times `mag`; float32 rows take them in float64).  `unit_norm`: the norm without
//                        weights (queries and keys are divided by their root mean square and nothing
//                        else).  `qt_every` > 0: a query at position p is multiplied by
//                        1 + qt_coef * ln(floor((p + 1) / qt_every) + 1), a temperature that grows with
//                        the position; keys are not.
//   rms_mean             out = (1/n) sum_i rms(x_i) * w_i  over n = 2 inputs of one width
//                        (branches of a mixer that run side by side)
//   gated_rmsnorm        out = rms(x) * w * sigmoid(g)     (x float32, g in the activation dtype)
//
// rms(x) = x / sqrt(mean(x^2) + eps), eps inside the root.  One warp a head or one block a
// row; the order of a row's additions depends on its width only.
#include "common.cuh"
#include <math.h>

#define HN_WARPS 4

// qkv: T rows of [nq * dk | nkv * dk | nkv * dv] with row stride `stride`.
template <typename T, typename TW>
__global__ void __launch_bounds__(32 * HN_WARPS)
head_norm_kv_write_kernel(T* qkv, int stride, const int* positions, const int* token_seq, const TW* wq, const TW* wk,
                          float eps, const int* block_table, int max_blocks, T* kcache, T* vcache, int T_tokens, int nq,
                          int nkv, int dk, int dv, int dkp, int dvp, T* q_out, int page_size, int num_pages,
                          int write_kv, const float* __restrict__ bias, const double* __restrict__ inv_freq, int rd,
                          float mag, int unit_norm, float qt_coef, int qt_every, int* err) {
  pdl_wait();
  pdl_launch();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int heads = nq + 2 * nkv;
  const long long gw = (long long)blockIdx.x * HN_WARPS + warp;
  if (gw >= (long long)T_tokens * heads) return;
  const int t = (int)(gw / heads), h = (int)(gw - (long long)t * heads);
  T* row = qkv + (size_t)t * stride;
  T* dst = nullptr;
  const int pos = positions[t];
  if (h >= nq) {
    if (!write_kv) return;
    const int s = token_seq[t];
    const int blk = pos / page_size;
    const int page = (blk < max_blocks) ? block_table[(size_t)s * max_blocks + blk] : -1;
    if (page < 0 || page >= num_pages) {
      if (lane == 0) atomicOr(err, 2);
      return;
    }
    const int kvh = (h - nq) % nkv;
    dst = (h < nq + nkv) ? kcache + (((size_t)page * nkv + kvh) * page_size + pos % page_size) * dkp
                         : vcache + (((size_t)page * nkv + kvh) * page_size + pos % page_size) * dvp;
  } else if (q_out) {
    dst = q_out + ((size_t)t * nq + h) * dkp;
  }
  if (h >= nq + nkv) {                                    // a value head: copied (with its bias)
    const size_t at = (size_t)nq * dk + (size_t)nkv * dk + (size_t)(h - nq - nkv) * dv;
    const T* src = row + at;
    for (int i = lane; i < dvp; i += 32)
      dst[i] = (i >= dv) ? from_f32<T>(0.f) : (bias ? from_f32<T>(to_f32(src[i]) + bias[at + i]) : src[i]);
    return;
  }
  T* src = row + (size_t)h * dk;                          // query heads, then key heads: both dk wide
  const float* bs = bias ? bias + (size_t)h * dk : nullptr;
  const TW* w = (h < nq) ? wq : wk;
  const bool warm = h < nq && qt_every > 0;             // a query under a temperature that grows with its position
  const bool scaled = w || unit_norm || warm;
  if (!scaled && !bs && rd == 0) {
    if (dst) for (int i = lane; i < dkp; i += 32) dst[i] = (i < dk) ? src[i] : from_f32<T>(0.f);
    return;
  }
  float r = 1.0f;
  if (w || unit_norm) {
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) { const float v = to_f32(src[i]) + (bs ? bs[i] : 0.f); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    r = 1.0f / sqrtf(ss / (float)dk + eps);
  }
  if (warm) r *= 1.0f + qt_coef * logf((float)((pos + 1) / qt_every) + 1.0f);
  T* o = dst ? dst : src;
  const int half = rd >> 1;
  // a lane reads both members of its pairs before it writes them, and no other lane touches them: in place is safe
  for (int i = lane; i < half; i += 32) {
    float a = to_f32(src[i]) + (bs ? bs[i] : 0.f), b = to_f32(src[i + half]) + (bs ? bs[i + half] : 0.f);
    if (scaled) { a *= r * (w ? to_f32(w[i]) : 1.0f); b *= r * (w ? to_f32(w[i + half]) : 1.0f); }
    float c, sn;
    if (sizeof(T) == 4) {
      double sd, cd;
      sincos((double)pos * inv_freq[i], &sd, &cd);
      c = (float)(cd * (double)mag); sn = (float)(sd * (double)mag);
    } else {
      rope_cos_sin(pos, inv_freq[i], &c, &sn);
      c *= mag; sn *= mag;
    }
    o[i] = from_f32<T>(a * c - b * sn);
    o[i + half] = from_f32<T>(b * c + a * sn);
  }
  for (int i = rd + lane; i < (dst ? dkp : dk); i += 32) {
    if (i >= dk) { o[i] = from_f32<T>(0.f); continue; }
    float a = to_f32(src[i]) + (bs ? bs[i] : 0.f);
    if (scaled) a *= r * (w ? to_f32(w[i]) : 1.0f);
    o[i] = from_f32<T>(a);
  }
}

// The same without norm weights for bfloat16 rows whose heads are multiples of 8 wide and 16-byte aligned
// (rd a multiple of 16, no wider cache rows): a thread takes 8 neighbouring elements of a head (16 bytes), or,
// inside the rotated dims, the 8 elements at i .. i + 7 and their partners at i + rd / 2 ..; the arithmetic of
// every element is that of the kernel above.  Items of a token: (nq + nkv) * dk / 8 of q and k, nkv * dv / 8 of v.
__device__ __forceinline__ void hn_load8(const bf16* p, float* o) {
  const uint4 a = *(const uint4*)p;
  const __nv_bfloat162* h = (const __nv_bfloat162*)&a;
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void hn_store8(bf16* p, const float* v) {
  uint4 a;
  __nv_bfloat162* h = (__nv_bfloat162*)&a;
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *(uint4*)p = a;
}

__global__ void __launch_bounds__(256)
head_kv_write_bf16x8_kernel(bf16* qkv, int stride, const int* positions, const int* token_seq, const int* block_table,
                            int max_blocks, bf16* kcache, bf16* vcache, int T_tokens, int nq, int nkv, int dk, int dv,
                            int page_size, int num_pages, int write_kv, const float* __restrict__ bias,
                            const double* __restrict__ inv_freq, int rd, float mag, int* err) {
  pdl_wait();
  pdl_launch();
  const int ck = dk >> 3, cv = dv >> 3;
  const int per_tok = (nq + nkv) * ck + nkv * cv;
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= (long long)T_tokens * per_tok) return;
  const int t = (int)(item / per_tok), it = (int)(item - (long long)t * per_tok);
  const bool is_v = it >= (nq + nkv) * ck;
  const int h = is_v ? (it - (nq + nkv) * ck) / cv : it / ck;          // head among the v heads, or among q then k
  const int c = is_v ? (it - (nq + nkv) * ck) - h * cv : it - h * ck;  // which 8 elements of the head
  const int half = rd >> 1;
  if (!is_v && c * 8 >= half && c * 8 < rd) return;                    // partners: done by the thread of c - half / 8
  const bool to_cache = is_v || h >= nq;
  if (to_cache && !write_kv) return;
  const int pos = positions[t];
  bf16* row = qkv + (size_t)t * stride;
  const size_t at = is_v ? (size_t)(nq + nkv) * dk + (size_t)h * dv + c * 8 : (size_t)h * dk + c * 8;
  bf16* dst = row + at;
  if (to_cache) {
    const int s = token_seq[t];
    const int blk = pos / page_size;
    const int page = (blk < max_blocks) ? block_table[(size_t)s * max_blocks + blk] : -1;
    if (page < 0 || page >= num_pages) { atomicOr(err, 2); return; }
    const int kvh = is_v ? h : h - nq;
    dst = is_v ? vcache + (((size_t)page * nkv + kvh) * page_size + pos % page_size) * dv + c * 8
               : kcache + (((size_t)page * nkv + kvh) * page_size + pos % page_size) * dk + c * 8;
  }
  float a[8];
  hn_load8(row + at, a);
  if (bias) {
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] += bias[at + i];
  }
  if (is_v || c * 8 >= rd) {                                           // no rotation here
    if (to_cache || bias) hn_store8(dst, a);
    return;
  }
  float b[8];
  hn_load8(row + at + half, b);
  if (bias) {
#pragma unroll
    for (int i = 0; i < 8; ++i) b[i] += bias[at + half + i];
  }
  float lo[8], hi[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float cs, sn;
    rope_cos_sin(pos, inv_freq[c * 8 + i], &cs, &sn);
    cs *= mag; sn *= mag;
    lo[i] = a[i] * cs - b[i] * sn;
    hi[i] = b[i] * cs + a[i] * sn;
  }
  hn_store8(dst, lo);
  hn_store8(dst + half, hi);
}

RLLM_EXPORT int rllm_head_norm_kv_write(void* qkv, int dtype, int stride, const int* positions, const int* token_seq,
                                        const void* wq, const void* wk, int w_dtype, float eps, const int* block_table,
                                        int max_blocks, void* kcache, void* vcache, int T, int nq, int nkv, int dk,
                                        int dv, int dkp, int dvp, void* q_out, int page_size, int num_pages,
                                        int write_kv, const float* bias, const double* inv_freq, int rd, float mag,
                                        int unit_norm, float qt_coef, int qt_every, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (nq <= 0 || nkv < 0 || dk <= 0 || dv <= 0 || dkp < dk || dvp < dv) return RLLM_E_BADARG;
  if (rd < 0 || rd > dk || (rd & 1) || (rd > 0 && !inv_freq)) return RLLM_E_BADARG;
  if (dkp > dk && !q_out) return RLLM_E_BADARG;          // padded keys want padded queries
  if (write_kv && (page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || !kcache || !vcache)) return RLLM_E_BADARG;
  const int nkv_w = write_kv ? nkv : 0;
  if (qt_every < 0 || (unit_norm && (wq || wk))) return RLLM_E_BADARG;
  if (dtype == RLLM_DT_BF16 && !wq && !wk && !unit_norm && qt_every == 0 && !q_out && dkp == dk && dvp == dv && dk % 8 == 0 && dv % 8 == 0 &&
      rd % 16 == 0 && stride % 8 == 0 && (((uintptr_t)qkv | (uintptr_t)kcache | (uintptr_t)vcache) & 15) == 0) {
    const long long items = (long long)T * ((nq + nkv_w) * (dk / 8) + nkv_w * (dv / 8));
    const unsigned blocks8 = (unsigned)((items + 255) / 256);
    cudaError_t e8 = rllm_launch_pdl(head_kv_write_bf16x8_kernel, dim3(blocks8), dim3(256), (size_t)0, stream, (bf16*)qkv,
                                     stride, positions, token_seq, block_table, max_blocks, (bf16*)kcache, (bf16*)vcache,
                                     T, nq, nkv_w, dk, dv, page_size, num_pages, write_kv, bias, inv_freq, rd, mag, err);
    return (int)e8;
  }
  const long long warps = (long long)T * (nq + 2 * nkv);
  const unsigned blocks = (unsigned)((warps + HN_WARPS - 1) / HN_WARPS);
  RLLM_DISPATCH_DTYPE(dtype, TT, RLLM_DISPATCH_DTYPE(w_dtype, TW,
    (rllm_launch_pdl(head_norm_kv_write_kernel<TT, TW>, dim3(blocks), dim3(32 * HN_WARPS), (size_t)0, stream, (TT*)qkv,
                     stride, positions, token_seq, (const TW*)wq, (const TW*)wk, eps, block_table, max_blocks,
                     (TT*)kcache, (TT*)vcache, T, nq, nkv, dk, dv, dkp, dvp, (TT*)q_out, page_size, num_pages,
                     write_kv, bias, inv_freq, rd, mag, unit_norm, qt_coef, qt_every, err))));
  RLLM_LAUNCH_CHECK();
  return 0;
}

// out[r] = 1/2 (rms(a[r]) wa + rms(b[r]) wb)
template <typename T, typename TW>
__global__ void __launch_bounds__(256)
rms_mean2_kernel(const T* a, const T* b, const TW* wa, const TW* wb, T* out, int H, float eps) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const size_t base = (size_t)blockIdx.x * H;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float x = to_f32(a[base + i]), y = to_f32(b[base + i]);
    sa = fmaf(x, x, sa);
    sb = fmaf(y, y, sb);
  }
  sa = block_sum(sa, red);
  sb = block_sum(sb, red);
  const float ra = 1.0f / sqrtf(sa / (float)H + eps), rb = 1.0f / sqrtf(sb / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[base + i] = from_f32<T>(0.5f * (to_f32(a[base + i]) * ra * to_f32(wa[i]) + to_f32(b[base + i]) * rb * to_f32(wb[i])));
}

RLLM_EXPORT int rllm_rms_mean2(const void* a, const void* b, const void* wa, const void* wb, int w_dtype, void* out,
                               int dtype, int T, int H, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0) return RLLM_E_BADARG;
  RLLM_DISPATCH_DTYPE(dtype, TT, RLLM_DISPATCH_DTYPE(w_dtype, TW,
    (rllm_launch_pdl(rms_mean2_kernel<TT, TW>, dim3(T), dim3(256), (size_t)0, stream, (const TT*)a, (const TT*)b,
                     (const TW*)wa, (const TW*)wb, (TT*)out, H, eps))));
  RLLM_LAUNCH_CHECK();
  return 0;
}

// out[r] = rms(x[r]) * w * sigmoid(g[r]);  x float32 [T, H], g rows with stride g_stride
template <typename T, typename TW>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* x, const T* g, int g_stride, const TW* w, T* out, int H, float eps) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const size_t base = (size_t)blockIdx.x * H;
  const T* gr = g + (size_t)blockIdx.x * g_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) { const float v = x[base + i]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  const float r = 1.0f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float gate = 1.0f / (1.0f + expf(-to_f32(gr[i])));
    out[base + i] = from_f32<T>(x[base + i] * r * to_f32(w[i]) * gate);
  }
}

RLLM_EXPORT int rllm_gated_rmsnorm(const float* x, const void* g, int g_stride, const void* w, int w_dtype, void* out,
                                   int dtype, int T, int H, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0) return RLLM_E_BADARG;
  RLLM_DISPATCH_DTYPE(dtype, TT, RLLM_DISPATCH_DTYPE(w_dtype, TW,
    (rllm_launch_pdl(gated_rmsnorm_kernel<TT, TW>, dim3(T), dim3(256), (size_t)0, stream, x, (const TT*)g, g_stride,
                     (const TW*)w, (TT*)out, H, eps))));
  RLLM_LAUNCH_CHECK();
  return 0;
}
