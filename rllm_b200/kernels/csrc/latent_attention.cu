// Attention through a low-rank latent: a token keeps one row in the cache, its
// normalised latent c (kv_rank values) followed by a rotated key part that all
// heads share (rot values).  A head's key is W_uk c and its value W_uv c; both
// products are moved to the query side, so the cached rows are read as they are:
//   q~[h]   = [ W_uk[h]^T q_nope[h] , rotate(q_rot[h]) ]          (kv_rank + rot values)
//   score   = q~[h] . row * scale ;  softmax over the visible rows (all up to the
//             query's position, or the last `window` of them), optionally with a
//             sink: one more term exp(sink[h]) in the denominator, without a value
//   o~[h]   = sum_j p_j c_j ;  head output = W_uv[h] o~[h].
// This file holds: the per-token preparation (RMS norms of the two latents,
// rotation of the shared key part, cache write), the rotation of the queries'
// rotated part, the per-head products, and the attention over the cached rows on
// CUDA cores (float32 and bfloat16 rows; scores, softmax and sums in float32).
// Rotation pairs dimension 2i with 2i+1; angles are position * f_i in float64.
#include "tile_gemm.cuh"
#include "tile_gemm_mma.cuh"
#include <math.h>

// ---------------------------------------------------------------------------
// per token: c_q = rmsnorm(a[0:q_rank]) * wq  -> cq
//            c   = rmsnorm(a[q_rank : q_rank+kv_rank]) * wkv -> cache row [0:kv_rank]
//            rotate(a[q_rank+kv_rank : +rot]) -> cache row [kv_rank : kv_rank+rot]
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void rot_cos_sin(int pos, double f, float* c, float* s);
template <>
__device__ __forceinline__ void rot_cos_sin<float>(int pos, double f, float* c, float* s) {
  double sd, cd;
  sincos((double)pos * f, &sd, &cd);
  *c = (float)cd; *s = (float)sd;
}
template <>
__device__ __forceinline__ void rot_cos_sin<bf16>(int pos, double f, float* c, float* s) {
  rope_cos_sin(pos, f, c, s);
}

template <typename T, typename TW>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const T* a, int a_stride, int q_rank, int kv_rank, int rot, int rot_dims,
                   const TW* wq, const TW* wkv, float eps, T* cq,
                   T* cache, const int* block_table, int max_blocks,
                   const int* positions, const int* token_seq,
                   const double* inv_freq, float mag, int page_size, int num_pages, int write_kv,
                   int* err) {
  // (Every kernel of this file starts with the wait for the kernel ahead of it in the stream and lets the
  // next one in right after: launches overlap the tails of their predecessors.  The pointer parameters
  // carry no __restrict__, so that no load is proved independent of that wait and moved above it.)
  pdl_wait();
  pdl_launch();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const T* row = a + (size_t)t * a_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) { const float v = to_f32(row[i]); ss += v * v; }
  ss = block_sum(ss, red);
  float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq[(size_t)t * q_rank + i] = from_f32<T>(to_f32(row[i]) * inv * to_f32(wq[i]));
  if (!write_kv) return;
  const int pos = positions[t], s = token_seq[t];
  const int page = block_table[(size_t)s * max_blocks + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(err, 2);
    return;
  }
  const int width = kv_rank + rot;
  T* dst = cache + ((size_t)page * page_size + (pos % page_size)) * width;
  const T* kv = row + q_rank;
  ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) { const float v = to_f32(kv[i]); ss += v * v; }
  ss = block_sum(ss, red);
  inv = 1.0f / sqrtf(ss / (float)kv_rank + eps);
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x)
    dst[i] = from_f32<T>(to_f32(kv[i]) * inv * to_f32(wkv[i]));
  const T* kr = kv + kv_rank;
  for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) {
    const float u = to_f32(kr[2 * i]), v = to_f32(kr[2 * i + 1]);
    if (2 * i + 1 < rot_dims) {
      float c, sn;
      rot_cos_sin<T>(pos, inv_freq[i], &c, &sn);
      c *= mag; sn *= mag;              // the factor that a rescaled rotation puts on cosine and sine (1: none)
      dst[kv_rank + 2 * i] = from_f32<T>(u * c - v * sn);
      dst[kv_rank + 2 * i + 1] = from_f32<T>(v * c + u * sn);
    } else {
      dst[kv_rank + 2 * i] = from_f32<T>(u);
      dst[kv_rank + 2 * i + 1] = from_f32<T>(v);
    }
  }
}

RLLM_EXPORT int rllm_latent_prep(const void* a, int a_stride, int q_rank, int kv_rank, int rot, int rot_dims,
                                 const void* wq, const void* wkv, float eps, void* cq, void* cache,
                                 const int* block_table, int max_blocks, const int* positions,
                                 const int* token_seq, const double* inv_freq, float mag, int page_size,
                                 int num_pages, int write_kv, int T, int dtype, int w_dtype, int* err,
                                 cudaStream_t stream) {
  if (T <= 0) return 0;
  if (q_rank <= 0 || (write_kv && (kv_rank <= 0 || rot < 0 || (rot & 1) || rot_dims > rot || (rot_dims & 1) ||
                                   page_size <= 0 || num_pages <= 0 || max_blocks <= 0)))
    return RLLM_E_BADARG;
#define LP_LAUNCH(T_, TW_)                                                                                \
  rllm_launch_pdl(latent_prep_kernel<T_, TW_>, dim3(T), dim3(128), (size_t)(0), stream, (const T_*)a, a_stride, q_rank, kv_rank, rot, rot_dims, \
      (const TW_*)wq, (const TW_*)wkv, eps, (T_*)cq, (T_*)cache, block_table, max_blocks, positions,      \
      token_seq, inv_freq, mag, page_size, num_pages, write_kv, err)
  RLLM_DISPATCH_DTYPE(dtype, TT, RLLM_DISPATCH_DTYPE(w_dtype, TW, LP_LAUNCH(TT, TW)));
#undef LP_LAUNCH
  RLLM_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// the queries' rotated part: q[t, h, dim : dim+rot] rotated -> qt[t, h, kv_rank : kv_rank+rot]
// ---------------------------------------------------------------------------
template <typename T>
__global__ void latent_q_rot_kernel(const T* q, T* qt, const int* positions,
                                    const double* inv_freq, float mag, int heads, int dim, int rot,
                                    int rot_dims, int kv_rank, long long total) {
  pdl_wait();
  pdl_launch();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int half = rot / 2;
  const int i = (int)(idx % half);
  const long long th = idx / half;
  const int h = (int)(th % heads);
  const long long t = th / heads;
  const T* src = q + ((size_t)t * heads + h) * (dim + rot) + dim;
  T* dst = qt + ((size_t)t * heads + h) * (kv_rank + rot) + kv_rank;
  const float u = to_f32(src[2 * i]), v = to_f32(src[2 * i + 1]);
  if (2 * i + 1 < rot_dims) {
    float c, sn;
    rot_cos_sin<T>(positions[t], inv_freq[i], &c, &sn);
    c *= mag; sn *= mag;
    dst[2 * i] = from_f32<T>(u * c - v * sn);
    dst[2 * i + 1] = from_f32<T>(v * c + u * sn);
  } else {
    dst[2 * i] = from_f32<T>(u);
    dst[2 * i + 1] = from_f32<T>(v);
  }
}

RLLM_EXPORT int rllm_latent_q_rot(const void* q, void* qt, const int* positions, const double* inv_freq, float mag, int T,
                                  int heads, int dim, int rot, int rot_dims, int kv_rank, int dtype,
                                  cudaStream_t stream) {
  const long long total = (long long)T * heads * (rot / 2);
  if (total <= 0) return 0;
  if (rot & 1 || rot_dims > rot || (rot_dims & 1)) return RLLM_E_BADARG;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  RLLM_DISPATCH_DTYPE(dtype, TT, (rllm_launch_pdl(latent_q_rot_kernel<TT>, dim3(blocks), dim3(256), (size_t)(0), stream, 
      (const TT*)q, (TT*)qt, positions, inv_freq, mag, heads, dim, rot, rot_dims, kv_rank, total)));
  RLLM_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// products per head: C[m, h, 0:N] = A[m, h, 0:K] . B[h], with B[h] either [N, K] or [K, N];
// A, B and C are slices with their own row and head strides (elements)
// ---------------------------------------------------------------------------
template <typename T, int BM, bool B_KN>
__global__ void __launch_bounds__(TG_THREADS)
head_gemm_kernel(const T* A, long long lda, long long a_head, const T* B, long long ldb,
                 long long b_head, T* C, long long ldc, long long c_head, int M, int N, int K) {
  pdl_wait();
  pdl_launch();
  __shared__ TileGemmSmem<BM> sm;
  const int h = blockIdx.z, m0 = blockIdx.y * BM, n0 = blockIdx.x * TG_BN;
  if (threadIdx.x < BM) {
    const int m = m0 + threadIdx.x;
    sm.rows[threadIdx.x] = (m < M) ? (const void*)(A + (size_t)m * lda + (size_t)h * a_head) : nullptr;
  }
  __syncthreads();
  float acc[BM / 16][4];
  tile_gemm_accumulate<T, BM, B_KN>(sm, B + (size_t)h * b_head, ldb, n0, N, K, acc);
  const int tm = (threadIdx.x / 16) * (BM / 16), tn = (threadIdx.x % 16) * 4;
#pragma unroll
  for (int i = 0; i < BM / 16; ++i) {
    const int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + j;
      if (n < N) C[(size_t)m * ldc + (size_t)h * c_head + n] = from_f32<T>(acc[i][j]);
    }
  }
}

template <int BM>
__global__ void __launch_bounds__(TGM_THREADS)
head_gemm_mma_kernel(const bf16* A, long long lda, long long a_head, const bf16* B,
                     long long ldb, long long b_head, bf16* C, long long ldc, long long c_head, int M,
                     int N, int K) {
  pdl_wait();
  pdl_launch();
  MmaTileSmem<BM, 1>& sm = tgm_smem<BM, 1>();
  const int h = blockIdx.z, m0 = blockIdx.y * BM, n0 = blockIdx.x * TGM_BN;
  if (threadIdx.x < BM) {
    const int m = m0 + threadIdx.x;
    sm.rows[threadIdx.x] = (m < M) ? (const void*)(A + (size_t)m * lda + (size_t)h * a_head) : nullptr;
  }
  __syncthreads();
  float acc[1][TgmShape<BM>::NT][4];
  const bf16* const Bh[1] = {B + (size_t)h * b_head};
  tile_gemm_mma<BM, 1>(sm, Bh, ldb, n0, N, K, acc);
#pragma unroll
  for (int nt = 0; nt < TgmShape<BM>::NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int tr, tc;
      tgm_coord<BM>(nt, i, tr, tc);
      const int m = m0 + tr, n = n0 + tc;
      if (m < M && n < N) C[(size_t)m * ldc + (size_t)h * c_head + n] = __float2bfloat16_rn(acc[0][nt][i]);
    }
}

RLLM_EXPORT int rllm_head_gemm(const void* A, long long lda, long long a_head, const void* B, long long ldb,
                               long long b_head, int b_kn, void* C, long long ldc, long long c_head, int M, int N,
                               int K, int heads, int dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || heads <= 0) return 0;
  if (K <= 0 || heads > 65535) return RLLM_E_BADARG;
  const bool small = M <= 16;
  const int bm = small ? 16 : 64;
  dim3 grid((N + TG_BN - 1) / TG_BN, (M + bm - 1) / bm, heads);
  if (grid.y > 65535) return RLLM_E_UNSUPPORTED;
  if (dtype == RLLM_DT_BF16 && !b_kn && !tgm_disabled() && K % 8 == 0 && lda % 8 == 0 && a_head % 8 == 0 &&
      ldb % 8 == 0 && b_head % 8 == 0 && (((uintptr_t)A | (uintptr_t)B) & 15) == 0) {
    if (small)
      rllm_launch_pdl(head_gemm_mma_kernel<16>, dim3(grid), dim3(TGM_THREADS), (size_t)(sizeof(MmaTileSmem<16, 1>)), stream, (const bf16*)A, lda, a_head, (const bf16*)B, ldb,
                                                                 b_head, (bf16*)C, ldc, c_head, M, N, K);
    else
      rllm_launch_pdl(head_gemm_mma_kernel<64>, dim3(grid), dim3(TGM_THREADS), (size_t)(sizeof(MmaTileSmem<64, 1>)), stream, (const bf16*)A, lda, a_head, (const bf16*)B, ldb,
                                                                 b_head, (bf16*)C, ldc, c_head, M, N, K);
    RLLM_LAUNCH_CHECK();
    return 0;
  }
#define HG_LAUNCH(T_, BM_, KN_)                                                                          \
  rllm_launch_pdl(head_gemm_kernel<T_, BM_, KN_>, dim3(grid), dim3(TG_THREADS), (size_t)(0), stream, (const T_*)A, lda, a_head, (const T_*)B, \
      ldb, b_head, (T_*)C, ldc, c_head, M, N, K)
  RLLM_DISPATCH_DTYPE(dtype, TT, {
    if (small) { if (b_kn) HG_LAUNCH(TT, 16, true); else HG_LAUNCH(TT, 16, false); }
    else { if (b_kn) HG_LAUNCH(TT, 64, true); else HG_LAUNCH(TT, 64, false); }
  });
#undef HG_LAUNCH
  RLLM_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// attention over the cached rows, one warp per (query token, head).  Keys are walked
// in groups of 32 aligned to absolute positions, so a row's arithmetic does not depend
// on the cut of the sequence, on the batch or on the pages.
// ---------------------------------------------------------------------------
#define LA_WARPS 4

template <typename T, int R>
__global__ void __launch_bounds__(32 * LA_WARPS)
latent_attention_simt_kernel(const T* q, T* out, const T* cache,
                             const int* block_table, int max_blocks,
                             const int* positions, const int* token_seq, int T_tokens,
                             int heads, int dk, int dv, int page_size, int num_pages, int window, float scale,
                             const float* sink, int* err) {
  pdl_wait();
  pdl_launch();
  extern __shared__ float qs[];  // [LA_WARPS][dk]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long gw = (long long)blockIdx.x * LA_WARPS + warp;
  if (gw >= (long long)T_tokens * heads) return;
  const int t = (int)(gw / heads), h = (int)(gw - (long long)t * heads);
  const int s = token_seq[t];
  const int qpos = positions[t];
  const int kend = qpos + 1;
  const int kstart = (window > 0 && qpos - window + 1 > 0) ? qpos - window + 1 : 0;
  float* myq = qs + warp * dk;
  const T* qrow = q + ((size_t)t * heads + h) * dk;
  for (int i = lane; i < dk; i += 32) myq[i] = to_f32(qrow[i]);
  __syncwarp();
  // a sink is one more term of the denominator: the running max starts at it, the running sum at 1
  float m = sink ? sink[h] : -INFINITY, l = sink ? 1.f : 0.f;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  const int* bt = block_table + (size_t)s * max_blocks;
  const bool vec = (dk % 8 == 0) && ((uintptr_t)cache % 16 == 0);
  for (int j0 = (kstart / 32) * 32; j0 < kend; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = (j >= kstart) && (j < kend);
    float score = -INFINITY;
    int page = -1;
    if (valid) {
      page = bt[j / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, 4);
        page = -1;
      } else {
        const T* kp = cache + ((size_t)page * page_size + (j % page_size)) * dk;
        float dot = 0.f;
        if (vec) {
          for (int i = 0; i < dk; i += 8) {
            float kv[8];
            if (sizeof(T) == 4) {
              const float4 a = *(const float4*)(kp + i), b = *(const float4*)(kp + i + 4);
              kv[0] = a.x; kv[1] = a.y; kv[2] = a.z; kv[3] = a.w; kv[4] = b.x; kv[5] = b.y; kv[6] = b.z; kv[7] = b.w;
            } else {
              const uint4 a = *(const uint4*)(kp + i);
              const __nv_bfloat162* hh = (const __nv_bfloat162*)&a;
#pragma unroll
              for (int u = 0; u < 4; ++u) { const float2 f = __bfloat1622float2(hh[u]); kv[2 * u] = f.x; kv[2 * u + 1] = f.y; }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) dot = fmaf(myq[i + u], kv[u], dot);
          }
        } else {
          for (int i = 0; i < dk; ++i) dot = fmaf(myq[i], to_f32(kp[i]), dot);
        }
        score = dot * scale;
      }
    }
    const float cmax = warp_max(score);
    const float m_new = fmaxf(m, cmax);
    if (m_new == -INFINITY) continue;  // nothing visible in this group (warp-uniform)
    const float p = (score == -INFINITY) ? 0.f : expf(score - m_new);
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] *= corr;
    m = m_new;
    const int jn = min(32, kend - j0);
    for (int jj = max(0, kstart - j0); jj < jn; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int pg = __shfl_sync(0xffffffffu, page, jj);
      if (pg < 0) continue;
      const T* vp = cache + ((size_t)pg * page_size + ((j0 + jj) % page_size)) * dk;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = lane + 32 * r;
        if (i < dv) acc[r] = fmaf(pj, to_f32(vp[i]), acc[r]);
      }
    }
  }
  T* orow = out + ((size_t)t * heads + h) * dv;
  const float inv = (l > 0.f) ? 1.0f / l : 0.f;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
    if (i < dv) orow[i] = from_f32<T>(acc[r] * inv);
  }
}

RLLM_EXPORT int rllm_latent_attention_simt(const void* q, void* out, const void* cache, int dtype,
                                           const int* block_table, int max_blocks, const int* positions,
                                           const int* token_seq, int T, int heads, int dk, int dv, int page_size,
                                           int num_pages, int window, float scale, const float* sink, int* err,
                                           cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads <= 0 || dk <= 0 || dv <= 0 || dv > dk || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 ||
      window < 0)
    return RLLM_E_BADARG;
  if (dv > 1024 || (size_t)LA_WARPS * dk * sizeof(float) > 48 * 1024) return RLLM_E_UNSUPPORTED;
  const long long warps = (long long)T * heads;
  const unsigned blocks = (unsigned)((warps + LA_WARPS - 1) / LA_WARPS);
  const size_t smem = (size_t)LA_WARPS * dk * sizeof(float);
#define LA_LAUNCH(T_, R_)                                                                                   \
  rllm_launch_pdl(latent_attention_simt_kernel<T_, R_>, dim3(blocks), dim3(32 * LA_WARPS), (size_t)(smem), stream, (const T_*)q, (T_*)out,     \
      (const T_*)cache, block_table, max_blocks, positions, token_seq, T, heads, dk, dv, page_size, num_pages, \
      window, scale, sink, err)
  RLLM_DISPATCH_DTYPE(dtype, TT, {
    if (dv <= 128) LA_LAUNCH(TT, 4);
    else if (dv <= 256) LA_LAUNCH(TT, 8);
    else if (dv <= 512) LA_LAUNCH(TT, 16);
    else LA_LAUNCH(TT, 32);
  });
#undef LA_LAUNCH
  RLLM_LAUNCH_CHECK();
  return 0;
}
