// A feed-forward of routed experts.
//   route:    z = W_r h in float32, s = softmax(z) over all experts; the `top` experts
//             with the largest s (lowest index on ties) and their s, as they are.
//   sort:     the (token, choice) pairs ordered by expert: offsets per expert, the
//             pairs in that order, and a list of row tiles (expert, first row), all on
//             the device, so that no size is read back to the host.
//   gate_up:  per expert, y = act(W_gate h, W_up h) for its rows, with
//             act(g, u) = g' sigmoid(alpha g') (u' + shift), g' = min(g, limit),
//             u' = clamp(u, -limit, limit)  (alpha, limit and shift are arguments; alpha 1,
//             no limit and shift 0 give silu(g) u).
//   down:     per expert, W_down y, written to the pair's own row; the weighted sum
//             over a token's pairs is taken by the kernel that reads the result, in
//             the order of the choices.
// A pair's result depends on its token and its expert only: not on the rows beside
// it in a tile, not on the order of the pairs.
#include "tile_gemm.cuh"
#include "tile_gemm_mma.cuh"
#include <math.h>

#define ROUTE_WARPS 4

template <typename T>
__global__ void __launch_bounds__(32 * ROUTE_WARPS)
moe_route_kernel(const T* h, const T* wr, int* ids,
                 float* weights, int T_tokens, int H, int E, int top) {
  // (Every kernel of this file starts with the wait for the kernel ahead of it in the stream and lets the
  // next one in right after: launches overlap the tails of their predecessors.  The pointer parameters
  // carry no __restrict__, so that no load is proved independent of that wait and moved above it.)
  pdl_wait();
  pdl_launch();
  extern __shared__ float zs[];   // [ROUTE_WARPS][E]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T_tokens) return;
  float* z = zs + warp * E;
  const T* x = h + (size_t)t * H;
  for (int e = 0; e < E; ++e) {
    const T* w = wr + (size_t)e * H;
    float part = 0.f;
    for (int i = lane; i < H; i += 32) part = fmaf(to_f32(x[i]), to_f32(w[i]), part);
    part = warp_sum(part);
    if (lane == 0) z[e] = part;
  }
  __syncwarp();
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) sum += expf(z[e] - mx);
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < E; e += 32) z[e] = expf(z[e] - mx) / sum;
  __syncwarp();
  for (int k = 0; k < top; ++k) {
    float best = -1.f;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      float v = z[e];
      if (v != v) v = 0.f;                 // a NaN score still leaves an expert index inside the range
      if (v > best) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) {
      ids[(size_t)t * top + k] = bi;
      weights[(size_t)t * top + k] = best;
      z[bi] = -2.f;
    }
    __syncwarp();
  }
}

// the same choice from logits that a matrix product left in float32: z [T, E].
// groups > 0: the experts form `groups` equal groups of neighbours; a group's score is the largest score in
// it, and only experts of the `keep` groups with the largest scores (lowest index among equals) can be
// chosen.  renorm: the chosen experts' weights are divided by their sum + 1e-20.
__global__ void __launch_bounds__(32 * ROUTE_WARPS)
moe_choose_kernel(const float* logits, int* ids, float* weights,
                  int T_tokens, int E, int top, int groups, int keep, int renorm) {
  pdl_wait();
  pdl_launch();
  extern __shared__ float zs[];   // [ROUTE_WARPS][E + groups]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T_tokens) return;
  float* z = zs + warp * (E + groups);
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) { z[e] = logits[(size_t)t * E + e]; mx = fmaxf(mx, z[e]); }
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) sum += expf(z[e] - mx);
  sum = warp_sum(sum);
  for (int e = lane; e < E; e += 32) z[e] = expf(z[e] - mx) / sum;
  __syncwarp();
  if (groups > 0) {
    float* gs = z + E;
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float b = -1.f;
      for (int e = g * per; e < (g + 1) * per; ++e) { float v = z[e]; if (v != v) v = 0.f; b = fmaxf(b, v); }
      gs[g] = b;
    }
    __syncwarp();
    // a group stays if fewer than `keep` groups stand ahead of it (a larger score, or the same and a lower index)
    for (int g = lane; g < groups; g += 32) {
      int ahead = 0;
      for (int o = 0; o < groups; ++o) ahead += (gs[o] > gs[g] || (gs[o] == gs[g] && o < g)) ? 1 : 0;
      if (ahead >= keep)
        for (int e = g * per; e < (g + 1) * per; ++e) z[e] = -2.f;
    }
    __syncwarp();
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -1.f;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      float v = z[e];
      if (v != v) v = 0.f;
      if (v > best) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    total += best;
    if (lane == 0) {
      ids[(size_t)t * top + k] = bi;
      weights[(size_t)t * top + k] = best;
      z[bi] = -2.f;
    }
    __syncwarp();
  }
  if (renorm && lane == 0) {
    const float inv = 1.0f / (total + 1e-20f);
    for (int k = 0; k < top; ++k) weights[(size_t)t * top + k] *= inv;
  }
}

// Scores that do not compete: s = sigmoid(z) per expert.  The `top` experts with the largest s + bias are
// chosen (bias [E] may be absent; lowest index among equals); their weights are s * scale, the bias left out.
__global__ void __launch_bounds__(32 * ROUTE_WARPS)
moe_choose_sigmoid_kernel(const float* logits, const float* bias, float scale, int* ids, float* weights,
                          int T_tokens, int E, int top) {
  pdl_wait();
  pdl_launch();
  extern __shared__ float zs[];   // [ROUTE_WARPS][2 E]: choice scores, then the scores themselves
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T_tokens) return;
  float* z = zs + warp * 2 * E;
  float* sc = z + E;
  for (int e = lane; e < E; e += 32) {
    float v = 1.0f / (1.0f + expf(-logits[(size_t)t * E + e]));
    if (v != v) v = 0.f;                   // a NaN score still leaves an expert index inside the range
    sc[e] = v;
    z[e] = v + (bias ? bias[e] : 0.f);
  }
  __syncwarp();
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best || (bi == 0x7fffffff && v > -INFINITY)) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (bi >= E) bi = 0;
    if (lane == 0) {
      ids[(size_t)t * top + k] = bi;
      weights[(size_t)t * top + k] = sc[bi] * scale;
      z[bi] = -INFINITY;
    }
    __syncwarp();
  }
}

RLLM_EXPORT int rllm_moe_choose_sigmoid(const float* logits, const float* bias, float scale, int* ids, float* weights,
                                        int T, int E, int top, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || E > 2048) return RLLM_E_BADARG;
  const unsigned blocks = (unsigned)((T + ROUTE_WARPS - 1) / ROUTE_WARPS);
  rllm_launch_pdl(moe_choose_sigmoid_kernel, dim3(blocks), dim3(32 * ROUTE_WARPS),
                  (size_t)((size_t)ROUTE_WARPS * 2 * E * sizeof(float)), stream, logits, bias, scale, ids, weights, T, E, top);
  RLLM_LAUNCH_CHECK();
  return 0;
}

RLLM_EXPORT int rllm_moe_choose(const float* logits, int* ids, float* weights, int T, int E, int top, int groups,
                                int keep, int renorm, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || E > 2048) return RLLM_E_BADARG;
  if (groups < 0 || (groups > 0 && (E % groups || keep < 1 || keep > groups || keep * (E / groups) < top))) return RLLM_E_BADARG;
  const unsigned blocks = (unsigned)((T + ROUTE_WARPS - 1) / ROUTE_WARPS);
  rllm_launch_pdl(moe_choose_kernel, dim3(blocks), dim3(32 * ROUTE_WARPS),
                  (size_t)((size_t)ROUTE_WARPS * (E + groups) * sizeof(float)), stream, logits, ids, weights, T, E, top, groups,
                  keep, renorm);
  RLLM_LAUNCH_CHECK();
  return 0;
}

RLLM_EXPORT int rllm_moe_route(const void* h, const void* wr, int* ids, float* weights, int T, int H, int E,
                               int top, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || E <= 0 || top <= 0 || top > E || E > 2048) return RLLM_E_BADARG;
  const unsigned blocks = (unsigned)((T + ROUTE_WARPS - 1) / ROUTE_WARPS);
  const size_t smem = (size_t)ROUTE_WARPS * E * sizeof(float);
  RLLM_DISPATCH_DTYPE(dtype, TT, (rllm_launch_pdl(moe_route_kernel<TT>, dim3(blocks), dim3(32 * ROUTE_WARPS), (size_t)(smem), stream, 
      (const TT*)h, (const TT*)wr, ids, weights, T, H, E, top)));
  RLLM_LAUNCH_CHECK();
  return 0;
}

// meta: [0] number of tiles.  offsets [E + 1].  sorted [P]: pair indices by expert.
// tile_expert, tile_row0 [max_tiles].
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* ids, int P, int E, int bm, int* offsets,
                int* sorted, int* tile_expert, int* tile_row0,
                int* meta) {
  pdl_wait();
  pdl_launch();
  extern __shared__ int sh[];      // counts [E], start [E + 1], tile_start [E + 1], cursor [E]
  int* cnt = sh;
  int* start = cnt + E;
  int* tstart = start + E + 1;
  int* cur = tstart + E + 1;
  for (int e = threadIdx.x; e < E; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&cnt[min(max(ids[p], 0), E - 1)], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0, b = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = a; tstart[e] = b;
      a += cnt[e];
      b += (cnt[e] + bm - 1) / bm;
    }
    start[E] = a; tstart[E] = b;
    meta[0] = b;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = start[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int n = tstart[e + 1] - tstart[e];
    for (int i = 0; i < n; ++i) {
      tile_expert[tstart[e] + i] = e;
      tile_row0[tstart[e] + i] = start[e] + i * bm;
    }
  }
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = min(max(ids[p], 0), E - 1);
    sorted[start[e] + atomicAdd(&cur[e], 1)] = p;
  }
}

RLLM_EXPORT int rllm_moe_sort(const int* ids, int P, int E, int bm, int* offsets, int* sorted, int* tile_expert,
                              int* tile_row0, int* meta, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (E <= 0 || E > 2048 || (bm != 16 && bm != 64)) return RLLM_E_BADARG;
  const size_t smem = (size_t)(4 * E + 2) * sizeof(int);
  rllm_launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), (size_t)(smem), stream, ids, P, E, bm, offsets, sorted, tile_expert, tile_row0, meta);
  RLLM_LAUNCH_CHECK();
  return 0;
}

// y[row, n] = act(h[token(row)] . Wg[e][n], h[token(row)] . Wu[e][n]);  w: [E, 2 F, H], gate rows then up rows
template <typename T, int BM>
__global__ void __launch_bounds__(TG_THREADS)
moe_gate_up_kernel(const T* h, const T* w, T* y,
                   const int* offsets, const int* sorted,
                   const int* tile_expert, const int* tile_row0,
                   const int* meta, int H, int F, int top, float limit, float alpha, float up_shift) {
  pdl_wait();
  pdl_launch();
  __shared__ TileGemmSmem<BM> sm;
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int e = tile_expert[tile], r0 = tile_row0[tile], rend = offsets[e + 1];
  const int n0 = blockIdx.x * TG_BN;
  if (threadIdx.x < BM) {
    const int r = r0 + threadIdx.x;
    sm.rows[threadIdx.x] = (r < rend) ? (const void*)(h + (size_t)(sorted[r] / top) * H) : nullptr;
  }
  __syncthreads();
  float g[BM / 16][4], u[BM / 16][4];
  const T* we = w + (size_t)e * 2 * F * H;
  tile_gemm_accumulate<T, BM, false>(sm, we, H, n0, F, H, g);
  tile_gemm_accumulate<T, BM, false>(sm, we + (size_t)F * H, H, n0, F, H, u);
  const int tm = (threadIdx.x / 16) * (BM / 16), tn = (threadIdx.x % 16) * 4;
#pragma unroll
  for (int i = 0; i < BM / 16; ++i) {
    const int r = r0 + tm + i;
    if (r >= rend) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + j;
      if (n >= F) continue;
      const float gg = fminf(g[i][j], limit), uu = fminf(fmaxf(u[i][j], -limit), limit);
      y[(size_t)r * F + n] = from_f32<T>(gg * (1.0f / (1.0f + expf(-alpha * gg))) * (uu + up_shift));
    }
  }
}

// out[pair(row), n] = y[row] . Wd[e][n];  w: [E, H, F]
template <typename T, int BM>
__global__ void __launch_bounds__(TG_THREADS)
moe_down_kernel(const T* y, const T* w, T* out,
                const int* offsets, const int* sorted,
                const int* tile_expert, const int* tile_row0,
                const int* meta, int H, int F) {
  pdl_wait();
  pdl_launch();
  __shared__ TileGemmSmem<BM> sm;
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int e = tile_expert[tile], r0 = tile_row0[tile], rend = offsets[e + 1];
  const int n0 = blockIdx.x * TG_BN;
  if (threadIdx.x < BM) {
    const int r = r0 + threadIdx.x;
    sm.rows[threadIdx.x] = (r < rend) ? (const void*)(y + (size_t)r * F) : nullptr;
  }
  __syncthreads();
  float acc[BM / 16][4];
  tile_gemm_accumulate<T, BM, false>(sm, w + (size_t)e * H * F, F, n0, H, F, acc);
  const int tm = (threadIdx.x / 16) * (BM / 16), tn = (threadIdx.x % 16) * 4;
#pragma unroll
  for (int i = 0; i < BM / 16; ++i) {
    const int r = r0 + tm + i;
    if (r >= rend) continue;
    const int pair = sorted[r];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + j;
      if (n < H) out[(size_t)pair * H + n] = from_f32<T>(acc[i][j]);
    }
  }
}

// the same two kernels on the tensor cores (bfloat16)
template <int BM>
__global__ void __launch_bounds__(TGM_THREADS)
moe_gate_up_mma_kernel(const bf16* h, const bf16* w, bf16* y,
                       const int* offsets, const int* sorted,
                       const int* tile_expert, const int* tile_row0,
                       const int* meta, int H, int F, int top, float limit, float alpha, float up_shift) {
  pdl_wait();
  pdl_launch();
  MmaTileSmem<BM, 2>& sm = tgm_smem<BM, 2>();
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int e = tile_expert[tile], r0 = tile_row0[tile], rend = offsets[e + 1];
  const int n0 = blockIdx.x * TGM_BN;
  if (threadIdx.x < BM) {
    const int r = r0 + threadIdx.x;
    sm.rows[threadIdx.x] = (r < rend) ? (const void*)(h + (size_t)(sorted[r] / top) * H) : nullptr;
  }
  __syncthreads();
  float acc[2][TgmShape<BM>::NT][4];
  const bf16* we = w + (size_t)e * 2 * F * H;
  const bf16* const B[2] = {we, we + (size_t)F * H};
  tile_gemm_mma<BM, 2>(sm, B, H, n0, F, H, acc);
#pragma unroll
  for (int nt = 0; nt < TgmShape<BM>::NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int tr, tc;
      tgm_coord<BM>(nt, i, tr, tc);
      const int r = r0 + tr, n = n0 + tc;
      if (r >= rend || n >= F) continue;
      const float gg = fminf(acc[0][nt][i], limit), uu = fminf(fmaxf(acc[1][nt][i], -limit), limit);
      y[(size_t)r * F + n] = __float2bfloat16_rn(gg * (1.0f / (1.0f + expf(-alpha * gg))) * (uu + up_shift));
    }
}

template <int BM>
__global__ void __launch_bounds__(TGM_THREADS)
moe_down_mma_kernel(const bf16* y, const bf16* w, bf16* out,
                    const int* offsets, const int* sorted,
                    const int* tile_expert, const int* tile_row0,
                    const int* meta, int H, int F) {
  pdl_wait();
  pdl_launch();
  MmaTileSmem<BM, 1>& sm = tgm_smem<BM, 1>();
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int e = tile_expert[tile], r0 = tile_row0[tile], rend = offsets[e + 1];
  const int n0 = blockIdx.x * TGM_BN;
  if (threadIdx.x < BM) {
    const int r = r0 + threadIdx.x;
    sm.rows[threadIdx.x] = (r < rend) ? (const void*)(y + (size_t)r * F) : nullptr;
  }
  __syncthreads();
  float acc[1][TgmShape<BM>::NT][4];
  const bf16* const B[1] = {w + (size_t)e * H * F};
  tile_gemm_mma<BM, 1>(sm, B, F, n0, H, F, acc);
#pragma unroll
  for (int nt = 0; nt < TgmShape<BM>::NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int tr, tc;
      tgm_coord<BM>(nt, i, tr, tc);
      const int r = r0 + tr, n = n0 + tc;
      if (r >= rend || n >= H) continue;
      out[(size_t)sorted[r] * H + n] = __float2bfloat16_rn(acc[0][nt][i]);
    }
}

// out[t, :] = sum_k c[t, k] y[t * K + k, :], the k terms in order; then, if `extra` is given,
// + sigmoid(extra_gate[t]) * extra[t, :]  (a part that runs for every token, gated by one number a token)
template <typename T>
__global__ void weighted_slot_sum_kernel(const T* y, const float* c, T* out,
                                         int slots, int H, long long total, const T* extra, const float* extra_gate) {
  pdl_wait();
  pdl_launch();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / H;
  const int i = (int)(idx - t * H);
  float v = 0.f;
  for (int k = 0; k < slots; ++k) v = fmaf(c[t * slots + k], to_f32(y[((size_t)t * slots + k) * H + i]), v);
  if (extra) v = fmaf(extra_gate ? 1.0f / (1.0f + expf(-extra_gate[t])) : 1.0f, to_f32(extra[idx]), v);
  out[idx] = from_f32<T>(v);
}

RLLM_EXPORT int rllm_weighted_slot_sum(const void* y, const float* c, void* out, int T, int slots, int H,
                                       const void* extra, const float* extra_gate, int dtype, cudaStream_t stream) {
  const long long total = (long long)T * H;
  if (total <= 0) return 0;
  if (slots <= 0) return RLLM_E_BADARG;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  RLLM_DISPATCH_DTYPE(dtype, TT, (rllm_launch_pdl(weighted_slot_sum_kernel<TT>, dim3(blocks), dim3(256), (size_t)(0), stream, 
      (const TT*)y, c, (TT*)out, slots, H, total, (const TT*)extra, extra_gate)));
  RLLM_LAUNCH_CHECK();
  return 0;
}

RLLM_EXPORT int rllm_moe_experts(const void* h, const void* w_gate_up, const void* w_down, void* y, void* out,
                                 const int* offsets, const int* sorted, const int* tile_expert,
                                 const int* tile_row0, const int* meta, int max_tiles, int bm, int H, int F,
                                 int top, float limit, float alpha, float up_shift, int dtype, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (H <= 0 || F <= 0 || top <= 0 || (bm != 16 && bm != 64)) return RLLM_E_BADARG;
  if (max_tiles > 65535) return RLLM_E_UNSUPPORTED;
  dim3 g1((F + TG_BN - 1) / TG_BN, max_tiles), g2((H + TG_BN - 1) / TG_BN, max_tiles);
  const bool aligned = H % 8 == 0 && F % 8 == 0 &&
                       (((uintptr_t)h | (uintptr_t)w_gate_up | (uintptr_t)w_down | (uintptr_t)y) & 15) == 0;
  if (dtype == RLLM_DT_BF16 && aligned && !tgm_disabled()) {
#define MOE_MMA(BM_)                                                                                         \
  do {                                                                                                       \
    tgm_allow_smem<decltype(&moe_gate_up_mma_kernel<BM_>), BM_, 2>(moe_gate_up_mma_kernel<BM_>);             \
    rllm_launch_pdl(moe_gate_up_mma_kernel<BM_>, dim3(g1), dim3(TGM_THREADS), (size_t)(sizeof(MmaTileSmem<BM_, 2>)), stream, (const bf16*)h, (const bf16*)w_gate_up,      \
        (bf16*)y, offsets, sorted, tile_expert, tile_row0, meta, H, F, top, limit, alpha, up_shift);                   \
    tgm_allow_smem<decltype(&moe_down_mma_kernel<BM_>), BM_, 1>(moe_down_mma_kernel<BM_>);                   \
    rllm_launch_pdl(moe_down_mma_kernel<BM_>, dim3(g2), dim3(TGM_THREADS), (size_t)(sizeof(MmaTileSmem<BM_, 1>)), stream, (const bf16*)y, (const bf16*)w_down, (bf16*)out, \
        offsets, sorted, tile_expert, tile_row0, meta, H, F);                                                \
  } while (0)
    if (bm == 16) MOE_MMA(16); else MOE_MMA(64);
#undef MOE_MMA
    RLLM_LAUNCH_CHECK();
    return 0;
  }
#define MOE_LAUNCH(T_, BM_)                                                                                  \
  do {                                                                                                       \
    rllm_launch_pdl(moe_gate_up_kernel<T_, BM_>, dim3(g1), dim3(TG_THREADS), (size_t)(0), stream, (const T_*)h, (const T_*)w_gate_up, (T_*)y,    \
        offsets, sorted, tile_expert, tile_row0, meta, H, F, top, limit, alpha, up_shift);                             \
    rllm_launch_pdl(moe_down_kernel<T_, BM_>, dim3(g2), dim3(TG_THREADS), (size_t)(0), stream, (const T_*)y, (const T_*)w_down, (T_*)out, offsets, \
        sorted, tile_expert, tile_row0, meta, H, F);                                                         \
  } while (0)
  RLLM_DISPATCH_DTYPE(dtype, TT, { if (bm == 16) MOE_LAUNCH(TT, 16); else MOE_LAUNCH(TT, 64); });
#undef MOE_LAUNCH
  RLLM_LAUNCH_CHECK();
  return 0;
}
