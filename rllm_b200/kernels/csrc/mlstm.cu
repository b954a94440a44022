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
//   mlstm_scan           one block per (sequence, head, 64 or 128 value columns): it walks the
//                        sequence's tokens of this step in order with its slice of S in
//                        registers (a warp 16 rows, a lane two or four columns; n alike; every block
//                        of a head carries n, the first writes it back).  Long portions are cut into chunks of 64
//                        tokens that run side by side: every chunk's end state from zero, then
//                        the states at the chunks' starts chunk after chunk (an elementwise
//                        pass), then every chunk's tokens from its start state.  Either way a
//                        token's result is the recurrence's; the two ways differ by rounding.
//   head_gated_rmsnorm   out = o / sqrt(mean_head(o^2) + eps) * w * sigmoid(g): the norm runs
//                        over each head's dv values, w is [heads * dv]; one warp a (token, head).
#include "common.cuh"
#include <math.h>

#define ML_MAX_D 256

__device__ __forceinline__ float ml_soft_cap(float z, float cap) { return cap > 0.f ? cap * tanhf(z / cap) : z; }
__device__ __forceinline__ float ml_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// MODE 0: a unit is a sequence: all its tokens of this step, from its state slot and back into it.
// MODE 1: a unit is a chunk of ML_CHUNK tokens of a sequence: its end state from a zero state under a maximum of
//         its own that starts at minus infinity (S, n, that maximum, and the sum of the chunk's log forget gates)
//         goes to `local`; nothing else is written.
// MODE 2: a unit is such a chunk, started from the state that `start` holds for it; outputs are written, and the
//         sequence's last chunk writes the slot.
// Units of MODE 1 and 2 are numbered sequence by sequence; a block finds its sequence by walking q_start.
#define ML_CHUNK 64

#define ML_R 16                 // rows of S a thread keeps in registers

// the gates' pre-activations become the log gates, in place: gates[t][h] <- a, gates[t][heads + h] <- b
__global__ void __launch_bounds__(256)
mlstm_gates_kernel(float* gates, const float* bias_i, const float* bias_f, float cap, long long n, int heads) {
  pdl_wait();
  pdl_launch();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const long long t = idx / heads;
  const int h = (int)(idx - t * heads);
  float* g = gates + t * 2 * heads;
  g[h] = ml_soft_cap(g[h] + (bias_i ? bias_i[h] : 0.f), cap);
  g[heads + h] = ml_logsigmoid(ml_soft_cap(g[heads + h] + (bias_f ? bias_f[h] : 0.f), cap));
}

// A block: (32 NC value columns, head, unit); warp w keeps rows w * ML_R .. of its columns of S in registers (a
// lane NC columns, 32 apart) and lanes 0 .. ML_R - 1 of it the same rows of n.  Tokens go in segments of
// ML_SEG: first the segment's factors exp(b + m' - m), exp(a - m) and maxima m are made once for all threads
// (the gates fetched side by side, the chain over m walked by one thread) and the segment's keys, queries and
// values are put into shared memory as float32, all loads in flight together.  Then four tokens at a time: every
// thread updates its rows token after token and adds up its parts of S^T q; the warps' parts (and those of n . q)
// meet in shared memory (two buffers, so one barrier a group serves), and the first warp finishes the group
// before last while the others work on.
#define ML_G 4                  // tokens between two barriers
#define ML_SEG 32               // tokens whose rows are staged in shared memory at a time

// NC: value columns a lane (a block covers 32 NC columns)
template <typename T, int MODE, int NC>
__global__ void __launch_bounds__(512)
mlstm_scan_kernel(const T* q, const T* k, const T* v, int stride, const float* gates, float qscale, float* state,
                  const int* q_start, const int* slots, float* out, int num_seqs, int heads, int d, int dv,
                  int num_slots, float* local, float* start, int* err) {
  pdl_wait();
  pdl_launch();
  extern __shared__ __align__(16) float sm[];
  __shared__ float g_keep[ML_CHUNK], g_take[ML_CHUNK], g_m[ML_CHUNK];
  constexpr int ML_COLS = 32 * NC, ML_PART = ML_COLS + 1;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, W = blockDim.x >> 5;
  const int dpad = W * ML_R;
  float* kf = sm;                                  // [ML_SEG][dpad]: the segment's keys
  float* qf = kf + ML_SEG * dpad;                  // [ML_SEG][dpad]: its queries
  float* vf = qf + ML_SEG * dpad;                  // [ML_SEG][32 NC]: its values of this block's columns
  float* part = vf + ML_SEG * ML_COLS;             // [2][ML_G][W][65]: the warps' parts of S^T q for 64 columns, and of n . q
  const int j0 = blockIdx.x * ML_COLS + lane;                    // this lane's value columns: j0 + 32 c
  const int h = blockIdx.y;
  int s = blockIdx.z, t0, t1;
  const int unit = blockIdx.z;
  bool last_chunk = true;
  if (MODE == 0) {
    t0 = q_start[s];
    t1 = q_start[s + 1];
  } else {
    int left = blockIdx.z;
    s = -1;
    for (int i = 0; i < num_seqs; ++i) {
      const int n = (q_start[i + 1] - q_start[i] + ML_CHUNK - 1) / ML_CHUNK;
      if (left < n) { s = i; break; }
      left -= n;
    }
    if (s < 0) return;
    t0 = q_start[s] + left * ML_CHUNK;
    t1 = min(t0 + ML_CHUNK, q_start[s + 1]);
    last_chunk = t1 == q_start[s + 1];
    if (MODE == 1 && last_chunk) return;             // nobody reads the end state of a sequence's last chunk
  }
  if (t1 <= t0) return;
  const int slot = slots[s];
  if (slot < 0 || slot >= num_slots) {
    if (tid == 0) atomicOr(err, 8);
    return;
  }
  const size_t per_head = (size_t)d * dv + d + 1;
  float* st = state + ((size_t)slot * heads + h) * per_head;
  // (MODE 2 reads every chunk's start state, the first one's too, from `start`: the slot is written by the
  // sequence's last chunk, which may run at the same time)
  const float* from = MODE == 2 ? start + ((size_t)unit * heads + h) * per_head : st;
  bool live[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) live[c] = j0 + 32 * c < dv;
  const int i0 = w * ML_R;
  const int ni = i0 + lane;              // the row of n this lane keeps (lanes below ML_R)
  float S[NC][ML_R];
  float nreg = 0.f, m = -INFINITY, bsum = 0.f;       // m, bsum: the first thread's
#pragma unroll
  for (int c = 0; c < NC; ++c)
#pragma unroll
    for (int r = 0; r < ML_R; ++r)
      S[c][r] = (MODE != 1 && live[c] && i0 + r < d) ? from[(size_t)(i0 + r) * dv + j0 + 32 * c] : 0.f;
  if (MODE != 1) {
    if (lane < ML_R && ni < d) nreg = from[(size_t)d * dv + ni];
    m = from[(size_t)d * dv + d];
  }
  auto finish = [&](int t, int end, int buf, int g0) { // the first warp: the parts of tokens t .. become outputs
    for (int x = 0; x < ML_G && t + x < end; ++x) {
      float num[NC], dot = 0.f;
#pragma unroll
      for (int c = 0; c < NC; ++c) num[c] = 0.f;
      const float* pp = part + (size_t)((buf * ML_G + x) * W) * ML_PART;
      for (int y = 0; y < W; ++y) {
#pragma unroll
        for (int c = 0; c < NC; ++c) num[c] += pp[y * ML_PART + 32 * c + lane];
        dot += pp[y * ML_PART + ML_COLS];
      }
      // (the queries' scale is applied here, to both sums)
      const float inv = qscale / (fmaxf(fabsf(dot * qscale), expf(-g_m[g0 + x])) + 1e-6f);
#pragma unroll
      for (int c = 0; c < NC; ++c)
        if (live[c]) out[(size_t)(t + x) * heads * dv + (size_t)h * dv + j0 + 32 * c] = num[c] * inv;
    }
  };
  const int cols = min(ML_COLS, dv - blockIdx.x * ML_COLS);
  for (int seg = t0; seg < t1; seg += ML_SEG) {
    const int seg_end = min(seg + ML_SEG, t1);
    const int count = seg_end - seg;
    const int padded = (count + ML_G - 1) / ML_G * ML_G;                   // the last group is filled up
    // the segment's rows into shared memory as float32 (all loads of a segment are in flight together), zeros
    // behind its end; its gates side by side, then the chain over the maximum by one thread
    for (int idx = tid; idx < padded * dpad; idx += blockDim.x) {
      const int x = idx / dpad, e = idx - x * dpad;
      const bool in = x < count && e < d;
      kf[idx] = in ? to_f32(k[(size_t)(seg + x) * stride + (size_t)h * d + e]) : 0.f;
      if (MODE != 1) qf[idx] = in ? to_f32(q[(size_t)(seg + x) * stride + (size_t)h * d + e]) : 0.f;
    }
    for (int idx = tid; idx < padded * ML_COLS; idx += blockDim.x) {
      const int x = idx / ML_COLS, c = idx - x * ML_COLS;
      vf[idx] = (x < count && c < cols) ? to_f32(v[(size_t)(seg + x) * stride + (size_t)h * dv + blockIdx.x * ML_COLS + c]) : 0.f;
    }
    for (int x = tid; x < count; x += blockDim.x) {
      g_keep[x] = gates[(size_t)(seg + x) * 2 * heads + heads + h];         // b
      g_take[x] = gates[(size_t)(seg + x) * 2 * heads + h];                 // a
    }
    __syncthreads();
    if (tid == 0) {
      for (int x = 0; x < padded; ++x) {
        if (x >= count) { g_keep[x] = 1.f; g_take[x] = 0.f; g_m[x] = m; continue; }
        const float b = g_keep[x], a = g_take[x];
        const float m_new = fmaxf(b + m, a);
        g_keep[x] = expf(b + m - m_new);
        g_take[x] = expf(a - m_new);
        g_m[x] = m_new;
        m = m_new;
        bsum += b;
      }
    }
    __syncthreads();
    int grp = 0;
    for (int t = seg; t < seg_end; t += ML_G, ++grp) {
      const int buf = grp & 1, g0 = grp * ML_G;
      if (grp > 0) {
        __syncthreads();                 // the parts of the group before are in
        if (MODE != 1 && w == 0) finish(t - ML_G, seg_end, buf ^ 1, g0 - ML_G);
      }
#pragma unroll
      for (int x = 0; x < ML_G; ++x) {
        const float keep = g_keep[g0 + x], take = g_take[g0 + x];
        const float4* k4 = (const float4*)(kf + (size_t)(g0 + x) * dpad + i0);
        const float4* q4 = (const float4*)(qf + (size_t)(g0 + x) * dpad + i0);
        float vv[NC], acc[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) { vv[c] = take * vf[(g0 + x) * ML_COLS + 32 * c + lane]; acc[c] = 0.f; }
#pragma unroll
        for (int r4 = 0; r4 < ML_R / 4; ++r4) {
          const float4 kk = k4[r4];
          float4 qq = make_float4(0.f, 0.f, 0.f, 0.f);
          if (MODE != 1) qq = q4[r4];
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            S[c][4 * r4 + 0] = fmaf(keep, S[c][4 * r4 + 0], kk.x * vv[c]);
            S[c][4 * r4 + 1] = fmaf(keep, S[c][4 * r4 + 1], kk.y * vv[c]);
            S[c][4 * r4 + 2] = fmaf(keep, S[c][4 * r4 + 2], kk.z * vv[c]);
            S[c][4 * r4 + 3] = fmaf(keep, S[c][4 * r4 + 3], kk.w * vv[c]);
            if (MODE != 1) {
              acc[c] = fmaf(S[c][4 * r4 + 0], qq.x, acc[c]);
              acc[c] = fmaf(S[c][4 * r4 + 1], qq.y, acc[c]);
              acc[c] = fmaf(S[c][4 * r4 + 2], qq.z, acc[c]);
              acc[c] = fmaf(S[c][4 * r4 + 3], qq.w, acc[c]);
            }
          }
        }
        float pd = 0.f;
        if (lane < ML_R) {
          nreg = fmaf(keep, nreg, take * kf[(size_t)(g0 + x) * dpad + ni]);
          if (MODE != 1) pd = nreg * qf[(size_t)(g0 + x) * dpad + ni];
        }
        if (MODE != 1) {
          pd = warp_sum(pd);
          float* pp = part + (size_t)((buf * ML_G + x) * W + w) * ML_PART;
#pragma unroll
          for (int c = 0; c < NC; ++c) pp[32 * c + lane] = acc[c];
          if (lane == 0) pp[ML_COLS] = pd;
        }
      }
    }
    __syncthreads();          // the segment's last parts are in; and everybody is through with its rows and factors
    if (MODE != 1 && w == 0) finish(seg + (grp - 1) * ML_G, seg_end, (grp - 1) & 1, (grp - 1) * ML_G);
  }
  float* to = nullptr;
  if (MODE == 0 || (MODE == 2 && last_chunk)) to = st;
  if (MODE == 1) to = local + ((size_t)unit * heads + h) * (per_head + 1);
  if (to == nullptr) return;
#pragma unroll
  for (int c = 0; c < NC; ++c)
#pragma unroll
    for (int r = 0; r < ML_R; ++r)
      if (live[c] && i0 + r < d) to[(size_t)(i0 + r) * dv + j0 + 32 * c] = S[c][r];
  if (blockIdx.x == 0) {
    if (lane < ML_R && ni < d) to[(size_t)d * dv + ni] = nreg;
    if (tid == 0) {
      to[(size_t)d * dv + d] = m;
      if (MODE == 1) to[(size_t)d * dv + d + 1] = bsum;
    }
  }
}

// Between the two chunked passes: from the chunks' local end states to the state at every chunk's start, chunk
// after chunk.  With (X, m) the state at a chunk's start, (L, m', B) the chunk's local end state, its maximum and
// the sum of its log forget gates:  m_end = max(m + B, m'),  X_end = exp(m + B - m_end) X + exp(m' - m_end) L.
// One thread an element of a head's state; grid (elements / 256, heads, sequences).
__global__ void __launch_bounds__(256)
mlstm_chunk_starts_kernel(const float* state, const int* q_start, const int* slots, const float* local, float* start,
                          int num_seqs, int heads, int d, int dv, int num_slots) {
  pdl_wait();
  pdl_launch();
  const int s = blockIdx.z, h = blockIdx.y;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const int per = d * dv + d;                       // S and n; the maximum lies behind them
  int base = 0;
  for (int i = 0; i < s; ++i) base += (q_start[i + 1] - q_start[i] + ML_CHUNK - 1) / ML_CHUNK;
  const int nc = (q_start[s + 1] - q_start[s] + ML_CHUNK - 1) / ML_CHUNK;
  const int slot = slots[s];
  if (nc < 1 || slot < 0 || slot >= num_slots || e >= per) return;
  const size_t per_head = (size_t)per + 1;
  const float* st = state + ((size_t)slot * heads + h) * per_head;
  float x = st[e], m = st[per];
  for (int c = 0; c < nc; ++c) {
    float* X = start + ((size_t)(base + c) * heads + h) * per_head;
    X[e] = x;                                       // (the first chunk's start is the slot's state)
    if (e == 0) X[per] = m;
    if (c + 1 == nc) break;
    const float* L = local + ((size_t)(base + c) * heads + h) * (per_head + 1);
    const float ml = L[per], B = L[per + 1];
    const float m_end = fmaxf(m + B, ml);
    x = fmaf(expf(m + B - m_end), x, expf(ml - m_end) * L[e]);
    m = m_end;
  }
}

// q, k: rows of heads * d; v: rows of heads * dv; all three with the row stride `stride` (views into one
// product's result).  gates float32 [T, 2 heads]: the input gates' pre-activations, then the forget gates'.
// They are turned into the log gates in place by a first launch.
// state float32 [slots, heads, d * dv + d + 1]; out float32 [T, heads * dv].
// chunks > 0 (the number of chunks of ML_CHUNK tokens over all sequences, each sequence cut from its first token
// of this step) with workspaces local [chunks, heads, d * dv + d + 2] and start [chunks, heads, d * dv + d + 1]:
// three launches that work on all chunks side by side; chunks == 0: one warp walks a sequence's tokens.
RLLM_EXPORT int rllm_mlstm_scan(const void* q, const void* k, const void* v, int stride, int dtype, float* gates,
                                const float* bias_i, const float* bias_f, float cap, float qscale, float* state,
                                const int* q_start, const int* slots, float* out, int num_tokens, int num_seqs,
                                int heads, int d, int dv, int num_slots, int chunks, float* local, float* start,
                                int* err, cudaStream_t stream) {
  if (num_seqs <= 0 || num_tokens <= 0) return 0;
  if (heads <= 0 || d <= 0 || dv <= 0 || num_slots <= 0 || !(cap >= 0.f) || chunks < 0) return RLLM_E_BADARG;
  if (chunks > 0 && (!local || !start)) return RLLM_E_BADARG;
  if (d > ML_MAX_D || heads > 65535 || num_seqs > 65535 || chunks > 65535) return RLLM_E_UNSUPPORTED;
  const int W = (d + ML_R - 1) / ML_R;
  // the walk over a sequence's tokens (decoding, short portions) takes two value columns a lane, so that a few
  // sequences still make many blocks; the chunk passes take four where the head is wide enough
  const long long warps4 = (long long)((dv + 127) / 128) * heads * (chunks > 0 ? chunks : num_seqs) * W;
  const int nc_chunks = (dv > 64 && warps4 >= 148LL * 16) ? 4 : 2;      // (four only while the GPU stays filled)
#define ML_SMEM(NC_) (((size_t)2 * ML_SEG * W * ML_R + (size_t)ML_SEG * 32 * (NC_) + 2 * (size_t)ML_G * W * (32 * (NC_) + 1)) * sizeof(float))
  const long long ng = (long long)num_tokens * heads;
  rllm_launch_pdl(mlstm_gates_kernel, dim3((unsigned)((ng + 255) / 256)), dim3(256), (size_t)0, stream, gates, bias_i,
                  bias_f, cap, ng, heads);
  RLLM_LAUNCH_CHECK();
#define ML_GO_NC(T_, MODE_, NC_, UNITS_)                                                                       \
  do {                                                                                                         \
    const size_t smem = ML_SMEM(NC_);                                                                          \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(mlstm_scan_kernel<T_, MODE_, NC_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    rllm_launch_pdl(mlstm_scan_kernel<T_, MODE_, NC_>, dim3((dv + 32 * NC_ - 1) / (32 * NC_), heads, UNITS_),   \
                    dim3(32 * W), smem, stream, (const T_*)q, (const T_*)k, (const T_*)v, stride,              \
                    (const float*)gates, qscale, state, q_start, slots, out, num_seqs, heads, d, dv, num_slots, \
                    local, start, err);                                                                        \
  } while (0)
#define ML_GO(T_, MODE_, UNITS_)                                                                               \
  do {                                                                                                         \
    if (MODE_ != 0 && nc_chunks == 4) ML_GO_NC(T_, MODE_, 4, UNITS_); else ML_GO_NC(T_, MODE_, 2, UNITS_);     \
  } while (0)
  if (chunks == 0) {
    RLLM_DISPATCH_DTYPE(dtype, TT, ML_GO(TT, 0, num_seqs));
  } else {
    RLLM_DISPATCH_DTYPE(dtype, TT, ML_GO(TT, 1, chunks));
    RLLM_LAUNCH_CHECK();
    rllm_launch_pdl(mlstm_chunk_starts_kernel, dim3((d * dv + d + 255) / 256, heads, num_seqs), dim3(256), (size_t)0,
                    stream, (const float*)state, q_start, slots, (const float*)local, start, num_seqs, heads, d, dv,
                    num_slots);
    RLLM_LAUNCH_CHECK();
    RLLM_DISPATCH_DTYPE(dtype, TT, ML_GO(TT, 2, chunks));
  }
#undef ML_GO
#undef ML_GO_NC
#undef ML_SMEM
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
