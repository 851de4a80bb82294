// Linear recurrences with one decay per head and token, as mixers with per-sequence state:
//     S_t = a_t S_(t-1) + b_t k_t v_t^T        o_t = S_t^T q_t        (S is [dk, dv] per head, 32-bit)
// Two designs of mixer reduce to it.  A state-space layer (state-space duality): k = B_t, q = C_t of
// the head's group, v = x_t, a = exp(-exp(A_log) dt), b = dt, dt = softplus(raw + bias).  A matrix
// memory with exponential gates (mLSTM): a = exp(f + m_(t-1) - m_t), b = exp(i - m_t) with the
// running maximum m_t = max(f + m_(t-1), i) and capped gate pre-activations; its normaliser
// n_t = a n + b k is one more column of S whose v is 1.
//
// A column of S never meets another, so the scan runs one column per group of 8 lanes, the column's
// rows in the lanes' registers, sequentially over a sequence's tokens and in parallel over sequences,
// heads and columns.  All kernels take packed rows of several sequences (prompts, portions, single
// tokens); rows whose position is negative belong to finished sequences and are skipped.
//
//   conv_silu        causal convolution per channel with bias, then SiLU; predecessors are found in the
//                    step by slot and position, or in the state's tail
//   conv_tail        the last taps-1 convolution inputs of every sequence -> its state
//   ssm_gates        a, b of the state-space layer
//   xgate_scan       a, b and the running maximum of the matrix memory (a warp a head, 32 tokens a pass)
//   decay_scan       the recurrence; reads and writes S in the state
//   ssm_out          (o + D x) silu(z), RMS norm in equal parts, weight -> activation type
//   xlstm_out        o / (max(|n.q|, exp(-m)) + 1e-6), RMS norm per head, weight, sigmoid gate
// and a recurrence with a decay per CHANNEL and no matrix state (a gated linear recurrent unit):
//   lru_gates        both gates from block-diagonal products, the decay and the gated input
//   lru_scan         S_t = a_t S_(t-1) + x_t per channel, times the GELU of a side branch
// Everything here is 32-bit; only the two output kernels round, once, to the activation type.
#include "common.cuh"

namespace ek {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
// ln(1 + e^x); beyond 20 the sum rounds to e^x in 32 bits, so x itself is the exact result
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// Predecessors of token t inside the step (same slot, positions counting down), at most `most`.
__device__ __forceinline__ int step_predecessors(const int* positions, const int* token_slot, int t, int most) {
  const int slot = token_slot[t], pos = positions[t];
  int n = 0;
  while (n < most && t - n - 1 >= 0 && token_slot[t - n - 1] == slot && positions[t - n - 1] == pos - n - 1) ++n;
  return n;
}

// grid (token tiles, channel tiles).  out[t, c] = silu(bias[c] + sum_j w[c][K-1-j] x[t-j, c]) with
// x = proj[., col0 + c] (+ in_bias[c] for tokens that exist; `act` 0: no SiLU).  tail of a slot: [channels][K-1], oldest first.  A block takes `per_block`
// neighbouring tokens (at most 16), so that a prompt's rows are fetched once into L1 for all their taps.
constexpr int kConvTokens = 16;
__global__ void __launch_bounds__(256)
conv_silu_kernel(float* __restrict__ out, int out_stride, const float* __restrict__ proj, int proj_stride, int col0,
                 const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                 const float* __restrict__ state, size_t slot_stride, size_t tail_offset,
                 const int* __restrict__ positions, const int* __restrict__ token_slot, int n_tokens, int channels,
                 int K, int per_block, const float* __restrict__ in_bias, int act) {
  __shared__ int n_prev_s[kConvTokens], slot_s[kConvTokens], pos_s[kConvTokens];
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * per_block, nt = min(per_block, n_tokens - t0);
  if ((int)threadIdx.x < nt) {
    const int t = t0 + threadIdx.x;
    const bool live = positions[t] >= 0;
    n_prev_s[threadIdx.x] = live ? step_predecessors(positions, token_slot, t, K - 1) : -1;
    slot_s[threadIdx.x] = live ? token_slot[t] : 0;
    pos_s[threadIdx.x] = positions[t];
  }
  __syncthreads();
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    const float* w = conv_w + (size_t)c * K;
    const float bias = conv_b ? conv_b[c] : 0.f;
    const float xb = in_bias ? in_bias[c] : 0.f;       // a bias of the projection itself: only real tokens carry it
    for (int i = 0; i < nt; ++i) {
      const int n_prev = n_prev_s[i], t = t0 + i;
      if (n_prev < 0) continue;
      const float* tail = state + (size_t)slot_s[i] * slot_stride + tail_offset;
      float acc = bias + w[K - 1] * (proj[(size_t)t * proj_stride + col0 + c] + xb);
      for (int j = 1; j < K; ++j) {
        float x = j <= n_prev ? proj[(size_t)(t - j) * proj_stride + col0 + c]
                              : tail[(size_t)c * (K - 1) + (n_prev - j + K - 1)];
        if (pos_s[i] - j >= 0) x += xb;
        acc = fmaf(w[K - 1 - j], x, acc);
      }
      out[(size_t)t * out_stride + c] = act ? acc * sigmoid_f(acc) : acc;
    }
  }
}

// grid (sequences, channel tiles).  After the step the tail holds the sequence's last taps-1 inputs.
__global__ void conv_tail_kernel(float* __restrict__ state, size_t slot_stride, size_t tail_offset,
                                 const float* __restrict__ proj, int proj_stride, int col0,
                                 const int* __restrict__ cu_seqlens, const int* __restrict__ positions,
                                 const int* __restrict__ token_slot, int channels, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
  if (n <= 0 || positions[start] < 0) return;
  float* tail = state + (size_t)token_slot[start] * slot_stride + tail_offset;
  const int keep = taps - 1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float* tc = tail + (size_t)c * keep;
    for (int m = 0; m < keep; ++m) {
      const int from_step = n - keep + m;       // row of the step that lands at place m
      tc[m] = from_step >= 0 ? proj[(size_t)(start + from_step) * proj_stride + col0 + c] : tc[m + n];
    }
  }
}

// The gates of a gated linear recurrence over R = parts * size channels (the real-gated linear recurrent
// unit of Griffin): with u the recurrence's input, cut into `parts` equal parts,
//     r = sigmoid(W_a[p] u_p + b_a),  i = sigmoid(W_i[p] u_p + b_i)          (square matrices per part)
//     log a = -rate * r * softplus(lam),  a = exp(log a),  x = sqrt(1 - a^2) * i * u
// so that the recurrence itself is S_t = a_t S_(t-1) + x_t.  1 - a^2 is taken as -expm1(2 log a), which
// keeps its digits when a is close to 1.  grid (token tiles of 32, parts, output tiles of 128); a block
// stages its tokens' u_p in shared memory, a thread owns one output channel for all 32 tokens, and the
// weights come transposed ([in][out]) so that neighbouring threads read neighbouring words.
constexpr int kLruTokens = 32;
__global__ void __launch_bounds__(128)
lru_gates_kernel(float* __restrict__ a_out, float* __restrict__ x_out, const float* __restrict__ u, int u_stride,
                 const float* __restrict__ w_a, const float* __restrict__ b_a, const float* __restrict__ w_i,
                 const float* __restrict__ b_i, const float* __restrict__ lam, float rate, int n_tokens, int parts,
                 int size) {
  extern __shared__ __align__(16) float u_s[];     // [kLruTokens][ld], ld = size rounded up to 4
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * kLruTokens, p = blockIdx.y, tid = threadIdx.x;
  const int nt = min(kLruTokens, n_tokens - t0);
  const int R = parts * size, ld = (size + 3) & ~3;
  for (int idx = tid; idx < kLruTokens * ld; idx += blockDim.x) {
    const int tt = idx / ld, r = idx % ld;
    u_s[idx] = (tt < nt && r < size) ? u[(size_t)(t0 + tt) * u_stride + p * size + r] : 0.f;
  }
  __syncthreads();
  const int o = blockIdx.z * 128 + tid;
  if (o >= size) return;
  const int c = p * size + o;
  float ra[kLruTokens], ri[kLruTokens];
  const float ba = b_a ? b_a[c] : 0.f, bi = b_i ? b_i[c] : 0.f;
#pragma unroll
  for (int tt = 0; tt < kLruTokens; ++tt) { ra[tt] = ba; ri[tt] = bi; }
  const float* wa = w_a + (size_t)p * size * size + o;
  const float* wi = w_i + (size_t)p * size * size + o;
  int r = 0;
  for (; r + 4 <= size; r += 4) {               // eight weights, then one 16-byte read of a token's four inputs
    float va[4], vi[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { va[j] = wa[(size_t)(r + j) * size]; vi[j] = wi[(size_t)(r + j) * size]; }
#pragma unroll
    for (int tt = 0; tt < kLruTokens; ++tt) {
      const float4 x = *reinterpret_cast<const float4*>(u_s + tt * ld + r);
      ra[tt] = fmaf(va[3], x.w, fmaf(va[2], x.z, fmaf(va[1], x.y, fmaf(va[0], x.x, ra[tt]))));
      ri[tt] = fmaf(vi[3], x.w, fmaf(vi[2], x.z, fmaf(vi[1], x.y, fmaf(vi[0], x.x, ri[tt]))));
    }
  }
  for (; r < size; ++r) {
    const float va = wa[(size_t)r * size], vi = wi[(size_t)r * size];
#pragma unroll
    for (int tt = 0; tt < kLruTokens; ++tt) {
      const float x = u_s[tt * ld + r];
      ra[tt] = fmaf(va, x, ra[tt]);
      ri[tt] = fmaf(vi, x, ri[tt]);
    }
  }
  const float sp = rate * softplus_f(lam[c]);
#pragma unroll
  for (int tt = 0; tt < kLruTokens; ++tt) {
    if (tt < nt) {
      const float log_a = -sp * sigmoid_f(ra[tt]);
      const size_t at = (size_t)(t0 + tt) * R + c;
      a_out[at] = expf(log_a);
      x_out[at] = sqrtf(-expm1f(2.f * log_a)) * sigmoid_f(ri[tt]) * u_s[tt * ld + o];
    }
  }
}

// The same for few tokens (single tokens of a batch): a warp an output channel, its lanes spread over the
// part's inputs, so that a step's few rows still give a block to every SM and every weight is read once, in
// whole lines.  Weights here lie as stored, [part][out][in].  grid (parts * output tiles of 8, token tiles of 8);
// a block stages its tokens' inputs of its part in shared memory once for its eight warps.
constexpr int kLruFewTokens = 8;
__global__ void __launch_bounds__(256)
lru_gates_few_kernel(float* __restrict__ a_out, float* __restrict__ x_out, const float* __restrict__ u, int u_stride,
                     const float* __restrict__ w_a, const float* __restrict__ b_a, const float* __restrict__ w_i,
                     const float* __restrict__ b_i, const float* __restrict__ lam, float rate, int n_tokens, int parts,
                     int size) {
  extern __shared__ __align__(16) float u_few[];              // [kLruFewTokens][size]
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = (size + 7) / 8;
  const int p = blockIdx.x / tiles, o = (blockIdx.x % tiles) * 8 + warp;
  const bool live = o < size;
  const int c = p * size + (live ? o : 0), R = parts * size;
  const float* wa = w_a + (size_t)c * size;     // row c of the part's matrix: [out][in]
  const float* wi = w_i + (size_t)c * size;
  const int t0 = blockIdx.y * kLruFewTokens;
  const int nt = min(kLruFewTokens, n_tokens - t0);
  float va[8], vi[8];                           // the weights do not depend on the kernel before: fetch, then wait
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int r = j * 32 + lane;
    va[j] = (live && r < size) ? wa[r] : 0.f;
    vi[j] = (live && r < size) ? wi[r] : 0.f;
  }
  pdl_wait();
  for (int idx = threadIdx.x; idx < kLruFewTokens * size; idx += blockDim.x) {
    const int tt = idx / size, r = idx % size;
    u_few[idx] = tt < nt ? u[(size_t)(t0 + tt) * u_stride + p * size + r] : 0.f;
  }
  __syncthreads();
  if (!live) return;
  float ra[kLruFewTokens], ri[kLruFewTokens];
#pragma unroll
  for (int tt = 0; tt < kLruFewTokens; ++tt) ra[tt] = ri[tt] = 0.f;
  for (int r0 = 0; r0 < size; r0 += 256) {
    if (r0 > 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int r = r0 + j * 32 + lane;
        va[j] = r < size ? wa[r] : 0.f;
        vi[j] = r < size ? wi[r] : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int r = r0 + j * 32 + lane;
      if (r < size) {
#pragma unroll
        for (int tt = 0; tt < kLruFewTokens; ++tt) {
          const float x = u_few[tt * size + r];
          ra[tt] = fmaf(va[j], x, ra[tt]);
          ri[tt] = fmaf(vi[j], x, ri[tt]);
        }
      }
    }
  }
#pragma unroll
  for (int tt = 0; tt < kLruFewTokens; ++tt) { ra[tt] = warp_sum(ra[tt]); ri[tt] = warp_sum(ri[tt]); }
  if (lane < nt) {
    float sa = 0.f, si = 0.f;
#pragma unroll
    for (int tt = 0; tt < kLruFewTokens; ++tt) if (tt == lane) { sa = ra[tt]; si = ri[tt]; }
    const float log_a = -rate * softplus_f(lam[c]) * sigmoid_f(sa + (b_a ? b_a[c] : 0.f));
    const size_t at = (size_t)(t0 + lane) * R + c;
    a_out[at] = expf(log_a);
    x_out[at] = sqrtf(-expm1f(2.f * log_a)) * sigmoid_f(si + (b_i ? b_i[c] : 0.f)) * u_few[lane * size + o];
  }
}

// S_t = a_t S_(t-1) + x_t per channel and sequence, S read from and written back to the slot's state
// (its first `channels` values, 32-bit); out[t, c] = S_t * gelu_tanh(side[t, side_col + c] + side_bias[c]),
// rounded to the activation type.  grid (sequences, channel tiles of 128): a thread walks one channel's
// tokens; only the multiply-add is on the chain, the loads of the tokens ahead are independent of it.
template <typename T>
__global__ void __launch_bounds__(128)
lru_scan_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ x,
                const float* __restrict__ side, int side_stride, int side_col, const float* __restrict__ side_bias,
                float* __restrict__ state, size_t slot_stride, const int* __restrict__ cu_seqlens,
                const int* __restrict__ positions, const int* __restrict__ token_slot, int channels,
                int write_state) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, c = blockIdx.y * 128 + threadIdx.x;
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
  if (c >= channels || n <= 0) return;
  if (positions[start] < 0) {                   // rows of a finished sequence: zeros, the state untouched
    for (int i = 0; i < n; ++i) out[(size_t)(start + i) * channels + c] = from_f<T>(0.f);
    return;
  }
  float* sp = state + (size_t)token_slot[start] * slot_stride + c;
  float S = *sp;
  const float sb = side_bias ? side_bias[c] : 0.f;
  constexpr int U = 8;
  int i = 0;
  for (; i + U <= n; i += U) {
    float av[U], xv[U], yv[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const size_t row = (size_t)(start + i + j);
      av[j] = a[row * channels + c];
      xv[j] = x[row * channels + c];
      yv[j] = side[row * side_stride + side_col + c] + sb;
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
      S = fmaf(av[j], S, xv[j]);
      const float z = yv[j];
      const float g = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
      out[(size_t)(start + i + j) * channels + c] = from_f<T>(S * g);
    }
  }
  for (; i < n; ++i) {
    const size_t row = (size_t)(start + i);
    S = fmaf(a[row * channels + c], S, x[row * channels + c]);
    const float z = side[row * side_stride + side_col + c] + sb;
    const float g = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    out[row * channels + c] = from_f<T>(S * g);
  }
  if (write_state) *sp = S;
}

// The same recurrence for prompts: a block of 32 warps takes 16 channels and walks a sequence 1,024 tokens a
// pass - 64 neighbouring stretches of 16 tokens, two to a warp (a half-warp a stretch, a lane a channel).  The map
// S -> a S + x of a stretch composes to S -> A S + B; every half-warp forms its stretch's (A, B) from zero, the 64
// meet in shared memory, every half-warp applies the stretches before its own to the state the pass was handed,
// and then walks its tokens again (they are still in L1 / L2) with the true state.  The chain from token to
// token is 16 long instead of the whole run, and a prompt of one sequence still fills the machine's schedulers.
constexpr int kLruWarps = 32, kLruStretch = 16, kLruLanes = 16;
constexpr int kLruSubs = kLruWarps * 32 / kLruLanes;          // stretches a pass
template <typename T>
__global__ void __launch_bounds__(kLruWarps * 32)
lru_scan_wide_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ x,
                     const float* __restrict__ side, int side_stride, int side_col,
                     const float* __restrict__ side_bias, float* __restrict__ state, size_t slot_stride,
                     const int* __restrict__ cu_seqlens, const int* __restrict__ positions,
                     const int* __restrict__ token_slot, int channels, int write_state) {
  __shared__ float A_s[kLruSubs][kLruLanes], B_s[kLruSubs][kLruLanes];
  pdl_launch_dependents();
  pdl_wait();
  const int sub = threadIdx.x / kLruLanes, cl = threadIdx.x % kLruLanes;
  const int b = blockIdx.x, c = blockIdx.y * kLruLanes + cl;
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
  if (n <= 0) return;
  const bool live = c < channels;
  if (positions[start] < 0) {                   // rows of a finished sequence: zeros, the state untouched
    if (live)
      for (int i = sub; i < n; i += kLruSubs) out[(size_t)(start + i) * channels + c] = from_f<T>(0.f);
    return;
  }
  float* sp = state + (size_t)token_slot[start] * slot_stride + c;
  float S0 = live ? *sp : 0.f;
  const float sb = (side_bias && live) ? side_bias[c] : 0.f;
  for (int base = 0; base < n; base += kLruSubs * kLruStretch) {
    const int lo = base + sub * kLruStretch, hi = min(lo + kLruStretch, n);
    float A = 1.f, B = 0.f;
    if (live) {
#pragma unroll 8
      for (int i = lo; i < hi; ++i) {
        const size_t at = (size_t)(start + i) * channels + c;
        const float av = a[at];
        A *= av;
        B = fmaf(av, B, x[at]);
      }
    }
    A_s[sub][cl] = A;
    B_s[sub][cl] = B;
    __syncthreads();
    float S = S0;
    for (int w = 0; w < sub; ++w) S = fmaf(A_s[w][cl], S, B_s[w][cl]);
    if (live) {
#pragma unroll 4
      for (int i = lo; i < hi; ++i) {
        const size_t row = (size_t)(start + i);
        S = fmaf(a[row * channels + c], S, x[row * channels + c]);
        const float z = side[row * side_stride + side_col + c] + sb;
        const float g = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        out[row * channels + c] = from_f<T>(S * g);
      }
    }
    if (base + kLruSubs * kLruStretch < n) {    // the state the next pass starts from
      float all = S;
      for (int w = sub + 1; w < kLruSubs; ++w) all = fmaf(A_s[w][cl], all, B_s[w][cl]);
      S0 = all;
    } else if (write_state && live && lo < n && hi == n) {
      *sp = S;                                  // the stretch that ends the run leaves the state
    }
    __syncthreads();                            // before the next pass overwrites A_s, B_s
  }
}

// a[t, h] = exp(-exp(a_log[h]) dt), b[t, h] = dt, dt = softplus(proj[t, col0 + h] + dt_bias[h]).
__global__ void ssm_gates_kernel(float* __restrict__ a, float* __restrict__ b, const float* __restrict__ proj,
                                 int proj_stride, int col0, const float* __restrict__ dt_bias,
                                 const float* __restrict__ a_log, int n_tokens, int heads) {
  pdl_launch_dependents();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_tokens * heads) return;
  const int t = idx / heads, h = idx % heads;
  const float dt = softplus_f(proj[(size_t)t * proj_stride + col0 + h] + dt_bias[h]);
  a[idx] = expf(-expf(a_log[h]) * dt);
  b[idx] = dt;
}

// grid (sequences, heads); a block a head, 32 tokens a warp.  Log input gate i = cap tanh((x_i + b_i) / cap),
// log forget gate f = logsigmoid(cap tanh((x_f + b_f) / cap)); m_t = max(f_t + m_(t-1), i_t) from the
// state's m; a = exp(f + m_(t-1) - m_t), b = exp(i - m_t), m_run[t, h] = m_t.  The maximum is a scan: the
// maps m -> max(m + F, I) compose as (F1 + F2, max(I1 + F2, I2)); a warp composes its 32 tokens by shuffles,
// the warps' totals meet in shared memory, and 256 tokens are done a pass with no chain from token to token.
constexpr int kGateWarps = 8;
__global__ void __launch_bounds__(kGateWarps * 32)
xgate_scan_kernel(float* __restrict__ a, float* __restrict__ b, float* __restrict__ m_run,
                  const float* __restrict__ proj, int proj_stride, int col_i, int col_f,
                  const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
                  float* __restrict__ state, size_t slot_stride, size_t m_offset,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ positions,
                  const int* __restrict__ token_slot, int heads, int write_state) {
  __shared__ float F_s[2][kGateWarps], I_s[2][kGateWarps];
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int start = cu_seqlens[seq], n = cu_seqlens[seq + 1] - start;
  if (n <= 0 || positions[start] < 0) return;
  float* m_state = state + (size_t)token_slot[start] * slot_stride + m_offset + h;
  float m_in = *m_state;
  const float bi = bias_i[h], bf = bias_f[h];
  // raw gate inputs of the next pass are fetched while this one runs
  auto raw = [&](int c0, float& xi, float& xf) {
    xi = xf = 0.f;
    if (c0 + (int)threadIdx.x < n) {
      const float* row = proj + (size_t)(start + c0 + threadIdx.x) * proj_stride;
      xi = row[col_i + h];
      xf = row[col_f + h];
    }
  };
  float xi_next, xf_next;
  raw(0, xi_next, xf_next);
  int buf = 0;
  for (int c0 = 0; c0 < n; c0 += kGateWarps * 32, buf ^= 1) {
    const int t = start + c0 + threadIdx.x;
    const bool live = c0 + (int)threadIdx.x < n;
    const float xi = xi_next, xf = xf_next;
    if (c0 + kGateWarps * 32 < n) raw(c0 + kGateWarps * 32, xi_next, xf_next);
    float gi = 0.f, gf = 0.f;                    // the identity map for tokens past the end: F = 0, I = -inf
    if (live) {
      gi = cap * tanhf((xi + bi) / cap);
      gf = -softplus_f(-(cap * tanhf((xf + bf) / cap)));
    }
    float F = live ? gf : 0.f, I = live ? gi : -INFINITY;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {           // inclusive scan: the maps of this warp's tokens up to the lane's
      const float F1 = __shfl_up_sync(0xffffffffu, F, o), I1 = __shfl_up_sync(0xffffffffu, I, o);
      if (lane >= o) { I = fmaxf(I1 + F, I); F = F1 + F; }
    }
    if (lane == 31) { F_s[buf][warp] = F; I_s[buf][warp] = I; }
    __syncthreads();                             // (two buffers: the pass after writes the other one)
    float m_warp = m_in;                         // m before this warp's first token
#pragma unroll
    for (int w = 0; w < kGateWarps; ++w) {
      if (w == warp) m_warp = m_in;
      m_in = fmaxf(m_in + F_s[buf][w], I_s[buf][w]);
    }
    const float m = fmaxf(m_warp + F, I);
    float m_prev = __shfl_up_sync(0xffffffffu, m, 1);
    if (lane == 0) m_prev = m_warp;
    if (live) {
      a[(size_t)t * heads + h] = expf(gf + m_prev - m);
      b[(size_t)t * heads + h] = expf(gi - m);
      m_run[(size_t)t * heads + h] = m;
    }
  }
  if (write_state && threadIdx.x == 0) *m_state = m_in;
}

constexpr int kScanCols = 16;        // columns of S a block takes
constexpr int kScanLanes = 8;        // lanes that share a column
constexpr int kScanThreads = kScanCols * kScanLanes;
constexpr int kScanFloats = 2048;    // values of keys (and of queries) fetched into shared memory at a time

// grid (sequences, heads, column tiles).  RPL rows of a column a lane: lane l holds rows 32 g + 4 l + c
// (g < RPL / 4, c < 4), so that the 8 lanes of a column read 128 neighbouring bytes of a key at a time.
// S of a slot: state[((h * C + j) * DK + i], DK = 8 RPL rows (keys padded with zeros), C = dv + ones_col columns.
// Column dv (with ones_col) has v = 1: it carries n_t = a n + b k and gives n.q.
// Tokens come 2048 / DK at a time: while one portion is worked through from shared memory, the next one's
// keys, queries, values and gates are already on their way into registers.
template <int RPL>
__global__ void __launch_bounds__(kScanThreads)
decay_scan_kernel(float* __restrict__ out, int out_stride, const float* __restrict__ q, int q_stride,
                  const float* __restrict__ k, int k_stride, const float* __restrict__ v, int v_stride,
                  const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ state,
                  size_t slot_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ positions,
                  const int* __restrict__ token_slot, int heads, int kv_heads, int dk, int dv, int ones_col,
                  int write_state) {
  constexpr int DK = 8 * RPL, G4 = RPL / 4, DK4 = DK / 4;
  constexpr int CH = kScanFloats / DK;                       // tokens a portion: 64, 32, 16 or 8
  constexpr int NV4 = kScanFloats / 4 / kScanThreads;        // float4 of keys (of queries) a thread fetches
  constexpr int NV = CH * kScanCols / kScanThreads;          // values a thread fetches
  static_assert(CH <= kScanThreads && CH * kScanCols % kScanThreads == 0, "portion sizes");
  __shared__ __align__(16) float k_s[CH][DK];
  __shared__ __align__(16) float q_s[CH][DK];
  __shared__ float v_s[CH][kScanCols];
  __shared__ float a_s[CH], b_s[CH];
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * kScanCols;
  const int start = cu_seqlens[seq], n = cu_seqlens[seq + 1] - start;
  if (n <= 0 || positions[start] < 0) return;
  const int tid = threadIdx.x, col = tid / kScanLanes, lane = tid % kScanLanes;
  const int C = dv + ones_col, j = col0 + col;
  const bool live = j < C;
  const int kv = h / (heads / kv_heads);
  // whole float4 loads need rows and head offsets on 16-byte boundaries
  const bool vec = dk % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 &&
                   (((uintptr_t)q | (uintptr_t)k) & 15) == 0;
  float* sp = state + (size_t)token_slot[start] * slot_stride + ((size_t)h * C + (live ? j : 0)) * DK;
  float4 S[G4];
#pragma unroll
  for (int g = 0; g < G4; ++g)
    S[g] = live ? *reinterpret_cast<const float4*>(sp + 32 * g + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);

  float4 k_r[NV4], q_r[NV4];
  float v_r[NV], a_r = 1.f, b_r = 0.f;
  // rows past the portion's end, and keys past dk, stay zero: the loads are predicated, nothing is selected
  // from a loaded value, so a fetch does not wait for what it asked for
  auto row4 = [&](float4& r, const float* base, size_t t, int stride, int i) {
    const float* p = base + t * stride + (size_t)kv * dk + i;
    if (vec) {
      if (i < dk) r = *reinterpret_cast<const float4*>(p);
    } else {
      if (i < dk) r.x = p[0];
      if (i + 1 < dk) r.y = p[1];
      if (i + 2 < dk) r.z = p[2];
      if (i + 3 < dk) r.w = p[3];
    }
  };
  auto fetch = [&](int c0) {
    const int nc = min(CH, n - c0);
#pragma unroll
    for (int m = 0; m < NV4; ++m) {
      const int f = tid + m * kScanThreads, tt = f / DK4, i = (f % DK4) * 4;
      k_r[m] = q_r[m] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tt < nc) {
        row4(k_r[m], k, (size_t)start + c0 + tt, k_stride, i);
        row4(q_r[m], q, (size_t)start + c0 + tt, q_stride, i);
      }
    }
#pragma unroll
    for (int m = 0; m < NV; ++m) {
      const int f = tid + m * kScanThreads, tt = f / kScanCols, jj = col0 + f % kScanCols;
      v_r[m] = jj >= dv && jj < C ? 1.f : 0.f;
      if (tt < nc && jj < dv) v_r[m] = v[((size_t)start + c0 + tt) * v_stride + (size_t)h * dv + jj];
    }
    a_r = 1.f, b_r = 0.f;                        // tokens past the end leave S as it is
    if (tid < nc) {
      a_r = a[((size_t)start + c0 + tid) * heads + h];
      b_r = b[((size_t)start + c0 + tid) * heads + h];
    }
  };
  fetch(0);
  for (int c0 = 0; c0 < n; c0 += CH) {
    const int nc = min(CH, n - c0);
    __syncthreads();                             // the portion before is worked through
#pragma unroll
    for (int m = 0; m < NV4; ++m) {
      const int f = tid + m * kScanThreads;
      reinterpret_cast<float4*>(&k_s[0][0])[f] = k_r[m];
      reinterpret_cast<float4*>(&q_s[0][0])[f] = q_r[m];
    }
#pragma unroll
    for (int m = 0; m < NV; ++m) (&v_s[0][0])[tid + m * kScanThreads] = v_r[m];
    if (tid < CH) { a_s[tid] = a_r; b_s[tid] = b_r; }
    __syncthreads();
    if (c0 + CH < n) fetch(c0 + CH);
    auto token = [&](int tt) {                   // S <- a S + b v k, returns this lane's part of S^T q
      const float aa = a_s[tt], bv = b_s[tt] * v_s[tt][col];
      float acc[G4];
#pragma unroll
      for (int g = 0; g < G4; ++g) {
        const float4 kk = *reinterpret_cast<const float4*>(&k_s[tt][32 * g + 4 * lane]);
        const float4 qq = *reinterpret_cast<const float4*>(&q_s[tt][32 * g + 4 * lane]);
        S[g].x = fmaf(aa, S[g].x, bv * kk.x);
        S[g].y = fmaf(aa, S[g].y, bv * kk.y);
        S[g].z = fmaf(aa, S[g].z, bv * kk.z);
        S[g].w = fmaf(aa, S[g].w, bv * kk.w);
        acc[g] = fmaf(S[g].w, qq.w, fmaf(S[g].z, qq.z, fmaf(S[g].y, qq.y, S[g].x * qq.x)));
      }
      float sum = acc[0];
#pragma unroll
      for (int g = 1; g < G4; ++g) sum += acc[g];
      return sum;
    };
    int tt = 0;
    // eight tokens at a time: their partial sums are exchanged so that lane l ends with token l's total
    // (7 shuffles in 3 levels for 8 tokens instead of 24 in 24)
    for (; tt + 8 <= nc; tt += 8) {
      float p[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) p[u] = token(tt + u);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float send = (lane & 4) ? p[u] : p[u + 4], keep = (lane & 4) ? p[u + 4] : p[u];
        p[u] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const float send = (lane & 2) ? p[u] : p[u + 2], keep = (lane & 2) ? p[u + 2] : p[u];
        p[u] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
      }
      const float send = (lane & 1) ? p[0] : p[1], keep = (lane & 1) ? p[1] : p[0];
      const float total = keep + __shfl_xor_sync(0xffffffffu, send, 1);
      if (live) out[(size_t)(start + c0 + tt + lane) * out_stride + (size_t)h * C + j] = total;
    }
    for (; tt < nc; ++tt) {
      float sum = token(tt);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      if (lane == 0 && live) out[(size_t)(start + c0 + tt) * out_stride + (size_t)h * C + j] = sum;
    }
  }
  if (write_state && live) {
#pragma unroll
    for (int g = 0; g < G4; ++g) *reinterpret_cast<float4*>(sp + 32 * g + 4 * lane) = S[g];
  }
}

// grid (tokens, parts).  y[t, c] = rms-normed over the part ((o + D[h] x) silu(z)) * w[c]; o [T, inner] from
// the scan, x [T, .] the convolved inputs (stride x_stride), z = proj[t, col_z + c]; a head is vdim channels.
constexpr int kOutKeep = 8;          // values a thread keeps in registers between the sum of squares and the write
template <typename T>
__global__ void __launch_bounds__(1024)
ssm_out_kernel(T* __restrict__ y, const float* __restrict__ o, const float* __restrict__ x, int x_stride,
               const float* __restrict__ proj, int proj_stride, int col_z, const float* __restrict__ d_skip,
               const float* __restrict__ w, float eps, const int* __restrict__ positions, int inner, int vdim,
               int parts) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, part = blockIdx.y;
  if (positions[t] < 0) return;
  const int size = inner / parts, c0 = part * size;
  auto value = [&](int c) {
    const float z = proj[(size_t)t * proj_stride + col_z + c];
    return (o[(size_t)t * inner + c] + d_skip[c / vdim] * x[(size_t)t * x_stride + c]) * (z * sigmoid_f(z));
  };
  float ss = 0.f;
  if (size <= (int)blockDim.x * kOutKeep) {      // every value is fetched once and waits in a register for the norm
    float u[kOutKeep];
#pragma unroll
    for (int m = 0; m < kOutKeep; ++m) {
      const int i = threadIdx.x + m * blockDim.x;
      u[m] = i < size ? value(c0 + i) : 0.f;
      ss += u[m] * u[m];
    }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)size + eps);
#pragma unroll
    for (int m = 0; m < kOutKeep; ++m) {
      const int i = threadIdx.x + m * blockDim.x;
      if (i < size) y[(size_t)t * inner + c0 + i] = from_f<T>(u[m] * rstd * w[c0 + i]);
    }
    return;
  }
  for (int i = threadIdx.x; i < size; i += blockDim.x) { const float u = value(c0 + i); ss += u * u; }
  const float rstd = rsqrtf(block_sum(ss, scratch) / (float)size + eps);
  for (int i = threadIdx.x; i < size; i += blockDim.x)
    y[(size_t)t * inner + c0 + i] = from_f<T>(value(c0 + i) * rstd * w[c0 + i]);
}

// A warp a token and head, 8 warps a block.  o [T, heads * (vdim + 1)] from the scan with n.q in each head's last
// column, both still to be multiplied by q_scale; y[t, h, j] = u / rms(u) * w[h vdim + j] * sigmoid(gate),
// u = o q_scale / (max(|n.q| q_scale, exp(-m)) + 1e-6), gate = proj[t, col_g + h vdim + j].
constexpr int kOutWarps = 8;
template <typename T>
__global__ void __launch_bounds__(32 * kOutWarps)
xlstm_out_kernel(T* __restrict__ y, const float* __restrict__ o, const float* __restrict__ m_run,
                 const float* __restrict__ proj, int proj_stride, int col_g, const float* __restrict__ w,
                 float eps, float q_scale, const int* __restrict__ positions, int n_tokens, int heads, int vdim) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long pair = (long long)blockIdx.x * kOutWarps + (threadIdx.x >> 5);
  if (pair >= (long long)n_tokens * heads) return;
  const int t = (int)(pair / heads), h = (int)(pair % heads);
  if (positions[t] < 0) return;
  const float* oh = o + ((size_t)t * heads + h) * (vdim + 1);
  const float den = fmaxf(fabsf(oh[vdim] * q_scale), expf(-m_run[(size_t)t * heads + h])) + 1e-6f;
  const float f = q_scale / den;
  float ss = 0.f;
  if (vdim <= 32 * kOutKeep) {                   // the head's values and gates are fetched once, all at a time
    float u[kOutKeep], g[kOutKeep];
#pragma unroll
    for (int m = 0; m < kOutKeep; ++m) {
      const int i = lane + 32 * m;
      u[m] = i < vdim ? oh[i] * f : 0.f;
      g[m] = i < vdim ? proj[(size_t)t * proj_stride + col_g + h * vdim + i] : 0.f;
      ss += u[m] * u[m];
    }
    const float rstd = rsqrtf(warp_sum(ss) / (float)vdim + eps);
#pragma unroll
    for (int m = 0; m < kOutKeep; ++m) {
      const int i = lane + 32 * m, c = h * vdim + i;
      if (i < vdim) y[((size_t)t * heads) * vdim + c] = from_f<T>(u[m] * rstd * w[c] * sigmoid_f(g[m]));
    }
    return;
  }
  for (int i = lane; i < vdim; i += 32) { const float u = oh[i] * f; ss += u * u; }
  const float rstd = rsqrtf(warp_sum(ss) / (float)vdim + eps);
  for (int i = lane; i < vdim; i += 32) {
    const int c = h * vdim + i;
    y[((size_t)t * heads) * vdim + c] =
        from_f<T>(oh[i] * f * rstd * w[c] * sigmoid_f(proj[(size_t)t * proj_stride + col_g + c]));
  }
}

}  // namespace ek

EK_EXPORT int ek_conv_silu(float* out, int out_stride, const float* proj, int proj_stride, int col0,
                           const float* conv_w, const float* conv_b, const float* state, long long slot_stride,
                           long long tail_offset, const int* positions, const int* token_slot, int n_tokens,
                           int channels, int taps, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (channels <= 0 || taps < 1) return EK_ERR_ARG;
  const int tiles = (channels + 255) / 256;
  const int per_block = n_tokens >= 2048 ? ek::kConvTokens : n_tokens >= 256 ? 4 : 1;
  return (int)ek::launch_pdl(ek::conv_silu_kernel, dim3((n_tokens + per_block - 1) / per_block, tiles < 65535 ? tiles : 65535),
                             dim3(256), 0, stream, out, out_stride, proj, proj_stride, col0, conv_w, conv_b, state,
                             (size_t)slot_stride, (size_t)tail_offset, positions, token_slot, n_tokens, channels,
                             taps, per_block, (const float*)nullptr, 1);
}

// The same convolution with two options: `in_bias` [channels] is added to every input that belongs to a
// token (the inputs before a sequence's start stay zero), and `act` 0 leaves the SiLU out.
EK_EXPORT int ek_conv_act(float* out, int out_stride, const float* proj, int proj_stride, int col0,
                          const float* conv_w, const float* conv_b, const float* in_bias, int act,
                          const float* state, long long slot_stride, long long tail_offset, const int* positions,
                          const int* token_slot, int n_tokens, int channels, int taps, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (channels <= 0 || taps < 1) return EK_ERR_ARG;
  const int tiles = (channels + 255) / 256;
  const int per_block = n_tokens >= 2048 ? ek::kConvTokens : n_tokens >= 256 ? 4 : 1;
  return (int)ek::launch_pdl(ek::conv_silu_kernel, dim3((n_tokens + per_block - 1) / per_block, tiles < 65535 ? tiles : 65535),
                             dim3(256), 0, stream, out, out_stride, proj, proj_stride, col0, conv_w, conv_b, state,
                             (size_t)slot_stride, (size_t)tail_offset, positions, token_slot, n_tokens, channels,
                             taps, per_block, in_bias, act);
}

// Both gates of the gated linear recurrence and what enters it: a[t, c] and x[t, c] (see lru_gates_kernel).
// u [T, R] 32-bit rows `u_stride` apart; w_a, w_i [parts][in][out] (transposed at load); w_a_rows, w_i_rows
// (nullable) the same matrices as stored, [parts][out][in], for steps of few tokens; R = parts * size.
EK_EXPORT int ek_lru_gates(float* a, float* x, const float* u, int u_stride, const float* w_a, const float* b_a,
                           const float* w_i, const float* b_i, const float* w_a_rows, const float* w_i_rows,
                           const float* lam, float rate, int n_tokens, int parts, int size, cudaStream_t stream) {
  using namespace ek;
  if (n_tokens <= 0) return 0;
  if (parts <= 0 || size <= 0 || parts > 65535) return EK_ERR_ARG;
  const size_t few_smem = (size_t)kLruFewTokens * size * sizeof(float);
  if (n_tokens <= 192 && w_a_rows && w_i_rows && few_smem <= 200 * 1024) {   // few tokens: a warp an output channel
    if (few_smem > 40 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(lru_gates_few_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)few_smem);
      if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(parts * ((size + 7) / 8), (n_tokens + kLruFewTokens - 1) / kLruFewTokens);
    return (int)launch_pdl(lru_gates_few_kernel, grid, dim3(256), few_smem, stream, a, x, u, u_stride, w_a_rows, b_a,
                           w_i_rows, b_i, lam, rate, n_tokens, parts, size);
  }
  const size_t smem = (size_t)kLruTokens * ((size + 3) & ~3) * sizeof(float);
  if (smem > 200 * 1024) return EK_ERR_ARG;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(lru_gates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((n_tokens + kLruTokens - 1) / kLruTokens, parts, (size + 127) / 128);
  return (int)launch_pdl(lru_gates_kernel, grid, dim3(128), smem, stream, a, x, u, u_stride, w_a, b_a, w_i, b_i, lam,
                         rate, n_tokens, parts, size);
}

#define EK_LRU_SCAN(SUFFIX, T)                                                                              \
  EK_EXPORT int ek_lru_scan_##SUFFIX(void* out, const float* a, const float* x, const float* side,            \
                                     int side_stride, int side_col, const float* side_bias, float* state,    \
                                     long long slot_stride, const int* cu_seqlens, const int* positions,     \
                                     const int* token_slot, int n_seqs, int channels, int write_state,       \
                                     int max_new, cudaStream_t stream) {                                     \
    if (n_seqs <= 0) return 0;                                                                               \
    if (channels <= 0) return EK_ERR_ARG;                                                                    \
    if (max_new > 16) {              /* some sequence brings a stretch of tokens: the form for prompts */    \
      dim3 wide(n_seqs, (channels + ek::kLruLanes - 1) / ek::kLruLanes);                                     \
      if (wide.y > 65535) return EK_ERR_ARG;                                                                 \
      return (int)ek::launch_pdl(ek::lru_scan_wide_kernel<T>, wide, dim3(ek::kLruWarps * 32), 0, stream,     \
                                 (T*)out, a, x, side, side_stride, side_col, side_bias, state,               \
                                 (size_t)slot_stride, cu_seqlens, positions, token_slot, channels,           \
                                 write_state);                                                               \
    }                                                                                                        \
    dim3 grid(n_seqs, (channels + 127) / 128);                                                               \
    if (grid.y > 65535) return EK_ERR_ARG;                                                                   \
    return (int)ek::launch_pdl(ek::lru_scan_kernel<T>, grid, dim3(128), 0, stream, (T*)out, a, x, side,      \
                               side_stride, side_col, side_bias, state, (size_t)slot_stride, cu_seqlens,     \
                               positions, token_slot, channels, write_state);                                \
  }
EK_LRU_SCAN(f32, float)
EK_LRU_SCAN(bf16, ek::bf16)

EK_EXPORT int ek_conv_tail(float* state, long long slot_stride, long long tail_offset, const float* proj,
                           int proj_stride, int col0, const int* cu_seqlens, const int* positions,
                           const int* token_slot, int n_seqs, int channels, int taps, cudaStream_t stream) {
  if (n_seqs <= 0 || taps <= 1) return 0;
  const int tiles = (channels + 255) / 256;
  return (int)ek::launch_pdl(ek::conv_tail_kernel, dim3(n_seqs, tiles < 64 ? tiles : 64), dim3(256), 0, stream, state,
                             (size_t)slot_stride, (size_t)tail_offset, proj, proj_stride, col0, cu_seqlens,
                             positions, token_slot, channels, taps);
}

EK_EXPORT int ek_ssm_gates(float* a, float* b, const float* proj, int proj_stride, int col0, const float* dt_bias,
                           const float* a_log, int n_tokens, int heads, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (heads <= 0) return EK_ERR_ARG;
  const long long total = (long long)n_tokens * heads;
  return (int)ek::launch_pdl(ek::ssm_gates_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, a, b,
                             proj, proj_stride, col0, dt_bias, a_log, n_tokens, heads);
}

EK_EXPORT int ek_xgate_scan(float* a, float* b, float* m_run, const float* proj, int proj_stride, int col_i,
                            int col_f, const float* bias_i, const float* bias_f, float cap, float* state,
                            long long slot_stride, long long m_offset, const int* cu_seqlens, const int* positions,
                            const int* token_slot, int n_seqs, int heads, int write_state, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || !(cap > 0.f)) return EK_ERR_ARG;
  if (heads > 65535) return EK_ERR_ARG;
  return (int)ek::launch_pdl(ek::xgate_scan_kernel, dim3(n_seqs, heads), dim3(ek::kGateWarps * 32), 0, stream, a, b, m_run, proj, proj_stride, col_i, col_f,
                             bias_i, bias_f, cap, state, (size_t)slot_stride, (size_t)m_offset, cu_seqlens,
                             positions, token_slot, heads, write_state);
}

// Rows of S per column that the scan keeps for keys of dk values: dk rounded up to 32, 64, 128 or 256.
EK_EXPORT int ek_decay_scan_rows(int dk) {
  return dk <= 0 || dk > 256 ? 0 : dk <= 32 ? 32 : dk <= 64 ? 64 : dk <= 128 ? 128 : 256;
}

EK_EXPORT int ek_decay_scan(float* out, int out_stride, const float* q, int q_stride, const float* k, int k_stride,
                            const float* v, int v_stride, const float* a, const float* b, float* state,
                            long long slot_stride, const int* cu_seqlens, const int* positions,
                            const int* token_slot, int n_seqs, int heads, int kv_heads, int dk, int dv,
                            int ones_col, int write_state, cudaStream_t stream) {
  using namespace ek;
  if (n_seqs <= 0) return 0;
  const int rows = ek_decay_scan_rows(dk);
  if (!rows || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dv <= 0 || heads > 65535 || slot_stride % 4 ||
      ((uintptr_t)state & 15))
    return EK_ERR_ARG;
  const int C = dv + (ones_col ? 1 : 0);
  dim3 grid(n_seqs, heads, (C + kScanCols - 1) / kScanCols);
  auto kernel = rows == 32 ? decay_scan_kernel<4> : rows == 64 ? decay_scan_kernel<8>
              : rows == 128 ? decay_scan_kernel<16> : decay_scan_kernel<32>;
  return (int)launch_pdl(kernel, grid, dim3(kScanThreads), 0, stream, out, out_stride, q, q_stride, k, k_stride, v,
                         v_stride, a, b, state, (size_t)slot_stride, cu_seqlens, positions, token_slot, heads,
                         kv_heads, dk, dv, ones_col ? 1 : 0, write_state);
}

#define EK_INSTANTIATE(SUFFIX, T)                                                                              \
  EK_EXPORT int ek_ssm_out_##SUFFIX(void* y, const float* o, const float* x, int x_stride, const float* proj,  \
                                    int proj_stride, int col_z, const float* d_skip, const float* w, float eps, \
                                    const int* positions, int n_tokens, int inner, int vdim, int parts,        \
                                    cudaStream_t stream) {                                                     \
    if (n_tokens <= 0) return 0;                                                                               \
    if (inner <= 0 || vdim <= 0 || parts <= 0 || inner % parts || inner % vdim || parts > 65535)               \
      return EK_ERR_ARG;                                                                                       \
    const int size = inner / parts; /* a thread takes up to four channels of a part */                         \
    const int threads = size >= 4096 ? 1024 : size <= 256 ? 64 : (size / 4 + 31) / 32 * 32;                    \
    return (int)ek::launch_pdl(ek::ssm_out_kernel<T>, dim3(n_tokens, parts), dim3(threads), 0, stream, (T*)y,  \
                               o, x, x_stride, proj, proj_stride, col_z, d_skip, w, eps, positions, inner,     \
                               vdim, parts);                                                                   \
  }                                                                                                            \
  EK_EXPORT int ek_xlstm_out_##SUFFIX(void* y, const float* o, const float* m_run, const float* proj,          \
                                      int proj_stride, int col_g, const float* w, float eps, float q_scale,    \
                                      const int* positions, int n_tokens, int heads, int vdim,                 \
                                      cudaStream_t stream) {                                                   \
    if (n_tokens <= 0) return 0;                                                                               \
    if (heads <= 0 || heads > 65535 || vdim <= 0) return EK_ERR_ARG;                                           \
    const long long blocks = ((long long)n_tokens * heads + ek::kOutWarps - 1) / ek::kOutWarps;                \
    if (blocks > 0x7fffffffLL) return EK_ERR_ARG;                                                              \
    return (int)ek::launch_pdl(ek::xlstm_out_kernel<T>, dim3((unsigned)blocks), dim3(32 * ek::kOutWarps), 0,   \
                               stream, (T*)y, o, m_run, proj, proj_stride, col_g, w, eps, q_scale, positions,  \
                               n_tokens, heads, vdim);                                                         \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)
