// Gated delta rule with one decay per key channel (or one per head), as a recurrent mixer with per-sequence state.
//
// Per token and head (S is [d, e], 32-bit, carried from token to token):
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// with q, k unit vectors per head (q also times d^-1/2) made from projections that pass a short
// causal convolution over time and SiLU, beta = sigmoid(.), g = exp(-exp(A) softplus(a + bias)).
// A column of S (one value channel) never meets another column, so the scan runs one column per
// group of 8 lanes, the column's d rows spread over the lanes' registers, sequentially over the
// tokens of a sequence and in parallel over sequences, heads and columns.
//
// Five kernels, all taking packed rows of several sequences (prompts, chunks, single tokens):
//   delta_low_rank   the second halves of the two low-rank pairs: decays and output gates, a tile of
//                    tokens x channels a block so that a weight is fetched once for 16 tokens
//   delta_prepare    convolution + SiLU, unit norms, beta             (a block a token and key head)
//   delta_conv_tail  the last taps-1 convolution inputs of every sequence -> its state
//   delta_scan       the recurrence; reads and writes S in the state
//   delta_out_norm   o / rms(o) * w * gate per head, to the activation type
// State of a slot (32-bit): [heads][e][DP] for S (DP = d rounded up to the scan's row count), then
// [channels][taps-1] convolution inputs.  A fresh slot is all zeros.
// Everything that enters the recurrence is computed and kept in 32-bit.
#include "common.cuh"

namespace ek {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

struct DeltaShape {
  int heads, kv_heads, dim, vdim, taps;
  int rank_a, rank_g;          // inner sizes of the low-rank decay and gate projections
  // columns of a projected row: [q | k | v | beta | a1 | g1]
  __host__ __device__ int cq() const { return kv_heads * dim; }
  __host__ __device__ int cv() const { return heads * vdim; }
  __host__ __device__ int channels() const { return 2 * cq() + cv(); }
  __host__ __device__ int off_beta() const { return channels(); }
  __host__ __device__ int off_a() const { return channels() + heads; }
  __host__ __device__ int off_g() const { return off_a() + rank_a; }
  __host__ __device__ int row() const { return off_g() + rank_g; }
};

// out[t, c] = f(bias[c] + sum_r w2t[r][c] * proj[t, offset + r]) for c < channels: f = sigmoid (mode 1), or
// the decay exp(-exp(a_log[c / dim]) * softplus(.)) (mode 0).  grid (token tiles of 16, channel tiles of 128).
constexpr int kRankTokens = 16;
__global__ void __launch_bounds__(128)
delta_low_rank_kernel(float* __restrict__ out, const float* __restrict__ proj, int proj_stride, int offset,
                      int rank, const float* __restrict__ w2t, const float* __restrict__ bias,
                      const float* __restrict__ a_log, int dim, int channels, int n_tokens, int mode) {
  extern __shared__ __align__(16) float x_s[];  // [kRankTokens][ld], ld = rank rounded up to 4
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * kRankTokens, tid = threadIdx.x;
  const int nt = min(kRankTokens, n_tokens - t0);
  const int ld = (rank + 3) & ~3;
  for (int idx = tid; idx < kRankTokens * rank; idx += blockDim.x) {
    const int tt = idx / rank, r = idx % rank;
    x_s[tt * ld + r] = tt < nt ? proj[(size_t)(t0 + tt) * proj_stride + offset + r] : 0.f;
  }
  __syncthreads();
  const int c = blockIdx.y * 128 + tid;
  if (c >= channels) return;
  float acc[kRankTokens];
  const float b = bias ? bias[c] : 0.f;
#pragma unroll
  for (int tt = 0; tt < kRankTokens; ++tt) acc[tt] = b;
  int r = 0;
  for (; r + 4 <= rank; r += 4) {               // four weights, then one 16-byte read of a token's four inputs
    const float w0 = w2t[(size_t)r * channels + c], w1 = w2t[(size_t)(r + 1) * channels + c];
    const float w2 = w2t[(size_t)(r + 2) * channels + c], w3 = w2t[(size_t)(r + 3) * channels + c];
#pragma unroll
    for (int tt = 0; tt < kRankTokens; ++tt) {
      const float4 x = *reinterpret_cast<const float4*>(x_s + tt * ld + r);
      acc[tt] = fmaf(w3, x.w, fmaf(w2, x.z, fmaf(w1, x.y, fmaf(w0, x.x, acc[tt]))));
    }
  }
  for (; r < rank; ++r) {
    const float wv = w2t[(size_t)r * channels + c];
#pragma unroll
    for (int tt = 0; tt < kRankTokens; ++tt) acc[tt] = fmaf(wv, x_s[tt * ld + r], acc[tt]);
  }
  const float rate = mode == 0 ? expf(a_log[c / dim]) : 0.f;
#pragma unroll
  for (int tt = 0; tt < kRankTokens; ++tt)      // (a fixed trip count keeps acc in registers)
    if (tt < nt)
      out[(size_t)(t0 + tt) * channels + c] = mode == 0 ? expf(-rate * softplus_f(acc[tt])) : sigmoid_f(acc[tt]);
}

// grid (tokens, key heads): a block convolves one q head, one k head and the v channels of the value
// heads that read them (few tokens: many short blocks).  proj [T, >= row()] 32-bit.  conv_w [channels][taps] (last column: the current
// token).  Outputs (32-bit): qn, kn [T, kv_heads * dim]; vc [T, heads * vdim]; beta [T, heads].
__global__ void __launch_bounds__(128)
delta_prepare_kernel(float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vc,
                     float* __restrict__ beta,
                     const float* __restrict__ proj, int proj_stride, const float* __restrict__ conv_w,
                     const float* __restrict__ state,
                     size_t slot_stride, size_t tail_offset, const int* __restrict__ positions,
                     const int* __restrict__ token_slot, DeltaShape sh) {
  extern __shared__ float qk_s[];               // [2][dim] convolved q and k of this key head
  __shared__ int n_prev_s;
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int pos = positions[t];
  if (pos < 0) return;
  const int slot = token_slot[t];
  const int K = sh.taps, cq = sh.cq(), rep = sh.heads / sh.kv_heads;
  if (tid == 0) {
    int n = 0;                                  // predecessors of this token inside the step
    while (n < K - 1 && t - n - 1 >= 0 && token_slot[t - n - 1] == slot && positions[t - n - 1] == pos - n - 1) ++n;
    n_prev_s = n;
  }
  const float* row = proj + (size_t)t * proj_stride;
  __syncthreads();
  const int n_prev = n_prev_s;
  const float* tail = state + (size_t)slot * slot_stride + tail_offset;
  auto convolve = [&](int c) {                  // channel c of [q | k | v]: convolution, then SiLU
    const float* w = conv_w + (size_t)c * K;
    float acc = w[K - 1] * row[c];
    for (int j = 1; j < K; ++j) {
      const float x = j <= n_prev ? proj[(size_t)(t - j) * proj_stride + c]
                                  : tail[(size_t)c * (K - 1) + (n_prev - j + K - 1)];
      acc = fmaf(w[K - 1 - j], x, acc);
    }
    return acc * sigmoid_f(acc);
  };
  const int g = blockIdx.y;
  for (int i = tid; i < 2 * sh.dim; i += blockDim.x)
    qk_s[i] = convolve((i < sh.dim ? 0 : cq - sh.dim) + g * sh.dim + i);      // q head g, then k head g
  const int v0 = g * rep * sh.vdim;             // this key head's value channels
  for (int i = tid; i < rep * sh.vdim; i += blockDim.x)
    vc[(size_t)t * sh.cv() + v0 + i] = convolve(2 * cq + v0 + i);
  for (int h = g * rep + tid; h < (g + 1) * rep; h += blockDim.x)
    beta[(size_t)t * sh.heads + h] = sigmoid_f(row[sh.off_beta() + h]);
  __syncthreads();
  // unit vectors: q (also times dim^-1/2), then k
  for (int which = 0; which < 2; ++which) {
    const float* x = qk_s + which * sh.dim;
    float ss = 0.f;
    for (int i = tid; i < sh.dim; i += blockDim.x) ss += x[i] * x[i];
    ss = block_sum(ss, scratch);
    const float f = rsqrtf(ss + 1e-6f) * (which == 0 ? rsqrtf((float)sh.dim) : 1.f);
    float* dst = (which == 0 ? qn : kn) + (size_t)t * cq + (size_t)g * sh.dim;
    for (int i = tid; i < sh.dim; i += blockDim.x) dst[i] = x[i] * f;
  }
}

// The same with a block a token (many tokens: fewer, longer blocks).  grid: tokens.  proj [T, >= row()] 32-bit.  conv_w [channels][taps] (last column: the current
// token).  Outputs (32-bit): qn, kn [T, kv_heads * dim]; vc [T, heads * vdim]; beta [T, heads].
__global__ void __launch_bounds__(256)
delta_prepare_token_kernel(float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vc,
                     float* __restrict__ beta,
                     const float* __restrict__ proj, int proj_stride, const float* __restrict__ conv_w,
                     const float* __restrict__ state,
                     size_t slot_stride, size_t tail_offset, const int* __restrict__ positions,
                     const int* __restrict__ token_slot, DeltaShape sh) {
  extern __shared__ float qk_s[];               // [2 * cq] convolved q and k
  __shared__ int n_prev_s;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int pos = positions[t];
  if (pos < 0) return;
  const int slot = token_slot[t];
  const int K = sh.taps, cq = sh.cq(), nch = sh.channels();
  if (tid == 0) {
    int n = 0;                                  // predecessors of this token inside the step
    while (n < K - 1 && t - n - 1 >= 0 && token_slot[t - n - 1] == slot && positions[t - n - 1] == pos - n - 1) ++n;
    n_prev_s = n;
  }
  const float* row = proj + (size_t)t * proj_stride;
  __syncthreads();
  const int n_prev = n_prev_s;
  const float* tail = state + (size_t)slot * slot_stride + tail_offset;
  for (int c = tid; c < nch; c += blockDim.x) {
    const float* w = conv_w + (size_t)c * K;
    float acc = w[K - 1] * row[c];
    for (int j = 1; j < K; ++j) {
      const float x = j <= n_prev ? proj[(size_t)(t - j) * proj_stride + c]
                                  : tail[(size_t)c * (K - 1) + (n_prev - j + K - 1)];
      acc = fmaf(w[K - 1 - j], x, acc);
    }
    const float y = acc * sigmoid_f(acc);
    if (c < 2 * cq) qk_s[c] = y;
    else vc[(size_t)t * sh.cv() + (c - 2 * cq)] = y;
  }
  __syncthreads();
  // unit vectors per head: a warp a head
  const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  const float q_scale = rsqrtf((float)sh.dim);
  for (int hh = warp; hh < 2 * sh.kv_heads; hh += nwarps) {
    const float* x = qk_s + (size_t)hh * sh.dim;
    float ss = 0.f;
    for (int i = lane; i < sh.dim; i += 32) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const bool is_q = hh < sh.kv_heads;
    const float f = rsqrtf(ss + 1e-6f) * (is_q ? q_scale : 1.f);
    float* dst = (is_q ? qn : kn) + (size_t)t * cq + (size_t)(is_q ? hh : hh - sh.kv_heads) * sh.dim;
    for (int i = lane; i < sh.dim; i += 32) dst[i] = x[i] * f;
  }
  for (int h = tid; h < sh.heads; h += blockDim.x)
    beta[(size_t)t * sh.heads + h] = sigmoid_f(row[sh.off_beta() + h]);
}

// grid (sequences, channel tiles).  After the step the state's tail holds the last taps-1 inputs of the sequence.
__global__ void delta_conv_tail_kernel(float* __restrict__ state, size_t slot_stride, size_t tail_offset,
                                       const float* __restrict__ proj, int proj_stride,
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
      tc[m] = from_step >= 0 ? proj[(size_t)(start + from_step) * proj_stride + c] : tc[m + n];
    }
  }
}

constexpr int kScanCols = 16;        // columns of S a block takes
constexpr int kScanLanes = 8;        // lanes that share a column
constexpr int kScanChunk = 16;       // tokens fetched into shared memory at a time
constexpr int kScanThreads = kScanCols * kScanLanes;

// grid (sequences, heads, column tiles); 128 threads = 16 columns x 8 lanes (small blocks: the scan is a
// chain of latencies, and more blocks put it on more SMs); a lane holds RPL
// consecutive rows of its column.  The tokens' q, k, decays, v and beta come in chunks of 16 through
// two shared-memory buffers: while a chunk is worked through, the next one is on its way from global
// memory into registers and is put down behind the chunk's last token.  Only S^T k lies on the chain
// from token to token (a lane's share in four independent sums, then three exchanges among the eight
// lanes); the read-out S^T q is summed beside it.
template <int RPL>
__global__ void __launch_bounds__(kScanThreads)
delta_scan_kernel(float* __restrict__ out, const float* __restrict__ qn, const float* __restrict__ kn,
                  const float* __restrict__ vc, const float* __restrict__ beta,
                  const float* __restrict__ decay, float* __restrict__ state, size_t slot_stride,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ positions,
                  const int* __restrict__ token_slot, DeltaShape sh, int decay_per_head) {
  constexpr int DP = RPL * kScanLanes;          // rows held (>= dim; rows past dim stay zero)
  constexpr int LDS = RPL + 4;                  // a lane's stretch in shared memory, padded
  constexpr int ROW = kScanLanes * LDS;
  constexpr int PER = kScanChunk * DP / kScanThreads;       // staged values of q (k, g) per thread
  constexpr int PERV = kScanChunk * kScanCols / kScanThreads;
  extern __shared__ __align__(16) float scan_s[];
  float* q_s = scan_s;                          // [2][chunk][ROW]
  float* k_s = q_s + 2 * kScanChunk * ROW;
  float* g_s = k_s + 2 * kScanChunk * ROW;
  float* v_s = g_s + 2 * kScanChunk * ROW;      // [2][chunk][cols]
  float* b_s = v_s + 2 * kScanChunk * kScanCols;          // [2][chunk]
  float* o_s = b_s + 2 * kScanChunk;            // [chunk][cols]
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
  if (n <= 0 || positions[start] < 0) return;
  const int slot = token_slot[start];
  const int cl = tid / kScanLanes, lr = tid % kScanLanes;
  const int col = blockIdx.z * kScanCols + cl;
  const bool live = col < sh.vdim;
  const int kvh = h / (sh.heads / sh.kv_heads);
  const int cq = sh.cq(), cv = sh.cv(), nd = sh.heads * sh.dim;

  float S[RPL];
  float* sp = state + (size_t)slot * slot_stride + ((size_t)h * sh.vdim + (live ? col : 0)) * DP + lr * RPL;
#pragma unroll
  for (int i = 0; i < RPL; i += 4) {
    const float4 x = live ? *reinterpret_cast<const float4*>(sp + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    S[i] = x.x; S[i + 1] = x.y; S[i + 2] = x.z; S[i + 3] = x.w;
  }

  float rq[PER], rk[PER], rg[PER], rv[PERV], rb = 0.f;
  auto fetch = [&](int c0) {                    // chunk c0 .. c0+15 of the sequence -> registers
    const int nt = min(kScanChunk, n - c0);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int idx = tid + i * kScanThreads, tt = idx / DP, r = idx % DP;
      const bool ok = tt < nt && r < sh.dim;
      const size_t rowi = (size_t)(start + c0 + tt);
      rq[i] = ok ? qn[rowi * cq + (size_t)kvh * sh.dim + r] : 0.f;
      rk[i] = ok ? kn[rowi * cq + (size_t)kvh * sh.dim + r] : 0.f;
      rg[i] = ok ? (decay_per_head ? decay[rowi * sh.heads + h] : decay[rowi * nd + (size_t)h * sh.dim + r]) : 1.f;
    }
#pragma unroll
    for (int i = 0; i < PERV; ++i) {
      const int idx = tid + i * kScanThreads, tt = idx / kScanCols, c = idx % kScanCols;
      const int gc = blockIdx.z * kScanCols + c;
      rv[i] = (tt < nt && gc < sh.vdim) ? vc[(size_t)(start + c0 + tt) * cv + (size_t)h * sh.vdim + gc] : 0.f;
    }
    if (tid < kScanChunk) rb = tid < nt ? beta[(size_t)(start + c0 + tid) * sh.heads + h] : 0.f;
  };
  auto put = [&](int buf) {                     // registers -> buffer `buf`
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int idx = tid + i * kScanThreads, tt = idx / DP, r = idx % DP;
      const int at = (buf * kScanChunk + tt) * ROW + (r / RPL) * LDS + r % RPL;
      q_s[at] = rq[i]; k_s[at] = rk[i]; g_s[at] = rg[i];
    }
#pragma unroll
    for (int i = 0; i < PERV; ++i) v_s[buf * kScanChunk * kScanCols + tid + i * kScanThreads] = rv[i];
    if (tid < kScanChunk) b_s[buf * kScanChunk + tid] = rb;
  };

  fetch(0);
  put(0);
  __syncthreads();
  int buf = 0;
  for (int c0 = 0; c0 < n; c0 += kScanChunk, buf ^= 1) {
    const int nt = min(kScanChunk, n - c0);
    const bool more = c0 + kScanChunk < n;
    if (more) fetch(c0 + kScanChunk);           // in flight while this chunk is worked through
    for (int tt = 0; tt < nt; ++tt) {
      const float* kk = k_s + (buf * kScanChunk + tt) * ROW + lr * LDS;
      const float* gg = g_s + (buf * kScanChunk + tt) * ROW + lr * LDS;
      const float* qq = q_s + (buf * kScanChunk + tt) * ROW + lr * LDS;
      float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
      for (int i = 0; i < RPL; i += 4) {
        const float4 g4 = *reinterpret_cast<const float4*>(gg + i);
        const float4 k4 = *reinterpret_cast<const float4*>(kk + i);
        S[i] *= g4.x; S[i + 1] *= g4.y; S[i + 2] *= g4.z; S[i + 3] *= g4.w;
        p0 = fmaf(S[i], k4.x, p0);
        p1 = fmaf(S[i + 1], k4.y, p1);
        p2 = fmaf(S[i + 2], k4.z, p2);
        p3 = fmaf(S[i + 3], k4.w, p3);
      }
      float part = (p0 + p1) + (p2 + p3);
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      part += __shfl_xor_sync(0xffffffffu, part, 4);
      const float u = b_s[buf * kScanChunk + tt] * (v_s[(buf * kScanChunk + tt) * kScanCols + cl] - part);
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int i = 0; i < RPL; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kk + i);
        const float4 q4 = *reinterpret_cast<const float4*>(qq + i);
        S[i] = fmaf(k4.x, u, S[i]);
        S[i + 1] = fmaf(k4.y, u, S[i + 1]);
        S[i + 2] = fmaf(k4.z, u, S[i + 2]);
        S[i + 3] = fmaf(k4.w, u, S[i + 3]);
        o0 = fmaf(S[i], q4.x, o0);
        o1 = fmaf(S[i + 1], q4.y, o1);
        o2 = fmaf(S[i + 2], q4.z, o2);
        o3 = fmaf(S[i + 3], q4.w, o3);
      }
      float po = (o0 + o1) + (o2 + o3);
      po += __shfl_xor_sync(0xffffffffu, po, 1);
      po += __shfl_xor_sync(0xffffffffu, po, 2);
      po += __shfl_xor_sync(0xffffffffu, po, 4);
      if (lr == 0) o_s[tt * kScanCols + cl] = po;
    }
    if (more) put(buf ^ 1);                     // (the other buffer: nobody reads it during this chunk)
    __syncthreads();
    for (int idx = tid; idx < nt * kScanCols; idx += kScanThreads) {
      const int tt = idx / kScanCols, c = idx % kScanCols;
      const int gc = blockIdx.z * kScanCols + c;
      if (gc < sh.vdim) out[(size_t)(start + c0 + tt) * cv + (size_t)h * sh.vdim + gc] = o_s[idx];
    }
    __syncthreads();                            // o_s is written again in the next chunk
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RPL; i += 4)
      *reinterpret_cast<float4*>(sp + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
  }
}

template <int RPL>
static cudaError_t launch_scan(dim3 grid, cudaStream_t stream, float* out, const float* qn, const float* kn,
                               const float* vc, const float* beta, const float* decay, float* state,
                               size_t slot_stride, const int* cu_seqlens, const int* positions,
                               const int* token_slot, DeltaShape sh, int decay_per_head) {
  constexpr int ROW = kScanLanes * (RPL + 4);
  const size_t smem = sizeof(float) * (size_t)(6 * kScanChunk * ROW + 2 * kScanChunk * kScanCols + 2 * kScanChunk +
                                               kScanChunk * kScanCols);
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<RPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  delta_scan_kernel<RPL><<<grid, kScanThreads, smem, stream>>>(out, qn, kn, vc, beta, decay, state, slot_stride,
                                                              cu_seqlens, positions, token_slot, sh, decay_per_head);
  return cudaGetLastError();
}

// grid: tokens.  y[t, h, j] = o[t, h, j] / rms_j(o[t, h, :]) * w[j] * f(gate[t, h, j]); gate rows are
// `gate_stride` apart; f is the identity (gate_act 0: the gate is finished) or SiLU (1: it is a raw projection).
template <typename T>
__global__ void __launch_bounds__(256)
delta_out_norm_kernel(T* __restrict__ y, const float* __restrict__ o, const float* __restrict__ gate,
                      const float* __restrict__ w, float eps, const int* __restrict__ positions,
                      DeltaShape sh, int gate_stride, int gate_act) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int cv = sh.cv();
  if (positions[t] < 0) {
    for (int c = tid; c < cv; c += blockDim.x) y[(size_t)t * cv + c] = from_f<T>(0.f);
    return;
  }
  const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  for (int h = warp; h < sh.heads; h += nwarps) {
    const float* x = o + (size_t)t * cv + (size_t)h * sh.vdim;
    float ss = 0.f;
    for (int j = lane; j < sh.vdim; j += 32) ss += x[j] * x[j];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)sh.vdim + eps);
    for (int j = lane; j < sh.vdim; j += 32) {
      const int c = h * sh.vdim + j;
      float g = gate[(size_t)t * gate_stride + c];
      if (gate_act == 1) g = g * sigmoid_f(g);
      y[(size_t)t * cv + c] = from_f<T>(x[j] * inv * w[j] * g);
    }
  }
}

static bool shape_ok(const DeltaShape& sh) {
  return sh.heads > 0 && sh.kv_heads > 0 && sh.heads % sh.kv_heads == 0 && sh.dim > 0 && sh.vdim > 0 &&
         sh.taps >= 1 && sh.rank_a > 0 && sh.rank_g > 0 && sh.heads <= 65535;
}

}  // namespace ek

// Rows of S the scan holds for a key size `dim` (the state's [heads][vdim][rows] uses it); 0: too large.
EK_EXPORT int ek_delta_state_rows(int dim) {
  if (dim <= 0 || dim > 256) return 0;
  if (dim <= 32) return 32;
  if (dim <= 64) return 64;
  if (dim <= 128) return 128;
  return 256;
}

// mode 0: decays (bias = dt_bias, a_log per head of `dim` channels); mode 1: sigmoid gates.
EK_EXPORT int ek_delta_low_rank(float* out, const float* proj, int proj_stride, int offset, int rank,
                                const float* w2t, const float* bias, const float* a_log, int dim,
                                int channels, int n_tokens, int mode, cudaStream_t stream) {
  using namespace ek;
  if (n_tokens <= 0) return 0;
  if (rank <= 0 || rank > 2048 || channels <= 0 || dim <= 0 || offset < 0 || proj_stride < offset + rank ||
      (mode == 0 && !a_log) || (channels + 127) / 128 > 65535)
    return EK_ERR_ARG;
  dim3 grid((n_tokens + kRankTokens - 1) / kRankTokens, (channels + 127) / 128);
  const size_t smem = (size_t)kRankTokens * ((rank + 3) & ~3) * sizeof(float);
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_low_rank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  delta_low_rank_kernel<<<grid, 128, smem, stream>>>(out, proj, proj_stride, offset, rank, w2t, bias, a_log, dim,
                                                     channels, n_tokens, mode);
  EK_RETURN_LAUNCH_STATUS();
}

EK_EXPORT int ek_delta_prepare(float* qn, float* kn, float* vc, float* beta,
                               const float* proj, int proj_stride, const float* conv_w, const float* state,
                               long long slot_stride, long long tail_offset, const int* positions,
                               const int* token_slot, int n_tokens, int heads, int kv_heads, int dim,
                               int vdim, int taps, int rank_a, int rank_g, cudaStream_t stream) {
  using namespace ek;
  if (n_tokens <= 0) return 0;
  DeltaShape sh{heads, kv_heads, dim, vdim, taps, rank_a, rank_g};
  if (!shape_ok(sh) || proj_stride < sh.row()) return EK_ERR_ARG;
  if (n_tokens >= 512) {
    const size_t smem = (size_t)(2 * sh.cq()) * sizeof(float);
    if (smem > 200 * 1024) return EK_ERR_ARG;
    if (smem > 40 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(delta_prepare_token_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    delta_prepare_token_kernel<<<n_tokens, 256, smem, stream>>>(qn, kn, vc, beta, proj, proj_stride, conv_w, state,
                                                                (size_t)slot_stride, (size_t)tail_offset, positions,
                                                                token_slot, sh);
    EK_RETURN_LAUNCH_STATUS();
  }
  const size_t smem = (size_t)(2 * dim) * sizeof(float);
  if (smem > 40 * 1024 || kv_heads > 65535) return EK_ERR_ARG;
  delta_prepare_kernel<<<dim3(n_tokens, kv_heads), 128, smem, stream>>>(qn, kn, vc, beta, proj, proj_stride, conv_w,
                                                                       state, (size_t)slot_stride,
                                                                       (size_t)tail_offset, positions, token_slot, sh);
  EK_RETURN_LAUNCH_STATUS();
}

EK_EXPORT int ek_delta_conv_tail(float* state, long long slot_stride, long long tail_offset,
                                 const float* proj, int proj_stride, const int* cu_seqlens,
                                 const int* positions, const int* token_slot, int n_seqs, int channels,
                                 int taps, cudaStream_t stream) {
  if (n_seqs <= 0 || taps <= 1) return 0;
  if (channels <= 0 || proj_stride < channels) return EK_ERR_ARG;
  dim3 grid(n_seqs, (channels + 255) / 256 > 64 ? 64 : (channels + 255) / 256);
  ek::delta_conv_tail_kernel<<<grid, 256, 0, stream>>>(state, (size_t)slot_stride, (size_t)tail_offset,
                                                         proj, proj_stride, cu_seqlens, positions,
                                                         token_slot, channels, taps);
  EK_RETURN_LAUNCH_STATUS();
}

EK_EXPORT int ek_delta_scan(float* out, const float* qn, const float* kn, const float* vc,
                            const float* beta, const float* decay, float* state, long long slot_stride,
                            const int* cu_seqlens, const int* positions, const int* token_slot,
                            int n_seqs, int heads, int kv_heads, int dim, int vdim, int decay_per_head,
                            cudaStream_t stream) {
  using namespace ek;
  if (n_seqs <= 0) return 0;
  DeltaShape sh{heads, kv_heads, dim, vdim, 1, 1, 1};
  // S is read and written four values at a time: every slot's S must start on a 16-byte boundary
  if (!shape_ok(sh) || slot_stride % 4 || ((uintptr_t)state & 15)) return EK_ERR_ARG;
  dim3 grid(n_seqs, heads, (vdim + kScanCols - 1) / kScanCols);
  if (grid.z > 65535) return EK_ERR_ARG;
  const int rows = ek_delta_state_rows(dim);
#define EK_SCAN(RPL)                                                                                 \
  return (int)launch_scan<RPL>(grid, stream, out, qn, kn, vc, beta, decay, state, (size_t)slot_stride, \
                               cu_seqlens, positions, token_slot, sh, decay_per_head)
  switch (rows) {
    case 32: EK_SCAN(4);
    case 64: EK_SCAN(8);
    case 128: EK_SCAN(16);
    case 256: EK_SCAN(32);
    default: return EK_ERR_ARG;
  }
#undef EK_SCAN
}

#define EK_INSTANTIATE(SUFFIX, T)                                                                    \
  EK_EXPORT int ek_delta_out_norm_##SUFFIX(void* y, const float* o, const float* gate,                \
                                           const float* w, float eps,                                \
                                           const int* positions, int n_tokens, int heads,            \
                                           int kv_heads, int dim, int vdim, int taps, int rank_a,    \
                                           int rank_g, int gate_stride, int gate_act,                \
                                           cudaStream_t stream) {                                    \
    using namespace ek;                                                                              \
    if (n_tokens <= 0) return 0;                                                                     \
    DeltaShape sh{heads, kv_heads, dim, vdim, taps, rank_a, rank_g};                                 \
    if (!shape_ok(sh) || gate_stride < sh.cv() || gate_act < 0 || gate_act > 1) return EK_ERR_ARG;   \
    delta_out_norm_kernel<T><<<n_tokens, 256, 0, stream>>>((T*)y, o, gate, w, eps, positions, sh,    \
                                                           gate_stride, gate_act);                   \
    EK_RETURN_LAUNCH_STATUS();                                                                       \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)
