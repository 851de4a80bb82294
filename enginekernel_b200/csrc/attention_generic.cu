// Attention over the paged cache for any head size, head count and group size, in
// 32-bit or bfloat16 storage with 32-bit arithmetic throughout.  One block per
// (token, query head, key split) walks the keys the token may see:
//     lo = max(0, pos - window + 1) (window <= 0: 0)  ...  pos
// with a running maximum and sum (online softmax) so that no score row is stored.
// An optional sink - a key without a value whose fixed score `sink` every query sees - adds
// exp(sink) to the softmax denominator once per (token, head); -INFINITY switches it off.
// `sinks`, if given, holds one such score per query head and takes the place of `sink`.
// `keep_first` > 0 (with a window): the first keep_first positions of the sequence stay visible to
// every later token at their true positions, beside the window.  `gate`, if given, holds one value
// per token and query head (row stride `gate_stride`): the head's output is multiplied by its sigmoid.
// `cross` > 1 (entry point ..._cross): every head's weights are applied to the values of every key/value
// head and the results are kept in 32-bit, for designs that mix the heads' weights behind the softmax;
// mix_heads_kernel forms the mixed results from them.
// It serves whole prompts, chunks and single decoded tokens alike, since each token
// carries its own position and slot; the faster bfloat16 kernels in attention_bf16.cu
// cover the common head sizes, this one covers everything and is the 32-bit path.
//
// Formula: engine/ek_model.py:475-488 (scores q.k * scale in 32-bit, softmax in 32-bit,
// weighted sum of values in 32-bit); query head h reads KV head h / (heads / kv heads).
// Splitting the keys and merging partial (max, sum, accumulator) triples in split order
// is the reference's flash-decoding scheme (engine/ek_kernels.py:534-615, 988-1019).
#include "common.cuh"

namespace ek {

constexpr int kAttnThreads = 128;
constexpr int kGenericMaxDim = 1024;  // this kernel's own limit on the head size: 8 values a thread
constexpr int kGenericAcc = kGenericMaxDim / kAttnThreads;

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ row, const float* __restrict__ q, int d);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ row,
                                                const float* __restrict__ q, int d) {
  float s = 0.f;
  if (d % 4) {                                 // rows that do not start on 16-byte boundaries
    for (int i = 0; i < d; ++i) s += row[i] * q[i];
    return s;
  }
  const float4* r4 = reinterpret_cast<const float4*>(row);
  for (int i = 0; i < d / 4; ++i) {
    const float4 v = r4[i];
    s += v.x * q[4 * i] + v.y * q[4 * i + 1] + v.z * q[4 * i + 2] + v.w * q[4 * i + 3];
  }
  return s;
}

template <>
__device__ __forceinline__ float dot_row<bf16>(const bf16* __restrict__ row,
                                               const float* __restrict__ q, int d) {
  float s = 0.f;
  if (d % 8) {                                 // rows that do not start on 16-byte boundaries
    for (int i = 0; i < d; ++i) s += __bfloat162float(row[i]) * q[i];
    return s;
  }
  const uint4* r4 = reinterpret_cast<const uint4*>(row);
  for (int i = 0; i < d / 8; ++i) {
    const uint4 v = r4[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      s += f.x * q[8 * i + 2 * j] + f.y * q[8 * i + 2 * j + 1];
    }
  }
  return s;
}

template <typename T>
__global__ void attention_generic_kernel(T* __restrict__ out, const T* __restrict__ q,
                                         int q_row_stride, const int* __restrict__ positions,
                                         const int* __restrict__ token_slot, PagedKV cache,
                                         int n_q_heads, float scale, int window, int n_splits,
                                         int keys_per_split, float* __restrict__ part_acc,
                                         float* __restrict__ part_ml, float sink,
                                         const float* __restrict__ sinks, int keep_first,
                                         const T* __restrict__ gate, int gate_stride, int cross,
                                         float* __restrict__ out32) {
  __shared__ float q_s[kGenericMaxDim];
  __shared__ float p_s[kAttnThreads];
  __shared__ size_t voff_s[kAttnThreads];
  __shared__ float scratch[33];

  // cross > 1: grid.y runs over (query head, value head) pairs - the head's softmax weights, taken
  // against its own key head, are applied to the values of EVERY key/value head in turn
  const int t = blockIdx.x, h = blockIdx.y / cross, split = blockIdx.z;
  const int tid = threadIdx.x;
  if (sinks != nullptr) sink = sinks[h];        // a sink score of its own for every query head
  const int d = cache.head_dim;
  const int kv_head = h / (n_q_heads / cache.heads);
  const int v_head = cross > 1 ? (int)(blockIdx.y % cross) : kv_head;
  const int pos = positions[t];
  const size_t part_index = ((size_t)t * gridDim.y + blockIdx.y) * n_splits + split;

  int lo = 0, hi = -1;                          // keys [lo, hi] ...
  int f_lo = 0, f_hi = -1;                      // ... and the kept first keys [f_lo, f_hi] before them
  if (pos >= 0) {
    lo = window > 0 ? max(0, pos - window + 1) : 0;
    hi = pos;
    f_hi = min(keep_first, lo) - 1;
    if (n_splits > 1) {
      lo = max(lo, split * keys_per_split);
      hi = min(hi, (split + 1) * keys_per_split - 1);
      f_lo = max(f_lo, split * keys_per_split);
      f_hi = min(f_hi, (split + 1) * keys_per_split - 1);
    }
  }
  const int n_first = max(0, f_hi - f_lo + 1);
  const int total = n_first + max(0, hi - lo + 1);

  float acc[kGenericAcc];                       // dims tid, tid + 128, ... (those below d)
#pragma unroll
  for (int a = 0; a < kGenericAcc; ++a) acc[a] = 0.f;
  float m = -INFINITY, l = 0.f;
  if (total > 0) {
    const int slot = token_slot[t];
    const int* table = cache.block_table + (size_t)slot * cache.table_stride;
    const T* qrow = q + (size_t)t * q_row_stride + (size_t)h * d;
    for (int i = tid; i < d; i += kAttnThreads) q_s[i] = to_f<T>(qrow[i]) * scale;
    __syncthreads();
    const T* kbase = (const T*)cache.k;
    const T* vbase = (const T*)cache.v;
    for (int start = 0; start < total; start += kAttnThreads) {
      const int x = start + tid;
      const int j = x < n_first ? f_lo + x : lo + (x - n_first);
      const bool seen = x < total;
      float s = -INFINITY;
      if (seen) {
        const int page = table[j / EK_PAGE];
        voff_s[tid] = page_offset(cache, page, v_head, j);
        s = dot_row<T>(kbase + page_offset(cache, page, kv_head, j), q_s, d);
      }
      const float m_new = fmaxf(m, block_max(s, scratch));
      const float p = seen ? expf(s - m_new) : 0.f;
      p_s[tid] = p;
      const float alpha = expf(m - m_new);      // m = -inf on the first chunk: 0
      l = l * alpha + block_sum(p, scratch);    // the barriers inside also publish p_s, voff_s
      m = m_new;
      const int n = min(kAttnThreads, total - start);
#pragma unroll
      for (int a = 0; a < kGenericAcc; ++a) {
        acc[a] *= alpha;
        if (tid + a * kAttnThreads < d) {
          float s2 = acc[a];
          for (int i = 0; i < n; ++i) s2 += p_s[i] * to_f<T>(vbase[voff_s[i] + tid + a * kAttnThreads]);
          acc[a] = s2;
        }
      }
      __syncthreads();                          // before p_s / voff_s are overwritten
    }
  }

  if (n_splits == 1) {
    const size_t o_at = ((size_t)t * gridDim.y + blockIdx.y) * d;
    // a sink: one more term exp(sink) in the denominator, with no value (-inf: none)
    if (sink > -INFINITY && l > 0.f) l += expf(sink - m);
    float inv = l > 0.f ? 1.f / l : 0.f;
    if (gate != nullptr) inv *= 1.f / (1.f + expf(-to_f<T>(gate[(size_t)t * gate_stride + h])));
#pragma unroll
    for (int a = 0; a < kGenericAcc; ++a)
      if (tid + a * kAttnThreads < d) {
        if (out32) out32[o_at + tid + a * kAttnThreads] = acc[a] * inv;
        else out[o_at + tid + a * kAttnThreads] = from_f<T>(acc[a] * inv);
      }
  } else {
    float* pa = part_acc + part_index * d;
#pragma unroll
    for (int a = 0; a < kGenericAcc; ++a)
      if (tid + a * kAttnThreads < d) pa[tid + a * kAttnThreads] = acc[a];
    if (tid == 0) {
      part_ml[2 * part_index] = m;
      part_ml[2 * part_index + 1] = l;
    }
  }
}

// Merge the partial results of the key splits in split order.
template <typename T>
__global__ void attention_combine_kernel(T* __restrict__ out, const float* __restrict__ part_acc,
                                         const float* __restrict__ part_ml, int n_q_heads,
                                         int head_dim, int n_splits, float sink,
                                         const float* __restrict__ sinks, const T* __restrict__ gate,
                                         int gate_stride, int cross, float* __restrict__ out32) {
  const int h = blockIdx.y / cross;
  if (sinks != nullptr) sink = sinks[h];
  const size_t th = (size_t)blockIdx.x * gridDim.y + blockIdx.y;
  const float* ml = part_ml + 2 * th * n_splits;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, ml[2 * s]);
  float l = 0.f;
  for (int s = 0; s < n_splits; ++s)
    if (ml[2 * s + 1] > 0.f) l += ml[2 * s + 1] * expf(ml[2 * s] - m);
  if (sink > -INFINITY && l > 0.f) l += expf(sink - m);                 // the sink, counted once
  float inv = l > 0.f ? 1.f / l : 0.f;
  if (gate != nullptr) inv *= 1.f / (1.f + expf(-to_f<T>(gate[(size_t)blockIdx.x * gate_stride + h])));
  for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s)
      if (ml[2 * s + 1] > 0.f) acc += part_acc[(th * n_splits + s) * head_dim + i] * expf(ml[2 * s] - m);
    if (out32) out32[th * head_dim + i] = acc * inv;
    else out[th * head_dim + i] = from_f<T>(acc * inv);
  }
}

template <typename T>
static int launch(void* out, const void* q, int q_row_stride, const int* positions,
                  const int* token_slot, const void* k_pages, const void* v_pages,
                  const int* block_table, int table_stride, int n_tokens, int n_q_heads,
                  int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                  int keys_per_split, float* part_acc, float* part_ml, float sink,
                  const float* sinks, int keep_first, const void* gate, int gate_stride,
                  cudaStream_t stream, int cross = 1, float* out32 = nullptr) {
  if (n_tokens <= 0) return 0;
  if (head_dim <= 0 || head_dim > kGenericMaxDim || n_kv_heads <= 0 ||
      n_q_heads % n_kv_heads || n_q_heads > 65535 || n_splits < 1 || n_splits > 65535 ||
      (n_splits > 1 && (!part_acc || !part_ml || keys_per_split <= 0)) ||
      (cross != 1 && cross != n_kv_heads) || (long long)n_q_heads * cross > 65535)
    return EK_ERR_ARG;
  PagedKV cache{(void*)k_pages, (void*)v_pages, block_table, table_stride, n_kv_heads, head_dim};
  dim3 grid(n_tokens, n_q_heads * cross, n_splits);
  attention_generic_kernel<T><<<grid, kAttnThreads, 0, stream>>>(
      (T*)out, (const T*)q, q_row_stride, positions, token_slot, cache, n_q_heads, scale, window,
      n_splits, keys_per_split, part_acc, part_ml, sink, sinks, window > 0 ? keep_first : 0,
      (const T*)gate, gate_stride, cross, out32);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || n_splits == 1) return (int)e;
  dim3 cgrid(n_tokens, n_q_heads * cross);
  attention_combine_kernel<T><<<cgrid, 64, 0, stream>>>((T*)out, part_acc, part_ml, n_q_heads,
                                                        head_dim, n_splits, sink, sinks,
                                                        (const T*)gate, gate_stride, cross, out32);
  EK_RETURN_LAUNCH_STATUS();
}

// Heads that share their softmax weights ("talking heads" behind the softmax): with
// weight_h <- sum_g mix[h, g] weight_g and head h applying its mixed weights to the values of its own
// key/value head c(h) = h / (H / G), the result is  out_h = sum_g mix[h, g] * A[g, c(h)],  A[g, c] being
// head g's weights applied to value head c - what the attention kernels above write with cross = G
// (32-bit, [T, H, G, head size]).  This kernel forms the sums, multiplies element by element by the
// sigmoid of a gate row (optional) and rounds: out [T, H * vdim].  grid: tokens.
template <typename T>
__global__ void mix_heads_kernel(T* __restrict__ out, const float* __restrict__ parts, const float* __restrict__ mix,
                                 const T* __restrict__ gate, int gate_stride, int n_q_heads, int n_kv_heads,
                                 int head_dim, int vdim, const int* __restrict__ positions) {
  // grid (tokens, value heads): a block stages A[., c] of its token - every head's weights on value head c -
  // once, and forms the results of the heads that own value head c from it
  extern __shared__ __align__(16) float mix_s[];              // [H][H] mix, then [H][vdim] parts
  float* a_s = mix_s + n_q_heads * n_q_heads;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, c = blockIdx.y;
  const int per = n_q_heads / n_kv_heads;
  if (positions[t] < 0) {                       // a row of a finished sequence: zeros
    for (int i = threadIdx.x; i < per * vdim; i += blockDim.x)
      out[(size_t)t * n_q_heads * vdim + (size_t)c * per * vdim + i] = from_f<T>(0.f);
    return;
  }
  for (int i = threadIdx.x; i < n_q_heads * n_q_heads; i += blockDim.x) mix_s[i] = mix[i];
  const float* a = parts + ((size_t)t * n_q_heads * n_kv_heads + c) * head_dim;
  for (int i = threadIdx.x; i < n_q_heads * vdim; i += blockDim.x) {
    const int g = i / vdim, j = i % vdim;
    a_s[i] = a[(size_t)g * n_kv_heads * head_dim + j];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < per * vdim; i += blockDim.x) {
    const int h = c * per + i / vdim, j = i % vdim;
    float acc = 0.f;
    for (int g = 0; g < n_q_heads; ++g) acc = fmaf(mix_s[h * n_q_heads + g], a_s[g * vdim + j], acc);
    const size_t at = (size_t)h * vdim + j;
    if (gate != nullptr) acc *= 1.f / (1.f + expf(-to_f<T>(gate[(size_t)t * gate_stride + at])));
    out[(size_t)t * n_q_heads * vdim + at] = from_f<T>(acc);
  }
}

}  // namespace ek

#define EK_INSTANTIATE(SUFFIX, T)                                                              \
  EK_EXPORT int ek_attention_generic_##SUFFIX(                                                  \
      void* out, const void* q, int q_row_stride, const int* positions, const int* token_slot, \
      const void* k_pages, const void* v_pages, const int* block_table, int table_stride,      \
      int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, float scale, int window,      \
      int n_splits, int keys_per_split, float* part_acc, float* part_ml, float sink,           \
      const float* sinks, int keep_first, const void* gate, int gate_stride,                   \
      cudaStream_t stream) {                                                                   \
    return ek::launch<T>(out, q, q_row_stride, positions, token_slot, k_pages, v_pages,        \
                         block_table, table_stride, n_tokens, n_q_heads, n_kv_heads, head_dim, \
                         scale, window, n_splits, keys_per_split, part_acc, part_ml, sink,     \
                         sinks, keep_first, gate, gate_stride, stream);                        \
  }

#define EK_INSTANTIATE_CROSS(SUFFIX, T)                                                        \
  /* Every query head's weights applied to the values of every key/value head: out32          */ \
  /* [T, heads, kv heads, head size] in 32-bit (see mix_heads_kernel).                        */ \
  EK_EXPORT int ek_attention_generic_cross_##SUFFIX(                                            \
      float* out32, const void* q, int q_row_stride, const int* positions, const int* token_slot, \
      const void* k_pages, const void* v_pages, const int* block_table, int table_stride,      \
      int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, float scale, int window,      \
      int n_splits, int keys_per_split, float* part_acc, float* part_ml, int keep_first,       \
      cudaStream_t stream) {                                                                   \
    if (!out32) return EK_ERR_ARG;                                                             \
    return ek::launch<T>(nullptr, q, q_row_stride, positions, token_slot, k_pages, v_pages,    \
                         block_table, table_stride, n_tokens, n_q_heads, n_kv_heads, head_dim, \
                         scale, window, n_splits, keys_per_split, part_acc, part_ml, -INFINITY, \
                         nullptr, keep_first, nullptr, 0, stream, n_kv_heads, out32);          \
  }                                                                                            \
  EK_EXPORT int ek_mix_heads_##SUFFIX(void* out, const float* parts, const float* mix, const void* gate, \
                                      int gate_stride, const int* positions, int n_tokens, int n_q_heads, \
                                      int n_kv_heads, int head_dim, int vdim, cudaStream_t stream) { \
    if (n_tokens <= 0) return 0;                                                               \
    if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads || vdim <= 0 || vdim > head_dim || \
        n_q_heads > 96 || (gate && gate_stride < n_q_heads * vdim))                            \
      return EK_ERR_ARG;                                                                       \
    const size_t smem = (size_t)n_q_heads * (n_q_heads + vdim) * sizeof(float);                \
    if (smem > 200 * 1024 || n_kv_heads > 65535) return EK_ERR_ARG;                            \
    if (smem > 40 * 1024) {                                                                    \
      cudaError_t e = cudaFuncSetAttribute(ek::mix_heads_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                         \
      if (e != cudaSuccess) return (int)e;                                                     \
    }                                                                                          \
    return (int)ek::launch_pdl(ek::mix_heads_kernel<T>, dim3(n_tokens, n_kv_heads), dim3(128), smem, stream, \
                               (T*)out, parts, mix, (const T*)gate, gate_stride, n_q_heads, n_kv_heads, \
                               head_dim, vdim, positions);                                     \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)
EK_INSTANTIATE_CROSS(f32, float)
EK_INSTANTIATE_CROSS(bf16, ek::bf16)
