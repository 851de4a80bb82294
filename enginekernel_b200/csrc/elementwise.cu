// Embedding lookup (also through a hashed table of token pairs), RMSNorm (plain, with the residual add
// folded in, on gathered rows, behind a sum of scaled results, and as the pair "norm of a result, add,
// norm of the stream"), the SwiGLU gate, and bias + activation on a projection's rows.
//
// The residual stream is held in 32-bit in both precisions; T is the type of the
// normalised activations that feed the matrix products (float or bfloat16).
// Mean of squares, the scaling and the residual sum are computed in 32-bit
// (the reference does the same inside its norm kernels, engine/ek_kernels.py:89-123,
// but stores the stream in bfloat16).
#include "common.cuh"

namespace ek {

// resid[t] = table[ids[t]] * scale (+ pos_table[positions[t]] if the model has learned positions);
// with `accumulate` the same is added to what resid[t] holds (a model that feeds its embedding
// output into the stream again at a later layer).
template <typename T>
__global__ void embed_kernel(float* __restrict__ resid, const T* __restrict__ table,
                             const int* ids, int hidden, int vocab, float scale,
                             const T* __restrict__ pos_table, const int* positions, int max_positions,
                             int accumulate) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T* row = table + (size_t)id * hidden;
  float* out = resid + (size_t)t * hidden;
  const T* prow = nullptr;
  if (pos_table != nullptr) {
    const int p = positions[t];                // rows of finished sequences (negative) get no position
    if (p >= 0) prow = pos_table + (size_t)min(p, max_positions - 1) * hidden;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    out[i] = (accumulate ? out[i] : 0.f) + (to_f<T>(row[i]) * scale + (prow ? to_f<T>(prow[i]) : 0.f));
}

__global__ void scale_f32_kernel(float* x, size_t n, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] *= scale;
}


// y = gain * x * rsqrt(mean(x^2) + eps) for each row; x is the 32-bit stream.
// If `add` is given, the stream first becomes stream + add (written back when
// `write_back`).  If `rows` is given, output row i reads stream row rows[i].
// VEC: the row length is a multiple of 4 and rows are accessed four values at a time.
template <typename T, bool VEC>
__global__ void rmsnorm_kernel(T* __restrict__ y, float* resid, const T* add,
                               const float* __restrict__ gain, const int* rows, float eps, int hidden,
                               int write_back) {
  __shared__ float scratch[33];
  extern __shared__ __align__(16) float row_cache[];          // `hidden` floats
  pdl_launch_dependents();
  pdl_wait();
  const int out_row = blockIdx.x;
  const int src_row = rows ? rows[out_row] : out_row;
  float* r = resid + (size_t)src_row * hidden;
  const T* a = add ? add + (size_t)src_row * hidden : nullptr;
  T* out = y + (size_t)out_row * hidden;
  float ss = 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(r + i);
      if (a) {
        const float4 w = Vec4<T>::load(a + i);
        v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        if (write_back) *reinterpret_cast<float4*>(r + i) = v;
      }
      *reinterpret_cast<float4*>(row_cache + i) = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = r[i];
      if (a) {
        v += to_f<T>(a[i]);
        if (write_back) r[i] = v;
      }
      row_cache[i] = v;
      ss += v * v;
    }
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row_cache + i);
      const float4 g = *reinterpret_cast<const float4*>(gain + i);
      Vec4<T>::store(out + i, make_float4(v.x * rstd * g.x, v.y * rstd * g.y, v.z * rstd * g.z,
                                          v.w * rstd * g.w));
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      out[i] = from_f<T>(row_cache[i] * rstd * gain[i]);
  }
}

// The same for rows of at most 4,096 values in steps of 4: 128 threads a row, the row held in
// registers (NV loads of 16 bytes a thread at most, all issued before the first use), no row in
// shared memory - so that an SM keeps more rows in flight, which is what a kernel that only moves
// memory needs.  Same arithmetic; the sum of squares is taken in another order.
constexpr int kNormRegThreads = 128, kNormRegVecs = 8;
template <typename T, int NV>
__global__ void __launch_bounds__(kNormRegThreads, NV <= 6 ? 8 : 5)
rmsnorm_reg_kernel(T* __restrict__ y, float* resid, const T* add, const float* __restrict__ gain,
                   const int* rows, float eps, int hidden, int write_back) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int out_row = blockIdx.x;
  const int src_row = rows ? rows[out_row] : out_row;
  float* r = resid + (size_t)src_row * hidden;
  const T* a = add ? add + (size_t)src_row * hidden : nullptr;
  T* out = y + (size_t)out_row * hidden;
  float4 v[NV], w[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = (threadIdx.x + j * kNormRegThreads) * 4;
    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    w[j] = v[j];
    if (i < hidden) {
      v[j] = *reinterpret_cast<const float4*>(r + i);
      if (a) w[j] = Vec4<T>::load(a + i);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = (threadIdx.x + j * kNormRegThreads) * 4;
    if (a) {
      v[j].x += w[j].x; v[j].y += w[j].y; v[j].z += w[j].z; v[j].w += w[j].w;
      if (write_back && i < hidden) *reinterpret_cast<float4*>(r + i) = v[j];
    }
    ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = (threadIdx.x + j * kNormRegThreads) * 4;
    if (i < hidden) {
      const float4 g = *reinterpret_cast<const float4*>(gain + i);
      Vec4<T>::store(out + i, make_float4(v[j].x * rstd * g.x, v[j].y * rstd * g.y, v[j].z * rstd * g.z,
                                          v[j].w * rstd * g.w));
    }
  }
}

// The same norm behind a sum of two sublayer outputs, each multiplied element by element by a 32-bit
// vector of the stream's width first (a learned scale per channel): stream += a * sa + b * sb, then
// y = gain * n(stream).  `b` (with `sb`) may be absent; `sa` / `sb` absent count as ones.  For layers
// whose mixer and feed-forward read the same normed input and are added together.
template <typename T>
__global__ void rmsnorm_scaled_sum_kernel(T* __restrict__ y, float* resid, const T* __restrict__ a,
                                          const float* __restrict__ sa, const T* __restrict__ b,
                                          const float* __restrict__ sb, const float* __restrict__ gain,
                                          const int* rows, float eps, int hidden, int write_back) {
  __shared__ float scratch[33];
  extern __shared__ __align__(16) float row_cache[];          // `hidden` floats
  pdl_launch_dependents();
  pdl_wait();
  const int out_row = blockIdx.x;
  const int src_row = rows ? rows[out_row] : out_row;
  float* r = resid + (size_t)src_row * hidden;
  const T* ar = a + (size_t)src_row * hidden;
  const T* br = b ? b + (size_t)src_row * hidden : nullptr;
  T* out = y + (size_t)out_row * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float add = to_f<T>(ar[i]) * (sa ? sa[i] : 1.f);
    if (br) add = fmaf(to_f<T>(br[i]), sb ? sb[i] : 1.f, add);
    const float v = r[i] + add;
    if (write_back) r[i] = v;
    row_cache[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    out[i] = from_f<T>(row_cache[i] * rstd * gain[i]);
}

// stream += add, without a norm (the last feed-forward output when no norm follows)
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ resid, const T* __restrict__ add, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) resid[i] += to_f<T>(add[i]);
}

// stream[r, i] += a[r, i] * sa[i] + b[r, i] * sb[i] without a norm (`b` may be absent; absent scales
// count as ones): the last layer's outputs of a model whose layers scale them per channel
template <typename T>
__global__ void add_scaled_kernel(float* __restrict__ resid, const T* __restrict__ a, const float* __restrict__ sa,
                                  const T* __restrict__ b, const float* __restrict__ sb, size_t n, int hidden) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int c = (int)(i % hidden);
  float add = to_f<T>(a[i]) * (sa ? sa[c] : 1.f);
  if (b) add = fmaf(to_f<T>(b[i]), sb ? sb[c] : 1.f, add);
  resid[i] += add;
}
// the same, four neighbours a thread (hidden a multiple of 4, every row on a 16-byte boundary)
template <typename T>
__global__ void add_scaled4_kernel(float* __restrict__ resid, const T* __restrict__ a, const float* __restrict__ sa,
                                   const T* __restrict__ b, const float* __restrict__ sb, size_t n4, int hidden4) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const int c = (int)(i % hidden4);
  const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
  const float4 fa = sa ? reinterpret_cast<const float4*>(sa)[c] : one, fb = sb ? reinterpret_cast<const float4*>(sb)[c] : one;
  float4 r = reinterpret_cast<float4*>(resid)[i];
  float va[4], vb[4] = {0.f, 0.f, 0.f, 0.f};
  if (sizeof(T) == 2) {
    const uint2 pa = reinterpret_cast<const uint2*>(a)[i];
    const T* ta = reinterpret_cast<const T*>(&pa);
#pragma unroll
    for (int j = 0; j < 4; ++j) va[j] = to_f<T>(ta[j]);
    if (b) {
      const uint2 pb = reinterpret_cast<const uint2*>(b)[i];
      const T* tb = reinterpret_cast<const T*>(&pb);
#pragma unroll
      for (int j = 0; j < 4; ++j) vb[j] = to_f<T>(tb[j]);
    }
  } else {
    const float4 pa = reinterpret_cast<const float4*>(a)[i];
    va[0] = pa.x, va[1] = pa.y, va[2] = pa.z, va[3] = pa.w;
    if (b) {
      const float4 pb = reinterpret_cast<const float4*>(b)[i];
      vb[0] = pb.x, vb[1] = pb.y, vb[2] = pb.z, vb[3] = pb.w;
    }
  }
  r.x += fmaf(vb[0], fb.x, va[0] * fa.x);
  r.y += fmaf(vb[1], fb.y, va[1] * fa.y);
  r.z += fmaf(vb[2], fb.z, va[2] * fa.z);
  r.w += fmaf(vb[3], fb.w, va[3] * fa.w);
  reinterpret_cast<float4*>(resid)[i] = r;
}

// out[r, i] = act(gu[r, i]) * gu[r, inter + i]    (silu: engine/ek_kernels.py:125-143)
// VEC: inter is a multiple of 4; a thread handles four neighbours.  A 16-bit result takes the
// fast exponential and division (a few 32-bit ulps, far below its own rounding); a 32-bit
// result the exact ones.
// ACT 0: silu(g) = g / (1 + exp(-g)).  ACT 1: the tanh form of GELU,
// 0.5 g (1 + tanh(u)) with u = sqrt(2/pi) (g + 0.044715 g^3), which is g / (1 + exp(-2u)).
template <typename T, int ACT = 0>
__device__ __forceinline__ float silu_of(float g) {
  if (ACT == 1) {
    const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    if (sizeof(T) == 2) return __fdividef(g, 1.f + __expf(-2.f * u));
    return 0.5f * g * (1.f + tanhf(u));
  }
  if (sizeof(T) == 2) return __fdividef(g, 1.f + __expf(-g));
  return g / (1.f + expf(-g));
}

// resid[t] += table[row], row = (previous * mul_prev + ids[t] * mul_cur) mod buckets, or row `buckets`
// (the table's last) for a sequence's first token.  The token before t is the step's token t - 1 when
// that belongs to the same sequence, else what the sequence's slot holds in `before` (a 32-bit integer
// per slot, `before_stride` apart).  A plain launch; rows whose position is negative are skipped.
template <typename T>
__global__ void embed_pair_kernel(float* __restrict__ resid, const T* __restrict__ table, const int* ids,
                                  const int* positions, const int* token_slot, const int* before,
                                  long long before_stride, int hidden, int buckets, long long mul_prev,
                                  long long mul_cur) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  if (pos < 0) return;
  int row = buckets;
  if (pos > 0) {
    const int slot = token_slot[t];
    const int prev = (t > 0 && token_slot[t - 1] == slot && positions[t - 1] == pos - 1)
                         ? ids[t - 1] : before[(size_t)slot * before_stride];
    row = (int)(((long long)prev * mul_prev + (long long)ids[t] * mul_cur) % (long long)buckets);
  }
  const T* src = table + (size_t)row * hidden;
  float* out = resid + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] += to_f<T>(src[i]);
}

// before[slot] = the last token a sequence brought in this step.
__global__ void keep_last_token_kernel(int* before, long long before_stride, const int* ids, const int* positions,
                                       const int* token_slot, int n_tokens) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tokens || positions[t] < 0) return;
  const int slot = token_slot[t];
  if (t + 1 < n_tokens && token_slot[t + 1] == slot && positions[t + 1] == positions[t] + 1) return;
  before[(size_t)slot * before_stride] = ids[t];
}

// dst[r, col0 + i] = src[r, i] rounded to T, for i < width (dst rows `dst_stride` apart).
template <typename T>
__global__ void cast_columns_kernel(T* __restrict__ dst, int dst_stride, int col0, const float* __restrict__ src,
                                    int width, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t r = i / width;
  const int c = (int)(i % width);
  dst[r * dst_stride + col0 + c] = from_f<T>(src[i]);
}

// A sublayer's result passes a norm of its own before it joins the stream, and the norm of the next
// reader follows in the same pass over the row:
//     u = a * wa + b * wb + bias          (b, bias optional; wa, wb plain numbers)
//     stream += gain_post * u * rsqrt(mean(u^2) + eps_post)
//     y = gain * stream * rsqrt(mean(stream^2) + eps)          (only when y is given)
// A block a row, the row in shared memory (2 x hidden floats).
template <typename T>
__global__ void rmsnorm_post_add_kernel(T* __restrict__ y, float* resid, const T* __restrict__ a, float wa,
                                        const T* __restrict__ b, float wb, const float* __restrict__ bias,
                                        const float* __restrict__ gain_post, float eps_post,
                                        const float* __restrict__ gain, float eps, int hidden) {
  __shared__ float scratch[33];
  extern __shared__ __align__(16) float row_cache[];          // u, then the stream's row
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  float* r = resid + row * hidden;
  const T* ar = a + row * hidden;
  const T* br = b ? b + row * hidden : nullptr;
  float* u_s = row_cache;
  float* x_s = row_cache + hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float u = to_f<T>(ar[i]) * wa;
    if (br) u = fmaf(to_f<T>(br[i]), wb, u);
    if (bias) u += bias[i];
    u_s[i] = u;
    x_s[i] = r[i];
    ss += u * u;
  }
  const float rstd_post = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps_post);
  ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = x_s[i] + u_s[i] * rstd_post * gain_post[i];
    r[i] = v;
    x_s[i] = v;
    ss += v * v;
  }
  if (y == nullptr) return;
  const float rstd = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
  T* out = y + row * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = from_f<T>(x_s[i] * rstd * gain[i]);
}

// Four neighbouring values a thread, a row a block row (grid (rows, column tiles)): for widths, offsets and
// strides that are multiples of 4 and pointers on 16-byte boundaries.
template <typename T>
__global__ void cast_columns4_kernel(T* __restrict__ dst, int dst_stride, int col0, const float* __restrict__ src,
                                     int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (c >= width) return;
  const size_t r = blockIdx.x;
  Vec4<T>::store(dst + r * dst_stride + col0 + c, *reinterpret_cast<const float4*>(src + r * width + c));
}

template <typename T, typename X>
__global__ void bias_act4_kernel(T* __restrict__ out, const X* __restrict__ x, int x_stride, int col0,
                                 const float* __restrict__ bias, int width, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (c >= width) return;
  const size_t r = blockIdx.x;
  float4 v = Vec4<X>::load(x + r * x_stride + col0 + c);
  if (bias) {
    const float4 b = *reinterpret_cast<const float4*>(bias + c);
    v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
  }
  if (act == 1) v = make_float4(silu_of<T, 1>(v.x), silu_of<T, 1>(v.y), silu_of<T, 1>(v.z), silu_of<T, 1>(v.w));
  else if (act == 2) v = make_float4(silu_of<T, 0>(v.x), silu_of<T, 0>(v.y), silu_of<T, 0>(v.z), silu_of<T, 0>(v.w));
  Vec4<T>::store(out + r * width + c, v);
}

// out[r, i] = act(x[r, col0 + i] + bias[i]) for i < width; act 0: none, 1: the tanh form of GELU, 2: SiLU.
// x is 32-bit or T (`x_is_f32`), rows `x_stride` apart.
template <typename T>
__global__ void bias_act_kernel(T* __restrict__ out, const void* __restrict__ x, int x_is_f32, int x_stride,
                                int col0, const float* __restrict__ bias, int width, size_t n, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t r = i / width;
  const int c = (int)(i % width);
  const size_t at = r * x_stride + col0 + c;
  float v = x_is_f32 ? ((const float*)x)[at] : to_f<T>(((const T*)x)[at]);
  if (bias) v += bias[c];
  if (act == 1) v = silu_of<T, 1>(v);
  else if (act == 2) v = silu_of<T, 0>(v);
  out[i] = from_f<T>(v);
}

template <typename T, bool VEC, int ACT>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int inter) {
  const size_t r = blockIdx.y;
  const T* g_row = gu + r * 2 * inter;
  T* o_row = out + r * inter;
  if (VEC) {
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= inter) return;
    const float4 g = Vec4<T>::load(g_row + i), u = Vec4<T>::load(g_row + inter + i);
    Vec4<T>::store(o_row + i, make_float4(silu_of<T, ACT>(g.x) * u.x, silu_of<T, ACT>(g.y) * u.y,
                                          silu_of<T, ACT>(g.z) * u.z, silu_of<T, ACT>(g.w) * u.w));
  } else {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const float g = to_f<T>(g_row[i]), u = to_f<T>(g_row[inter + i]);
    o_row[i] = from_f<T>(silu_of<T, ACT>(g) * u);
  }
}

// The same for bfloat16 rows whose halves start on 16-byte boundaries: eight neighbours a thread.
template <int ACT>
__global__ void silu_mul_wide_kernel(bf16* __restrict__ out, const bf16* __restrict__ gu, int inter) {
  const size_t r = blockIdx.y;
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= inter) return;
  const bf16* g_row = gu + r * 2 * inter;
  const uint4 g = *reinterpret_cast<const uint4*>(g_row + i);
  const uint4 u = *reinterpret_cast<const uint4*>(g_row + inter + i);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 a = __bfloat1622float2(g2[j]), b = __bfloat1622float2(u2[j]);
    __nv_bfloat162 h = __floats2bfloat162_rn(silu_of<bf16, ACT>(a.x) * b.x, silu_of<bf16, ACT>(a.y) * b.y);
    w[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(out + r * inter + i) = make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename T>
static int launch_rmsnorm(void* y, float* resid, const void* add, const float* gain,
                          const int* rows, float eps, int n_rows, int hidden, int write_back,
                          cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || (size_t)hidden * 4 > 200 * 1024) return EK_ERR_ARG;
  const size_t smem = (size_t)hidden * sizeof(float);
  const bool vec = hidden % 4 == 0 && ((uintptr_t)y % 8) == 0 && ((uintptr_t)add % 8) == 0;
  if (vec && hidden <= kNormRegThreads * kNormRegVecs * 4 && ((uintptr_t)resid % 16) == 0 &&
      ((uintptr_t)gain % 16) == 0)
  {
    const int nv = (hidden / 4 + kNormRegThreads - 1) / kNormRegThreads;
    auto reg_kernel = nv <= 2 ? rmsnorm_reg_kernel<T, 2> : nv <= 4 ? rmsnorm_reg_kernel<T, 4>
                    : nv <= 6 ? rmsnorm_reg_kernel<T, 6> : rmsnorm_reg_kernel<T, 8>;
    return (int)launch_pdl(reg_kernel, dim3(n_rows), dim3(kNormRegThreads), 0, stream, (T*)y, resid,
                           (const T*)add, gain, rows, eps, hidden, write_back);
  }
  auto kernel = vec ? rmsnorm_kernel<T, true> : rmsnorm_kernel<T, false>;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int per_thread = vec ? 4 : 1;
  int threads = hidden / per_thread >= 512 ? 512 : (hidden / per_thread >= 256 ? 256 : 128);
  return (int)launch_pdl(kernel, dim3(n_rows), dim3(threads), smem, stream, (T*)y, resid,
                         (const T*)add, gain, rows, eps, hidden, write_back);
}

template <typename T, int ACT>
static int launch_silu_mul(void* out, const void* gu, int rows, int inter, cudaStream_t stream) {
  if (rows <= 0 || inter <= 0) return 0;
  if (rows > 65535) return EK_ERR_ARG;
  if (sizeof(T) == 2 && inter % 8 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)gu % 16) == 0) {
    dim3 wide((inter / 8 + 255) / 256, rows);
    silu_mul_wide_kernel<ACT><<<wide, 256, 0, stream>>>((bf16*)out, (const bf16*)gu, inter);
    EK_RETURN_LAUNCH_STATUS();
  }
  const bool vec = inter % 4 == 0 && ((uintptr_t)out % 8) == 0 && ((uintptr_t)gu % 8) == 0;
  const int per_thread = vec ? 4 : 1;
  dim3 grid((inter / per_thread + 255) / 256 + (inter % per_thread ? 1 : 0), rows);
  if (vec) silu_mul_kernel<T, true, ACT><<<grid, 256, 0, stream>>>((T*)out, (const T*)gu, inter);
  else silu_mul_kernel<T, false, ACT><<<grid, 256, 0, stream>>>((T*)out, (const T*)gu, inter);
  EK_RETURN_LAUNCH_STATUS();
}

}  // namespace ek

using namespace ek;

#define EK_INSTANTIATE(SUFFIX, T)                                                               \
  EK_EXPORT int ek_embed_##SUFFIX(float* resid, const void* table, const int* ids, int n_tokens, \
                                  int hidden, int vocab, float scale, const void* pos_table,    \
                                  const int* positions, int max_positions, int accumulate,      \
                                  cudaStream_t stream) {                                        \
    if (n_tokens <= 0) return 0;                                                                \
    if (pos_table && (!positions || max_positions <= 0)) return EK_ERR_ARG;                     \
    /* A plain launch, on purpose: the first kernel of a step starts only when everything   */ \
    /* before it on the stream has finished and is visible.  The kernels behind it may then */ \
    /* read per-step state (positions, slots) before their own griddepcontrol.wait even     */ \
    /* when the step before was not a graph launch of its own (eager decode).               */ \
    embed_kernel<T><<<dim3(n_tokens), dim3(256), 0, stream>>>(resid, (const T*)table, ids,     \
                                                               hidden, vocab, scale,            \
                                                               (const T*)pos_table, positions,  \
                                                               max_positions, accumulate);      \
    EK_RETURN_LAUNCH_STATUS();                                                                  \
  }                                                                                             \
  EK_EXPORT int ek_rmsnorm_##SUFFIX(void* y, float* resid, const void* add, const float* gain,  \
                                    const int* rows, float eps, int n_rows, int hidden,         \
                                    int write_back, cudaStream_t stream) {                      \
    return launch_rmsnorm<T>(y, resid, add, gain, rows, eps, n_rows, hidden, write_back, stream); \
  }                                                                                             \
  EK_EXPORT int ek_rmsnorm_scaled_sum_##SUFFIX(void* y, float* resid, const void* a, const float* sa, \
                                               const void* b, const float* sb, const float* gain, \
                                               const int* rows, float eps, int n_rows, int hidden, \
                                               int write_back, cudaStream_t stream) {           \
    if (n_rows <= 0) return 0;                                                                  \
    if (hidden <= 0 || (size_t)hidden * 4 > 200 * 1024 || a == nullptr) return EK_ERR_ARG;      \
    const size_t smem = (size_t)hidden * sizeof(float);                                         \
    auto kernel = ek::rmsnorm_scaled_sum_kernel<T>;                                             \
    if (smem > 40 * 1024) {                                                                     \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                      \
    }                                                                                           \
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);                     \
    return (int)ek::launch_pdl(kernel, dim3(n_rows), dim3(threads), smem, stream, (T*)y, resid, \
                               (const T*)a, sa, (const T*)b, sb, gain, rows, eps, hidden,       \
                               write_back);                                                     \
  }                                                                                             \
  EK_EXPORT int ek_embed_pair_##SUFFIX(float* resid, const void* table, const int* ids,           \
                                       const int* positions, const int* token_slot, const int* before, \
                                       long long before_stride, int n_tokens, int hidden, int buckets, \
                                       long long mul_prev, long long mul_cur, cudaStream_t stream) { \
    if (n_tokens <= 0) return 0;                                                                \
    if (buckets <= 0 || mul_prev < 0 || mul_cur < 0 || hidden <= 0) return EK_ERR_ARG;          \
    embed_pair_kernel<T><<<dim3(n_tokens), dim3(256), 0, stream>>>(resid, (const T*)table, ids, positions, \
                                                                    token_slot, before, before_stride, \
                                                                    hidden, buckets, mul_prev, mul_cur); \
    EK_RETURN_LAUNCH_STATUS();                                                                  \
  }                                                                                             \
  EK_EXPORT int ek_cast_columns_##SUFFIX(void* dst, int dst_stride, int col0, const float* src, int width, \
                                         int n_rows, cudaStream_t stream) {                     \
    if (n_rows <= 0) return 0;                                                                  \
    if (width <= 0 || col0 < 0 || dst_stride < col0 + width) return EK_ERR_ARG;                 \
    const size_t n = (size_t)n_rows * width;                                                    \
    if (width % 4 == 0 && col0 % 4 == 0 && dst_stride % 4 == 0 && (((uintptr_t)dst | (uintptr_t)src) & 15) == 0 \
        && (width + 1023) / 1024 <= 65535)                                                      \
      return (int)ek::launch_pdl(ek::cast_columns4_kernel<T>, dim3(n_rows, (width + 1023) / 1024), dim3(256), 0, \
                                 stream, (T*)dst, dst_stride, col0, src, width);                \
    return (int)ek::launch_pdl(ek::cast_columns_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, \
                               stream, (T*)dst, dst_stride, col0, src, width, n);               \
  }                                                                                             \
  EK_EXPORT int ek_rmsnorm_post_add_##SUFFIX(void* y, float* resid, const void* a, float wa, const void* b, \
                                             float wb, const float* bias, const float* gain_post, \
                                             float eps_post, const float* gain, float eps, int n_rows, \
                                             int hidden, cudaStream_t stream) {                 \
    if (n_rows <= 0) return 0;                                                                  \
    if (hidden <= 0 || (size_t)hidden * 8 > 200 * 1024 || a == nullptr || gain_post == nullptr || \
        (y != nullptr && gain == nullptr))                                                      \
      return EK_ERR_ARG;                                                                        \
    const size_t smem = (size_t)hidden * 2 * sizeof(float);                                     \
    auto kernel = ek::rmsnorm_post_add_kernel<T>;                                               \
    if (smem > 40 * 1024) {                                                                     \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                      \
    }                                                                                           \
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);                     \
    return (int)ek::launch_pdl(kernel, dim3(n_rows), dim3(threads), smem, stream, (T*)y, resid, \
                               (const T*)a, wa, (const T*)b, wb, bias, gain_post, eps_post, gain, eps, hidden); \
  }                                                                                             \
  EK_EXPORT int ek_bias_act_##SUFFIX(void* out, const void* x, int x_is_f32, int x_stride, int col0, \
                                     const float* bias, int width, int n_rows, int act, cudaStream_t stream) { \
    if (n_rows <= 0) return 0;                                                                  \
    if (width <= 0 || col0 < 0 || x_stride < col0 + width || act < 0 || act > 2) return EK_ERR_ARG; \
    const size_t n = (size_t)n_rows * width;                                                    \
    if (width % 4 == 0 && col0 % 4 == 0 && x_stride % 4 == 0 && (width + 1023) / 1024 <= 65535 && \
        (((uintptr_t)out | (uintptr_t)x | (uintptr_t)bias) & 15) == 0) {                        \
      const dim3 grid(n_rows, (width + 1023) / 1024);                                           \
      if (x_is_f32)                                                                             \
        return (int)ek::launch_pdl(ek::bias_act4_kernel<T, float>, grid, dim3(256), 0, stream, (T*)out, \
                                   (const float*)x, x_stride, col0, bias, width, act);          \
      return (int)ek::launch_pdl(ek::bias_act4_kernel<T, T>, grid, dim3(256), 0, stream, (T*)out, (const T*)x, \
                                 x_stride, col0, bias, width, act);                             \
    }                                                                                           \
    return (int)ek::launch_pdl(ek::bias_act_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, \
                               stream, (T*)out, x, x_is_f32, x_stride, col0, bias, width, n, act); \
  }                                                                                             \
  EK_EXPORT int ek_add_residual_##SUFFIX(float* resid, const void* add, long long n,            \
                                         cudaStream_t stream) {                                 \
    if (n <= 0) return 0;                                                                       \
    add_residual_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(resid, (const T*)add, \
                                                                             (size_t)n);        \
    EK_RETURN_LAUNCH_STATUS();                                                                  \
  }                                                                                             \
  EK_EXPORT int ek_add_scaled_##SUFFIX(float* resid, const void* a, const float* sa, const void* b, \
                                       const float* sb, long long n, int hidden, cudaStream_t stream) { \
    if (n <= 0) return 0;                                                                       \
    if (hidden <= 0 || a == nullptr) return EK_ERR_ARG;                                         \
    const uintptr_t bits = (uintptr_t)resid | (uintptr_t)sa | (uintptr_t)sb |                   \
                           (((uintptr_t)a | (uintptr_t)b) * (16 / (4 * sizeof(T))));            \
    if (hidden % 4 == 0 && (bits & 15) == 0)                                                    \
      add_scaled4_kernel<T><<<(unsigned)((n / 4 + 255) / 256), 256, 0, stream>>>(               \
          resid, (const T*)a, sa, (const T*)b, sb, (size_t)n / 4, hidden / 4);                  \
    else                                                                                        \
      add_scaled_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(                    \
          resid, (const T*)a, sa, (const T*)b, sb, (size_t)n, hidden);                          \
    EK_RETURN_LAUNCH_STATUS();                                                                  \
  }                                                                                             \
  EK_EXPORT int ek_silu_mul_##SUFFIX(void* out, const void* gu, int rows, int inter,            \
                                     cudaStream_t stream) {                                     \
    return launch_silu_mul<T, 0>(out, gu, rows, inter, stream);                                 \
  }                                                                                             \
  /* act 0: silu, 1: gelu (tanh form) */                                                        \
  EK_EXPORT int ek_act_mul_##SUFFIX(void* out, const void* gu, int rows, int inter, int act,    \
                                    cudaStream_t stream) {                                      \
    if (act == 0) return launch_silu_mul<T, 0>(out, gu, rows, inter, stream);                   \
    if (act == 1) return launch_silu_mul<T, 1>(out, gu, rows, inter, stream);                   \
    return EK_ERR_ARG;                                                                          \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)

// before[slot] = the last token every sequence of the step brought (see embed_pair_kernel)
EK_EXPORT int ek_keep_last_token(int* before, long long before_stride, const int* ids, const int* positions,
                                 const int* token_slot, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  ek::keep_last_token_kernel<<<(unsigned)((n_tokens + 255) / 256), 256, 0, stream>>>(before, before_stride, ids,
                                                                                      positions, token_slot, n_tokens);
  EK_RETURN_LAUNCH_STATUS();
}

// x[i] *= scale for n 32-bit values (logits of a model with a logit multiplier)
EK_EXPORT int ek_scale_f32(float* x, long long n, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  return (int)ek::launch_pdl(ek::scale_f32_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x,
                             (size_t)n, scale);
}
