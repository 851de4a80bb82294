// Per-head RMSNorm of queries and keys, rotary position encoding, and the write of
// keys and values into the paged cache - one pass over the fused q/k/v rows.
//
// Same work as the reference's _qk_norm_rope_kv_kernel (engine/ek_kernels.py:223-279):
// normalise each head over its dimension, rotate pairs (j, j + rot/2) by the angle of
// the token's position (NeoX pairing, engine/ek_model.py:164-174), leave values
// untouched, store keys and values at the token's place in its sequence's cache.
// Differences: positions and slots come per token (no padded rectangle), the cache is
// paged, and all arithmetic is 32-bit with one rounding at the end.
#include "common.cuh"

namespace ek {

constexpr int kRopeWarps = 4;

// What a design may ask for beyond norm and rotation (all off in a zeroed struct):
// biases of the projections, added here in 32-bit before anything else ([heads * head size] each);
// a query temperature, q *= 1 + coef * ln(floor((position + 1) / every) + 1), which sharpens the
// scores of late positions step by step; and values that are the keys as projected (bias added,
// before the key norm and rotation): the row then has no value heads, and a key head is stored
// twice, raw in the value pages and normalised in the key pages.
// `norm_dim` > 0: heads are padded with zeros up to the cache's head size and the query / key norm takes
// its mean over the first norm_dim values only.  `v_unit`: every value head is divided by its root mean
// square over its first v_norm_dim values (eps v_eps, no gain) before it is stored.
struct QkExtras {
  const float* q_bias;
  const float* k_bias;
  const float* v_bias;
  float q_temp_coef;
  int q_temp_every;
  int v_from_k;
  int norm_dim;
  int v_unit;
  int v_norm_dim;
  float v_eps;
};


template <typename T>
__global__ void qk_norm_rope_kv_kernel(T* qkv, int row_stride,
                                       const float* __restrict__ q_gain,
                                       const float* __restrict__ k_gain,
                                       const float* __restrict__ cos_tab,
                                       const float* __restrict__ sin_tab, int rot_dim,
                                       const int* positions, const int* token_slot,
                                       PagedKV cache,
                                       int n_q_heads, float eps, int write_kv, QkExtras ex) {
  __shared__ __align__(16) float buf[kRopeWarps][EK_MAX_HEAD_DIM];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * kRopeWarps + warp;
  const int n_kv = cache.heads, d = cache.head_dim;
  if (head >= n_q_heads + (ex.v_from_k ? 1 : 2) * n_kv) return;
  const int pos = positions[t];
  if (pos < 0) return;                        // a row of a finished sequence
  const bool is_q = head < n_q_heads;
  const bool is_k = !is_q && head < n_q_heads + n_kv;
  if (!is_q && !write_kv) return;

  T* src = qkv + (size_t)t * row_stride + (size_t)head * d;
  T* dst = src;
  T* dst_raw = nullptr;                       // where a key head also goes as the value
  const float* bias = is_q ? ex.q_bias : (is_k ? ex.k_bias : ex.v_bias);
  if (bias) bias += (size_t)(is_q ? head : (is_k ? head - n_q_heads : head - n_q_heads - n_kv)) * d;
  if (!is_q) {
    const int slot = token_slot[t];
    const int page = cache.block_table[(size_t)slot * cache.table_stride + pos / EK_PAGE];
    const int kv_head = is_k ? head - n_q_heads : head - n_q_heads - n_kv;
    dst = (T*)(is_k ? cache.k : cache.v) + page_offset(cache, page, kv_head, pos);
    if (is_k && ex.v_from_k) dst_raw = (T*)cache.v + page_offset(cache, page, kv_head, pos);
  }

  // Four neighbouring dimensions a lane when the sizes allow (head size a multiple of 4 and
  // the rotated half a multiple of 4), else one.
  const bool vec = (d % 4 == 0) && (rot_dim % 8 == 0) && (row_stride % 4 == 0);
  if (!is_q && !is_k && ex.v_unit) {          // values over their root mean square
    float y[EK_MAX_HEAD_DIM / 32];
    float ssv = 0.f;
#pragma unroll
    for (int r = 0; r < EK_MAX_HEAD_DIM / 32; ++r) {
      const int i = lane + 32 * r;
      float v = 0.f;
      if (i < d) v = to_f<T>(src[i]) + (bias ? bias[i] : 0.f);
      y[r] = v;
      ssv += v * v;
    }
    const float rv = rsqrtf(warp_sum(ssv) / (float)(ex.v_norm_dim > 0 ? ex.v_norm_dim : d) + ex.v_eps);
#pragma unroll
    for (int r = 0; r < EK_MAX_HEAD_DIM / 32; ++r) {
      const int i = lane + 32 * r;
      if (i < d) dst[i] = from_f<T>(y[r] * rv);
    }
    return;
  }
  if (!is_q && !is_k) {                       // values: a copy (plus the bias)
    if (vec) {
      for (int i = lane * 4; i < d; i += 128) {
        float4 v = Vec4<T>::load(src + i);
        if (bias) { v.x += bias[i]; v.y += bias[i + 1]; v.z += bias[i + 2]; v.w += bias[i + 3]; }
        Vec4<T>::store(dst + i, v);
      }
    } else {
      for (int i = lane; i < d; i += 32) dst[i] = bias ? from_f<T>(to_f<T>(src[i]) + bias[i]) : src[i];
    }
    return;
  }

  const float* gain = is_q ? q_gain : k_gain;
  float ss = 0.f;
  if (vec) {
    for (int i = lane * 4; i < d; i += 128) {
      float4 v = Vec4<T>::load(src + i);
      if (bias) { v.x += bias[i]; v.y += bias[i + 1]; v.z += bias[i + 2]; v.w += bias[i + 3]; }
      if (dst_raw) Vec4<T>::store(dst_raw + i, v);
      *reinterpret_cast<float4*>(&buf[warp][i]) = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = lane; i < d; i += 32) {
      float v = to_f<T>(src[i]);
      if (bias) v += bias[i];
      if (dst_raw) dst_raw[i] = from_f<T>(v);
      buf[warp][i] = v;
      ss += v * v;
    }
  }
  float rstd = 1.f;
  if (gain) {
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / (float)(ex.norm_dim > 0 ? ex.norm_dim : d) + eps);
  }
  if (is_q && ex.q_temp_coef != 0.f)          // the rotation is linear: the factor may come first
    rstd *= 1.f + ex.q_temp_coef * logf((float)((pos + 1) / ex.q_temp_every) + 1.f);
  __syncwarp();
  const int half = rot_dim >> 1;
  const float* cs = cos_tab + (size_t)pos * half;
  const float* sn = sin_tab + (size_t)pos * half;
  auto rotated = [&](int i) {
    const float g = gain ? gain[i] : 1.f;
    const float x = buf[warp][i] * rstd * g;
    if (i < half) {
      const float partner = buf[warp][i + half] * rstd * (gain ? gain[i + half] : 1.f);
      return x * cs[i] - partner * sn[i];
    }
    if (i < rot_dim) {
      const int j = i - half;
      const float partner = buf[warp][j] * rstd * (gain ? gain[j] : 1.f);
      return x * cs[j] + partner * sn[j];
    }
    return x;
  };
  if (vec) {
    for (int i = lane * 4; i < d; i += 128)
      Vec4<T>::store(dst + i, make_float4(rotated(i), rotated(i + 1), rotated(i + 2), rotated(i + 3)));
  } else {
    for (int i = lane; i < d; i += 32) dst[i] = from_f<T>(rotated(i));
  }
}


// Rotation first, then the head divided by its root mean square - for designs that turn queries and
// keys before they normalise them, without a gain.  A warp a head.  The row of a token holds its query
// heads from column 0, its key heads from `k_col` and its value heads from `v_col` (each `d` = the
// cache's head size apart; key and value heads only when `write_kv`).  A head may be padded with zeros
// beyond the values it really has: `norm_dim` is the count the mean is taken over.  `unit` 0: no norm.
template <typename T>
__global__ void qk_rope_unit_kv_kernel(T* rows, int row_stride, int k_col, int v_col,
                                       const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                       int rot_dim, const int* positions, const int* token_slot,
                                       PagedKV cache, int n_q_heads, int norm_dim, float eps, int unit,
                                       int write_kv) {
  __shared__ float buf[kRopeWarps][EK_MAX_HEAD_DIM];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * kRopeWarps + warp;
  const int n_kv = cache.heads, d = cache.head_dim;
  if (head >= n_q_heads + (write_kv ? 2 * n_kv : 0)) return;
  const int pos = positions[t];
  if (pos < 0) return;
  const bool is_q = head < n_q_heads;
  const bool is_k = !is_q && head < n_q_heads + n_kv;
  const int kv_head = is_q ? 0 : (is_k ? head - n_q_heads : head - n_q_heads - n_kv);
  T* src = rows + (size_t)t * row_stride + (is_q ? (size_t)head * d : (size_t)(is_k ? k_col : v_col) + (size_t)kv_head * d);
  T* dst = src;
  if (!is_q) {
    const int page = cache.block_table[(size_t)token_slot[t] * cache.table_stride + pos / EK_PAGE];
    dst = (T*)(is_k ? cache.k : cache.v) + page_offset(cache, page, kv_head, pos);
  }
  if (!is_q && !is_k) {                         // values: a copy
    for (int i = lane; i < d; i += 32) dst[i] = src[i];
    return;
  }
  for (int i = lane; i < d; i += 32) buf[warp][i] = to_f<T>(src[i]);
  __syncwarp();
  const int half = rot_dim >> 1;
  const float* cs = cos_tab + (size_t)pos * half;
  const float* sn = sin_tab + (size_t)pos * half;
  float y[EK_MAX_HEAD_DIM / 32];
  float ss = 0.f;
#pragma unroll
  for (int r = 0; r < EK_MAX_HEAD_DIM / 32; ++r) {
    const int i = lane + 32 * r;
    float v = 0.f;
    if (i < d) {
      v = buf[warp][i];
      if (i < half) v = v * cs[i] - buf[warp][i + half] * sn[i];
      else if (i < rot_dim) v = v * cs[i - half] + buf[warp][i - half] * sn[i - half];
    }
    y[r] = v;
    ss += v * v;
  }
  float rstd = 1.f;
  if (unit) rstd = rsqrtf(warp_sum(ss) / (float)norm_dim + eps);
#pragma unroll
  for (int r = 0; r < EK_MAX_HEAD_DIM / 32; ++r) {
    const int i = lane + 32 * r;
    if (i < d) dst[i] = from_f<T>(y[r] * rstd);
  }
}

// Wide form for 16-bit rows whose head size is 64, 128 or 256 and fully rotated: a block takes
// every head of one token, D/8 lanes a head.  A lane holds 4 neighbouring dimensions of the head's
// first half and the 4 they turn with in the second half (two 8-byte loads, each a full 128-byte
// line over the head's lanes), so the rotation needs no exchange between lanes; only the sum of
// squares of the head norm goes through shuffles.  The kernel is bound by instruction issue, not by
// memory (with the arithmetic taken out it runs at the copy bandwidth), so the gain and the angle
// are multiplied once per token and lane - four products per pair of dimensions, for q and for k -
// and a head costs a lane two multiply-adds and one multiply per value:
//     y_lo = rstd * (x_lo * (g_lo cos) - x_hi * (g_hi sin)),   y_hi = rstd * (x_hi * (g_hi cos) + x_lo * (g_lo sin))
// which is gain * x * rstd rotated, with the 32-bit products taken in another order.  All loads of
// a token are issued before the first use.
constexpr int kWideThreads = 256;
constexpr int kWidePasses = 4;

template <int D>
__global__ void __launch_bounds__(kWideThreads, 4)
qk_norm_rope_kv_wide_kernel(bf16* qkv, int row_stride, const float* __restrict__ q_gain,
                            const float* __restrict__ k_gain, const float* __restrict__ cos_tab,
                            const float* __restrict__ sin_tab, const int* positions,
                            const int* token_slot, PagedKV cache, int n_q_heads, float eps,
                            int write_kv) {
  constexpr int LPH = D / 8;                       // lanes a head
  constexpr int HPP = kWideThreads / LPH;          // heads a pass
  constexpr int half = D / 2;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int n_kv = cache.heads;
  const int n_heads = write_kv ? n_q_heads + 2 * n_kv : n_q_heads;
  const int lih = threadIdx.x % LPH;               // lane in head
  const int head0 = threadIdx.x / LPH;
  const int d0 = 4 * lih;                          // this lane's dimensions: d0.. and half + d0..
  bf16* row = qkv + (size_t)t * row_stride;
  // the first heads are asked for before the position is known: one round trip less in the chain
  uint2 raw_lo[kWidePasses], raw_hi[kWidePasses];
  auto load_heads = [&](int base) {
#pragma unroll
    for (int p = 0; p < kWidePasses; ++p) {
      const int head = base + p * HPP + head0;
      if (head < n_heads) {
        raw_lo[p] = *reinterpret_cast<const uint2*>(row + (size_t)head * D + d0);
        raw_hi[p] = *reinterpret_cast<const uint2*>(row + (size_t)head * D + half + d0);
      }
    }
  };
  load_heads(0);
  const int pos = positions[t];
  if (pos < 0) return;
  // the lanes of this head within the warp: heads of one warp may take different branches
  const unsigned seg = LPH == 32 ? 0xffffffffu
                                 : ((1u << (LPH & 31)) - 1u) << ((threadIdx.x & 31) / LPH * LPH);
  size_t page_base = 0;
  if (write_kv) {
    const int page = cache.block_table[(size_t)token_slot[t] * cache.table_stride + pos / EK_PAGE];
    page_base = page_offset(cache, page, 0, pos);
  }
  // gain x angle, once per token and lane, for the query heads (most of a token's heads); a key
  // head takes its own four products when it comes
  float cs[4], sn[4];
  {
    const float4 c4 = *reinterpret_cast<const float4*>(cos_tab + (size_t)pos * half + d0);
    const float4 s4 = *reinterpret_cast<const float4*>(sin_tab + (size_t)pos * half + d0);
    cs[0] = c4.x; cs[1] = c4.y; cs[2] = c4.z; cs[3] = c4.w;
    sn[0] = s4.x; sn[1] = s4.y; sn[2] = s4.z; sn[3] = s4.w;
  }
  auto products = [&](const float* gain, float* lc, float* hs, float* hc, float* ls) {
    float gl[4] = {1.f, 1.f, 1.f, 1.f}, gh[4] = {1.f, 1.f, 1.f, 1.f};
    if (gain) {
      const float4 l4 = *reinterpret_cast<const float4*>(gain + d0);
      const float4 h4 = *reinterpret_cast<const float4*>(gain + half + d0);
      gl[0] = l4.x; gl[1] = l4.y; gl[2] = l4.z; gl[3] = l4.w;
      gh[0] = h4.x; gh[1] = h4.y; gh[2] = h4.z; gh[3] = h4.w;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lc[i] = gl[i] * cs[i];
      hs[i] = gh[i] * sn[i];
      hc[i] = gh[i] * cs[i];
      ls[i] = gl[i] * sn[i];
    }
  };
  float q_lc[4], q_hs[4], q_hc[4], q_ls[4];
  products(q_gain, q_lc, q_hs, q_hc, q_ls);
  const bool q_norm = q_gain != nullptr, k_norm = k_gain != nullptr;
  for (int base = 0; base < n_heads; base += HPP * kWidePasses) {
    if (base > 0) load_heads(base);
#pragma unroll
    for (int p = 0; p < kWidePasses; ++p) {
      const int head = base + p * HPP + head0;
      // shuffles below are among the D/8 lanes of a head, which are all in or all out
      if (head >= n_heads) continue;
      const bool is_q = head < n_q_heads;
      const bool is_k = !is_q && head < n_q_heads + n_kv;
      bf16* dst = row + (size_t)head * D + d0;
      if (!is_q) {
        const int kv_head = is_k ? head - n_q_heads : head - n_q_heads - n_kv;
        dst = (bf16*)(is_k ? cache.k : cache.v) + page_base + (size_t)kv_head * EK_PAGE * D + d0;
      }
      if (!is_q && !is_k) {
        *reinterpret_cast<uint2*>(dst) = raw_lo[p];
        *reinterpret_cast<uint2*>(dst + half) = raw_hi[p];
        continue;
      }
      float lo[4], hi[4];
      {
        const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&raw_lo[p]);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw_hi[p]);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float2 f = __bfloat1622float2(l2[i]), g = __bfloat1622float2(h2[i]);
          lo[2 * i] = f.x; lo[2 * i + 1] = f.y;
          hi[2 * i] = g.x; hi[2 * i + 1] = g.y;
        }
      }
      float rstd = 1.f;
      if (is_q ? q_norm : k_norm) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) ss += lo[i] * lo[i] + hi[i] * hi[i];
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(seg, ss, o, LPH);
        rstd = rsqrtf(ss / (float)D + eps);
      }
      float ylo[4], yhi[4];
      if (is_q) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ylo[i] = (lo[i] * q_lc[i] - hi[i] * q_hs[i]) * rstd;
          yhi[i] = (hi[i] * q_hc[i] + lo[i] * q_ls[i]) * rstd;
        }
      } else {
        float k_lc[4], k_hs[4], k_hc[4], k_ls[4];
        products(k_gain, k_lc, k_hs, k_hc, k_ls);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ylo[i] = (lo[i] * k_lc[i] - hi[i] * k_hs[i]) * rstd;
          yhi[i] = (hi[i] * k_hc[i] + lo[i] * k_ls[i]) * rstd;
        }
      }
      __nv_bfloat162 l0 = __floats2bfloat162_rn(ylo[0], ylo[1]), l1 = __floats2bfloat162_rn(ylo[2], ylo[3]);
      __nv_bfloat162 h0 = __floats2bfloat162_rn(yhi[0], yhi[1]), h1 = __floats2bfloat162_rn(yhi[2], yhi[3]);
      *reinterpret_cast<uint2*>(dst) =
          make_uint2(*reinterpret_cast<uint32_t*>(&l0), *reinterpret_cast<uint32_t*>(&l1));
      *reinterpret_cast<uint2*>(dst + half) =
          make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
    }
  }
}

// Wide form without rotation, with the options of QkExtras, for 16-bit rows of many tokens: a block
// takes every head of one token, D/8 lanes a head, a lane 8 neighbouring dimensions (one 16-byte
// load and store).  Bias, sum of squares, 1/rms times the query's temperature, gain - all in
// 32-bit, one rounding at the end; a key head is stored twice when the values are the keys as
// projected.  All loads of a pass are issued before the first use.
template <int D>
__global__ void __launch_bounds__(kWideThreads, 4)
qk_prepare_kv_wide_kernel(bf16* qkv, int row_stride, const float* __restrict__ q_gain,
                          const float* __restrict__ k_gain, const int* positions, const int* token_slot,
                          PagedKV cache, int n_q_heads, float eps, int write_kv, QkExtras ex) {
  constexpr int LPH = D / 8;                       // lanes a head
  constexpr int HPP = kWideThreads / LPH;          // heads a pass
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int n_kv = cache.heads;
  const int n_heads = write_kv ? n_q_heads + (ex.v_from_k ? 1 : 2) * n_kv : n_q_heads;
  const int lih = threadIdx.x % LPH, head0 = threadIdx.x / LPH;
  const int d0 = 8 * lih;
  bf16* row = qkv + (size_t)t * row_stride;
  uint4 raw[kWidePasses];
  auto load_heads = [&](int base) {
#pragma unroll
    for (int p = 0; p < kWidePasses; ++p) {
      const int head = base + p * HPP + head0;
      if (head < n_heads) raw[p] = *reinterpret_cast<const uint4*>(row + (size_t)head * D + d0);
    }
  };
  load_heads(0);
  const int pos = positions[t];
  if (pos < 0) return;
  const unsigned seg = LPH == 32 ? 0xffffffffu
                                 : ((1u << (LPH & 31)) - 1u) << ((threadIdx.x & 31) / LPH * LPH);
  size_t page_base = 0;
  if (write_kv) {
    const int page = cache.block_table[(size_t)token_slot[t] * cache.table_stride + pos / EK_PAGE];
    page_base = page_offset(cache, page, 0, pos);
  }
  const float temp = ex.q_temp_coef != 0.f
                         ? 1.f + ex.q_temp_coef * logf((float)((pos + 1) / ex.q_temp_every) + 1.f) : 1.f;
  auto eight = [&](const float* p, float* v, float fill) {
    if (p) {
      const float4 a = *reinterpret_cast<const float4*>(p + d0), b = *reinterpret_cast<const float4*>(p + d0 + 4);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = fill;
    }
  };
  float qg[8], kg[8];
  eight(q_gain, qg, 1.f);
  eight(k_gain, kg, 1.f);
  auto pack = [](const float* y) {
    uint4 o;
    __nv_bfloat162 a = __floats2bfloat162_rn(y[0], y[1]), b = __floats2bfloat162_rn(y[2], y[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(y[4], y[5]), d = __floats2bfloat162_rn(y[6], y[7]);
    o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
    o.z = *reinterpret_cast<uint32_t*>(&c); o.w = *reinterpret_cast<uint32_t*>(&d);
    return o;
  };
  for (int base = 0; base < n_heads; base += HPP * kWidePasses) {
    if (base > 0) load_heads(base);
#pragma unroll
    for (int p = 0; p < kWidePasses; ++p) {
      const int head = base + p * HPP + head0;
      if (head >= n_heads) continue;               // (the D/8 lanes of a head are all in or all out)
      const bool is_q = head < n_q_heads;
      const bool is_k = !is_q && head < n_q_heads + n_kv;
      const int local = is_q ? head : (is_k ? head - n_q_heads : head - n_q_heads - n_kv);
      float x[8], b[8];
      {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[p]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h2[i]);
          x[2 * i] = f.x; x[2 * i + 1] = f.y;
        }
      }
      const float* bias = is_q ? ex.q_bias : (is_k ? ex.k_bias : ex.v_bias);
      eight(bias ? bias + (size_t)local * D : nullptr, b, 0.f);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] += b[i];
      if (!is_q && !is_k) {                        // a value head: as projected
        *reinterpret_cast<uint4*>((bf16*)cache.v + page_base + (size_t)local * EK_PAGE * D + d0) = pack(x);
        continue;
      }
      if (is_k && ex.v_from_k)
        *reinterpret_cast<uint4*>((bf16*)cache.v + page_base + (size_t)local * EK_PAGE * D + d0) = pack(x);
      float factor = is_q ? temp : 1.f;
      if (is_q ? q_gain != nullptr : k_gain != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(seg, ss, o, LPH);
        factor *= rsqrtf(ss / (float)D + eps);
      }
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = x[i] * factor * (is_q ? qg[i] : kg[i]);
      bf16* dst = is_q ? row + (size_t)head * D + d0
                       : (bf16*)cache.k + page_base + (size_t)local * EK_PAGE * D + d0;
      *reinterpret_cast<uint4*>(dst) = pack(y);
    }
  }
}

template <int D>
static int launch_prepare_wide(bf16* qkv, int row_stride, const float* q_gain, const float* k_gain,
                               const int* positions, const int* token_slot, PagedKV cache, int n_tokens,
                               int n_q_heads, float eps, int write_kv, QkExtras ex, cudaStream_t stream) {
  return (int)launch_pdl(qk_prepare_kv_wide_kernel<D>, dim3(n_tokens), dim3(kWideThreads), 0, stream, qkv,
                         row_stride, q_gain, k_gain, positions, token_slot, cache, n_q_heads, eps, write_kv, ex);
}

template <int D>
static int launch_wide(bf16* qkv, int row_stride, const float* q_gain, const float* k_gain,
                       const float* cos_tab, const float* sin_tab, const int* positions,
                       const int* token_slot, PagedKV cache, int n_tokens, int n_q_heads, float eps,
                       int write_kv, cudaStream_t stream) {
  return (int)launch_pdl(qk_norm_rope_kv_wide_kernel<D>, dim3(n_tokens), dim3(kWideThreads), 0, stream,
                         qkv, row_stride, q_gain, k_gain, cos_tab, sin_tab, positions, token_slot, cache,
                         n_q_heads, eps, write_kv);
}

// The wide form needs 16-byte rows and tables; one token a block pays once there are enough
// tokens to fill the machine.
template <typename T>
static bool wide_takes(const void*, int, const float*, const float*, const float*, const float*, int,
                       const void*, const void*, int, int) {
  return false;
}
template <>
bool wide_takes<bf16>(const void* qkv, int row_stride, const float* q_gain, const float* k_gain,
                      const float* cos_tab, const float* sin_tab, int rot_dim, const void* k_pages,
                      const void* v_pages, int n_tokens, int head_dim) {
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  return (head_dim == 64 || head_dim == 128 || head_dim == 256) && rot_dim == head_dim &&
         n_tokens >= 128 && row_stride % 8 == 0 && aligned(qkv) && aligned(q_gain) && aligned(k_gain) &&
         aligned(cos_tab) && aligned(sin_tab) && aligned(k_pages) && aligned(v_pages);
}

template <typename T>
static int launch(void* qkv, int row_stride, const float* q_gain, const float* k_gain,
                  const float* cos_tab, const float* sin_tab, int rot_dim, const int* positions,
                  const int* token_slot, void* k_pages, void* v_pages, const int* block_table,
                  int table_stride, int n_tokens, int n_q_heads, int n_kv_heads, int head_dim,
                  float eps, int write_kv, QkExtras ex, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (head_dim <= 0 || head_dim > EK_MAX_HEAD_DIM || rot_dim < 0 || rot_dim > head_dim ||
      (rot_dim & 1) || n_tokens > 2147483647 / 2 || (ex.q_temp_coef != 0.f && ex.q_temp_every <= 0))
    return EK_ERR_ARG;
  PagedKV cache{k_pages, v_pages, block_table, table_stride, n_kv_heads, head_dim};
  const bool padded = ex.norm_dim > 0 || ex.v_unit;      // only the warp-a-head kernel knows these
  const bool plain = !ex.q_bias && !ex.k_bias && !ex.v_bias && ex.q_temp_coef == 0.f && !ex.v_from_k && !padded;
  if (!plain && !padded && rot_dim == 0 && sizeof(T) == 2 && (head_dim == 64 || head_dim == 128 || head_dim == 256) &&
      n_tokens >= 128 && row_stride % 8 == 0) {
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if (aligned(qkv) && aligned(q_gain) && aligned(k_gain) && aligned(k_pages) && aligned(v_pages) &&
        aligned(ex.q_bias) && aligned(ex.k_bias) && aligned(ex.v_bias)) {
      bf16* rows = (bf16*)qkv;
      if (head_dim == 64)
        return launch_prepare_wide<64>(rows, row_stride, q_gain, k_gain, positions, token_slot, cache,
                                       n_tokens, n_q_heads, eps, write_kv, ex, stream);
      if (head_dim == 128)
        return launch_prepare_wide<128>(rows, row_stride, q_gain, k_gain, positions, token_slot, cache,
                                        n_tokens, n_q_heads, eps, write_kv, ex, stream);
      return launch_prepare_wide<256>(rows, row_stride, q_gain, k_gain, positions, token_slot, cache,
                                      n_tokens, n_q_heads, eps, write_kv, ex, stream);
    }
  }
  if (plain && wide_takes<T>(qkv, row_stride, q_gain, k_gain, cos_tab, sin_tab, rot_dim, k_pages, v_pages,
                    n_tokens, head_dim)) {
    bf16* rows = (bf16*)qkv;
    if (head_dim == 64)
      return launch_wide<64>(rows, row_stride, q_gain, k_gain, cos_tab, sin_tab, positions, token_slot,
                             cache, n_tokens, n_q_heads, eps, write_kv, stream);
    if (head_dim == 128)
      return launch_wide<128>(rows, row_stride, q_gain, k_gain, cos_tab, sin_tab, positions, token_slot,
                              cache, n_tokens, n_q_heads, eps, write_kv, stream);
    return launch_wide<256>(rows, row_stride, q_gain, k_gain, cos_tab, sin_tab, positions, token_slot,
                            cache, n_tokens, n_q_heads, eps, write_kv, stream);
  }
  const int heads = n_q_heads + (ex.v_from_k ? 1 : 2) * n_kv_heads;
  dim3 grid(n_tokens, (heads + kRopeWarps - 1) / kRopeWarps);
  return (int)launch_pdl(qk_norm_rope_kv_kernel<T>, grid, dim3(kRopeWarps * 32), 0, stream, (T*)qkv,
                         row_stride, q_gain, k_gain, cos_tab, sin_tab, rot_dim, positions,
                         token_slot, cache, n_q_heads, eps, write_kv, ex);
}

}  // namespace ek

#define EK_INSTANTIATE(SUFFIX, T)                                                              \
  EK_EXPORT int ek_qk_norm_rope_kv_##SUFFIX(                                                    \
      void* qkv, int row_stride, const float* q_gain, const float* k_gain, const float* cos_tab, \
      const float* sin_tab, int rot_dim, const int* positions, const int* token_slot,          \
      void* k_pages, void* v_pages, const int* block_table, int table_stride, int n_tokens,    \
      int n_q_heads, int n_kv_heads, int head_dim, float eps, int write_kv,                    \
      cudaStream_t stream) {                                                                   \
    return ek::launch<T>(qkv, row_stride, q_gain, k_gain, cos_tab, sin_tab, rot_dim, positions, \
                         token_slot, k_pages, v_pages, block_table, table_stride, n_tokens,    \
                         n_q_heads, n_kv_heads, head_dim, eps, write_kv, ek::QkExtras{},       \
                         stream);                                                              \
  }                                                                                            \
  /* The same with the options of ek::QkExtras: biases (32-bit, nullable), the query         */ \
  /* temperature (coef 0: none) and values taken from the keys as projected (the rows then   */ \
  /* hold (NQ + NKV) heads).                                                                  */ \
  EK_EXPORT int ek_qk_prepare_kv_##SUFFIX(                                                      \
      void* qkv, int row_stride, const float* q_gain, const float* k_gain, const float* cos_tab, \
      const float* sin_tab, int rot_dim, const int* positions, const int* token_slot,          \
      void* k_pages, void* v_pages, const int* block_table, int table_stride, int n_tokens,    \
      int n_q_heads, int n_kv_heads, int head_dim, float eps, int write_kv,                    \
      const float* q_bias, const float* k_bias, const float* v_bias, float q_temp_coef,        \
      int q_temp_every, int v_from_k, cudaStream_t stream) {                                   \
    ek::QkExtras ex{q_bias, k_bias, v_bias, q_temp_coef, q_temp_every, v_from_k, 0, 0, 0, 0.f}; \
    return ek::launch<T>(qkv, row_stride, q_gain, k_gain, cos_tab, sin_tab, rot_dim, positions, \
                         token_slot, k_pages, v_pages, block_table, table_stride, n_tokens,    \
                         n_q_heads, n_kv_heads, head_dim, eps, write_kv, ex, stream);          \
  }                                                                                            \
  /* The same for heads padded with zeros to the cache's head size: the gained query / key    */ \
  /* norm takes its mean over norm_dim values, and with v_unit a value head is divided by its */ \
  /* root mean square over v_norm_dim values before it is stored.                             */ \
  EK_EXPORT int ek_qk_prepare_padded_kv_##SUFFIX(                                               \
      void* qkv, int row_stride, const float* q_gain, const float* k_gain, const float* cos_tab, \
      const float* sin_tab, int rot_dim, const int* positions, const int* token_slot,          \
      void* k_pages, void* v_pages, const int* block_table, int table_stride, int n_tokens,    \
      int n_q_heads, int n_kv_heads, int head_dim, float eps, int write_kv,                    \
      const float* q_bias, const float* k_bias, const float* v_bias, int norm_dim, int v_unit, \
      int v_norm_dim, float v_eps, cudaStream_t stream) {                                      \
    if (norm_dim <= 0 || norm_dim > head_dim || (v_unit && (v_norm_dim <= 0 || v_norm_dim > head_dim))) \
      return EK_ERR_ARG;                                                                       \
    ek::QkExtras ex{q_bias, k_bias, v_bias, 0.f, 1, 0, norm_dim, v_unit, v_norm_dim, v_eps};   \
    return ek::launch<T>(qkv, row_stride, q_gain, k_gain, cos_tab, sin_tab, rot_dim, positions, \
                         token_slot, k_pages, v_pages, block_table, table_stride, n_tokens,    \
                         n_q_heads, n_kv_heads, head_dim, eps, write_kv, ex, stream);          \
  }                                                                                            \
  /* Rotation, then every query and key head over its root mean square (no gain); the row    */ \
  /* holds query heads from column 0, key heads from k_col, value heads from v_col.          */ \
  EK_EXPORT int ek_qk_rope_unit_kv_##SUFFIX(                                                    \
      void* rows, int row_stride, int k_col, int v_col, const float* cos_tab,                  \
      const float* sin_tab, int rot_dim, const int* positions, const int* token_slot,          \
      void* k_pages, void* v_pages, const int* block_table, int table_stride, int n_tokens,    \
      int n_q_heads, int n_kv_heads, int head_dim, int norm_dim, float eps, int unit,          \
      int write_kv, cudaStream_t stream) {                                                     \
    using namespace ek;                                                                        \
    if (n_tokens <= 0) return 0;                                                               \
    if (head_dim <= 0 || head_dim > EK_MAX_HEAD_DIM || rot_dim < 0 || rot_dim % 2 ||           \
        rot_dim > head_dim || norm_dim <= 0 || norm_dim > head_dim || n_q_heads <= 0 ||        \
        n_kv_heads <= 0)                                                                       \
      return EK_ERR_ARG;                                                                       \
    PagedKV cache{k_pages, v_pages, block_table, table_stride, n_kv_heads, head_dim};          \
    const int heads = n_q_heads + (write_kv ? 2 * n_kv_heads : 0);                             \
    dim3 grid(n_tokens, (heads + kRopeWarps - 1) / kRopeWarps);                                \
    return (int)launch_pdl(qk_rope_unit_kv_kernel<T>, grid, dim3(kRopeWarps * 32), 0, stream,  \
                           (T*)rows, row_stride, k_col, v_col, cos_tab, sin_tab, rot_dim,      \
                           positions, token_slot, cache, n_q_heads, norm_dim, eps, unit,       \
                           write_kv);                                                          \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)
