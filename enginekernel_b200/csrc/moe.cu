// Routed experts: a router that picks `top` of E small feed-forwards per token, and the experts'
// products for the tokens that chose them.
//
//   route     scores = softmax(logits) over all experts (32-bit); experts form `n_groups` equal
//             groups of neighbours, a group's score is its best expert's, only experts of the
//             `keep` best groups can be chosen; the `top` largest of those; weights = chosen
//             scores / (their sum + 1e-20) * scale.  A warp a token.  `among_chosen`: the weights are
//             the softmax over the chosen logits alone (times scale), taken from the logits with the
//             chosen maximum off, so that no score can vanish against an unchosen expert's.
//   plan      the (token, choice) pairs sorted by expert, and the row tiles of every expert's
//             stretch, made on the device: the host never sees who chose what.
//   expert product  out[row] = f(x[row] . W_e^T) over the tiles of the plan: FFMA with 32-bit
//             sums in ascending k (the 32-bit path, and 16-bit rows that cannot be read 16 bytes
//             at a time), or mma.sync on bfloat16 tiles with 32-bit accumulators; either way a
//             pair's result does not depend on its neighbours.  The up form gathers its rows by
//             token and applies the activation, the down form scales by the pair's weight and
//             scatters 32-bit rows by pair.  `gated` up form: the expert's weight rows alternate
//             gate, up, gate, up ...; column pair (2c, 2c + 1) of the product gives out[c] =
//             act(gate) * up from the 32-bit sums (N counts the weight rows, the output has N / 2).
//   combine   out[t] = sum over the token's choices, in the order they were chosen.
#include "common.cuh"

namespace ek {

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

constexpr int kRouteWarps = 4;

// logits [T, E] 32-bit -> sel_expert [T, top] int32, sel_weight [T, top] 32-bit.
__global__ void __launch_bounds__(kRouteWarps * 32)
moe_route_kernel(int* __restrict__ sel_expert, float* __restrict__ sel_weight,
                 const float* __restrict__ logits, int n_tokens, int E, int n_groups, int keep, int top,
                 float scale, int among_chosen) {
  extern __shared__ float route_s[];            // per warp: scores [E], candidates [E], groups [n_groups]
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  if (t >= n_tokens) return;
  float* s = route_s + (size_t)warp * (2 * E + n_groups);
  float* cand = s + E;
  float* gs = cand + E;
  const float* z = logits + (size_t)t * E;
  float m = -INFINITY;
  for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
  m = warp_max(m);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) { const float x = expf(z[e] - m); s[e] = x; sum += x; }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  // candidates: the scores; with weights among the chosen the logits themselves, so that the order of
  // two experts whose scores both round to nothing is still the order of their logits
  const float shut = among_chosen ? -INFINITY : -2.f;
  for (int e = lane; e < E; e += 32) { s[e] *= inv; cand[e] = among_chosen ? z[e] : s[e]; }
  __syncwarp();
  if (n_groups > 1 && keep < n_groups) {
    const int per = E / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float best = -1.f;
      for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, s[e]);
      gs[g] = best;
    }
    __syncwarp();
    for (int round = 0; round < keep; ++round) {
      float bv = -2.f; int bi = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32)
        if (gs[g] > bv) { bv = gs[g]; bi = g; }
      warp_argmax(bv, bi);
      if (lane == 0) gs[bi] = -3.f;             // kept
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gs[e / per] != -3.f) cand[e] = among_chosen ? -INFINITY : -1.f;
    __syncwarp();
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float bv = shut; int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (cand[e] > bv) { bv = cand[e]; bi = e; }
    warp_argmax(bv, bi);
    if (bi >= E) bi = 0;                        // (no finite candidate left: logits that are not numbers)
    const float sc = s[bi];
    total += sc;
    if (lane == 0) {
      sel_expert[(size_t)t * top + k] = bi;
      sel_weight[(size_t)t * top + k] = sc;     // scaled below
      cand[bi] = shut;
    }
    __syncwarp();
  }
  if (among_chosen) {                           // softmax over the chosen logits: the first chosen is the largest
    __syncwarp();
    const float z0 = z[sel_expert[(size_t)t * top]];
    float den = 0.f;
    for (int k = 0; k < top; ++k) den += expf(z[sel_expert[(size_t)t * top + k]] - z0);
    for (int k = lane; k < top; k += 32)
      sel_weight[(size_t)t * top + k] = expf(z[sel_expert[(size_t)t * top + k]] - z0) / den * scale;
    return;
  }
  const float f = scale / (total + 1e-20f);
  for (int k = lane; k < top; k += 32) sel_weight[(size_t)t * top + k] *= f;
}

constexpr int kTileRows = 64;

// One block.  sel_expert [P] -> sorted_pair [P] (pairs grouped by expert), tiles [max_tiles][3] =
// (expert, first sorted row, rows), n_tiles[0].
__global__ void __launch_bounds__(1024)
moe_plan_kernel(int* __restrict__ sorted_pair, int* __restrict__ tiles, int* __restrict__ n_tiles,
                const int* __restrict__ sel_expert, int P, int E) {
  extern __shared__ int plan_s[];               // counts [E], first row [E], first tile [E + 1]
  pdl_launch_dependents();
  pdl_wait();
  int* counts = plan_s;
  int* first = counts + E;
  int* tile0 = first + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = sel_expert[p];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int row = 0, tile = 0;
    for (int e = 0; e < E; ++e) {
      first[e] = row;
      tile0[e] = tile;
      row += counts[e];
      tile += (counts[e] + kTileRows - 1) / kTileRows;
    }
    tile0[E] = tile;
    n_tiles[0] = tile;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int n = counts[e];
    for (int i = 0, tile = tile0[e]; i < n; i += kTileRows, ++tile) {
      tiles[3 * tile] = e;
      tiles[3 * tile + 1] = first[e] + i;
      tiles[3 * tile + 2] = min(kTileRows, n - i);
    }
    counts[e] = first[e];                       // from here on: the next free row of the expert
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = sel_expert[p];
    if (e >= 0 && e < E) sorted_pair[atomicAdd(&counts[e], 1)] = p;
  }
}

constexpr int ACT_RELU2 = 1, ACT_SILU = 2, ACT_GELU_TANH = 3;      // 0: none

__device__ __forceinline__ float activate(float z, int act) {
  if (act == ACT_RELU2) { const float r = fmaxf(z, 0.f); return r * r; }
  if (act == ACT_SILU) return z / (1.f + expf(-z));
  if (act == ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z;
}

// grid (max tiles, column tiles).  UP: a[row] = x[pair / top], out T [sorted row][N] = act(.).
// DOWN: a[row] = in[sorted row], out 32-bit [pair][N] = weight[pair] * (.).
template <typename T, bool UP>
__global__ void __launch_bounds__(256)
moe_expert_product_kernel(void* __restrict__ out_, const T* __restrict__ a, const T* __restrict__ w,
                          const int* __restrict__ tiles, const int* __restrict__ n_tiles,
                          const int* __restrict__ sorted_pair, const float* __restrict__ pair_weight,
                          int top, int N, int K, int act, int gated) {
  constexpr int BM = kTileRows, BN = 64, BK = 16, TM = 4, TN = 4, PAD = 4;
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Ws[BK][BN + PAD];
  __shared__ int src_row[BM];
  __shared__ int pair_s[BM];
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.x >= n_tiles[0]) return;
  const int e = tiles[3 * blockIdx.x], row0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
  const int tid = threadIdx.x;
  if (tid < BM) {
    const int p = tid < rows ? sorted_pair[row0 + tid] : -1;
    pair_s[tid] = p;
    src_row[tid] = p < 0 ? -1 : (UP ? p / top : row0 + tid);
  }
  __syncthreads();
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int n0 = blockIdx.y * BN;
  const T* we = w + (size_t)e * N * K;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int idx = tid; idx < BM * BK; idx += 256) {
      const int row = idx / BK, kk = idx % BK;
      const int src = src_row[row], gk = k0 + kk;
      As[kk][row] = (src >= 0 && gk < K) ? to_f<T>(a[(size_t)src * K + gk]) : 0.f;
    }
    for (int idx = tid; idx < BN * BK; idx += 256) {
      const int row = idx / BK, kk = idx % BK;
      const int gn = n0 + row, gk = k0 + kk;
      Ws[kk][row] = (gn < N && gk < K) ? to_f<T>(we[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[TM], bv[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) av[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) bv[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = ty * TM + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      if (UP && gated) {                          // columns (gn, gn + 1) = (gate, up); N is even
        if (!(j & 1)) ((T*)out_)[(size_t)(row0 + r) * (N / 2) + gn / 2] =
            from_f<T>(activate(acc[i][j], act) * acc[i][j + 1]);
      } else if (UP) {
        ((T*)out_)[(size_t)(row0 + r) * N + gn] = from_f<T>(activate(acc[i][j], act));
      } else {
        const int p = pair_s[r];
        ((float*)out_)[(size_t)p * N + gn] = acc[i][j] * pair_weight[p];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The same product on the tensor cores (bfloat16 operands, 32-bit accumulators): a block takes a
// 64-row tile of the plan and 128 columns, eight warps of 32 x 32 each, K in steps of 64 through a
// ring of three shared-memory stages filled by cp.async (rows padded by 16 bytes: ldmatrix without
// bank conflicts).  K % 8 == 0.
__device__ __forceinline__ void ldsm_x4(uint32_t r[4], const bf16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16_16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 16 bytes global -> shared without passing through registers; `bytes` = 0 writes zeros instead.
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, int bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr int kTcCols = 128, kTcK = 64, kTcLd = kTcK + 8, kTcStages = 3;
constexpr size_t kTcSmem = (size_t)kTcStages * (kTileRows + kTcCols) * kTcLd * sizeof(bf16);

template <bool UP>
__global__ void __launch_bounds__(256)
moe_expert_product_tc_kernel(void* __restrict__ out_, const bf16* __restrict__ a, const bf16* __restrict__ w,
                             const int* __restrict__ tiles, const int* __restrict__ n_tiles,
                             const int* __restrict__ sorted_pair, const float* __restrict__ pair_weight,
                             int top, int N, int K, int act, int gated) {
  constexpr int BM = kTileRows, BN = kTcCols, BK = kTcK, LD = kTcLd, STAGES = kTcStages;
  extern __shared__ __align__(16) unsigned char tc_smem[];
  typedef bf16 (*Tile)[LD];
  bf16* const a_base = reinterpret_cast<bf16*>(tc_smem);                  // [STAGES][BM][LD]
  bf16* const w_base = a_base + STAGES * BM * LD;                          // [STAGES][BN][LD]
  __shared__ int src_row[BM];
  __shared__ int pair_s[BM];
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.x >= n_tiles[0]) return;
  const int e = tiles[3 * blockIdx.x], row0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < BM) {
    const int p = tid < rows ? sorted_pair[row0 + tid] : -1;
    pair_s[tid] = p;
    src_row[tid] = p < 0 ? -1 : (UP ? p / top : row0 + tid);
  }
  __syncthreads();
  const int n0 = blockIdx.y * BN;
  const bf16* we = w + (size_t)e * N * K;
  const int wm = warp >> 2, wn = warp & 3;      // the warp's 32 x 32 piece: rows wm * 32, columns wn * 32
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

  // a K step is (64 + 128) rows of 8 pieces of 16 bytes: six pieces a thread
  auto load = [&](int stage, int kt) {
    const int k0 = kt * BK;
#pragma unroll
    for (int it = 0; it < (BM + BN) * (BK / 8) / 256; ++it) {
      const int idx = tid + it * 256, row = idx / (BK / 8), piece = idx % (BK / 8);
      const int gk = k0 + piece * 8;
      if (row < BM) {
        const int src = src_row[row];
        const bool ok = src >= 0 && gk < K;
        cp_async_16(a_base + ((size_t)stage * BM + row) * LD + piece * 8, ok ? a + (size_t)src * K + gk : a, ok ? 16 : 0);
      } else {
        const int gn = n0 + row - BM;
        const bool ok = gn < N && gk < K;
        cp_async_16(w_base + ((size_t)stage * BN + row - BM) * LD + piece * 8, ok ? we + (size_t)gn * K + gk : w, ok ? 16 : 0);
      }
    }
  };
  const int KT = (K + BK - 1) / BK;
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < KT) load(st, st);
    cp_async_commit();
  }
  for (int kt = 0; kt < KT; ++kt) {
    cp_async_wait_group<STAGES - 2>();           // this step's tiles have landed
    __syncthreads();                             // ... for everyone, and the stage refilled below is free
    if (kt + STAGES - 1 < KT) load((kt + STAGES - 1) % STAGES, kt + STAGES - 1);
    cp_async_commit();
    const int st = kt % STAGES;
    Tile As = reinterpret_cast<Tile>(a_base + (size_t)st * BM * LD);
    Tile Ws = reinterpret_cast<Tile>(w_base + (size_t)st * BN * LD);
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t af[2][4], bfr[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)                // rows (lane % 16), k half (lane / 16)
        ldsm_x4(af[i], &As[wm * 32 + i * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int j = 0; j < 2; ++j)                // two n8 tiles a load: n = (lane / 16) * 8 + lane % 8, k half (lane / 8) % 2
        ldsm_x4(bfr[j], &Ws[wn * 32 + j * 16 + (lane >> 4) * 8 + (lane & 7)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          mma_bf16_16816(acc[i][j], af[i], bfr[j >> 1][(j & 1) * 2], bfr[j >> 1][(j & 1) * 2 + 1]);
    }
  }
  cp_async_wait_group<0>();
  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 32 + i * 16 + g + half * 8;
      if (r >= rows) continue;
      const int p = pair_s[r];
      const float pw = UP ? 1.f : pair_weight[p];
      if (UP && gated) {                          // a lane's two neighbouring columns are (gate, up)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int gn = n0 + wn * 32 + j * 8 + tq * 2;
          if (gn + 1 < N)
            ((bf16*)out_)[(size_t)(row0 + r) * (N / 2) + gn / 2] =
                __float2bfloat16_rn(activate(acc[i][j][half * 2], act) * acc[i][j][half * 2 + 1]);
        }
        continue;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int gn = n0 + wn * 32 + j * 8 + tq * 2 + c;
          if (gn >= N) continue;
          const float v = acc[i][j][half * 2 + c];
          if (UP) ((bf16*)out_)[(size_t)(row0 + r) * N + gn] = __float2bfloat16_rn(activate(v, act));
          else ((float*)out_)[(size_t)p * N + gn] = v * pw;
        }
    }
}

// out[t, :] = sum_k pair_out[t * top + k, :], k ascending.
template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const float* __restrict__ pair_out, int top,
                                   int width) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; ++k) a += pair_out[(t * top + k) * width + i];
    out[t * width + i] = from_f<T>(a);
  }
}

}  // namespace ek

EK_EXPORT int ek_moe_tile_rows() { return ek::kTileRows; }

EK_EXPORT int ek_moe_route(int* sel_expert, float* sel_weight, const float* logits, int n_tokens, int E,
                           int n_groups, int keep, int top, float scale, int among_chosen,
                           cudaStream_t stream) {
  using namespace ek;
  if (n_tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || n_groups < 1 || E % n_groups || keep < 1 || keep > n_groups ||
      top > keep * (E / n_groups))
    return EK_ERR_ARG;
  const size_t smem = (size_t)kRouteWarps * (2 * E + n_groups) * sizeof(float);
  if (smem > 200 * 1024) return EK_ERR_ARG;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  moe_route_kernel<<<(n_tokens + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, smem, stream>>>(
      sel_expert, sel_weight, logits, n_tokens, E, n_groups, keep, top, scale, among_chosen);
  EK_RETURN_LAUNCH_STATUS();
}

EK_EXPORT int ek_moe_plan(int* sorted_pair, int* tiles, int* n_tiles, const int* sel_expert, int P, int E,
                          cudaStream_t stream) {
  if (P <= 0) return 0;
  if (E <= 0 || E > 8192) return EK_ERR_ARG;
  ek::moe_plan_kernel<<<1, 1024, (size_t)(3 * E + 1) * sizeof(int), stream>>>(sorted_pair, tiles, n_tiles,
                                                                             sel_expert, P, E);
  EK_RETURN_LAUNCH_STATUS();
}

// The tensor-core forms: bfloat16, K a multiple of 8, operands on 16-byte boundaries.
EK_EXPORT int ek_moe_expert_up_tc(void* out, const void* x, const void* w, const int* tiles, const int* n_tiles,
                                  const int* sorted_pair, int max_tiles, int top, int N, int K, int act,
                                  int gated, cudaStream_t stream) {
  using namespace ek;
  if (max_tiles <= 0) return 0;
  if (gated && N % 2) return EK_ERR_ARG;
  if (N <= 0 || K <= 0 || K % 8 || top <= 0 || (N + 127) / 128 > 65535 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
    return EK_ERR_ARG;
  dim3 grid(max_tiles, (N + 127) / 128);
  cudaError_t e = cudaFuncSetAttribute(moe_expert_product_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)kTcSmem);
  if (e != cudaSuccess) return (int)e;
  moe_expert_product_tc_kernel<true><<<grid, 256, kTcSmem, stream>>>(out, (const bf16*)x, (const bf16*)w, tiles, n_tiles,
                                                              sorted_pair, nullptr, top, N, K, act, gated);
  EK_RETURN_LAUNCH_STATUS();
}

EK_EXPORT int ek_moe_expert_down_tc(float* out, const void* a, const void* w, const int* tiles, const int* n_tiles,
                                    const int* sorted_pair, const float* pair_weight, int max_tiles, int N, int K,
                                    cudaStream_t stream) {
  using namespace ek;
  if (max_tiles <= 0) return 0;
  if (N <= 0 || K <= 0 || K % 8 || (N + 127) / 128 > 65535 || ((uintptr_t)a & 15) || ((uintptr_t)w & 15))
    return EK_ERR_ARG;
  dim3 grid(max_tiles, (N + 127) / 128);
  cudaError_t e = cudaFuncSetAttribute(moe_expert_product_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)kTcSmem);
  if (e != cudaSuccess) return (int)e;
  moe_expert_product_tc_kernel<false><<<grid, 256, kTcSmem, stream>>>(out, (const bf16*)a, (const bf16*)w, tiles, n_tiles,
                                                               sorted_pair, pair_weight, 1, N, K, 0, 0);
  EK_RETURN_LAUNCH_STATUS();
}

#define EK_INSTANTIATE(SUFFIX, T)                                                                     \
  EK_EXPORT int ek_moe_expert_up_##SUFFIX(void* out, const void* x, const void* w, const int* tiles,  \
                                          const int* n_tiles, const int* sorted_pair, int max_tiles,  \
                                          int top, int N, int K, int act, int gated,                  \
                                          cudaStream_t stream) {                                      \
    using namespace ek;                                                                               \
    if (max_tiles <= 0) return 0;                                                                     \
    if (N <= 0 || K <= 0 || top <= 0 || (N + 63) / 64 > 65535 || (gated && N % 2)) return EK_ERR_ARG; \
    dim3 grid(max_tiles, (N + 63) / 64);                                                              \
    moe_expert_product_kernel<T, true><<<grid, 256, 0, stream>>>(                                     \
        out, (const T*)x, (const T*)w, tiles, n_tiles, sorted_pair, nullptr, top, N, K, act, gated);  \
    EK_RETURN_LAUNCH_STATUS();                                                                        \
  }                                                                                                   \
  EK_EXPORT int ek_moe_expert_down_##SUFFIX(float* out, const void* a, const void* w, const int* tiles, \
                                            const int* n_tiles, const int* sorted_pair,               \
                                            const float* pair_weight, int max_tiles, int N, int K,    \
                                            cudaStream_t stream) {                                    \
    using namespace ek;                                                                               \
    if (max_tiles <= 0) return 0;                                                                     \
    if (N <= 0 || K <= 0 || (N + 63) / 64 > 65535) return EK_ERR_ARG;                                 \
    dim3 grid(max_tiles, (N + 63) / 64);                                                              \
    moe_expert_product_kernel<T, false><<<grid, 256, 0, stream>>>(                                    \
        out, (const T*)a, (const T*)w, tiles, n_tiles, sorted_pair, pair_weight, 1, N, K, 0, 0);      \
    EK_RETURN_LAUNCH_STATUS();                                                                        \
  }                                                                                                   \
  EK_EXPORT int ek_moe_combine_##SUFFIX(void* out, const float* pair_out, int n_tokens, int top,      \
                                        int width, cudaStream_t stream) {                             \
    if (n_tokens <= 0) return 0;                                                                      \
    ek::moe_combine_kernel<T><<<n_tokens, 256, 0, stream>>>((T*)out, pair_out, top, width);           \
    EK_RETURN_LAUNCH_STATUS();                                                                        \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)
