// Mixture of experts: routing, the experts' products over rows grouped by expert, the join.
//
// A step's rows each choose `top` of E experts. A (row, choice) is a *pair*; pair p = row *
// top + choice. Four launches, none of which needs the host to know a count:
//   route:   per row, the `top` largest router logits (fp32; ties to the smaller index) and
//            the softmax over just those (or, `over_all`, their part of the softmax over
//            every expert) -> chosen[p], share[p];
//   align:   pairs grouped by expert into a list whose every expert's stretch is padded to
//            a multiple of the tile's rows (-1 = no pair), and the expert of every tile;
//   experts: two grouped products over those tiles. The first computes, per pair,
//            g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit) and writes
//            y = g sigmoid(alpha g) (u + shift); the second writes W_down y per pair in
//            fp32 (limit = infinity, alpha = 1, shift = 0: silu(g) u);
//   join:    dst[row] (+)= scale * sum_choice share * (W_down y)[pair], choices in order.
// A pair's result does not depend on its place in a tile or on the other pairs: every output
// element is one sum over k in a fixed order. Experts' matrices lie one under the other:
// w_in [E][2 * ff][width] (an expert's gate rows, then its up rows), w_out [E][width][ff]. An
// expert without a gate (`single`: y = relu(W_up h)^2) has w_in [E][ff][width].
//
// The tile products run on the CUDA cores with fp32 FMA for float32 and on the warp-level
// tensor cores (mma.sync m16n8k16, fp32 accumulators) for bfloat16.
#include <limits.h>

#include "common.cuh"

namespace ayk {

constexpr int MOE_TM = 32;   // pairs per tile: few rows, and float32
constexpr int MOE_TM_WIDE = 128;  // pairs per tile of the tensor-core products of many rows
constexpr int MOE_TN = 64;   // output columns per tile
constexpr int MOE_TK = 32;   // k per turn on the CUDA cores (the tensor-core tiles take 64)
constexpr int MOE_MAX_EXPERTS = 1024;

// ---------------------------------------------------------------------------------------------
// One warp per row. Lane l holds logits l, l + 32, ...; `top` times the largest not yet taken.
__global__ void moe_route_kernel(const float* __restrict__ logits, int ld, int rows, int E,
                                 int top, int over_all, int* __restrict__ chosen,
                                 float* __restrict__ share) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  pdl_wait_for(logits);
  const float* z = logits + (size_t)row * ld;
  uint32_t taken = 0;  // bit m: entry lane + 32 m is chosen
  float first = 0.f, total = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int at = INT_MAX;
    for (int m = 0; lane + 32 * m < E; ++m) {
      if (taken >> m & 1u) continue;
      const float v = z[lane + 32 * m];
      if (v > best || at == INT_MAX) {
        best = v;
        at = lane + 32 * m;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_at = __shfl_xor_sync(0xffffffffu, at, o);
      if (other_at != INT_MAX && (at == INT_MAX || other > best ||
                                  (other == best && other_at < at))) {
        best = other;
        at = other_at;
      }
    }
    if ((at & 31) == lane) taken |= 1u << (at >> 5);
    if (j == 0) first = best;
    const float e = expf(best - first);  // the first is the largest: no overflow
    total += e;
    if (lane == 0) {
      chosen[(size_t)row * top + j] = at;
      share[(size_t)row * top + j] = e;
    }
  }
  if (over_all) {  // the softmax's sum runs over every expert: the shares are not renormalised
    float all = 0.f;
    for (int e = lane; e < E; e += 32) all += expf(z[e] - first);
    total = warp_sum(all);
  }
  __syncwarp();
  if (lane < top) share[(size_t)row * top + lane] /= total;
  for (int j = 32 + lane; j < top; j += 32) share[(size_t)row * top + j] /= total;
}

// Routing by scores with groups: s = sigmoid(logit); the experts form `groups` equal groups of
// neighbours, a group's score is the sum of its two largest s (its only one when a group is one
// expert), and only experts of the `keep` best groups can be chosen; of those the `top` largest
// s are taken (ties to the smaller index, also among groups). share = factor * s, divided by
// the chosen ones' sum when `renorm` is set. One warp per row; the row's scores, the groups'
// scores and the kept groups' marks lie in the warp's part of shared memory.
__global__ void moe_route_scored_kernel(const float* __restrict__ logits, int ld, int rows, int E,
                                        int top, int groups, int keep, float factor, int renorm,
                                        int* __restrict__ chosen, float* __restrict__ share) {
  extern __shared__ float route_smem[];
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= rows) return;
  float* s = route_smem + (size_t)warp * (E + 2 * groups);
  float* gs = s + E;
  int* kept = reinterpret_cast<int*>(gs + groups);
  const int per = E / groups;
  pdl_wait_for(logits);
  const float* z = logits + (size_t)row * ld;
  for (int e = lane; e < E; e += 32) s[e] = 1.f / (1.f + expf(-z[e]));
  __syncwarp();
  // the largest entry of v[0 .. n) not yet taken (taken ones are -inf), ties to the smaller index
  auto arg_max = [&](const float* v, int n, float& best, int& at) {
    best = -INFINITY;
    at = INT_MAX;
    for (int i = lane; i < n; i += 32) {
      if (v[i] > best || at == INT_MAX) {
        best = v[i];
        at = i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_at = __shfl_xor_sync(0xffffffffu, at, o);
      if (other_at != INT_MAX && (at == INT_MAX || other > best ||
                                  (other == best && other_at < at))) {
        best = other;
        at = other_at;
      }
    }
  };
  if (keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;
      for (int i = 0; i < per; ++i) {
        const float v = s[g * per + i];
        if (v > a) {
          b = a;
          a = v;
        } else if (v > b) {
          b = v;
        }
      }
      gs[g] = per > 1 ? a + b : a;
      kept[g] = 0;
    }
    __syncwarp();
    for (int j = 0; j < keep; ++j) {
      float best;
      int at;
      arg_max(gs, groups, best, at);
      if (lane == 0) {
        gs[at] = -INFINITY;
        kept[at] = 1;
      }
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32) {
      if (!kept[e / per]) s[e] = -INFINITY;
    }
    __syncwarp();
  }
  float total = 0.f;
  for (int j = 0; j < top; ++j) {
    float best;
    int at;
    arg_max(s, E, best, at);
    total += best;
    if (lane == 0) {
      s[at] = -INFINITY;
      chosen[(size_t)row * top + j] = at;
      share[(size_t)row * top + j] = best * factor;
    }
    __syncwarp();
  }
  if (renorm) {
    for (int j = lane; j < top; j += 32) share[(size_t)row * top + j] /= total;
  }
}

// One CTA. sorted: [max_tiles * tile_rows] pair indices or -1; tile_expert: [max_tiles], -1 for a
// tile past the last.
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ chosen, int pairs, int E, int max_tiles, int tile_rows,
                 int* __restrict__ sorted, int* __restrict__ tile_expert) {
  __shared__ int counts[MOE_MAX_EXPERTS];
  __shared__ int starts[MOE_MAX_EXPERTS];
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += blockDim.x) counts[e] = 0;
  pdl_wait_for(chosen);
  __syncthreads();
  for (int p = tid; p < pairs; p += blockDim.x) {
    const int e = chosen[p];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  for (int i = tid; i < max_tiles * tile_rows; i += blockDim.x) sorted[i] = -1;
  __syncthreads();
  if (tid == 0) {
    int tile = 0;
    for (int e = 0; e < E; ++e) {
      starts[e] = tile * tile_rows;
      const int tiles = (counts[e] + tile_rows - 1) / tile_rows;
      for (int t = 0; t < tiles && tile < max_tiles; ++t) tile_expert[tile++] = e;
      counts[e] = 0;  // now the cursor of the expert's stretch
    }
    for (; tile < max_tiles; ++tile) tile_expert[tile] = -1;
  }
  __syncthreads();
  for (int p = tid; p < pairs; p += blockDim.x) {
    const int e = chosen[p];
    if (e >= 0 && e < E) sorted[starts[e] + atomicAdd(&counts[e], 1)] = p;
  }
}

// ---------------------------------------------------------------------------------------------
// A tile's product. PHASE 0: rows of `a` are the pairs' rows of the normed input (row = pair /
// top), the weight tile is rows n0.. of the expert's gate part and of its up part, the result
// y[place][n] in the compute type. PHASE 1: rows of `a` are y[place], the weight tile rows
// n0.. of the expert's down matrix, the result out[pair][n] in fp32.
__device__ __forceinline__ float expert_unit(float g, float u, float limit, float alpha, float shift,
                                             int single) {
  if (single) {  // one matrix, the square of relu
    g = fmaxf(g, 0.f);
    return g * g;
  }
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + shift);
}

template <typename T, int PHASE, int TM> struct TileAcc;

// fp32: thread (ty, tx) of 16 x 16 owns rows 2 ty .. +1 and columns 4 tx .. +3
template <int PHASE> struct TileAcc<float, PHASE, MOE_TM> {
  static constexpr int TK = MOE_TK;
  static constexpr int LDS = MOE_TK + 1;
  float acc[PHASE == 0 ? 2 : 1][2][4];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int w = 0; w < (PHASE == 0 ? 2 : 1); ++w)
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[w][i][j] = 0.f;
  }
  __device__ __forceinline__ void step(const float* As, const float* Bs, const float* Bs2,
                                       bool both) {
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
    for (int k = 0; k < MOE_TK; ++k) {
      float av[2], bv[4];
#pragma unroll
      for (int i = 0; i < 2; ++i) av[i] = As[(ty * 2 + i) * LDS + k];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[(tx * 4 + j) * LDS + k];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[0][i][j] = fmaf(av[i], bv[j], acc[0][i][j]);
      if (PHASE == 0 && both) {
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = Bs2[(tx * 4 + j) * LDS + k];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[PHASE == 0 ? 1 : 0][i][j] =
              fmaf(av[i], bv[j], acc[PHASE == 0 ? 1 : 0][i][j]);
      }
    }
  }
  template <typename F> __device__ __forceinline__ void each(F f) {
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        f(ty * 2 + i, tx * 4 + j, acc[0][i][j], acc[PHASE == 0 ? 1 : 0][i][j]);
      }
  }
};

// bfloat16: eight warps as (TM / 16 MT) x the rest; a warp holds MT x NT m16n8 accumulators
// per matrix (tiles of 32 pairs: 2 x 4 warps of 16 x 16; of 128 pairs: 4 x 2 warps of
// 32 x 32, four times the products per turn and a quarter of the weights' re-reads). Shared
// rows are padded by 8 entries so that the eight rows of an ldmatrix tile fall into
// different banks.
template <int PHASE, int TM> struct TileAcc<__nv_bfloat16, PHASE, TM> {
  static constexpr int TK = 64;
  static constexpr int LDS = TK + 8;
  static constexpr int MT = TM >= 128 ? 2 : 1;    // m16 tiles of a warp
  static constexpr int WARPS_M = TM / (16 * MT);  // warps down the rows
  static constexpr int WARPS_N = 8 / WARPS_M;
  static constexpr int NT = MOE_TN / (8 * WARPS_N);  // n8 tiles of a warp (2 or 4)
  static constexpr int W = PHASE == 0 ? 2 : 1;
  float acc[W][MT][NT][4];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int w = 0; w < W; ++w)
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[w][m][n][i] = 0.f;
  }
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4],
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  // four 8 x 8 tiles of 16-bit entries, one 16-byte row address per lane
  static __device__ __forceinline__ void load_tiles(uint32_t (&r)[4], const __nv_bfloat16* p) {
    const uint32_t address = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(address));
  }
  __device__ __forceinline__ void step(const __nv_bfloat16* As, const __nv_bfloat16* Bs,
                                       const __nv_bfloat16* Bs2, bool both) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = (warp / WARPS_N) * 16 * MT, n0 = (warp % WARPS_N) * 8 * NT;
    // A: lanes 0-15 give rows 0-15 at k, lanes 16-31 the same rows at k + 8 (a0..a3);
    // B (kept [n][k]): lanes 0-7 rows n.. at k, 8-15 the same at k + 8 (b0, b1 of eight
    // columns), 16-31 likewise for the next eight
    const __nv_bfloat16* a_at = As + (m0 + (lane & 15)) * LDS + (lane >> 4) * 8;
    const int b_offset = (n0 + (lane >> 4) * 8 + (lane & 7)) * LDS + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int k0 = 0; k0 < TK; k0 += 16) {
      uint32_t a[MT][4], b[4];
#pragma unroll
      for (int m = 0; m < MT; ++m) load_tiles(a[m], a_at + m * 16 * LDS + k0);
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        load_tiles(b, Bs + b_offset + n * 8 * LDS + k0);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          mma(acc[0][m][n], a[m], b[0], b[1]);
          mma(acc[0][m][n + 1], a[m], b[2], b[3]);
        }
        if (PHASE == 0 && both) {
          load_tiles(b, Bs2 + b_offset + n * 8 * LDS + k0);
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            mma(acc[W - 1][m][n], a[m], b[0], b[1]);
            mma(acc[W - 1][m][n + 1], a[m], b[2], b[3]);
          }
        }
      }
    }
  }
  template <typename F> __device__ __forceinline__ void each(F f) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = (warp / WARPS_N) * 16 * MT, n0 = (warp % WARPS_N) * 8 * NT;
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          f(m0 + 16 * m + g + (i >> 1) * 8, n0 + 8 * n + 2 * t + (i & 1), acc[0][m][n][i],
            acc[W - 1][m][n][i]);
        }
  }
};

template <typename T, int PHASE, int TM>
__global__ void __launch_bounds__(256, 2)  // two CTAs an SM: one's copies under the other's products
moe_tile_kernel(const T* __restrict__ a, int lda, const T* __restrict__ weight,
                const int* __restrict__ sorted, const int* __restrict__ tile_expert, int top,
                int K, int N, float limit, float alpha, float shift, T* __restrict__ y, int ld_y,
                float* __restrict__ out, int ld_out, int wide, int single) {
  using Acc = TileAcc<T, PHASE, TM>;
  constexpr int LDS = Acc::LDS, TK = Acc::TK;
  constexpr bool BF16 = sizeof(T) == 2;
  __shared__ __align__(16) T As[TM * LDS];
  __shared__ __align__(16) T Bs[MOE_TN * LDS];
  __shared__ __align__(16) T Bs2[PHASE == 0 ? MOE_TN * LDS : 8];
  __shared__ int pair_s[TM];
  pdl_launch_dependents();
  const int tile = blockIdx.x, n0 = blockIdx.y * MOE_TN, tid = threadIdx.x;
  pdl_wait_for(a, sorted, tile_expert);
  const int e = tile_expert[tile];
  if (e < 0) return;
  if (tid < TM) pair_s[tid] = sorted[tile * TM + tid];
  __syncthreads();
  // an expert's matrices: PHASE 0 [2 N][K] (gate rows, then up rows), PHASE 1 [N][K]
  // (`single`: an expert without a gate, PHASE 0 [N][K] too)
  const bool both = PHASE == 0 && !single;
  const T* w = weight + (size_t)e * (both ? 2 : 1) * N * K;
  Acc acc;
  acc.zero();
  if (BF16 && wide) {
    // 16-byte pieces: the tile's rows of 64 k are eight pieces each; a thread brings one
    // piece of the pairs' rows and two of each weight tile, and the next turn's pieces are
    // on their way while this turn's products run
    const int pr = tid >> 3, pk = (tid & 7) * 8;  // piece: row pr (+32, +64, ...), k pk
    constexpr int AP = TM / 32;                   // pieces of the pairs' rows per thread
    const T* a_row[AP];
#pragma unroll
    for (int i = 0; i < AP; ++i) {
      const int pair = pair_s[pr + 32 * i];
      a_row[i] = pair < 0 ? nullptr
                          : a + (PHASE == 0 ? (size_t)(pair / top)
                                            : (size_t)tile * TM + pr + 32 * i) * lda;
    }
    uint4 ra[AP], rb[2], rb2[2];
    auto fetch = [&](int k0) {
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
      const bool in_k = k0 + pk < K;  // (K is a multiple of 8: a piece is inside or outside)
#pragma unroll
      for (int i = 0; i < AP; ++i) {
        ra[i] = (a_row[i] != nullptr && in_k)
                    ? *reinterpret_cast<const uint4*>(a_row[i] + k0 + pk) : zero;
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = n0 + pr + 32 * i;
        const bool in = in_k && r < N;
        rb[i] = in ? *reinterpret_cast<const uint4*>(w + (size_t)r * K + k0 + pk) : zero;
        if (both) {
          rb2[i] = in ? *reinterpret_cast<const uint4*>(w + (size_t)(N + r) * K + k0 + pk) : zero;
        }
      }
    };
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
      for (int i = 0; i < AP; ++i) {
        *reinterpret_cast<uint4*>(As + (pr + 32 * i) * LDS + pk) = ra[i];
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        *reinterpret_cast<uint4*>(Bs + (pr + 32 * i) * LDS + pk) = rb[i];
        if (both) *reinterpret_cast<uint4*>(Bs2 + (pr + 32 * i) * LDS + pk) = rb2[i];
      }
      __syncthreads();
      if (k0 + TK < K) fetch(k0 + TK);
      acc.step(As, Bs, Bs2, both);
      __syncthreads();
    }
  } else {
    for (int k0 = 0; k0 < K; k0 += TK) {
      for (int idx = tid; idx < TM * TK; idx += 256) {
        const int r = idx / TK, k = idx % TK;
        const int pair = pair_s[r];
        T v = T(0.f);
        if (pair >= 0 && k0 + k < K) {
          const size_t row = PHASE == 0 ? (size_t)(pair / top) : (size_t)tile * TM + r;
          v = a[row * lda + k0 + k];
        }
        As[r * LDS + k] = v;
      }
      for (int idx = tid; idx < MOE_TN * TK; idx += 256) {
        const int r = idx / TK, k = idx % TK;
        const bool in = n0 + r < N && k0 + k < K;
        Bs[r * LDS + k] = in ? w[(size_t)(n0 + r) * K + k0 + k] : T(0.f);
        if (both) Bs2[r * LDS + k] = in ? w[(size_t)(N + n0 + r) * K + k0 + k] : T(0.f);
      }
      __syncthreads();
      acc.step(As, Bs, Bs2, both);
      __syncthreads();
    }
  }
  acc.each([&](int r, int c, float first, float second) {
    const int pair = pair_s[r];
    if (pair < 0 || n0 + c >= N) return;
    if (PHASE == 0) {
      stf(y + ((size_t)tile * TM + r) * ld_y + n0 + c,
          expert_unit(first, second, limit, alpha, shift, single));
    } else {
      out[(size_t)pair * ld_out + n0 + c] = first;
    }
  });
}

// dst[row][c] (+)= scale[c] * sum_j share[row * top + j] * pair_out[row * top + j][c]
__global__ void moe_join_kernel(const float* __restrict__ pair_out, int ld, const float* __restrict__ share,
                                int top, const float* __restrict__ scale,
                                float* __restrict__ dst, int ld_dst, int width, int accumulate) {
  pdl_launch_dependents();
  const int row = blockIdx.x;
  pdl_wait_for(pair_out, share, dst);
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    float sum = 0.f;
    for (int j = 0; j < top; ++j) {
      const size_t pair = (size_t)row * top + j;
      sum = fmaf(share[pair], pair_out[pair * ld + c], sum);
    }
    if (scale != nullptr) sum *= scale[c];
    float* to = dst + (size_t)row * ld_dst + c;
    *to = accumulate ? *to + sum : sum;
  }
}

template <typename T, int TM>
int moe_experts(const void* hidden, int ld_hidden, const void* w_in, const void* w_out,
                const int* sorted, const int* tile_expert, int max_tiles, int top, int width,
                int ff, float limit, float alpha, float shift, int single, void* y, int ld_y,
                float* pair_out, int ld_out, cudaStream_t stream) {
  // 16-byte pieces when every row of every operand starts on a 16-byte boundary
  const auto aligned = [](const void* p) { return ((uintptr_t)p % 16) == 0; };
  const int wide_in = sizeof(T) == 2 && width % 8 == 0 && ld_hidden % 8 == 0 &&
                      aligned(hidden) && aligned(w_in);
  const int wide_out = sizeof(T) == 2 && ff % 8 == 0 && ld_y % 8 == 0 && aligned(y) &&
                       aligned(w_out);
  // (room in shared memory for two CTAs an SM: the default split may leave less)
  static const bool carved = [] {
    cudaFuncSetAttribute(moe_tile_kernel<T, 0, TM>,
                         cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    cudaFuncSetAttribute(moe_tile_kernel<T, 1, TM>,
                         cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    return true;
  }();
  (void)carved;
  const dim3 grid_in(max_tiles, (ff + MOE_TN - 1) / MOE_TN);
  int status = launch_kernel(moe_tile_kernel<T, 0, TM>, grid_in, dim3(256), 0, stream, 1,
                             (const T*)hidden, ld_hidden, (const T*)w_in, sorted, tile_expert,
                             top, width, ff, limit, alpha, shift, (T*)y, ld_y, (float*)nullptr, 0,
                             wide_in, single);
  if (status != AYK_OK) return status;
  const dim3 grid_out(max_tiles, (width + MOE_TN - 1) / MOE_TN);
  return launch_kernel(moe_tile_kernel<T, 1, TM>, grid_out, dim3(256), 0, stream, 1, (const T*)y,
                       ld_y, (const T*)w_out, sorted, tile_expert, top, ff, width, limit, alpha, shift,
                       (T*)nullptr, 0, pair_out, ld_out, wide_out, 0);
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

AYK_API int ayk_moe_tile_rows() { return ayk::MOE_TM; }
AYK_API int ayk_moe_tile_rows_wide() { return ayk::MOE_TM_WIDE; }

AYK_API int ayk_moe_route(const float* logits, int ld, int rows, int experts, int top,
                          int over_all, int* chosen, float* share, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || experts < 1 || top < 1 || top > experts || ld < experts ||
      logits == nullptr || chosen == nullptr || share == nullptr) {
    return AYK_BAD_ARGUMENT;
  }
  if (experts > MOE_MAX_EXPERTS) return AYK_TOO_LARGE;
  const int warps = 4;
  return launch_kernel(moe_route_kernel, dim3((rows + warps - 1) / warps), dim3(32 * warps), 0,
                       (cudaStream_t)stream, 1, logits, ld, rows, experts, top, over_all, chosen,
                       share);
}

// Scores instead of a softmax: see moe_route_scored_kernel. `groups` divides `experts`,
// 1 <= keep <= groups, and the kept groups hold at least `top` experts.
AYK_API int ayk_moe_route_scored(const float* logits, int ld, int rows, int experts, int top,
                                 int groups, int keep, float factor, int renorm, int* chosen,
                                 float* share, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || experts < 1 || top < 1 || groups < 1 || experts % groups || keep < 1 ||
      keep > groups || top > keep * (experts / groups) || ld < experts || logits == nullptr ||
      chosen == nullptr || share == nullptr) {
    return AYK_BAD_ARGUMENT;
  }
  if (experts > MOE_MAX_EXPERTS) return AYK_TOO_LARGE;
  const int per_warp = experts + 2 * groups;
  const int warps = per_warp <= 1024 ? 4 : 1;
  return launch_kernel(moe_route_scored_kernel, dim3((rows + warps - 1) / warps),
                       dim3(32 * warps), (size_t)warps * per_warp * sizeof(float),
                       (cudaStream_t)stream, 1, logits, ld, rows, experts, top, groups, keep,
                       factor, renorm, chosen, share);
}

// Three launches: align, the two grouped products. `sorted` holds max_tiles * tile_rows ints,
// `tile_expert` max_tiles, `y` max_tiles * tile_rows rows of ff, `pair_out` rows * top rows
// of width. type: 0 = float32, 1 = bfloat16. tile_rows: 32, or 128 (bfloat16 only).
AYK_API int ayk_moe_experts(const void* hidden, int ld_hidden, const void* w_in,
                            const void* w_out, const int* chosen, int rows, int experts, int top,
                            int width, int ff, float limit, float alpha, float shift, int single,
                            int* sorted,
                            int* tile_expert, int max_tiles, int tile_rows, void* y, int ld_y,
                            float* pair_out, int ld_out, int type, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  const long long pairs = (long long)rows * top;
  if (rows < 0 || experts < 1 || top < 1 || width < 1 || ff < 1 || hidden == nullptr ||
      w_in == nullptr || w_out == nullptr || chosen == nullptr || sorted == nullptr ||
      tile_expert == nullptr || y == nullptr || pair_out == nullptr || ld_hidden < width ||
      ld_y < ff || ld_out < width || !(limit > 0.f) ||
      (tile_rows != MOE_TM && !(tile_rows == MOE_TM_WIDE && type == 1)) ||
      (long long)max_tiles * tile_rows <
          pairs + (long long)min(experts, (int)pairs) * (tile_rows - 1)) {
    return AYK_BAD_ARGUMENT;
  }
  if (experts > MOE_MAX_EXPERTS || max_tiles > 2000000) return AYK_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  int status = launch_kernel(moe_align_kernel, dim3(1), dim3(1024), 0, s, 1, chosen, (int)pairs,
                             experts, max_tiles, tile_rows, sorted, tile_expert);
  if (status != AYK_OK) return status;
  if (type == 0) {
    return moe_experts<float, MOE_TM>(hidden, ld_hidden, w_in, w_out, sorted, tile_expert, max_tiles,
                              top, width, ff, limit, alpha, shift, single, y, ld_y, pair_out,
                              ld_out, s);
  }
  if (type == 1 && tile_rows == MOE_TM_WIDE) {
    return moe_experts<__nv_bfloat16, MOE_TM_WIDE>(hidden, ld_hidden, w_in, w_out, sorted,
                                                   tile_expert, max_tiles, top, width, ff, limit,
                                                   alpha, shift, single, y, ld_y, pair_out, ld_out, s);
  }
  if (type == 1) {
    return moe_experts<__nv_bfloat16, MOE_TM>(hidden, ld_hidden, w_in, w_out, sorted,
                                              tile_expert, max_tiles, top, width, ff, limit,
                                              alpha, shift, single, y, ld_y, pair_out, ld_out, s);
  }
  return AYK_BAD_ARGUMENT;
}

AYK_API int ayk_moe_join(const float* pair_out, int ld, const float* share, int rows, int top,
                         const float* scale, float* dst, int ld_dst, int width, int accumulate,
                         void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || top < 1 || width < 1 || pair_out == nullptr || share == nullptr ||
      dst == nullptr || ld < width || ld_dst < width) {
    return AYK_BAD_ARGUMENT;
  }
  const int threads = 256, tiles = min(8, (width + threads - 1) / threads);
  return launch_kernel(moe_join_kernel, dim3(rows, tiles), dim3(threads), 0,
                       (cudaStream_t)stream, 1, pair_out, ld, share, top, scale, dst, ld_dst,
                       width, accumulate);
}
