// Latent attention: attention whose keys and values are up-projections W_uk c, W_uv c of one
// small latent row c per token, beside one rotated key piece kr that all heads share. The
// cache keeps only [c | kr] per token ("latent pages": [page][slot][rank + rot], one pool row
// per token whatever the number of heads).
//
// The up-projections are never applied to cached rows. With q_h = [q_plain | q_rot]:
//   q_plain . (W_uk,h c) = (W_uk,h^T q_plain) . c        (the query is taken to latent space)
//   sum_s w_s W_uv,h c_s = W_uv,h (sum_s w_s c_s)        (the weighted sum stays latent)
// so a step is: prepare (norm of c, rotation of kr and q_rot, store of [c | kr]), one small
// product per head that forms qa_h = [W_uk,h^T q_plain | q_rot], attention of all heads over
// the same latent rows (scores qa_h . [c | kr], values = the first `rank` entries of the key
// row), one small product per head W_uv,h (.) with the output gate in its epilogue. The three
// kernels of this file; the projections before and after are the engine's matrix products.
//
// All arithmetic in fp32; T is the type of the cache, of the queries and of the outputs.
#include <type_traits>

#include "rope.cuh"

namespace ayk {

// ---------------------------------------------------------------------------------------------
// prepare: one CTA per row of the step.
//   proj row (fp32): [ q: heads x (dim + rot) | c_raw: rank | kr_raw: rot | ... ]
//   latent page row <- [ c_raw * rsqrt(mean(c_raw^2) + eps) * w_c | rotate(kr_raw) ]
//   q_plain[row]    <- the heads' unrotated parts            [heads x dim]
//   qa[row]         <- rotate(q_rot) at [h][rank ..]          [heads x (rank + rot)]
// Only the first rot_dims entries of a rotated piece are turned; the rest passes.
template <typename T>
__global__ void latent_prepare_kernel(const float* __restrict__ proj, int ld_proj, int kv_offset,
                                      const float* __restrict__ latent_weight, float eps,
                                      const int* __restrict__ positions,
                                      const int* __restrict__ slots,
                                      const double* __restrict__ freq, int rot_dims, int layout,
                                      T* __restrict__ pages, T* __restrict__ q_plain,
                                      int ld_plain, T* __restrict__ qa, int ld_qa, int heads,
                                      int dim, int rot, int rank) {
  __shared__ float cos_s[ROPE_MAX_PAIRS], sin_s[ROPE_MAX_PAIRS];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int row = blockIdx.x, pairs = rot_dims / 2;
  rope_fill_table(cos_s, sin_s, positions[row], freq, pairs);
  const int slot = slots != nullptr ? slots[row] : -1;
  pdl_wait_for(proj);
  const float* src = proj + (size_t)row * ld_proj;
  const float* c_raw = src + kv_offset;
  float inv = 0.f;
  if (pages != nullptr) {  // (a layer that reads another's latents has no raw latent at all)
    float s = 0.f;
    for (int j = threadIdx.x; j < rank; j += blockDim.x) s += c_raw[j] * c_raw[j];
    inv = 1.f / sqrtf(block_sum(s, scratch) / (float)rank + eps);  // (also a barrier)
  } else {
    __syncthreads();  // the table of sines is read below
  }
  if (pages != nullptr && slot >= 0) {
    T* dst = pages + (size_t)slot * (rank + rot);
    for (int j = threadIdx.x; j < rank; j += blockDim.x) {
      stf(dst + j, c_raw[j] * inv * latent_weight[j]);
    }
    const float* kr = c_raw + rank;
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
      int a, b;
      rope_members(i, rot_dims, layout, a, b);
      const float u = kr[a], v = kr[b];
      stf(dst + rank + a, u * cos_s[i] - v * sin_s[i]);
      stf(dst + rank + b, v * cos_s[i] + u * sin_s[i]);
    }
    for (int j = rot_dims + threadIdx.x; j < rot; j += blockDim.x) stf(dst + rank + j, kr[j]);
  }
  T* plain = q_plain + (size_t)row * ld_plain;
  for (int idx = threadIdx.x; idx < heads * dim; idx += blockDim.x) {
    const int h = idx / dim, j = idx % dim;
    stf(plain + idx, src[(size_t)h * (dim + rot) + j]);
  }
  T* turned = qa + (size_t)row * ld_qa;
  for (int idx = threadIdx.x; idx < heads * pairs; idx += blockDim.x) {
    const int h = idx / pairs, i = idx % pairs;
    int a, b;
    rope_members(i, rot_dims, layout, a, b);
    const float* q_rot = src + (size_t)h * (dim + rot) + dim;
    T* dst = turned + (size_t)h * (rank + rot) + rank;
    const float u = q_rot[a], v = q_rot[b];
    stf(dst + a, u * cos_s[i] - v * sin_s[i]);
    stf(dst + b, v * cos_s[i] + u * sin_s[i]);
  }
  const int rest = rot - rot_dims;
  for (int idx = threadIdx.x; idx < heads * rest; idx += blockDim.x) {
    const int h = idx / rest, j = rot_dims + idx % rest;
    stf(turned + (size_t)h * (rank + rot) + rank + j, src[(size_t)h * (dim + rot) + dim + j]);
  }
}

// ---------------------------------------------------------------------------------------------
// One small product per head: out[n][h][j] = sum_i a[n][h][i] * W_h(i, j), fp32 sums in the
// order of i whatever the batch. W_h(i, j) sits at w + h * w_head + i * w_in + j * w_out, so a
// head's matrix is used as stored ([in, out] rows: w_in = cols, w_out = 1) or transposed
// ([out, in] rows: w_in = 1, w_out = cols). With `gate` (fp32 [n][h * J + j]) the result is
// multiplied by sigmoid(gate). Tiles go through shared memory a slice of the inner dimension
// at a time.
constexpr int HL_BN = 64;

// A CTA of 256 threads computes (256 / (BN / TN)) * TM rows x BN columns, BK of the inner
// dimension at a time: <2, 4, 16> is 32 rows x 64 columns for prompt portions; <1, 1, 64, 16>
// (<1, 1, 256, 16> for a longer inner dimension) is 16 rows x 16 columns in a quarter (a
// sixteenth) of the turns, for the few rows of a decode step, where
// what counts is the number of trips to memory and of CTAs that make them at once (a head's
// 64 columns over four CTAs), not the arithmetic.
template <typename T, int TM, int TN, int BK, int BN = HL_BN>
__global__ void __launch_bounds__(256)
head_linear_kernel(const T* __restrict__ a, int ld_a, int a_head, const T* __restrict__ w,
                   long long w_head, int w_in, int w_out, const float* __restrict__ gate,
                   int ld_gate, T* __restrict__ out, int ld_out, int out_head, int rows, int I,
                   int J) {
  constexpr int TX = BN / TN, TY = 256 / TX, BM = TY * TM;
  __shared__ float a_s[BK][BM + 1];
  __shared__ float w_s[BK][BN + 1];
  pdl_launch_dependents();
  const int h = blockIdx.z, m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
  const T* wh = w + (size_t)h * w_head;
  pdl_wait_for(a, gate);
  const T* ah = a + (size_t)h * a_head;
  float acc[TM][TN] = {};
  for (int k0 = 0; k0 < I; k0 += BK) {
    for (int idx = threadIdx.x; idx < BK * BM; idx += 256) {
      const int kk = idx % BK, mm = idx / BK;
      const int m = m0 + mm, k = k0 + kk;
      a_s[kk][mm] = (m < rows && k < I) ? ldf(ah + (size_t)m * ld_a + k) : 0.f;
    }
    for (int idx = threadIdx.x; idx < BK * BN; idx += 256) {
      int kk, nn;
      if (w_out == 1) {  // consecutive threads along the unit stride
        nn = idx % BN;
        kk = idx / BN;
      } else {
        kk = idx % BK;
        nn = idx / BK;
      }
      const int n = n0 + nn, k = k0 + kk;
      w_s[kk][nn] = (n < J && k < I) ? ldf(wh + (size_t)k * w_in + (size_t)n * w_out) : 0.f;
    }
    __syncthreads();
    const int kmax = min(BK, I - k0);  // (what lies beyond holds zeros)
#pragma unroll 16
    for (int kk = 0; kk < kmax; ++kk) {
      float av[TM];
#pragma unroll
      for (int r = 0; r < TM; ++r) av[r] = a_s[kk][ty * TM + r];
#pragma unroll
      for (int c = 0; c < TN; ++c) {
        const float wv = w_s[kk][tx * TN + c];
#pragma unroll
        for (int r = 0; r < TM; ++r) acc[r][c] = fmaf(av[r], wv, acc[r][c]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < TM; ++r) {
    const int m = m0 + ty * TM + r;
    if (m >= rows) continue;
#pragma unroll
    for (int c = 0; c < TN; ++c) {
      const int n = n0 + tx * TN + c;
      if (n >= J) continue;
      float v = acc[r][c];
      if (gate != nullptr) {
        const float z = gate[(size_t)m * ld_gate + (size_t)h * J + n];
        v *= 1.f / (1.f + expf(-z));
      }
      stf(out + (size_t)m * ld_out + (size_t)h * out_head + n, v);
    }
  }
}

// ---- the same product for bfloat16 prompt portions, on the warp-level tensor cores -----------
// (warp-level fragments; also used by the decode kernel further down)
__device__ __forceinline__ void lm_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lm_ldmatrix_x4_trans(uint32_t* r, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ uint32_t lm_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ void lm_ldmatrix_x4(uint32_t* r, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void lm_cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;  // (0: the 16 bytes are zero-filled, nothing is read)
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes)
               : "memory");
}

// A CTA of four warps computes 64 rows x 64 columns of one head, 64 of the inner dimension at
// a time through two stages of asynchronous 16-byte copies (zero fill past the edges); a warp
// owns 16 rows. K_ROWS: W_h is stored [j][i] (i contiguous: the B operand's own layout);
// otherwise [i][j] (j contiguous: fragments by transposing loads). fp32 accumulators summed
// in the order of i whatever the batch; the gate and the one rounding in the epilogue.
// Sizes: I, J, ld_a, a_head, ld_w and w_head multiples of 8, ld_out and out_head even.
constexpr int HM_TILE = 64, HM_STRIDE = HM_TILE + 8;

template <bool K_ROWS>
__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const __nv_bfloat16* __restrict__ a, int ld_a, int a_head,
                       const __nv_bfloat16* __restrict__ w, long long w_head, int ld_w,
                       const float* __restrict__ gate, int ld_gate,
                       __nv_bfloat16* __restrict__ out, int ld_out, int out_head, int rows,
                       int I, int J) {
  __shared__ __align__(16) __nv_bfloat16 a_s[2][HM_TILE * HM_STRIDE];
  __shared__ __align__(16) __nv_bfloat16 w_s[2][HM_TILE * HM_STRIDE];
  pdl_launch_dependents();
  const int h = blockIdx.z, m0 = blockIdx.x * HM_TILE, n0 = blockIdx.y * HM_TILE;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* wh = w + (size_t)h * w_head;
  pdl_wait_for(a, gate);
  const __nv_bfloat16* ah = a + (size_t)h * a_head;

  auto load = [&](int stage, int k0) {
    for (int idx = threadIdx.x; idx < HM_TILE * 8; idx += 128) {
      const int r = idx >> 3, c = (idx & 7) * 8;
      const bool valid = m0 + r < rows && k0 + c < I;
      lm_cp_async16(&a_s[stage][r * HM_STRIDE + c],
                    valid ? ah + (size_t)(m0 + r) * ld_a + k0 + c : ah, valid);
      if (K_ROWS) {  // row r of the tile is column n0 + r of the result
        const bool ok = n0 + r < J && k0 + c < I;
        lm_cp_async16(&w_s[stage][r * HM_STRIDE + c],
                      ok ? wh + (size_t)(n0 + r) * ld_w + k0 + c : wh, ok);
      } else {       // row r of the tile is inner index k0 + r
        const bool ok = k0 + r < I && n0 + c < J;
        lm_cp_async16(&w_s[stage][r * HM_STRIDE + c],
                      ok ? wh + (size_t)(k0 + r) * ld_w + n0 + c : wh, ok);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float acc[HM_TILE / 8][4];
#pragma unroll
  for (int t = 0; t < HM_TILE / 8; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
  const int turns = (I + HM_TILE - 1) / HM_TILE;
  load(0, 0);
  for (int turn = 0; turn < turns; ++turn) {
    const int stage = turn & 1;
    if (turn + 1 < turns) {
      load(stage ^ 1, (turn + 1) * HM_TILE);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const __nv_bfloat16* at = a_s[stage];
    const __nv_bfloat16* wt = w_s[stage];
#pragma unroll
    for (int kk = 0; kk < HM_TILE / 16; ++kk) {
      uint32_t af[4];
      lm_ldmatrix_x4(af, at + (warp * 16 + (lane & 15)) * HM_STRIDE + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int t = 0; t < HM_TILE / 16; ++t) {
        uint32_t bf[4];
        if (K_ROWS) {
          // lanes 0-7: columns 16t..+7, inner piece 0; 8-15: the same columns, piece 1;
          // 16-23: columns +8, piece 0; 24-31: columns +8, piece 1
          lm_ldmatrix_x4(bf, wt + (t * 16 + (lane & 7) + ((lane >> 4) << 3)) * HM_STRIDE +
                                 kk * 16 + ((lane >> 3) & 1) * 8);
        } else {
          // transposed: lanes 0-7: inner 16kk..+7 at column piece 2t; 8-15: inner +8, the same
          // piece; 16-23: inner 16kk..+7 at piece 2t + 1; 24-31: inner +8, piece 2t + 1
          lm_ldmatrix_x4_trans(bf, wt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) *
                                            HM_STRIDE + t * 16 + (lane >> 4) * 8);
        }
        lm_mma(acc[2 * t], af, bf[0], bf[1]);
        lm_mma(acc[2 * t + 1], af, bf[2], bf[3]);
      }
    }
    __syncthreads();  // the stage is filled again at the next turn
  }
  const int r0 = m0 + warp * 16 + (lane >> 2);
#pragma unroll
  for (int t = 0; t < HM_TILE / 8; ++t) {
    const int n = n0 + t * 8 + (lane & 3) * 2;
    if (n >= J) continue;  // (J is even: n + 1 < J too)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = r0 + half * 8;
      if (m >= rows) continue;
      float v0 = acc[t][2 * half], v1 = acc[t][2 * half + 1];
      if (gate != nullptr) {
        const float* z = gate + (size_t)m * ld_gate + (size_t)h * J + n;
        v0 *= 1.f / (1.f + expf(-z[0]));
        v1 *= 1.f / (1.f + expf(-z[1]));
      }
      *reinterpret_cast<uint32_t*>(out + (size_t)m * ld_out + (size_t)h * out_head + n) =
          lm_pack(v0, v1);
    }
  }
}

inline bool head_linear_mma_takes(const void* a, int ld_a, int a_head, const void* w,
                                  long long w_head, int ld_w, const void* out, int ld_out,
                                  int out_head, int rows, int I, int J) {
  return rows > 16 && I % 8 == 0 && J % 8 == 0 && ld_a % 8 == 0 && a_head % 8 == 0 &&
         ld_w % 8 == 0 && w_head % 8 == 0 && ld_out % 2 == 0 && out_head % 2 == 0 &&
         ((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 3) == 0;
}

template <typename T>
int head_linear(const void* a, int ld_a, int a_head, const void* w, long long w_head, int w_in,
                int w_out, const float* gate, int ld_gate, void* out, int ld_out, int out_head,
                int rows, int heads, int I, int J, cudaStream_t s) {
  const int tiles = (J + HL_BN - 1) / HL_BN;
  if (tiles > 65535) return AYK_TOO_LARGE;
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    const int ld_w = w_in == 1 ? w_out : w_in;
    if (head_linear_mma_takes(a, ld_a, a_head, w, w_head, ld_w, out, ld_out, out_head, rows, I,
                              J)) {
      const dim3 grid((rows + HM_TILE - 1) / HM_TILE, tiles, heads);
      if (w_in == 1) {
        return launch_kernel(head_linear_mma_kernel<true>, grid, dim3(128), 0, s, 1,
                             (const T*)a, ld_a, a_head, (const T*)w, w_head, ld_w, gate,
                             ld_gate, (T*)out, ld_out, out_head, rows, I, J);
      }
      return launch_kernel(head_linear_mma_kernel<false>, grid, dim3(128), 0, s, 1,
                           (const T*)a, ld_a, a_head, (const T*)w, w_head, ld_w, gate, ld_gate,
                           (T*)out, ld_out, out_head, rows, I, J);
    }
  }
  if (rows <= 16) {
    if (I > 64) {  // up to 256 of the inner dimension in one trip to memory
      return launch_kernel(head_linear_kernel<T, 1, 1, 256, 16>, dim3(1, (J + 15) / 16, heads),
                           dim3(256), 0, s, 1, (const T*)a, ld_a, a_head, (const T*)w, w_head,
                           w_in, w_out, gate, ld_gate, (T*)out, ld_out, out_head, rows, I, J);
    }
    return launch_kernel(head_linear_kernel<T, 1, 1, 64, 16>, dim3(1, (J + 15) / 16, heads),
                         dim3(256), 0, s, 1, (const T*)a, ld_a, a_head, (const T*)w, w_head,
                         w_in, w_out, gate, ld_gate, (T*)out, ld_out, out_head, rows, I, J);
  }
  return launch_kernel(head_linear_kernel<T, 2, 4, 16>, dim3((rows + 31) / 32, tiles, heads),
                       dim3(256), 0, s, 1, (const T*)a, ld_a, a_head, (const T*)w, w_head, w_in,
                       w_out, gate, ld_gate, (T*)out, ld_out, out_head, rows, I, J);
}

// ---------------------------------------------------------------------------------------------
// attention over latent pages: one warp per (row, head); the warps of a CTA take neighbouring
// heads of one row, so the key rows they share are fetched from memory once. The row at
// position p of request b sees keys max(0, p - window + 1) .. p (window 0: all), read through
// the block table in tiles of 32 keys counted from a multiple of 32: lane j scores key t0 + j
// over all rank + rot entries, the warp keeps a running maximum and sum (fp32, expf), then the
// lanes split the first `rank` entries of the key rows and add w_j * row_j. The tiling depends
// only on the position: a row's result is the same alone, in a portion or in a mixed batch.
constexpr int LA_WARPS = 4;

template <typename T> struct Chunk8;
template <> struct Chunk8<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct Chunk8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

template <typename T, int R>  // a lane holds R of the rank output entries: rank <= 32 * R
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(const T* __restrict__ qa, int ld_qa, const T* __restrict__ pages,
                        const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ request_of_row,
                        const int* __restrict__ positions, T* __restrict__ out, int ld_out,
                        int num_heads, int rank, int key_dim, int key_pad, int page_size,
                        float scale, int window, int vector_ok) {
  extern __shared__ __align__(16) float la_smem[];
  float* q_s = la_smem + (size_t)(threadIdx.x >> 5) * key_pad;
  __shared__ float w_s[LA_WARPS][32];
  __shared__ long long off_s[LA_WARPS][32];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x, head = blockIdx.y * LA_WARPS + warp;
  if (head >= num_heads) return;  // (no block barrier below)
  const int b = request_of_row[row], p = positions[row];
  pdl_wait_for(qa, pages);
  T* dst = out + (size_t)row * ld_out + (size_t)head * rank;
  if (b < 0) {
    for (int d = lane; d < rank; d += 32) stf(dst + d, 0.f);
    return;
  }
  const T* q = qa + (size_t)row * ld_qa + (size_t)head * key_dim;
  for (int d = lane; d < key_dim; d += 32) q_s[d] = ldf(q + d) * scale;
  __syncwarp();
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int* table = block_table + (size_t)b * table_stride;
  float m = -INFINITY, l = 0.f;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  for (int t0 = (lo / 32) * 32; t0 <= p; t0 += 32) {
    const int t = t0 + lane;
    const bool valid = t >= lo && t <= p;
    long long off = -1;
    float score = -INFINITY;
    if (valid) {
      off = ((long long)table[t / page_size] * page_size + t % page_size) * key_dim;
      const T* key = pages + off;
      float dot = 0.f;
      if (vector_ok) {
        for (int d = 0; d < key_dim; d += 8) {
          float kv[8];
          Chunk8<T>::load(key + d, kv);
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(q_s[d + e], kv[e], dot);
        }
      } else {
        for (int d = 0; d < key_dim; ++d) dot = fmaf(q_s[d], ldf(key + d), dot);
      }
      score = dot;
    }
    const float m_new = fmaxf(m, warp_max(score));  // every tile holds at least one key
    const float wgt = valid ? expf(score - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(wgt);
    m = m_new;
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] *= corr;
    w_s[warp][lane] = wgt;
    off_s[warp][lane] = off;
    __syncwarp();
    const int count = min(32, p - t0 + 1);
    for (int j = 0; j < count; ++j) {
      const long long oj = off_s[warp][j];
      if (oj < 0) continue;
      const float wj = w_s[warp][j];
      const T* value = pages + oj;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int d = lane + 32 * r;
        if (d < rank) acc[r] = fmaf(wj, ldf(value + d), acc[r]);
      }
    }
    __syncwarp();
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = lane + 32 * r;
    if (d < rank) stf(dst + d, acc[r] * inv);
  }
}

// ---------------------------------------------------------------------------------------------
// The same attention for steps of single rows (decode), where the time is the rows' trip from
// memory: a CTA takes one row and one share of its keys for ALL heads, so a latent row is
// fetched once whatever the number of heads. Tiles of 32 keys travel by 16-byte asynchronous
// copies into two padded shared-memory buffers (row stride + 16 bytes: a quarter warp's
// 16-byte reads of eight different rows fall on different banks); warp w takes heads w, w + 8,
// ...: lane j scores key j of the tile, the warp keeps the head's running maximum and sum, then
// lane l adds up entries 8 l .. 8 l + 7 of the rows. Every share writes (maximum, sum, weighted
// rows) to scratch and a second launch merges the shares in share order. The walk over a
// row's keys is cut at multiples of 32 counted from key 0, by position alone.
constexpr int LD_WARPS = 8, LD_HEADS = 4;  // heads per warp at most: 32 heads per CTA

__device__ __forceinline__ void la_copy16(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(LD_WARPS * 32)
latent_decode_kernel(const T* __restrict__ qa, int ld_qa, const T* __restrict__ pages,
                     const int* __restrict__ block_table, int table_stride,
                     const int* __restrict__ request_of_row, const int* __restrict__ positions,
                     float* __restrict__ partial, int num_heads, int rank, int key_dim,
                     int page_size, float scale, int window, int splits) {
  extern __shared__ __align__(16) unsigned char ld_smem[];
  constexpr int PER16 = 16 / sizeof(T);          // elements of a 16-byte piece
  const int row_elems = key_dim + PER16;         // padded row
  T* tile_s = reinterpret_cast<T*>(ld_smem);     // [2][32][row_elems]
  float* q_s = reinterpret_cast<float*>(ld_smem + (size_t)2 * 32 * row_elems * sizeof(T));
  __shared__ float w_s[LD_WARPS][32];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x, split = blockIdx.y, head0 = blockIdx.z * LD_WARPS * LD_HEADS;
  const int heads_here = min(num_heads - head0, LD_WARPS * LD_HEADS);
  const int b = request_of_row[row], p = positions[row];
  pdl_wait_for(qa, pages);
  float* mine = partial + (((size_t)row * num_heads + head0) * splits + split) * (rank + 2);
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  // tiles of 32 keys from a multiple of 32; this share's tiles
  const int first_tile = lo / 32, tiles = b < 0 ? 0 : p / 32 - first_tile + 1;
  const int per = (tiles + splits - 1) / splits;
  const int t_begin = first_tile + split * per, t_end = min(first_tile + tiles, t_begin + per);
  for (int idx = threadIdx.x; idx < heads_here * key_dim; idx += LD_WARPS * 32) {
    const int h = idx / key_dim, d = idx % key_dim;
    q_s[idx] = ldf(qa + (size_t)row * ld_qa + (size_t)(head0 + h) * key_dim + d) * scale;
  }
  const int* table = block_table + (size_t)max(b, 0) * table_stride;
  const int pieces = key_dim / PER16;
  auto stage = [&](int tile, int buffer) {
    T* at = tile_s + (size_t)buffer * 32 * row_elems;
    for (int idx = threadIdx.x; idx < 32 * pieces; idx += LD_WARPS * 32) {
      const int j = idx / pieces, c = idx % pieces, t = tile * 32 + j;
      T* to = at + (size_t)j * row_elems + c * PER16;
      if (t >= lo && t <= p) {
        const T* src = pages + ((size_t)table[t / page_size] * page_size + t % page_size) * key_dim;
        la_copy16(to, src + c * PER16);
      } else {  // a key out of sight: zeros, so that its weight of 0 meets no stale NaN
        *reinterpret_cast<uint4*>(to) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float m[LD_HEADS], l[LD_HEADS], acc[LD_HEADS][8];
#pragma unroll
  for (int u = 0; u < LD_HEADS; ++u) {
    m[u] = -INFINITY;
    l[u] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
  }
  if (t_begin < t_end) stage(t_begin, 0);
  for (int tile = t_begin; tile < t_end; ++tile) {
    const int buffer = (tile - t_begin) & 1;
    if (tile + 1 < t_end) {
      stage(tile + 1, buffer ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const T* at = tile_s + (size_t)buffer * 32 * row_elems;
    const int t = tile * 32 + lane;
    const bool valid = t >= lo && t <= p;
#pragma unroll
    for (int u = 0; u < LD_HEADS; ++u) {
      const int h = warp + LD_WARPS * u;
      if (h >= heads_here) break;
      const float* q = q_s + (size_t)h * key_dim;
      float score = -INFINITY;
      if (valid) {
        const T* key = at + (size_t)lane * row_elems;
        float dot[4] = {0.f, 0.f, 0.f, 0.f};  // four chains: the sum is not one long wait
#pragma unroll 4
        for (int d = 0; d < key_dim; d += 8) {
          float kv[8];
          Chunk8<T>::load(key + d, kv);
          const float4 qa0 = *reinterpret_cast<const float4*>(q + d);
          const float4 qa1 = *reinterpret_cast<const float4*>(q + d + 4);
          dot[0] = fmaf(qa0.x, kv[0], dot[0]); dot[1] = fmaf(qa0.y, kv[1], dot[1]);
          dot[2] = fmaf(qa0.z, kv[2], dot[2]); dot[3] = fmaf(qa0.w, kv[3], dot[3]);
          dot[0] = fmaf(qa1.x, kv[4], dot[0]); dot[1] = fmaf(qa1.y, kv[5], dot[1]);
          dot[2] = fmaf(qa1.z, kv[6], dot[2]); dot[3] = fmaf(qa1.w, kv[7], dot[3]);
        }
        score = (dot[0] + dot[1]) + (dot[2] + dot[3]);
      }
      const float m_new = fmaxf(m[u], warp_max(score));
      const float wgt = valid ? expf(score - m_new) : 0.f;
      const float corr = expf(m[u] - m_new);
      l[u] = l[u] * corr + warp_sum(wgt);
      m[u] = m_new;
      __syncwarp();
      w_s[warp][lane] = wgt;
      __syncwarp();
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[u][e] *= corr;
      if (lane * 8 < rank) {
#pragma unroll 8
        for (int j = 0; j < 32; ++j) {  // (rows out of sight are zeros with weight 0)
          const float wj = w_s[warp][j];
          float vv[8];
          Chunk8<T>::load(at + (size_t)j * row_elems + lane * 8, vv);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[u][e] = fmaf(wj, vv[e], acc[u][e]);
        }
      }
    }
    __syncthreads();  // the buffer is staged again at the next turn
  }
#pragma unroll
  for (int u = 0; u < LD_HEADS; ++u) {
    const int h = warp + LD_WARPS * u;
    if (h >= heads_here) break;
    float* to = mine + (size_t)h * splits * (rank + 2);
    if (lane == 0) {
      to[0] = m[u];
      to[1] = l[u];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (lane * 8 + e < rank) to[2 + lane * 8 + e] = acc[u][e];
    }
  }
}

constexpr int LD_MAX_SPLITS = 64;

template <typename T>
__global__ void latent_decode_merge_kernel(const float* __restrict__ partial,
                                           T* __restrict__ out, int ld_out, int out_head,
                                           int num_heads, int rank, int splits) {
  __shared__ float max_s[LD_MAX_SPLITS], weight_s[LD_MAX_SPLITS];
  pdl_launch_dependents();
  const int row = blockIdx.x, head = blockIdx.y;
  pdl_wait_for(partial);
  const float* from = partial + ((size_t)row * num_heads + head) * splits * (rank + 2);
  for (int s = threadIdx.x; s < splits; s += blockDim.x) {
    max_s[s] = from[(size_t)s * (rank + 2)];
    weight_s[s] = from[(size_t)s * (rank + 2) + 1];
  }
  __syncthreads();
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, max_s[s]);
  float l = 0.f;
  for (int s = 0; s < splits; ++s) {  // (a share without keys has sum 0 and maximum -inf)
    l += weight_s[s] > 0.f ? weight_s[s] * expf(max_s[s] - m) : 0.f;
  }
  __syncthreads();
  for (int s = threadIdx.x; s < splits; s += blockDim.x) {
    weight_s[s] = weight_s[s] > 0.f ? expf(max_s[s] - m) : 0.f;
  }
  __syncthreads();
  T* dst = out + (size_t)row * ld_out + (size_t)head * out_head;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float v = 0.f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) v = fmaf(from[(size_t)s * (rank + 2) + 2 + d], weight_s[s], v);
    stf(dst + d, l > 0.f ? v / l : 0.f);
  }
}

// ---------------------------------------------------------------------------------------------
// The same for bfloat16 on the warp-level tensor cores: the (up to) 16 heads of a request are
// the 16 rows of an mma.sync.m16n8k16 tile, so a tile of 32 latent rows is multiplied with all
// heads in 64 instructions (scores) and 2 x rank / 8 more (weighted sum) instead of being read
// once per head by the CUDA cores. A CTA of four warps takes one (row, share of keys, group
// of 16 heads); each warp walks every fourth tile of the share on its own (its own two
// buffers, filled by its own 16-byte asynchronous copies: no block barrier in the walk), keeps
// the heads' running maxima and sums and the [16 x rank] accumulator in registers, and the four
// warps' results are merged through shared memory into the share's (maximum, sum, weighted
// rows), which latent_decode_merge_kernel joins with the other shares'. Weights are rounded to
// bfloat16 as the A operand of the second product, like in the other tensor-core kernels.
// Rows of rank + rot entries, a multiple of 16 up to 320; rank up to 256.
constexpr int LM_WARPS = 4;
inline int& decode_tensor_cores() {
  static int enabled = 1;
  return enabled;
}

template <int NT16>  // the accumulator holds NT16 stretches of 16 entries: rank <= 16 * NT16
__global__ void __launch_bounds__(LM_WARPS * 32)
latent_decode_mma_kernel(const __nv_bfloat16* __restrict__ qa, int ld_qa,
                         const __nv_bfloat16* __restrict__ pages,
                         const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ request_of_row,
                         const int* __restrict__ positions, float* __restrict__ partial,
                         int num_heads, int rank, int key_dim, int page_size, float scale,
                         int window, int splits) {
  extern __shared__ __align__(16) unsigned char lm_smem[];
  const int stride = key_dim + 8;  // elements of a padded row (16 bytes more)
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(lm_smem);  // [16][stride]
  __nv_bfloat16* tiles_s = q_s + 16 * stride;                      // [warps][2][32][stride]
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int row = blockIdx.x, split = blockIdx.y, head0 = blockIdx.z * 16;
  const int heads_here = min(num_heads - head0, 16);
  const int b = request_of_row[row], p = positions[row];
  pdl_wait_for(qa, pages);
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int first_tile = lo / 32, tiles = b < 0 ? 0 : p / 32 - first_tile + 1;
  const int per = (tiles + splits - 1) / splits;
  const int t_begin = first_tile + split * per, t_end = min(first_tile + tiles, t_begin + per);
  const int pieces = key_dim / 8;
  for (int idx = threadIdx.x; idx < 16 * pieces; idx += LM_WARPS * 32) {
    const int h = idx / pieces, c = idx % pieces;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);  // heads beyond the model's are rows of zeros
    if (h < heads_here) {
      v = *reinterpret_cast<const uint4*>(qa + (size_t)row * ld_qa +
                                          (size_t)(head0 + h) * key_dim + c * 8);
    }
    *reinterpret_cast<uint4*>(q_s + (size_t)h * stride + c * 8) = v;
  }
  __syncthreads();
  const int* table = block_table + (size_t)max(b, 0) * table_stride;
  __nv_bfloat16* mine_s = tiles_s + (size_t)warp * 2 * 32 * stride;
  auto stage = [&](int tile, int buffer) {
    // key by key, the lanes side by side along the row: one request to memory brings 512
    // consecutive bytes (lane j fetching row j would scatter every request over 32 rows)
    // (lane j looks up where key j lies; the loop below asks it: a look-up inside the loop
    // would wait behind the copies, which no load may pass)
    const int t_mine = tile * 32 + lane;
    long long where = -1;
    if (t_mine >= lo && t_mine <= p) {
      where = ((long long)table[t_mine / page_size] * page_size + t_mine % page_size) * key_dim;
    }
#pragma unroll 4
    for (int j = 0; j < 32; ++j) {
      __nv_bfloat16* to = mine_s + ((size_t)buffer * 32 + j) * stride;
      const long long at = __shfl_sync(0xffffffffu, where, j);
      if (at >= 0) {
        const __nv_bfloat16* src = pages + at;
        for (int c = lane; c < pieces; c += 32) la_copy16(to + c * 8, src + c * 8);
      } else {
        for (int c = lane; c < pieces; c += 32) {
          *reinterpret_cast<uint4*>(to + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // heads g and g + 8
  float o[2 * NT16][4];
#pragma unroll
  for (int n = 0; n < 2 * NT16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  int turn = 0;
  if (t_begin + warp < t_end) stage(t_begin + warp, 0);
  for (int tile = t_begin + warp; tile < t_end; tile += LM_WARPS, ++turn) {
    const int buffer = turn & 1;
    if (tile + LM_WARPS < t_end) {
      stage(tile + LM_WARPS, buffer ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncwarp();
    const __nv_bfloat16* at = mine_s + (size_t)buffer * 32 * stride;
    // scores: [16 heads] x [32 keys], four stretches of 8 keys
    float sc[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
    for (int k0 = 0; k0 < key_dim; k0 += 16) {
      uint32_t a[4];
      a[0] = *reinterpret_cast<const uint32_t*>(q_s + (size_t)g * stride + k0 + 2 * t4);
      a[1] = *reinterpret_cast<const uint32_t*>(q_s + (size_t)(g + 8) * stride + k0 + 2 * t4);
      a[2] = *reinterpret_cast<const uint32_t*>(q_s + (size_t)g * stride + k0 + 8 + 2 * t4);
      a[3] = *reinterpret_cast<const uint32_t*>(q_s + (size_t)(g + 8) * stride + k0 + 8 + 2 * t4);
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const __nv_bfloat16* key = at + (size_t)(n * 8 + g) * stride + k0 + 2 * t4;
        lm_mma(sc[n], a, *reinterpret_cast<const uint32_t*>(key),
               *reinterpret_cast<const uint32_t*>(key + 8));
      }
    }
    // masks, running maxima and sums (a thread holds keys n * 8 + 2 t4 + {0, 1} of two heads)
    float top[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 4; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = tile * 32 + n * 8 + 2 * t4 + (e & 1);
        sc[n][e] = (t >= lo && t <= p) ? sc[n][e] * scale : -INFINITY;
        top[e >> 1] = fmaxf(top[e >> 1], sc[n][e]);
      }
    }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 1));
      top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 2));
      const float m_new = fmaxf(m_run[r], top[r]);  // (every tile holds a key in sight)
      corr[r] = expf(m_run[r] - m_new);
      m_run[r] = m_new;
      l_run[r] *= corr[r];
    }
    uint32_t pa[2][4];  // the weights as A operands: keys 0..15 and 16..31
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const float w0 = expf(sc[n][0] - m_run[0]), w1 = expf(sc[n][1] - m_run[0]);
      const float w2 = expf(sc[n][2] - m_run[1]), w3 = expf(sc[n][3] - m_run[1]);
      l_run[0] += w0 + w1;
      l_run[1] += w2 + w3;
      pa[n >> 1][(n & 1) * 2] = lm_pack(w0, w1);
      pa[n >> 1][(n & 1) * 2 + 1] = lm_pack(w2, w3);
    }
#pragma unroll
    for (int n = 0; n < 2 * NT16; ++n) {
      o[n][0] *= corr[0];
      o[n][1] *= corr[0];
      o[n][2] *= corr[1];
      o[n][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int c = 0; c < NT16; ++c) {
        if (c * 16 < key_dim) {
          uint32_t v[4];
          lm_ldmatrix_x4_trans(v, at + (size_t)(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) *
                                           stride + c * 16 + (lane >> 4) * 8);
          lm_mma(o[2 * c], pa[kk], v[0], v[1]);
          lm_mma(o[2 * c + 1], pa[kk], v[2], v[3]);
        }
      }
    }
    __syncwarp();  // the buffer is staged again at the next turn
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  // the four warps' results side by side in shared memory, then one (maximum, sum, rows)
  __syncthreads();
  const int width = 16 * NT16 + 2;
  float* merge_s = reinterpret_cast<float*>(tiles_s);  // [warps][16][width]
  {
    float* mine = merge_s + (size_t)warp * 16 * width;
    if (t4 == 0) {
      mine[(size_t)g * width] = m_run[0];
      mine[(size_t)g * width + 1] = l_run[0];
      mine[(size_t)(g + 8) * width] = m_run[1];
      mine[(size_t)(g + 8) * width + 1] = l_run[1];
    }
#pragma unroll
    for (int n = 0; n < 2 * NT16; ++n) {
      float* at = mine + 2 + n * 8 + 2 * t4;
      at[(size_t)g * width] = o[n][0];
      at[(size_t)g * width + 1] = o[n][1];
      at[(size_t)(g + 8) * width] = o[n][2];
      at[(size_t)(g + 8) * width + 1] = o[n][3];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < heads_here * (rank + 2); idx += LM_WARPS * 32) {
    const int h = idx / (rank + 2), d = idx % (rank + 2);
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < LM_WARPS; ++w) m = fmaxf(m, merge_s[((size_t)w * 16 + h) * width]);
    float value = 0.f;
    if (d == 0) {
      value = m;
    } else {
#pragma unroll
      for (int w = 0; w < LM_WARPS; ++w) {
        const float* from = merge_s + ((size_t)w * 16 + h) * width;
        if (from[1] > 0.f) value += from[d] * expf(from[0] - m);  // d = 1: the sum
      }
    }
    partial[(((size_t)row * num_heads + head0 + h) * splits + split) * (rank + 2) + d] = value;
  }
}

template <typename T>
int latent_attention(const void* qa, int ld_qa, const void* pages, const int* block_table,
                     int table_stride, const int* request_of_row, const int* positions, void* out,
                     int ld_out, int rows, int num_heads, int rank, int rot, int page_size,
                     float scale, int window, cudaStream_t stream) {
  const int key_dim = rank + rot;
  const int key_pad = (key_dim + 7) / 8 * 8;
  const int vector_ok =
      (key_dim % 8 == 0 && ((uintptr_t)pages % 16) == 0) ? 1 : 0;
  const size_t smem = (size_t)LA_WARPS * key_pad * sizeof(float);
  const dim3 grid(rows, (num_heads + LA_WARPS - 1) / LA_WARPS), block(LA_WARPS * 32);
#define AYK_LA(R)                                                                              \
  return launch_kernel(latent_attention_kernel<T, R>, grid, block, smem, stream, 1,            \
                       (const T*)qa, ld_qa, (const T*)pages, block_table, table_stride,        \
                       request_of_row, positions, (T*)out, ld_out, num_heads, rank, key_dim,   \
                       key_pad, page_size, scale, window, vector_ok)
  if (rank <= 64) AYK_LA(2);
  if (rank <= 128) AYK_LA(4);
  if (rank <= 256) AYK_LA(8);
  if (rank <= 512) AYK_LA(16);
  AYK_LA(32);
#undef AYK_LA
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// Whether single-row steps in bfloat16 may run on the warp-level tensor cores (the default) or
// stay on the CUDA-core kernel (tests of that kernel, measurements of one against the other).
AYK_API void ayk_set_latent_decode_tensor_cores(int on) { ayk::decode_tensor_cores() = on; }

// type: 0 = float32, 1 = bfloat16 (cache, queries). pages may be null (a run that reads a
// cache another run wrote) or a row's slot negative: nothing is stored then.
AYK_API int ayk_latent_prepare(const float* proj, int ld_proj, int kv_offset,
                               const float* latent_weight, float eps, const int* positions,
                               const int* slots, const double* freq, int rot_dims, int layout,
                               void* pages, void* q_plain, int ld_plain, void* qa, int ld_qa,
                               int rows, int heads, int dim, int rot, int rank, int type,
                               void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || heads < 1 || dim < 0 || rot < 0 || rank < 1 || rot_dims < 0 || rot_dims % 2 ||
      rot_dims > rot || kv_offset < heads * (dim + rot) || ld_proj < heads * (dim + rot) ||
      (pages != nullptr && ld_proj < kv_offset + rank + rot) ||
      ld_plain < heads * dim || ld_qa < heads * (rank + rot) || proj == nullptr ||
      latent_weight == nullptr || positions == nullptr || (rot_dims > 0 && freq == nullptr) ||
      q_plain == nullptr || qa == nullptr || !(eps > 0.f) ||
      (layout != ROPE_NEIGHBOURS && layout != ROPE_HALVES)) {
    return AYK_BAD_ARGUMENT;
  }
  if (rot_dims / 2 > ROPE_MAX_PAIRS) return AYK_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return launch_kernel(latent_prepare_kernel<float>, dim3(rows), dim3(256), 0, s, 1, proj,
                         ld_proj, kv_offset, latent_weight, eps, positions, slots, freq, rot_dims,
                         layout, (float*)pages, (float*)q_plain, ld_plain, (float*)qa, ld_qa,
                         heads, dim, rot, rank);
  }
  if (type == 1) {
    return launch_kernel(latent_prepare_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, s, 1,
                         proj, ld_proj, kv_offset, latent_weight, eps, positions, slots, freq,
                         rot_dims, layout, (__nv_bfloat16*)pages, (__nv_bfloat16*)q_plain,
                         ld_plain, (__nv_bfloat16*)qa, ld_qa, heads, dim, rot, rank);
  }
  return AYK_BAD_ARGUMENT;
}

AYK_API int ayk_head_linear(const void* a, int ld_a, int a_head, const void* w, long long w_head,
                            int w_in, int w_out, const float* gate, int ld_gate, void* out,
                            int ld_out, int out_head, int rows, int heads, int I, int J, int type,
                            void* stream) {
  using namespace ayk;
  if (rows == 0 || heads == 0 || J == 0) return AYK_OK;
  if (rows < 0 || heads < 0 || I < 1 || J < 0 || a == nullptr || w == nullptr || out == nullptr ||
      w_in < 1 || w_out < 1 || (w_in != 1 && w_out != 1) || heads > 65535) {
    return AYK_BAD_ARGUMENT;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return head_linear<float>(a, ld_a, a_head, w, w_head, w_in, w_out, gate, ld_gate, out, ld_out,
                              out_head, rows, heads, I, J, s);
  }
  if (type == 1) {
    return head_linear<__nv_bfloat16>(a, ld_a, a_head, w, w_head, w_in, w_out, gate, ld_gate, out,
                                      ld_out, out_head, rows, heads, I, J, s);
  }
  return AYK_BAD_ARGUMENT;
}

AYK_API int ayk_latent_attention(const void* qa, int ld_qa, const void* pages,
                                 const int* block_table, int table_stride,
                                 const int* request_of_row, const int* positions, void* out,
                                 int ld_out, int rows, int num_heads, int rank, int rot,
                                 int page_size, float scale, int window, int type, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || num_heads < 1 || rank < 1 || rot < 0 || page_size < 1 || window < 0 ||
      qa == nullptr || pages == nullptr || block_table == nullptr || request_of_row == nullptr ||
      positions == nullptr || out == nullptr || ld_qa < num_heads * (rank + rot) ||
      ld_out < num_heads * rank) {
    return AYK_BAD_ARGUMENT;
  }
  if (rank > 1024 || rank + rot > 2048 || num_heads > 65535 * ayk::LA_WARPS) return AYK_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return latent_attention<float>(qa, ld_qa, pages, block_table, table_stride, request_of_row,
                                   positions, out, ld_out, rows, num_heads, rank, rot, page_size,
                                   scale, window, s);
  }
  if (type == 1) {
    return latent_attention<__nv_bfloat16>(qa, ld_qa, pages, block_table, table_stride,
                                           request_of_row, positions, out, ld_out, rows, num_heads,
                                           rank, rot, page_size, scale, window, s);
  }
  return AYK_BAD_ARGUMENT;
}

// Attention over latent pages for steps of single rows, every head of a row in one CTA (see
// latent_decode_kernel). `partial`: rows * heads * splits * (rank + 2) floats of scratch.
// out rows hold the heads `out_head` entries apart. Refused (AYK_NOT_TAKEN, nothing ran) for
// sizes it does not take: rows of the cache that are no multiple of 8 entries or longer than
// 320, a rank over 256.
AYK_API int ayk_latent_decode(const void* qa, int ld_qa, const void* pages,
                              const int* block_table, int table_stride,
                              const int* request_of_row, const int* positions, float* partial,
                              void* out, int ld_out, int out_head, int rows, int num_heads,
                              int rank, int rot, int page_size, float scale, int window,
                              int splits, int type, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  const int key_dim = rank + rot;
  if (rows < 0 || num_heads < 1 || rank < 1 || rot < 0 || page_size < 1 || window < 0 ||
      splits < 1 || splits > LD_MAX_SPLITS || qa == nullptr || pages == nullptr ||
      block_table == nullptr || request_of_row == nullptr || positions == nullptr ||
      partial == nullptr || out == nullptr || ld_qa < num_heads * key_dim || out_head < rank ||
      (type != 0 && type != 1)) {
    return AYK_BAD_ARGUMENT;
  }
  if (key_dim % 8 || key_dim > 320 || rank > 256 || ((uintptr_t)pages % 16)) return AYK_NOT_TAKEN;
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 1 && key_dim % 16 == 0 && ld_qa % 8 == 0 && ((uintptr_t)qa % 16) == 0 &&
      decode_tensor_cores()) {
    const int stretches = rank <= 64 ? 4 : (rank <= 128 ? 8 : (rank <= 192 ? 12 : 16));
    const size_t walk = (size_t)LM_WARPS * 2 * 32 * (key_dim + 8) * 2;
    const size_t merge = (size_t)LM_WARPS * 16 * (16 * stretches + 2) * sizeof(float);
    const size_t bytes = (size_t)16 * (key_dim + 8) * 2 + (walk > merge ? walk : merge);
    const dim3 mma_grid(rows, splits, (num_heads + 15) / 16);
    int status = AYK_OK;
#define AYK_LM(NT16)                                                                           \
  {                                                                                            \
    static const bool allowed =                                                                \
        (cudaFuncSetAttribute(latent_decode_mma_kernel<NT16>,                                  \
                              cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), true); \
    (void)allowed;                                                                             \
    status = launch_kernel(latent_decode_mma_kernel<NT16>, mma_grid, dim3(LM_WARPS * 32),      \
                           bytes, s, 1, (const __nv_bfloat16*)qa, ld_qa,                       \
                           (const __nv_bfloat16*)pages, block_table, table_stride,             \
                           request_of_row, positions, partial, num_heads, rank, key_dim,       \
                           page_size, scale, window, splits);                                  \
  }
    if (rank <= 64) AYK_LM(4)
    else if (rank <= 128) AYK_LM(8)
    else if (rank <= 192) AYK_LM(12)
    else AYK_LM(16)
#undef AYK_LM
    if (status != AYK_OK) return status;
    return launch_kernel(latent_decode_merge_kernel<__nv_bfloat16>, dim3(rows, num_heads),
                         dim3(128), 0, s, 1, (const float*)partial, (__nv_bfloat16*)out, ld_out,
                         out_head, num_heads, rank, splits);
  }
  const int elem = type == 0 ? 4 : 2;
  const int group = LD_WARPS * LD_HEADS;
  const size_t smem = (size_t)2 * 32 * (key_dim + 16 / elem) * elem +
                      (size_t)(num_heads < group ? num_heads : group) * key_dim * sizeof(float);
  const dim3 grid(rows, splits, (num_heads + group - 1) / group);
  int status;
  if (type == 0) {
    static const bool allowed = (cudaFuncSetAttribute(
        latent_decode_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024), true);
    (void)allowed;
    status = launch_kernel(latent_decode_kernel<float>, grid, dim3(LD_WARPS * 32), smem, s, 1,
                           (const float*)qa, ld_qa, (const float*)pages, block_table,
                           table_stride, request_of_row, positions, partial, num_heads, rank,
                           key_dim, page_size, scale, window, splits);
    if (status != AYK_OK) return status;
    return launch_kernel(latent_decode_merge_kernel<float>, dim3(rows, num_heads), dim3(128), 0,
                         s, 1, (const float*)partial, (float*)out, ld_out, out_head, num_heads,
                         rank, splits);
  }
  static const bool allowed = (cudaFuncSetAttribute(
      latent_decode_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
      160 * 1024), true);
  (void)allowed;
  status = launch_kernel(latent_decode_kernel<__nv_bfloat16>, grid, dim3(LD_WARPS * 32), smem, s,
                         1, (const __nv_bfloat16*)qa, ld_qa, (const __nv_bfloat16*)pages,
                         block_table, table_stride, request_of_row, positions, partial, num_heads,
                         rank, key_dim, page_size, scale, window, splits);
  if (status != AYK_OK) return status;
  return launch_kernel(latent_decode_merge_kernel<__nv_bfloat16>, dim3(rows, num_heads),
                       dim3(128), 0, s, 1, (const float*)partial, (__nv_bfloat16*)out, ld_out,
                       out_head, num_heads, rank, splits);
}
