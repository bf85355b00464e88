// Softmax attention over paged keys and values with grouped heads, a value size of its own,
// a sliding window that keeps the first tokens of the sequence in sight, and an output gate.
//
// The query at position p of a request sees key j when j <= p and (p - j < window or
// j < keep_first); window 0 means every earlier key. Kept tokens are ordinary keys at their
// true positions: only the mask knows of them. Head h reads key/value head h / (H / G).
//
// prepare (one launch per layer): from a row of the fused projection in fp32, queries at
// column 0 (H * dim), keys at k_off (G * dim), values at v_off (G * vdim): with norm weights
// the whole query projection and the whole key projection are each divided by their root mean
// square (one mean over all heads' entries, eps inside the root) and multiplied by a weight
// per entry; queries go to `q` in the compute type, the key and value into the row's cache
// slot (pages [page][kv head][slot][dim or vdim]).
//
// attention: scores scale * (q . k), softmax and the weighted sum in fp32, the result times
// sigmoid(gate) entry by entry when a gate (fp32, [row][H * vdim]) is given. The visible keys
// are walked in a fixed order, first the kept ones that the window has left behind, then the
// window, in tiles that start at the first visible key: what a row computes depends on its
// position alone, not on the step's other rows.
// One CTA per (row, head) on the CUDA cores, any sizes, both types: the kernel of float32
// portions and of odd sizes. Steps of single rows cut a row's keys into shares (further
// down). Prompt portions in bfloat16 run on the tensor cores in attention_prefill.cu, which
// takes the same mask, value size and gate.
#include "common.cuh"

namespace ayk {

constexpr int GA_THREADS = 128;
constexpr int GA_MAX_VALUE = 4;  // value entries per thread of the generic kernel (vdim <= 512)

template <typename T>
__global__ void __launch_bounds__(256)
gated_prepare_kernel(const float* __restrict__ proj, int ld_proj, int k_off, int v_off,
                     const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                     float eps, const int* __restrict__ slots, T* __restrict__ k_pages,
                     T* __restrict__ v_pages, int page_size, T* __restrict__ q, int ld_q, int H,
                     int G, int dim, int vdim) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int row = blockIdx.x, tid = threadIdx.x;
  const int qn = H * dim, kn = G * dim, vn = G * vdim;
  const int slot = (slots != nullptr && k_pages != nullptr) ? slots[row] : -1;
  pdl_wait_for(proj);
  const float* src = proj + (size_t)row * ld_proj;
  float q_inv = 1.f, k_inv = 1.f;
  if (q_weight != nullptr) {
    float s = 0.f;
    for (int i = tid; i < qn; i += blockDim.x) s += src[i] * src[i];
    q_inv = 1.f / sqrtf(block_sum(s, scratch) / (float)qn + eps);
  }
  if (k_weight != nullptr) {
    float s = 0.f;
    for (int i = tid; i < kn; i += blockDim.x) s += src[k_off + i] * src[k_off + i];
    k_inv = 1.f / sqrtf(block_sum(s, scratch) / (float)kn + eps);
  }
  T* q_row = q + (size_t)row * ld_q;
  for (int i = tid; i < qn; i += blockDim.x) {
    stf(q_row + i, src[i] * q_inv * (q_weight != nullptr ? q_weight[i] : 1.f));
  }
  if (slot < 0) return;
  const size_t page = slot / page_size, at = slot % page_size;
  for (int i = tid; i < kn; i += blockDim.x) {
    const int g = i / dim, d = i % dim;
    stf(k_pages + ((page * G + g) * page_size + at) * dim + d,
        src[k_off + i] * k_inv * (k_weight != nullptr ? k_weight[i] : 1.f));
  }
  for (int i = tid; i < vn; i += blockDim.x) {
    const int g = i / vdim, d = i % vdim;
    stf(v_pages + ((page * G + g) * page_size + at) * vdim + d, src[v_off + i]);
  }
}

// q . k over one key row, by 16-byte pieces where the row's size allows (rows of the pages
// then start on 16-byte boundaries).
__device__ __forceinline__ float dot_row(const float* q, const float* k, int dim) {
  float sum = 0.f;
  if (dim % 4 == 0) {
    for (int d = 0; d < dim; d += 4) {
      const float4 v = *reinterpret_cast<const float4*>(k + d);
      sum = fmaf(q[d], v.x, sum);
      sum = fmaf(q[d + 1], v.y, sum);
      sum = fmaf(q[d + 2], v.z, sum);
      sum = fmaf(q[d + 3], v.w, sum);
    }
  } else {
    for (int d = 0; d < dim; ++d) sum = fmaf(q[d], k[d], sum);
  }
  return sum;
}
__device__ __forceinline__ float dot_row(const float* q, const __nv_bfloat16* k, int dim) {
  float sum = 0.f;
  if (dim % 8 == 0) {
    for (int d = 0; d < dim; d += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
      const __nv_bfloat162* pair = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(pair[i]);
        sum = fmaf(q[d + 2 * i], v.x, sum);
        sum = fmaf(q[d + 2 * i + 1], v.y, sum);
      }
    }
  } else {
    for (int d = 0; d < dim; ++d) sum = fmaf(q[d], __bfloat162float(k[d]), sum);
  }
  return sum;
}

// One CTA per (row, head). The visible keys, numbered 0 .. total - 1 (kept ones first), are
// taken GA_THREADS at a time: a thread scores one key, the CTA keeps a running maximum and
// sum, and thread c sums value entries c, c + GA_THREADS, ...
template <typename T>
__global__ void __launch_bounds__(GA_THREADS)
gated_attention_kernel(const T* __restrict__ q, int ld_q, const T* __restrict__ k_pages,
                       const T* __restrict__ v_pages, const int* __restrict__ block_table,
                       int ld_table, const int* __restrict__ request_of_row,
                       const int* __restrict__ positions, const float* __restrict__ gate,
                       int ld_gate, T* __restrict__ out, int ld_out, int H, int G, int dim,
                       int vdim, int page_size, float scale, int window, int keep_first) {
  extern __shared__ __align__(16) float ga_smem[];
  __shared__ float scratch[33];
  __shared__ float p_s[GA_THREADS];
  __shared__ long long base_s[GA_THREADS];
  pdl_launch_dependents();
  const int row = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  float* qv = ga_smem;  // dim
  const int b = request_of_row[row];
  T* dst = out + (size_t)row * ld_out + (size_t)h * vdim;
  if (b < 0) {  // a row of padding
    for (int c = tid; c < vdim; c += GA_THREADS) stf(dst + c, 0.f);
    return;
  }
  const int position = positions[row];
  const int lo = window > 0 ? max(0, position - window + 1) : 0;
  const int kept = min(keep_first, lo);  // kept keys the window no longer covers
  const int total = kept + position - lo + 1;
  const int kv = h / (H / G);
  const int* table = block_table + (size_t)b * ld_table;
  pdl_wait_for(q, k_pages, v_pages, gate);
  for (int i = tid; i < dim; i += GA_THREADS) qv[i] = ldf(q + (size_t)row * ld_q + (size_t)h * dim + i);
  __syncthreads();
  float m_run = -INFINITY, l_run = 0.f;
  float acc[GA_MAX_VALUE] = {};
  for (int j0 = 0; j0 < total; j0 += GA_THREADS) {
    const int j = j0 + tid;
    float score = -INFINITY;
    if (j < total) {
      const int at = j < kept ? j : lo + (j - kept);
      const long long page = table[at / page_size];
      const long long base = (page * G + kv) * page_size + at % page_size;
      base_s[tid] = base;
      score = dot_row(qv, k_pages + base * dim, dim) * scale;
    }
    float best = warp_max(score);
    __syncthreads();
    if ((tid & 31) == 0) scratch[tid >> 5] = best;
    __syncthreads();
    best = scratch[0];
    for (int w = 1; w < GA_THREADS / 32; ++w) best = fmaxf(best, scratch[w]);
    const float m_new = fmaxf(m_run, best);  // (finite: a tile holds at least one key)
    const float alpha = expf(m_run - m_new);
    const float e = j < total ? expf(score - m_new) : 0.f;
    p_s[tid] = e;
    const float tile_sum = block_sum(e, scratch);  // (its barriers also publish p_s, base_s)
    l_run = l_run * alpha + tile_sum;
    m_run = m_new;
    const int n = min(GA_THREADS, total - j0);
#pragma unroll
    for (int i = 0; i < GA_MAX_VALUE; ++i) {
      const int c = tid + i * GA_THREADS;
      if (c < vdim) {
        float sum = acc[i] * alpha;
        for (int jj = 0; jj < n; ++jj) {
          sum = fmaf(p_s[jj], ldf(v_pages + base_s[jj] * vdim + c), sum);
        }
        acc[i] = sum;
      }
    }
    __syncthreads();  // p_s and base_s are written again at the next turn
  }
#pragma unroll
  for (int i = 0; i < GA_MAX_VALUE; ++i) {
    const int c = tid + i * GA_THREADS;
    if (c < vdim) {
      float v = acc[i] / l_run;
      if (gate != nullptr) v /= 1.f + expf(-gate[(size_t)row * ld_gate + (size_t)h * vdim + c]);
      stf(dst + c, v);
    }
  }
}

// ---- single rows: the visible keys cut into shares ------------------------------------------
// A decode step has one row per request and nothing to reuse: the more CTAs fetch keys at
// once, the better. grid = (shares, heads, rows); the row's visible keys, numbered as above,
// are cut into `shares` contiguous shares of ceil(total / shares). A thread scores one key of
// a tile of GA_THREADS; for the weighted sum the threads form vdim / VEC columns of 16-byte
// pieces times GA_THREADS / columns groups of keys, each thread with VEC running sums, which
// are added up over the groups once, at the end, in the groups' order. With one share the
// CTA finishes the row itself; otherwise it leaves (maximum, sum, weighted values) in
// `partial` ([row][head][share][vdim + 2] floats) and gated_merge_kernel joins the shares in
// their order. Sizes: vdim a multiple of VEC (4 floats, 8 bfloat16) with at most GA_THREADS
// pieces.
template <typename T> struct Piece;
template <> struct Piece<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  }
};
template <> struct Piece<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* pair = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(pair[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};

template <typename T>
__global__ void __launch_bounds__(GA_THREADS)
gated_decode_kernel(const T* __restrict__ q, int ld_q, const T* __restrict__ k_pages,
                    const T* __restrict__ v_pages, const int* __restrict__ block_table,
                    int ld_table, const int* __restrict__ request_of_row,
                    const int* __restrict__ positions, const float* __restrict__ gate,
                    int ld_gate, float* __restrict__ partial, T* __restrict__ out, int ld_out,
                    int H, int G, int dim, int vdim, int page_size, float scale, int window,
                    int keep_first) {
  constexpr int VEC = Piece<T>::N;
  extern __shared__ __align__(16) float ga_smem[];
  __shared__ float scratch[33];
  __shared__ float p_s[GA_THREADS];
  __shared__ long long base_s[GA_THREADS];
  pdl_launch_dependents();
  const int share = blockIdx.x, shares = gridDim.x, h = blockIdx.y, row = blockIdx.z;
  const int tid = threadIdx.x;
  float* qv = ga_smem;         // dim
  float* sums = ga_smem + dim;  // [groups][vdim]
  const int columns = vdim / VEC, groups = GA_THREADS / columns;
  const int column = tid % columns, group = tid / columns;  // (group >= groups: idle)
  const int b = request_of_row[row];
  T* dst = out + (size_t)row * ld_out + (size_t)h * vdim;
  float* part = partial + (((size_t)row * H + h) * shares + share) * (vdim + 2);
  int first = 0, last = 0, lo = 0, kept = 0;
  if (b >= 0) {
    const int position = positions[row];
    lo = window > 0 ? max(0, position - window + 1) : 0;
    kept = min(keep_first, lo);  // kept keys the window no longer covers
    const int total = kept + position - lo + 1;
    const int each = (total + shares - 1) / shares;
    first = min(total, share * each);
    last = min(total, first + each);
  }
  pdl_wait_for(q, k_pages, v_pages, gate);
  if (first == last) {  // a row of padding, or a share without keys
    if (shares == 1) {
      for (int c = tid; c < vdim; c += GA_THREADS) stf(dst + c, 0.f);
    } else {
      for (int c = tid; c < vdim + 2; c += GA_THREADS) part[c] = c == 0 ? -INFINITY : 0.f;
    }
    return;
  }
  const int kv = h / (H / G);
  const int* table = block_table + (size_t)b * ld_table;
  for (int i = tid; i < dim; i += GA_THREADS) qv[i] = ldf(q + (size_t)row * ld_q + (size_t)h * dim + i);
  __syncthreads();
  float m_run = -INFINITY, l_run = 0.f;
  float acc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
  for (int j0 = first; j0 < last; j0 += GA_THREADS) {
    const int j = j0 + tid;
    float score = -INFINITY;
    if (j < last) {
      const int at = j < kept ? j : lo + (j - kept);
      const long long page = table[at / page_size];
      const long long base = (page * G + kv) * page_size + at % page_size;
      base_s[tid] = base;
      score = dot_row(qv, k_pages + base * dim, dim) * scale;
    }
    float best = warp_max(score);
    __syncthreads();
    if ((tid & 31) == 0) scratch[tid >> 5] = best;
    __syncthreads();
    best = scratch[0];
    for (int w = 1; w < GA_THREADS / 32; ++w) best = fmaxf(best, scratch[w]);
    const float m_new = fmaxf(m_run, best);  // (finite: a tile holds at least one key)
    const float alpha = expf(m_run - m_new);
    const float e = j < last ? expf(score - m_new) : 0.f;
    p_s[tid] = e;
    const float tile_sum = block_sum(e, scratch);  // (its barriers also publish p_s, base_s)
    l_run = l_run * alpha + tile_sum;
    m_run = m_new;
    const int n = min(GA_THREADS, last - j0);
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] *= alpha;
    if (group < groups) {
      for (int jj = group; jj < n; jj += groups) {
        float v[VEC];
        Piece<T>::load(v_pages + base_s[jj] * vdim + column * VEC, v);
        const float p = p_s[jj];
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = fmaf(p, v[i], acc[i]);
      }
    }
    __syncthreads();  // p_s and base_s are written again at the next turn
  }
  if (group < groups) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) sums[group * vdim + column * VEC + i] = acc[i];
  }
  __syncthreads();
  for (int c = tid; c < vdim; c += GA_THREADS) {
    float v = 0.f;
    for (int g = 0; g < groups; ++g) v += sums[g * vdim + c];
    if (shares == 1) {
      v /= l_run;
      if (gate != nullptr) v /= 1.f + expf(-gate[(size_t)row * ld_gate + (size_t)h * vdim + c]);
      stf(dst + c, v);
    } else {
      part[2 + c] = v;
    }
  }
  if (shares > 1 && tid == 0) {
    part[0] = m_run;
    part[1] = l_run;
  }
}

// One CTA per (row, head): the shares' results joined in the shares' order.
template <typename T>
__global__ void __launch_bounds__(GA_THREADS)
gated_merge_kernel(const float* __restrict__ partial, int shares,
                   const float* __restrict__ gate, int ld_gate, T* __restrict__ out, int ld_out,
                   int H, int vdim) {
  pdl_launch_dependents();
  const int row = blockIdx.x, h = blockIdx.y;
  pdl_wait_for(partial, gate);
  const float* part = partial + ((size_t)row * H + h) * shares * (vdim + 2);
  float m = -INFINITY;
  for (int s = 0; s < shares; ++s) m = fmaxf(m, part[(size_t)s * (vdim + 2)]);
  float l = 0.f;
  for (int s = 0; s < shares; ++s) {
    const float ms = part[(size_t)s * (vdim + 2)];
    if (ms > -INFINITY) l += part[(size_t)s * (vdim + 2) + 1] * expf(ms - m);
  }
  for (int c = threadIdx.x; c < vdim; c += GA_THREADS) {
    float v = 0.f;
    for (int s = 0; s < shares; ++s) {
      const float ms = part[(size_t)s * (vdim + 2)];
      if (ms > -INFINITY) v += part[(size_t)s * (vdim + 2) + 2 + c] * expf(ms - m);
    }
    v = l > 0.f ? v / l : 0.f;  // (a row of padding has no keys)
    if (gate != nullptr) v /= 1.f + expf(-gate[(size_t)row * ld_gate + (size_t)h * vdim + c]);
    stf(out + (size_t)row * ld_out + (size_t)h * vdim + c, v);
  }
}

template <typename T>
int gated_decode(const void* q, int ld_q, const void* k_pages, const void* v_pages,
                 const int* block_table, int ld_table, const int* request_of_row,
                 const int* positions, const float* gate, int ld_gate, float* partial,
                 void* out, int ld_out, int rows, int H, int G, int dim, int vdim,
                 int page_size, float scale, int window, int keep_first, int shares,
                 cudaStream_t s) {
  const int columns = vdim / Piece<T>::N;
  const size_t smem = ((size_t)dim + (size_t)(GA_THREADS / columns) * vdim) * sizeof(float);
  int status = launch_kernel(
      gated_decode_kernel<T>, dim3(shares, H, rows), dim3(GA_THREADS), smem, s, 1, (const T*)q,
      ld_q, (const T*)k_pages, (const T*)v_pages, block_table, ld_table, request_of_row,
      positions, gate, ld_gate, partial, (T*)out, ld_out, H, G, dim, vdim, page_size, scale,
      window, keep_first);
  if (status != AYK_OK || shares == 1) return status;
  return launch_kernel(gated_merge_kernel<T>, dim3(rows, H), dim3(GA_THREADS), 0, s, 1,
                       (const float*)partial, shares, gate, ld_gate, (T*)out, ld_out, H, vdim);
}

template <typename T>
int gated_attention(const void* q, int ld_q, const void* k_pages, const void* v_pages,
                    const int* block_table, int ld_table, const int* request_of_row,
                    const int* positions, const float* gate, int ld_gate, void* out, int ld_out,
                    int rows, int H, int G, int dim, int vdim, int page_size, float scale,
                    int window, int keep_first, cudaStream_t s) {
  return launch_kernel(gated_attention_kernel<T>, dim3(rows, H), dim3(GA_THREADS),
                       (size_t)dim * sizeof(float), s, 1, (const T*)q, ld_q, (const T*)k_pages,
                       (const T*)v_pages, block_table, ld_table, request_of_row, positions, gate,
                       ld_gate, (T*)out, ld_out, H, G, dim, vdim, page_size, scale, window,
                       keep_first);
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// type: 0 = float32, 1 = bfloat16 (of q and the pages). Norm weights, slots and pages may be
// null (no norm; nothing stored).
AYK_API int ayk_gated_prepare(const float* proj, int ld_proj, int k_off, int v_off,
                              const float* q_weight, const float* k_weight, float eps,
                              const int* slots, void* k_pages, void* v_pages, int page_size,
                              void* q, int ld_q, int rows, int heads, int kv_heads, int dim,
                              int vdim, int type, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || heads < 1 || kv_heads < 1 || heads % kv_heads || dim < 1 || vdim < 1 ||
      proj == nullptr || q == nullptr || ld_q < heads * dim || k_off < heads * dim ||
      v_off < k_off + kv_heads * dim || ld_proj < v_off + kv_heads * vdim ||
      (k_pages == nullptr) != (v_pages == nullptr) || (k_pages != nullptr && page_size < 1) ||
      !(eps > 0.f)) {
    return AYK_BAD_ARGUMENT;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return launch_kernel(gated_prepare_kernel<float>, dim3(rows), dim3(256), 0, s, 1, proj,
                         ld_proj, k_off, v_off, q_weight, k_weight, eps, slots, (float*)k_pages,
                         (float*)v_pages, page_size, (float*)q, ld_q, heads, kv_heads, dim, vdim);
  }
  if (type == 1) {
    return launch_kernel(gated_prepare_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, s, 1,
                         proj, ld_proj, k_off, v_off, q_weight, k_weight, eps, slots,
                         (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, page_size,
                         (__nv_bfloat16*)q, ld_q, heads, kv_heads, dim, vdim);
  }
  return AYK_BAD_ARGUMENT;
}

// Steps of single rows. type as above. `partial`: float32 scratch of rows * heads * shares *
// (vdim + 2) elements (not needed with one share). AYK_NOT_TAKEN, having run nothing, for
// value rows that are not whole 16-byte pieces.
AYK_API int ayk_gated_decode(const void* q, int ld_q, const void* k_pages, const void* v_pages,
                             const int* block_table, int ld_table, const int* request_of_row,
                             const int* positions, const float* gate, int ld_gate,
                             float* partial, void* out, int ld_out, int rows, int heads,
                             int kv_heads, int dim, int vdim, int page_size, float scale,
                             int window, int keep_first, int shares, int type, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || heads < 1 || kv_heads < 1 || heads % kv_heads || dim < 1 || vdim < 1 ||
      page_size < 1 || window < 0 || keep_first < 0 || shares < 1 || q == nullptr ||
      k_pages == nullptr || v_pages == nullptr || block_table == nullptr ||
      request_of_row == nullptr || positions == nullptr || out == nullptr ||
      ld_q < heads * dim || ld_out < heads * vdim || (shares > 1 && partial == nullptr) ||
      (gate != nullptr && ld_gate < heads * vdim) || (type != 0 && type != 1)) {
    return AYK_BAD_ARGUMENT;
  }
  const int piece = type == 0 ? 4 : 8;
  if (vdim % piece || vdim / piece > GA_THREADS || dim > 8192 || rows > 65535 ||
      heads > 65535) {
    return AYK_NOT_TAKEN;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return gated_decode<float>(q, ld_q, k_pages, v_pages, block_table, ld_table,
                               request_of_row, positions, gate, ld_gate, partial, out, ld_out,
                               rows, heads, kv_heads, dim, vdim, page_size, scale, window,
                               keep_first, shares, s);
  }
  return gated_decode<__nv_bfloat16>(q, ld_q, k_pages, v_pages, block_table, ld_table,
                                     request_of_row, positions, gate, ld_gate, partial, out,
                                     ld_out, rows, heads, kv_heads, dim, vdim, page_size, scale,
                                     window, keep_first, shares, s);
}

// mode: 0 = the generic kernel; 1 = the tensor-core kernel where the sizes allow (bfloat16).
AYK_API int ayk_gated_attention(const void* q, int ld_q, const void* k_pages,
                                const void* v_pages, const int* block_table, int ld_table,
                                const int* request_of_row, const int* positions,
                                const float* gate, int ld_gate, void* out, int ld_out, int rows,
                                int heads, int kv_heads, int dim, int vdim, int page_size,
                                float scale, int window, int keep_first, int mode, int type,
                                void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || heads < 1 || kv_heads < 1 || heads % kv_heads || dim < 1 || vdim < 1 ||
      page_size < 1 || window < 0 || keep_first < 0 || q == nullptr || k_pages == nullptr ||
      v_pages == nullptr || block_table == nullptr || request_of_row == nullptr ||
      positions == nullptr || out == nullptr || ld_q < heads * dim || ld_out < heads * vdim ||
      (gate != nullptr && ld_gate < heads * vdim)) {
    return AYK_BAD_ARGUMENT;
  }
  if (vdim > GA_THREADS * GA_MAX_VALUE || dim > 8192) return AYK_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  (void)mode;
  if (type == 0) {
    return gated_attention<float>(q, ld_q, k_pages, v_pages, block_table, ld_table,
                                  request_of_row, positions, gate, ld_gate, out, ld_out, rows,
                                  heads, kv_heads, dim, vdim, page_size, scale, window,
                                  keep_first, s);
  }
  if (type == 1) {
    return gated_attention<__nv_bfloat16>(q, ld_q, k_pages, v_pages, block_table, ld_table,
                                          request_of_row, positions, gate, ld_gate, out, ld_out,
                                          rows, heads, kv_heads, dim, vdim, page_size, scale,
                                          window, keep_first, s);
  }
  return AYK_BAD_ARGUMENT;
}
