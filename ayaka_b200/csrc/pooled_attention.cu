// Softmax attention over paged keys with a sliding window, pooled blocks behind the window,
// and a sink in the softmax.
//
// The query at position p of a request sees the keys j with 0 <= p - j < window (window 0:
// every earlier key, and nothing is pooled). With `pool` = P > 0 it also sees, as one key and
// one value each, the blocks of P positions that lie wholly behind its window: block e holds
// the positions e P .. e P + P - 1 and is seen when e P + P - 1 <= p - window, that is
// e < (p - window + 1) / P. A block's key is the mean of its P cached keys (as the cache
// holds them: normed, rotated, rounded), its value the mean of its P cached values. Keys and
// blocks share one softmax, whose denominator also holds exp(sink[h]) when a sink is given:
// an entry without key or value, not scaled, counted once. Head h reads key/value head
// h / (H / G).
//
// The pooled rows live beside the pages, under the same page numbers: a page of `page_size`
// tokens has ceil(page_size / P) pooled slots, and block e lies in the page that holds its
// first position e P, at slot (e P % page_size) / P (two blocks that start in one page start
// at least P apart, so their slots differ).
//
// prepare (one launch per layer): from a row of the fused projection in fp32, queries at
// column 0 (H * dim) and keys at k_off (G * dim): each head is divided by its own root mean
// square (eps inside the root) and multiplied by one weight of `dim` entries that all heads
// share; the first `rot_dims` entries of each head are rotated by the row's position (entry i
// pairs with entry i + rot_dims / 2; cosine and sine times `rot_gain`); queries go to `q` in
// the compute type, keys into the row's cache slot. Where value pages are given, a token's
// value is its key as projected, before norm and rotation.
// blocks (one launch per layer, after prepare): the means of every block whose last position
// is among the step's rows.
// attention: one CTA per (row, head) on the CUDA cores, any sizes, both types; steps of
// single rows cut a row's visible entries into shares (further down). The visible entries
// are numbered blocks first, then the window's keys, and walked in that order in tiles that
// start at entry 0: what a row computes depends on its position alone.
#include "common.cuh"
#include "rope.cuh"

namespace ayk {

constexpr int PA_THREADS = 128;
constexpr int PA_MAX_VALUE = 4;  // value entries per thread of the generic kernel (vdim <= 512)

template <typename T>
__global__ void __launch_bounds__(256)
pooled_prepare_kernel(const float* __restrict__ proj, int ld_proj, int k_off,
                      const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                      float eps, const int* __restrict__ positions,
                      const double* __restrict__ freq, int rot_dims, float rot_gain,
                      const int* __restrict__ slots, T* __restrict__ k_pages,
                      T* __restrict__ v_pages, int page_size, T* __restrict__ q, int ld_q, int H,
                      int G, int dim) {
  __shared__ float cos_s[ROPE_MAX_PAIRS];
  __shared__ float sin_s[ROPE_MAX_PAIRS];
  pdl_launch_dependents();
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5, pairs = rot_dims / 2;
  const int slot = (slots != nullptr && k_pages != nullptr) ? slots[row] : -1;
  if (pairs > 0) rope_fill_table(cos_s, sin_s, positions[row], freq, pairs);
  pdl_wait_for(proj);
  __syncthreads();
  const size_t page = slot < 0 ? 0 : slot / page_size, at = slot < 0 ? 0 : slot % page_size;
  for (int hh = warp; hh < H + G; hh += warps) {
    const bool query = hh < H;
    const float* src = proj + (size_t)row * ld_proj + (query ? hh * dim : k_off + (hh - H) * dim);
    const float* w = query ? q_weight : k_weight;
    float ss = 0.f;
    for (int i = lane; i < dim; i += 32) ss = fmaf(src[i], src[i], ss);
    const float inv = w == nullptr ? 1.f : 1.f / sqrtf(warp_sum(ss) / (float)dim + eps);
    T* dst = nullptr;
    if (query) {
      dst = q + (size_t)row * ld_q + (size_t)hh * dim;
    } else if (slot >= 0) {
      dst = k_pages + ((page * G + (hh - H)) * page_size + at) * dim;
    }
    if (dst == nullptr) continue;
    for (int i = lane; i < pairs; i += 32) {
      const float a = src[i] * inv * (w != nullptr ? w[i] : 1.f);
      const float b = src[i + pairs] * inv * (w != nullptr ? w[i + pairs] : 1.f);
      const float c = cos_s[i] * rot_gain, s = sin_s[i] * rot_gain;
      stf(dst + i, a * c - b * s);
      stf(dst + i + pairs, b * c + a * s);
    }
    for (int i = 2 * pairs + lane; i < dim; i += 32) {
      stf(dst + i, src[i] * inv * (w != nullptr ? w[i] : 1.f));
    }
    if (!query && v_pages != nullptr) {  // the value: the key as projected
      T* v = v_pages + ((page * G + (hh - H)) * page_size + at) * dim;
      for (int i = lane; i < dim; i += 32) stf(v + i, src[i]);
    }
  }
}

// grid (candidates, G). A request whose rows of this step run from position p0 to p1 ends the
// blocks p0 / P .. (p1 + 1) / P - 1; the blocks that all requests end are numbered through, and
// CTA x takes the x-th of them (none: it leaves). The grid is an upper bound that depends on
// the step's numbers of rows and requests alone, so that a captured graph's launch holds for
// every step of its shape. A block's rows are summed in their order, four loads in flight.
template <typename T>
__global__ void __launch_bounds__(128)
pooled_blocks_kernel(const int* __restrict__ positions, const int* __restrict__ request_of_row,
                     const int* __restrict__ row_start, int requests,
                     const int* __restrict__ block_table, int ld_table,
                     const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                     T* __restrict__ k_pool, T* __restrict__ v_pool, int page_size, int pool,
                     int pool_slots, int G, int dim, int vdim) {
  pdl_launch_dependents();
  const int g = blockIdx.y;
  int left = blockIdx.x, b = 0, block = -1;
  for (; b < requests; ++b) {
    const int r0 = row_start[b], count = row_start[b + 1] - r0;
    if (count <= 0 || request_of_row[r0] < 0) continue;  // (a request of padding)
    const int p0 = positions[r0];
    const int ends = (p0 + count) / pool - p0 / pool;
    if (left < ends) {
      block = p0 / pool + left;
      break;
    }
    left -= ends;
  }
  pdl_wait_for(k_pages, v_pages);
  if (block < 0) return;
  const int first = block * pool;
  const int* table = block_table + (size_t)b * ld_table;
  const size_t to_page = table[first / page_size];
  const size_t to = (to_page * G + g) * pool_slots + (first % page_size) / pool;
  const float share = 1.f / (float)pool;
  for (int d = threadIdx.x; d < dim + vdim; d += blockDim.x) {
    const bool key = d < dim;
    const int c = key ? d : d - dim, width = key ? dim : vdim;
    const T* pages = (key ? k_pages : v_pages) + c;
    auto row_of = [&](int at) {
      const size_t page = table[at / page_size];
      return ldf(pages + ((page * G + g) * page_size + at % page_size) * width);
    };
    float sum = 0.f;
    int t = 0;
    for (; t + 4 <= pool; t += 4) {
      const float v0 = row_of(first + t), v1 = row_of(first + t + 1);
      const float v2 = row_of(first + t + 2), v3 = row_of(first + t + 3);
      sum += v0;
      sum += v1;
      sum += v2;
      sum += v3;
    }
    for (; t < pool; ++t) sum += row_of(first + t);
    stf((key ? k_pool : v_pool) + to * width + c, sum * share);
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

// What a row sees: `blocks` pooled entries, then the keys lo .. position.
struct Sight {
  int lo, blocks, total;
};
__device__ __forceinline__ Sight sight_of(int position, int window, int pool) {
  Sight s;
  s.lo = window > 0 ? max(0, position - window + 1) : 0;
  s.blocks = (window > 0 && pool > 0) ? s.lo / pool : 0;
  s.total = s.blocks + position - s.lo + 1;
  return s;
}
// Where entry j of a row's sight lies: a row index into the pages (>= 0) or, for a pooled
// entry, the bitwise complement of a row index into the pooled tensors (< 0).
__device__ __forceinline__ long long entry_base(int j, const Sight& s, const int* table, int G,
                                                int kv, int page_size, int pool,
                                                int pool_slots) {
  if (j < s.blocks) {
    const int first = j * pool;
    const long long page = table[first / page_size];
    return ~((page * G + kv) * pool_slots + (first % page_size) / pool);
  }
  const int at = s.lo + (j - s.blocks);
  const long long page = table[at / page_size];
  return (page * G + kv) * page_size + at % page_size;
}

// One CTA per (row, head). The visible entries are taken PA_THREADS at a time: a thread
// scores one entry, the CTA keeps a running maximum and sum, and thread c sums value entries
// c, c + PA_THREADS, ...
template <typename T>
__global__ void __launch_bounds__(PA_THREADS)
pooled_attention_kernel(const T* __restrict__ q, int ld_q, const T* __restrict__ k_pages,
                        const T* __restrict__ v_pages, const T* __restrict__ k_pool,
                        const T* __restrict__ v_pool, const int* __restrict__ block_table,
                        int ld_table, const int* __restrict__ request_of_row,
                        const int* __restrict__ positions, const float* __restrict__ sink,
                        T* __restrict__ out, int ld_out, int H, int G, int dim, int vdim,
                        int page_size, float scale, int window, int pool, int pool_slots) {
  extern __shared__ __align__(16) float pa_smem[];
  __shared__ float scratch[33];
  __shared__ float p_s[PA_THREADS];
  __shared__ long long base_s[PA_THREADS];
  pdl_launch_dependents();
  const int row = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  float* qv = pa_smem;  // dim
  const int b = request_of_row[row];
  T* dst = out + (size_t)row * ld_out + (size_t)h * vdim;
  pdl_wait_for(q, k_pages, v_pages, k_pool, v_pool);
  if (b < 0) {  // a row of padding
    for (int c = tid; c < vdim; c += PA_THREADS) stf(dst + c, 0.f);
    return;
  }
  const Sight see = sight_of(positions[row], window, pool);
  const int kv = h / (H / G);
  const int* table = block_table + (size_t)b * ld_table;
  for (int i = tid; i < dim; i += PA_THREADS) {
    qv[i] = ldf(q + (size_t)row * ld_q + (size_t)h * dim + i);
  }
  __syncthreads();
  float m_run = -INFINITY, l_run = 0.f;
  float acc[PA_MAX_VALUE] = {};
  for (int j0 = 0; j0 < see.total; j0 += PA_THREADS) {
    const int j = j0 + tid;
    float score = -INFINITY;
    if (j < see.total) {
      const long long base = entry_base(j, see, table, G, kv, page_size, pool, pool_slots);
      base_s[tid] = base;
      score = (base < 0 ? dot_row(qv, k_pool + (~base) * dim, dim)
                        : dot_row(qv, k_pages + base * dim, dim)) * scale;
    }
    float best = warp_max(score);
    __syncthreads();
    if ((tid & 31) == 0) scratch[tid >> 5] = best;
    __syncthreads();
    best = scratch[0];
    for (int w = 1; w < PA_THREADS / 32; ++w) best = fmaxf(best, scratch[w]);
    const float m_new = fmaxf(m_run, best);  // (finite: a tile holds at least one entry)
    const float alpha = expf(m_run - m_new);
    const float e = j < see.total ? expf(score - m_new) : 0.f;
    p_s[tid] = e;
    const float tile_sum = block_sum(e, scratch);  // (its barriers also publish p_s, base_s)
    l_run = l_run * alpha + tile_sum;
    m_run = m_new;
    const int n = min(PA_THREADS, see.total - j0);
#pragma unroll
    for (int i = 0; i < PA_MAX_VALUE; ++i) {
      const int c = tid + i * PA_THREADS;
      if (c < vdim) {
        float sum = acc[i] * alpha;
        for (int jj = 0; jj < n; ++jj) {
          const long long base = base_s[jj];
          const float v = base < 0 ? ldf(v_pool + (~base) * vdim + c)
                                   : ldf(v_pages + base * vdim + c);
          sum = fmaf(p_s[jj], v, sum);
        }
        acc[i] = sum;
      }
    }
    __syncthreads();  // p_s and base_s are written again at the next turn
  }
  if (sink != nullptr) {  // one more entry of the denominator, without a value
    const float s = sink[h], m_new = fmaxf(m_run, s);
    const float alpha = expf(m_run - m_new);
    l_run = l_run * alpha + expf(s - m_new);
#pragma unroll
    for (int i = 0; i < PA_MAX_VALUE; ++i) acc[i] *= alpha;
  }
#pragma unroll
  for (int i = 0; i < PA_MAX_VALUE; ++i) {
    const int c = tid + i * PA_THREADS;
    if (c < vdim) stf(dst + c, acc[i] / l_run);
  }
}

// ---- single rows: the visible entries cut into shares ---------------------------------------
// grid = (shares, heads, rows); the row's visible entries, numbered as above, are cut into
// `shares` contiguous shares of ceil(total / shares). A thread scores one entry of a tile of
// PA_THREADS; for the weighted sum the threads form vdim / VEC columns of 16-byte pieces
// times PA_THREADS / columns groups of entries, each thread with VEC running sums, which are
// added up over the groups once, at the end, in the groups' order. With one share the CTA
// finishes the row itself; otherwise it leaves (maximum, sum, weighted values) in `partial`
// ([row][head][share][vdim + 2] floats) and pooled_merge_kernel joins the shares in their
// order and adds the sink. Sizes: vdim a multiple of VEC (4 floats, 8 bfloat16) with at most
// PA_THREADS pieces.
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
__global__ void __launch_bounds__(PA_THREADS)
pooled_decode_kernel(const T* __restrict__ q, int ld_q, const T* __restrict__ k_pages,
                     const T* __restrict__ v_pages, const T* __restrict__ k_pool,
                     const T* __restrict__ v_pool, const int* __restrict__ block_table,
                     int ld_table, const int* __restrict__ request_of_row,
                     const int* __restrict__ positions, const float* __restrict__ sink,
                     float* __restrict__ partial, T* __restrict__ out, int ld_out, int H, int G,
                     int dim, int vdim, int page_size, float scale, int window, int pool,
                     int pool_slots) {
  constexpr int VEC = Piece<T>::N;
  extern __shared__ __align__(16) float pa_smem[];
  __shared__ float scratch[33];
  __shared__ float p_s[PA_THREADS];
  __shared__ long long base_s[PA_THREADS];
  pdl_launch_dependents();
  const int share = blockIdx.x, shares = gridDim.x, h = blockIdx.y, row = blockIdx.z;
  const int tid = threadIdx.x;
  float* qv = pa_smem;         // dim
  float* sums = pa_smem + dim;  // [groups][vdim]
  const int columns = vdim / VEC, groups = PA_THREADS / columns;
  const int column = tid % columns, group = tid / columns;  // (group >= groups: idle)
  const int b = request_of_row[row];
  T* dst = out + (size_t)row * ld_out + (size_t)h * vdim;
  float* part = partial + (((size_t)row * H + h) * shares + share) * (vdim + 2);
  int first = 0, last = 0;
  Sight see = {0, 0, 0};
  if (b >= 0) {
    see = sight_of(positions[row], window, pool);
    const int each = (see.total + shares - 1) / shares;
    first = min(see.total, share * each);
    last = min(see.total, first + each);
  }
  pdl_wait_for(q, k_pages, v_pages, k_pool, v_pool);
  if (first == last) {  // a row of padding, or a share without entries
    if (shares == 1) {
      for (int c = tid; c < vdim; c += PA_THREADS) stf(dst + c, 0.f);
    } else {
      for (int c = tid; c < vdim + 2; c += PA_THREADS) part[c] = c == 0 ? -INFINITY : 0.f;
    }
    return;
  }
  const int kv = h / (H / G);
  const int* table = block_table + (size_t)b * ld_table;
  for (int i = tid; i < dim; i += PA_THREADS) {
    qv[i] = ldf(q + (size_t)row * ld_q + (size_t)h * dim + i);
  }
  __syncthreads();
  float m_run = -INFINITY, l_run = 0.f;
  float acc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
  for (int j0 = first; j0 < last; j0 += PA_THREADS) {
    const int j = j0 + tid;
    float score = -INFINITY;
    if (j < last) {
      const long long base = entry_base(j, see, table, G, kv, page_size, pool, pool_slots);
      base_s[tid] = base;
      score = (base < 0 ? dot_row(qv, k_pool + (~base) * dim, dim)
                        : dot_row(qv, k_pages + base * dim, dim)) * scale;
    }
    float best = warp_max(score);
    __syncthreads();
    if ((tid & 31) == 0) scratch[tid >> 5] = best;
    __syncthreads();
    best = scratch[0];
    for (int w = 1; w < PA_THREADS / 32; ++w) best = fmaxf(best, scratch[w]);
    const float m_new = fmaxf(m_run, best);  // (finite: a tile holds at least one entry)
    const float alpha = expf(m_run - m_new);
    const float e = j < last ? expf(score - m_new) : 0.f;
    p_s[tid] = e;
    const float tile_sum = block_sum(e, scratch);  // (its barriers also publish p_s, base_s)
    l_run = l_run * alpha + tile_sum;
    m_run = m_new;
    const int n = min(PA_THREADS, last - j0);
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] *= alpha;
    if (group < groups) {
      for (int jj = group; jj < n; jj += groups) {
        float v[VEC];
        const long long base = base_s[jj];
        Piece<T>::load(base < 0 ? v_pool + (~base) * vdim + column * VEC
                                : v_pages + base * vdim + column * VEC, v);
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
  float scale_out = 1.f;
  if (shares == 1) {
    if (sink != nullptr) {
      const float s = sink[h], m_new = fmaxf(m_run, s);
      const float alpha = expf(m_run - m_new);
      l_run = l_run * alpha + expf(s - m_new);
      scale_out = alpha;
    }
    scale_out /= l_run;
  }
  for (int c = tid; c < vdim; c += PA_THREADS) {
    float v = 0.f;
    for (int g = 0; g < groups; ++g) v += sums[g * vdim + c];
    if (shares == 1) {
      stf(dst + c, v * scale_out);
    } else {
      part[2 + c] = v;
    }
  }
  if (shares > 1 && tid == 0) {
    part[0] = m_run;
    part[1] = l_run;
  }
}

// One CTA per (row, head): the shares' results joined in the shares' order, then the sink.
template <typename T>
__global__ void __launch_bounds__(PA_THREADS)
pooled_merge_kernel(const float* __restrict__ partial, int shares,
                    const float* __restrict__ sink, T* __restrict__ out, int ld_out, int H,
                    int vdim) {
  pdl_launch_dependents();
  const int row = blockIdx.x, h = blockIdx.y;
  pdl_wait_for(partial);
  const float* part = partial + ((size_t)row * H + h) * shares * (vdim + 2);
  float m = -INFINITY;
  for (int s = 0; s < shares; ++s) m = fmaxf(m, part[(size_t)s * (vdim + 2)]);
  const bool any = m > -INFINITY;  // (a row of padding has no entries)
  if (sink != nullptr && any) m = fmaxf(m, sink[h]);
  float l = 0.f;
  for (int s = 0; s < shares; ++s) {
    const float ms = part[(size_t)s * (vdim + 2)];
    if (ms > -INFINITY) l += part[(size_t)s * (vdim + 2) + 1] * expf(ms - m);
  }
  if (sink != nullptr && any) l += expf(sink[h] - m);
  for (int c = threadIdx.x; c < vdim; c += PA_THREADS) {
    float v = 0.f;
    for (int s = 0; s < shares; ++s) {
      const float ms = part[(size_t)s * (vdim + 2)];
      if (ms > -INFINITY) v += part[(size_t)s * (vdim + 2) + 2 + c] * expf(ms - m);
    }
    stf(out + (size_t)row * ld_out + (size_t)h * vdim + c, l > 0.f ? v / l : 0.f);
  }
}

template <typename T>
int pooled_prepare(const float* proj, int ld_proj, int k_off, const float* q_weight,
                   const float* k_weight, float eps, const int* positions, const double* freq,
                   int rot_dims, float rot_gain, const int* slots, void* k_pages, void* v_pages,
                   int page_size, void* q, int ld_q, int rows, int H, int G, int dim,
                   cudaStream_t s) {
  return launch_kernel(pooled_prepare_kernel<T>, dim3(rows), dim3(256), 0, s, 1, proj, ld_proj,
                       k_off, q_weight, k_weight, eps, positions, freq, rot_dims, rot_gain,
                       slots, (T*)k_pages, (T*)v_pages, page_size, (T*)q, ld_q, H, G, dim);
}

template <typename T>
int pooled_blocks(const int* positions, const int* request_of_row, const int* row_start,
                  int requests, const int* block_table, int ld_table, const void* k_pages,
                  const void* v_pages, void* k_pool, void* v_pool, int page_size, int pool,
                  int pool_slots, int rows, int G, int dim, int vdim, cudaStream_t s) {
  // blocks a step of `rows` rows in `requests` requests can end, at most
  const int most = min(rows, rows / pool + requests);
  return launch_kernel(pooled_blocks_kernel<T>, dim3(most, G), dim3(128), 0, s, 1, positions,
                       request_of_row, row_start, requests, block_table, ld_table,
                       (const T*)k_pages, (const T*)v_pages, (T*)k_pool, (T*)v_pool, page_size,
                       pool, pool_slots, G, dim, vdim);
}

template <typename T>
int pooled_attention(const void* q, int ld_q, const void* k_pages, const void* v_pages,
                     const void* k_pool, const void* v_pool, const int* block_table,
                     int ld_table, const int* request_of_row, const int* positions,
                     const float* sink, float* partial, void* out, int ld_out, int rows, int H,
                     int G, int dim, int vdim, int page_size, float scale, int window, int pool,
                     int pool_slots, int shares, cudaStream_t s) {
  if (shares == 0) {
    return launch_kernel(pooled_attention_kernel<T>, dim3(rows, H), dim3(PA_THREADS),
                         (size_t)dim * sizeof(float), s, 1, (const T*)q, ld_q,
                         (const T*)k_pages, (const T*)v_pages, (const T*)k_pool,
                         (const T*)v_pool, block_table, ld_table, request_of_row, positions,
                         sink, (T*)out, ld_out, H, G, dim, vdim, page_size, scale, window, pool,
                         pool_slots);
  }
  const int columns = vdim / Piece<T>::N;
  const size_t smem = ((size_t)dim + (size_t)(PA_THREADS / columns) * vdim) * sizeof(float);
  int status = launch_kernel(
      pooled_decode_kernel<T>, dim3(shares, H, rows), dim3(PA_THREADS), smem, s, 1, (const T*)q,
      ld_q, (const T*)k_pages, (const T*)v_pages, (const T*)k_pool, (const T*)v_pool,
      block_table, ld_table, request_of_row, positions, sink, partial, (T*)out, ld_out, H, G,
      dim, vdim, page_size, scale, window, pool, pool_slots);
  if (status != AYK_OK || shares == 1) return status;
  return launch_kernel(pooled_merge_kernel<T>, dim3(rows, H), dim3(PA_THREADS), 0, s, 1,
                       (const float*)partial, shares, sink, (T*)out, ld_out, H, vdim);
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// type: 0 = float32, 1 = bfloat16 (of q and the pages). Norm weights, slots and pages may be
// null (no norm; nothing stored); v_pages null: values are stored by someone else. `freq`:
// rot_dims / 2 doubles (null with rot_dims 0).
AYK_API int ayk_pooled_prepare(const float* proj, int ld_proj, int k_off, const float* q_weight,
                               const float* k_weight, float eps, const int* positions,
                               const double* freq, int rot_dims, float rot_gain,
                               const int* slots, void* k_pages, void* v_pages, int page_size,
                               void* q, int ld_q, int rows, int heads, int kv_heads, int dim,
                               int type, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || heads < 1 || kv_heads < 1 || heads % kv_heads || dim < 1 || proj == nullptr ||
      q == nullptr || ld_q < heads * dim || k_off < heads * dim ||
      ld_proj < k_off + kv_heads * dim || (q_weight == nullptr) != (k_weight == nullptr) ||
      rot_dims < 0 || rot_dims % 2 || rot_dims > dim || (rot_dims > 0 && freq == nullptr) ||
      positions == nullptr || (k_pages != nullptr && (page_size < 1 || slots == nullptr)) ||
      (k_pages == nullptr && v_pages != nullptr) || !(eps > 0.f)) {
    return AYK_BAD_ARGUMENT;
  }
  if (rot_dims / 2 > ROPE_MAX_PAIRS) return AYK_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return pooled_prepare<float>(proj, ld_proj, k_off, q_weight, k_weight, eps, positions, freq,
                                 rot_dims, rot_gain, slots, k_pages, v_pages, page_size, q, ld_q,
                                 rows, heads, kv_heads, dim, s);
  }
  if (type == 1) {
    return pooled_prepare<__nv_bfloat16>(proj, ld_proj, k_off, q_weight, k_weight, eps,
                                         positions, freq, rot_dims, rot_gain, slots, k_pages,
                                         v_pages, page_size, q, ld_q, rows, heads, kv_heads, dim,
                                         s);
  }
  return AYK_BAD_ARGUMENT;
}

// The means of the blocks that end in this step. pool_slots = ceil(page_size / pool).
AYK_API int ayk_pooled_blocks(const int* positions, const int* request_of_row,
                              const int* row_start, int requests, const int* block_table,
                              int ld_table, const void* k_pages, const void* v_pages,
                              void* k_pool, void* v_pool, int page_size, int pool,
                              int pool_slots, int rows, int kv_heads, int dim, int vdim, int type,
                              void* stream) {
  using namespace ayk;
  if (rows == 0 || requests == 0) return AYK_OK;
  if (rows < 0 || requests < 0 || row_start == nullptr || kv_heads < 1 || dim < 1 || vdim < 1 ||
      page_size < 1 || pool < 1 ||
      pool_slots != (page_size + pool - 1) / pool || positions == nullptr ||
      request_of_row == nullptr || block_table == nullptr || k_pages == nullptr ||
      v_pages == nullptr || k_pool == nullptr || v_pool == nullptr || kv_heads > 65535) {
    return AYK_BAD_ARGUMENT;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return pooled_blocks<float>(positions, request_of_row, row_start, requests, block_table,
                                ld_table, k_pages, v_pages, k_pool, v_pool, page_size, pool,
                                pool_slots, rows, kv_heads, dim, vdim, s);
  }
  if (type == 1) {
    return pooled_blocks<__nv_bfloat16>(positions, request_of_row, row_start, requests,
                                        block_table, ld_table, k_pages, v_pages, k_pool, v_pool,
                                        page_size, pool, pool_slots, rows, kv_heads, dim, vdim,
                                        s);
  }
  return AYK_BAD_ARGUMENT;
}

// shares 0: the generic kernel (any sizes). shares >= 1: the kernel of single rows;
// `partial`: float32 scratch of rows * heads * shares * (vdim + 2) elements (not needed with
// one share); AYK_NOT_TAKEN, having run nothing, for value rows that are not whole 16-byte
// pieces. pool 0: no pooled blocks (the pooled tensors may be null).
AYK_API int ayk_pooled_attention(const void* q, int ld_q, const void* k_pages,
                                 const void* v_pages, const void* k_pool, const void* v_pool,
                                 const int* block_table, int ld_table, const int* request_of_row,
                                 const int* positions, const float* sink, float* partial,
                                 void* out, int ld_out, int rows, int heads, int kv_heads,
                                 int dim, int vdim, int page_size, float scale, int window,
                                 int pool, int pool_slots, int shares, int type, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || heads < 1 || kv_heads < 1 || heads % kv_heads || dim < 1 || vdim < 1 ||
      page_size < 1 || window < 0 || pool < 0 || shares < 0 || q == nullptr ||
      k_pages == nullptr || v_pages == nullptr || block_table == nullptr ||
      request_of_row == nullptr || positions == nullptr || out == nullptr ||
      ld_q < heads * dim || ld_out < heads * vdim || (shares > 1 && partial == nullptr) ||
      (pool > 0 && window > 0 && (k_pool == nullptr || v_pool == nullptr ||
                                  pool_slots != (page_size + pool - 1) / pool)) ||
      (type != 0 && type != 1)) {
    return AYK_BAD_ARGUMENT;
  }
  if (dim > 8192 || rows > 65535 || heads > 65535) return AYK_TOO_LARGE;
  if (shares == 0) {
    if (vdim > PA_THREADS * PA_MAX_VALUE) return AYK_TOO_LARGE;
  } else {
    const int piece = type == 0 ? 4 : 8;
    if (vdim % piece || vdim / piece > PA_THREADS) return AYK_NOT_TAKEN;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return pooled_attention<float>(q, ld_q, k_pages, v_pages, k_pool, v_pool, block_table,
                                   ld_table, request_of_row, positions, sink, partial, out,
                                   ld_out, rows, heads, kv_heads, dim, vdim, page_size, scale,
                                   window, pool, pool_slots, shares, s);
  }
  return pooled_attention<__nv_bfloat16>(q, ld_q, k_pages, v_pages, k_pool, v_pool, block_table,
                                         ld_table, request_of_row, positions, sink, partial, out,
                                         ld_out, rows, heads, kv_heads, dim, vdim, page_size,
                                         scale, window, pool, pool_slots, shares, s);
}
