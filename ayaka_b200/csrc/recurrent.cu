// Layers with a running per-request state instead of cached keys: the short causal
// convolution and the selective state-space recurrence of a Mamba-2 layer, the matrix
// memory of an mLSTM layer, and a gated linear attention with a decay per key channel. A step brings each request's next rows (a prompt portion or one
// token); the state a request left behind is read from its slot, carried over the rows in
// order, and written back. Everything here is fp32.
//
// Both recurrences have the shape S_t = a_t S_(t-1) + b_t k_t v_t^T, y_t = S_t^T q_t with S
// [n x p] per head, so the p columns of S never mix: a CTA owns one (head, request, tile of
// SCAN_COLS columns); a column's n entries are spread over LANES neighbouring lanes (8, 16 or
// a whole warp, by the size of n: entry n on lane n % LANES, so that a thread holds at most
// 16 entries and a device has thousands of warps to run), which add up their shares of y with
// shuffles. A column is kept with its n entries side by side ([head][p][n]). (A thread may
// take CP neighbouring columns, fetching B, C or k, q once for them: with two, the mLSTM scan
// of 256 x 256 heads took 870 against 680 microseconds a layer at 2 x 1,024 rows, because a
// device then has half the warps; every launch uses one.) The
// rows are taken in chunks: the chunk's inputs are brought to shared memory by all threads
// (and the gates turned into factors there, one thread per row), then every thread walks the
// chunk row by row.
#include <initializer_list>

#include "common.cuh"

namespace ayk {

constexpr int SCAN_COLS = 16;   // columns of the state per CTA
constexpr int SCAN_MAX_N = 512;  // entries of a column: 32 lanes x 16
constexpr int CONV_MAX_TAPS = 16;
constexpr int SCAN_STAGES = 4;  // buffers of staged chunks: three travel while one is walked

template <int LANES> __device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = 1; o < LANES; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float softplus_f(float z) {  // log(1 + e^z), exact for any z
  return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
}
__device__ __forceinline__ float log_sigmoid_f(float z) {  // -log(1 + e^-z)
  return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// ---------------------------------------------------------------------------------------------
// out[r][c] = silu(bias[c] + sum_l w[c][taps - 1 - l] * u[t - l][c]), l = 0 .. taps - 1, where
// u[t - l] is a row of this step if the request has it in this step, else one of the last
// taps - 1 inputs kept in the request's state (conv[k] = the input taps - 1 - k rows before the
// step's first), zeros before the sequence's start.
__global__ void causal_conv_silu_kernel(const float* __restrict__ in, int ld_in,
                                        const float* __restrict__ w,
                                        const float* __restrict__ bias,
                                        const float* __restrict__ state, long long state_stride,
                                        const int* __restrict__ request_of_row,
                                        const int* __restrict__ row_start,
                                        const int* __restrict__ state_slot,
                                        float* __restrict__ out, int ld_out, int channels,
                                        int taps) {
  pdl_launch_dependents();
  const int c = blockIdx.y * blockDim.x + threadIdx.x, r = blockIdx.x;
  const int b = request_of_row[r];
  if (c >= channels || b < 0) return;
  const int j = r - row_start[b];
  const float* kept = state + (size_t)state_slot[b] * state_stride;
  float wv[CONV_MAX_TAPS];
#pragma unroll
  for (int l = 0; l < CONV_MAX_TAPS; ++l) wv[l] = l < taps ? w[(size_t)c * taps + taps - 1 - l] : 0.f;
  float acc = bias != nullptr ? bias[c] : 0.f;
  pdl_wait_for(in, kept);
#pragma unroll
  for (int l = 0; l < CONV_MAX_TAPS; ++l) {
    if (l < taps) {
      const float u = j - l >= 0 ? in[(size_t)(r - l) * ld_in + c]
                                 : kept[(size_t)(taps - 1 + j - l) * channels + c];
      acc = fmaf(wv[l], u, acc);
    }
  }
  out[(size_t)r * ld_out + c] = silu_f(acc);
}

// After the convolution has read it, the kept inputs move on: conv[k] <- the input
// taps - 1 - k rows before the row that follows this step.
__global__ void conv_state_update_kernel(const float* __restrict__ in, int ld_in,
                                         float* __restrict__ state, long long state_stride,
                                         const int* __restrict__ row_start,
                                         const int* __restrict__ state_slot, int channels,
                                         int taps) {
  pdl_launch_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (c >= channels) return;
  const int r0 = row_start[b], rows = row_start[b + 1] - r0;
  if (state_slot[b] < 0) return;  // a row of padding (a graph's bucket): no request, no state
  float* kept = state + (size_t)state_slot[b] * state_stride;
  pdl_wait_for(in, kept);
  float next[CONV_MAX_TAPS];
#pragma unroll
  for (int k = 0; k < CONV_MAX_TAPS - 1; ++k) {
    if (k < taps - 1) {
      const int j = rows - (taps - 1) + k;  // index among the step's rows
      next[k] = j >= 0 ? in[(size_t)(r0 + j) * ld_in + c] : kept[(size_t)(k + rows) * channels + c];
    }
  }
#pragma unroll
  for (int k = 0; k < CONV_MAX_TAPS - 1; ++k) {
    if (k < taps - 1) kept[(size_t)k * channels + c] = next[k];
  }
}

// ---------------------------------------------------------------------------------------------
// Staging of a chunk's inputs: asynchronous copies (16 bytes each where every address allows
// it, else 4), all in flight at once, into one of two buffers, so that the copies of chunk
// c + 1 travel while chunk c is walked.
__device__ __forceinline__ void copy_async(float* dst, const float* src, int floats) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  if (floats == 4) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
  } else {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
  }
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// rows x width floats from rows `ld` apart into a dense tile; vec = 4 or 1 floats per copy
__device__ __forceinline__ void stage_tile(float* dst, const float* src, long long ld, int rows,
                                           int width, int vec) {
  const int per_row = width / vec;
  for (int idx = threadIdx.x; idx < rows * per_row; idx += blockDim.x) {
    const int i = idx / per_row, j = (idx % per_row) * vec;
    copy_async(dst + (size_t)i * width + j, src + (size_t)i * ld + j, vec);
  }
}
// the CTA's SCAN_COLS columns (from column p0 of a head of P columns; zeros beyond P)
__device__ __forceinline__ void stage_columns(float* dst, const float* src, long long ld,
                                              int rows, int p0, int P, int vec) {
  const int per_row = SCAN_COLS / vec;
  for (int idx = threadIdx.x; idx < rows * per_row; idx += blockDim.x) {
    const int i = idx / per_row, j = (idx % per_row) * vec;
    float* to = dst + i * SCAN_COLS + j;
    if (p0 + j < P) {  // (with vec 4, P is a multiple of 4: a group is inside or outside)
      copy_async(to, src + (size_t)i * ld + p0 + j, vec);
    } else {
      for (int e = 0; e < vec; ++e) to[e] = 0.f;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Mamba-2: per head h (group g = h / (heads / groups)), dt = softplus(dt_raw + dt_bias),
//   S <- exp(-exp(A_log) dt) S + dt B x^T,   y = S^T C + D x,    S: [N x P].
// xbc rows: [ x: heads x P | B: groups x N | C: groups x N ] (after convolution and silu).
// State of a request's slot: S as [heads][P][N] from `state`.
template <int RN, int LANES, int CP>  // entries of a column per lane: N <= LANES * RN;
__global__ void __launch_bounds__(SCAN_COLS / CP * LANES)  // CP columns per thread
mamba2_scan_kernel(const float* __restrict__ xbc, int ld_xbc, const float* __restrict__ dt_raw,
                   int ld_dt, const float* __restrict__ dt_bias,
                   const float* __restrict__ a_log, const float* __restrict__ skip,
                   float* __restrict__ state, long long state_stride,
                   const int* __restrict__ row_start, const int* __restrict__ state_slot,
                   float* __restrict__ y, int ld_y, int heads, int groups, int N, int P,
                   int chunk, int vec) {
  extern __shared__ __align__(16) float scan_smem[];
  const int stage_floats = chunk * (2 * N + SCAN_COLS + 4);
  pdl_launch_dependents();
  const int h = blockIdx.x, b = blockIdx.y, p0 = blockIdx.z * SCAN_COLS;
  const int col = threadIdx.x / LANES * CP, part = threadIdx.x % LANES;  // first of CP columns
  const int p = p0 + col;
  const int g = h / (heads / groups), inner = heads * P;
  const int r0 = row_start[b], rows = row_start[b + 1] - r0;
  const float rate = -expf(a_log[h]), bias = dt_bias[h], d_skip = skip != nullptr ? skip[h] : 0.f;
  if (state_slot[b] < 0) return;  // a row of padding (a graph's bucket): no request, no state
  float* mine = state + (size_t)state_slot[b] * state_stride + (size_t)h * N * P;
  pdl_wait_for(xbc, dt_raw, mine);
  float s[CP][RN];
#pragma unroll
  for (int c = 0; c < CP; ++c) {
#pragma unroll
    for (int k = 0; k < RN; ++k) {
      const int n = part + LANES * k;
      s[c][k] = (p + c < P && n < N) ? mine[(size_t)(p + c) * N + n] : 0.f;
    }
  }
  const int chunks = (rows + chunk - 1) / chunk;
  auto stage = [&](int c) {
    float* at = scan_smem + (size_t)(c % SCAN_STAGES) * stage_floats;
    const int t0 = c * chunk, count = min(chunk, rows - t0);
    const float* first = xbc + (size_t)(r0 + t0) * ld_xbc;
    stage_tile(at, first + inner + g * N, ld_xbc, count, N, vec);                          // B
    stage_tile(at + (size_t)chunk * N, first + inner + (groups + g) * N, ld_xbc, count, N, vec);
    stage_columns(at + (size_t)2 * chunk * N, first + h * P, ld_xbc, count, p0, P, vec);   // x
    for (int i = threadIdx.x; i < count; i += blockDim.x) {                              // dt
      copy_async(at + 2 * chunk * N + chunk * SCAN_COLS + i,
                 dt_raw + (size_t)(r0 + t0 + i) * ld_dt + h, 1);
    }
    copy_commit();
  };
  for (int c = 0; c < SCAN_STAGES - 1; ++c) {
    if (c < chunks) stage(c); else copy_commit();
  }
  for (int c = 0; c < chunks; ++c) {
    // (one group per turn, staged or empty, so that the count of groups in flight says
    // which chunk has landed)
    if (c + SCAN_STAGES - 1 < chunks) stage(c + SCAN_STAGES - 1); else copy_commit();
    copy_wait<SCAN_STAGES - 1>();
    __syncthreads();
    float* b_s = scan_smem + (size_t)(c % SCAN_STAGES) * stage_floats;
    float* c_s = b_s + (size_t)chunk * N;
    float* x_s = c_s + (size_t)chunk * N;
    float* dt_s = x_s + chunk * SCAN_COLS;   // raw, then the step size
    float* decay_s = dt_s + chunk;
    const int t0 = c * chunk, count = min(chunk, rows - t0);
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
      const float dt = softplus_f(dt_s[i] + bias);
      dt_s[i] = dt;
      decay_s[i] = expf(rate * dt);
    }
    __syncthreads();
    for (int i = 0; i < count; ++i) {
      const float decay = decay_s[i];
      float xv[CP], push[CP], acc[CP];
#pragma unroll
      for (int c = 0; c < CP; ++c) {
        xv[c] = x_s[i * SCAN_COLS + col + c];
        push[c] = dt_s[i] * xv[c];
        acc[c] = 0.f;
      }
      const float* bi = b_s + (size_t)i * N;
      const float* ci = c_s + (size_t)i * N;
#pragma unroll
      for (int k = 0; k < RN; ++k) {
        const int n = part + LANES * k;
        if (n < N) {
          const float bn = bi[n], cn = ci[n];  // fetched once for the thread's columns
#pragma unroll
          for (int c = 0; c < CP; ++c) {
            s[c][k] = fmaf(decay, s[c][k], push[c] * bn);
            acc[c] = fmaf(s[c][k], cn, acc[c]);
          }
        }
      }
#pragma unroll
      for (int c = 0; c < CP; ++c) {
        const float sum = group_sum<LANES>(acc[c]);
        if (part == 0 && p + c < P) {
          y[(size_t)(r0 + t0 + i) * ld_y + h * P + p + c] = sum + d_skip * xv[c];
        }
      }
    }
    __syncthreads();  // the buffer is staged again at the next turn
  }
#pragma unroll
  for (int c = 0; c < CP; ++c) {
#pragma unroll
    for (int k = 0; k < RN; ++k) {
      const int n = part + LANES * k;
      if (p + c < P && n < N) mine[(size_t)(p + c) * N + n] = s[c][k];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// mLSTM: per head, with log gates i = cap tanh((i_raw + b_i) / cap) and
// f = logsigmoid(cap tanh((f_raw + b_f) / cap)) and a running maximum m (0 at the start):
//   m' = max(f + m, i);  keep = e^(f + m - m'), take = e^(i - m');
//   S <- keep S + take k v^T;  n <- keep n + take k;
//   out = S^T q / (max(|n . q|, e^(-m')) + 1e-6),   q times dim^(-1/2).
// proj rows: [ q: H x dim | k: H x dim | v: H x P | (gate, not read here) | i_raw: H | f_raw: H ]
// at the given offsets. State of a slot: S [H][P][dim]; then, once per tile of SCAN_COLS
// columns so that no CTA reads what another writes, n [H][tiles][dim] and m [H][tiles].
template <int RN, int LANES, int CP>
__global__ void __launch_bounds__(SCAN_COLS / CP * LANES)
mlstm_scan_kernel(const float* __restrict__ proj, int ld_proj, int k_offset, int v_offset,
                  int i_offset, int f_offset, const float* __restrict__ gate_bias, float cap,
                  float* __restrict__ state, long long state_stride,
                  const int* __restrict__ row_start, const int* __restrict__ state_slot,
                  float* __restrict__ out, int ld_out, int heads, int dim, int P, int chunk,
                  int vec) {
  extern __shared__ __align__(16) float scan_smem[];
  const int stage_floats = chunk * (2 * dim + SCAN_COLS + 4);
  __shared__ float m_run;
  pdl_launch_dependents();
  const int h = blockIdx.x, b = blockIdx.y, tile = blockIdx.z, tiles = gridDim.z;
  const int p0 = tile * SCAN_COLS;
  const int col = threadIdx.x / LANES * CP, part = threadIdx.x % LANES;  // first of CP columns
  const int p = p0 + col;
  const int r0 = row_start[b], rows = row_start[b + 1] - r0;
  const float q_scale = 1.f / sqrtf((float)dim);
  const float bias_i = gate_bias != nullptr ? gate_bias[h] : 0.f;
  const float bias_f = gate_bias != nullptr ? gate_bias[heads + h] : 0.f;
  if (state_slot[b] < 0) return;  // a row of padding (a graph's bucket): no request, no state
  float* slot = state + (size_t)state_slot[b] * state_stride;
  float* mine = slot + (size_t)h * dim * P;
  float* norm_mine = slot + (size_t)heads * dim * P + ((size_t)h * tiles + tile) * dim;
  float* max_mine = slot + (size_t)heads * dim * P + (size_t)heads * tiles * dim + h * tiles + tile;
  pdl_wait_for(proj, mine, norm_mine, max_mine);
  float s[CP][RN], nrm[RN];
#pragma unroll
  for (int k = 0; k < RN; ++k) {
    const int n = part + LANES * k;
#pragma unroll
    for (int c = 0; c < CP; ++c) {
      s[c][k] = (p + c < P && n < dim) ? mine[(size_t)(p + c) * dim + n] : 0.f;
    }
    nrm[k] = n < dim ? norm_mine[n] : 0.f;
  }
  if (threadIdx.x == 0) m_run = *max_mine;
  const int chunks = (rows + chunk - 1) / chunk;
  auto stage = [&](int c) {
    float* at = scan_smem + (size_t)(c % SCAN_STAGES) * stage_floats;
    const int t0 = c * chunk, count = min(chunk, rows - t0);
    const float* first = proj + (size_t)(r0 + t0) * ld_proj;
    stage_tile(at, first + h * dim, ld_proj, count, dim, vec);                               // q
    stage_tile(at + (size_t)chunk * dim, first + k_offset + h * dim, ld_proj, count, dim, vec);
    stage_columns(at + (size_t)2 * chunk * dim, first + v_offset + h * P, ld_proj, count, p0, P,
                  vec);                                                                     // v
    float* gates = at + 2 * chunk * dim + chunk * SCAN_COLS;
    for (int i = threadIdx.x; i < 2 * count; i += blockDim.x) {
      const int row = i >> 1;
      copy_async(gates + (i & 1) * chunk + row,
                 first + (size_t)row * ld_proj + ((i & 1) ? i_offset : f_offset) + h, 1);
    }
    copy_commit();
  };
  for (int c = 0; c < SCAN_STAGES - 1; ++c) {
    if (c < chunks) stage(c); else copy_commit();
  }
  for (int c = 0; c < chunks; ++c) {
    // (one group per turn, staged or empty, so that the count of groups in flight says
    // which chunk has landed)
    if (c + SCAN_STAGES - 1 < chunks) stage(c + SCAN_STAGES - 1); else copy_commit();
    copy_wait<SCAN_STAGES - 1>();
    __syncthreads();
    float* q_s = scan_smem + (size_t)(c % SCAN_STAGES) * stage_floats;
    float* k_s = q_s + (size_t)chunk * dim;
    float* v_s = k_s + (size_t)chunk * dim;
    float* keep_s = v_s + chunk * SCAN_COLS;  // raw forget gate, log gate f, then the factor
    float* take_s = keep_s + chunk;           // raw input gate, log gate i, then the factor
    float* floor_s = take_s + chunk;          // e^(-m')
    const int t0 = c * chunk, count = min(chunk, rows - t0);
    if (threadIdx.x < 32) {
      // The gates of the chunk's rows, one lane each, and the running maximum by a scan:
      // row i maps m to max(f_i + m, i_i); two such maps compose to one of the same form,
      // (a, b) then (a', b') = (a + a', max(a' + b, b')), so five steps of a warp scan give
      // every row the map from the chunk's start to itself (chunk <= 32 rows).
      const int i = threadIdx.x;
      const bool row = i < count;
      const float ig = row ? cap * tanhf((take_s[i] + bias_i) / cap) : 0.f;
      const float f = row ? log_sigmoid_f(cap * tanhf((keep_s[i] + bias_f) / cap)) : 0.f;
      float a = f, bmax = row ? ig : -INFINITY;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float a_up = __shfl_up_sync(0xffffffffu, a, o);
        const float b_up = __shfl_up_sync(0xffffffffu, bmax, o);
        if (i >= o) {
          bmax = fmaxf(a + b_up, bmax);
          a += a_up;
        }
      }
      const float m_new = fmaxf(a + m_run, bmax);
      float m_old = __shfl_up_sync(0xffffffffu, m_new, 1);
      if (i == 0) m_old = m_run;
      __syncwarp();
      if (row) {
        keep_s[i] = expf(f + m_old - m_new);
        take_s[i] = expf(ig - m_new);
        floor_s[i] = expf(-m_new);
      }
      if (i == count - 1) m_run = m_new;
    }
    __syncthreads();
    for (int i = 0; i < count; ++i) {
      const float keep = keep_s[i], take = take_s[i];
      float tv[CP], acc[CP];
#pragma unroll
      for (int c = 0; c < CP; ++c) {
        tv[c] = take * v_s[i * SCAN_COLS + col + c];
        acc[c] = 0.f;
      }
      const float* qi = q_s + (size_t)i * dim;
      const float* ki = k_s + (size_t)i * dim;
      float dot = 0.f;
#pragma unroll
      for (int k = 0; k < RN; ++k) {
        const int n = part + LANES * k;
        if (n < dim) {
          const float kk = ki[n], qq = qi[n];  // fetched once for the thread's columns
          nrm[k] = fmaf(keep, nrm[k], take * kk);
          dot = fmaf(nrm[k], qq, dot);
#pragma unroll
          for (int c = 0; c < CP; ++c) {
            s[c][k] = fmaf(keep, s[c][k], tv[c] * kk);
            acc[c] = fmaf(s[c][k], qq, acc[c]);
          }
        }
      }
      dot = group_sum<LANES>(dot) * q_scale;
      const float below = fmaxf(fabsf(dot), floor_s[i]) + 1e-6f;
#pragma unroll
      for (int c = 0; c < CP; ++c) {
        const float sum = group_sum<LANES>(acc[c]) * q_scale;
        if (part == 0 && p + c < P) {
          out[(size_t)(r0 + t0 + i) * ld_out + h * P + p + c] = sum / below;
        }
      }
    }
    __syncthreads();  // the buffer is staged again at the next turn
  }
#pragma unroll
  for (int k = 0; k < RN; ++k) {
    const int n = part + LANES * k;
#pragma unroll
    for (int c = 0; c < CP; ++c) {
      if (p + c < P && n < dim) mine[(size_t)(p + c) * dim + n] = s[c][k];
    }
    if (col == 0 && n < dim) norm_mine[n] = nrm[k];
  }
  if (threadIdx.x == 0) *max_mine = m_run;
}

// ---------------------------------------------------------------------------------------------
// Gated linear attention with a decay per key channel: per head, with the raw decay z and
// alpha = sigmoid(z)^(1/tau) = exp(logsigmoid(z) / tau),
//   S <- diag(alpha) S + k v^T   (alpha_n scales row n of S: the entries of key channel n),
//   out = S^T q * q_scale,       S: [N x P].
// proj rows hold q at 0, k at k_offset (heads x N each) and v at v_offset (heads x P); z rows
// hold heads x N raw decays. State of a slot: S as [heads][P][N]. The decays are turned into
// factors in shared memory once per chunk, in fp32.
template <int RN, int LANES>
__global__ void __launch_bounds__(SCAN_COLS * LANES)
gla_scan_kernel(const float* __restrict__ proj, int ld_proj, int k_offset, int v_offset,
                const float* __restrict__ z, int ld_z, float inv_tau, float q_scale,
                float* __restrict__ state, long long state_stride,
                const int* __restrict__ row_start, const int* __restrict__ state_slot,
                float* __restrict__ out, int ld_out, int heads, int N, int P, int chunk,
                int vec) {
  extern __shared__ __align__(16) float scan_smem[];
  const int stage_floats = chunk * (3 * N + SCAN_COLS);
  pdl_launch_dependents();
  const int h = blockIdx.x, b = blockIdx.y, p0 = blockIdx.z * SCAN_COLS;
  const int col = threadIdx.x / LANES, part = threadIdx.x % LANES;
  const int p = p0 + col;
  const int r0 = row_start[b], rows = row_start[b + 1] - r0;
  if (state_slot[b] < 0) return;  // a row of padding (a graph's bucket): no request, no state
  float* mine = state + (size_t)state_slot[b] * state_stride + (size_t)h * N * P;
  pdl_wait_for(proj, z, mine);
  float s[RN];
#pragma unroll
  for (int k = 0; k < RN; ++k) {
    const int n = part + LANES * k;
    s[k] = (p < P && n < N) ? mine[(size_t)p * N + n] : 0.f;
  }
  const int chunks = (rows + chunk - 1) / chunk;
  auto stage = [&](int c) {
    float* at = scan_smem + (size_t)(c % SCAN_STAGES) * stage_floats;
    const int t0 = c * chunk, count = min(chunk, rows - t0);
    const float* first = proj + (size_t)(r0 + t0) * ld_proj;
    stage_tile(at, first + h * N, ld_proj, count, N, vec);                                  // q
    stage_tile(at + (size_t)chunk * N, first + k_offset + h * N, ld_proj, count, N, vec);   // k
    stage_tile(at + (size_t)2 * chunk * N, z + (size_t)(r0 + t0) * ld_z + h * N, ld_z, count, N,
               vec);                                                                        // z
    stage_columns(at + (size_t)3 * chunk * N, first + v_offset + h * P, ld_proj, count, p0, P,
                  vec);                                                                     // v
    copy_commit();
  };
  for (int c = 0; c < SCAN_STAGES - 1; ++c) {
    if (c < chunks) stage(c); else copy_commit();
  }
  for (int c = 0; c < chunks; ++c) {
    if (c + SCAN_STAGES - 1 < chunks) stage(c + SCAN_STAGES - 1); else copy_commit();
    copy_wait<SCAN_STAGES - 1>();
    __syncthreads();
    float* q_s = scan_smem + (size_t)(c % SCAN_STAGES) * stage_floats;
    float* k_s = q_s + (size_t)chunk * N;
    float* a_s = k_s + (size_t)chunk * N;  // raw decays, then the factors
    float* v_s = a_s + (size_t)chunk * N;
    const int t0 = c * chunk, count = min(chunk, rows - t0);
    for (int i = threadIdx.x; i < count * N; i += blockDim.x) {
      a_s[i] = expf(log_sigmoid_f(a_s[i]) * inv_tau);
    }
    __syncthreads();
#pragma unroll 4
    for (int i = 0; i < count; ++i) {
      const float vv = v_s[i * SCAN_COLS + col];
      const float* qi = q_s + (size_t)i * N;
      const float* ki = k_s + (size_t)i * N;
      const float* ai = a_s + (size_t)i * N;
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < RN; ++k) {
        const int n = part + LANES * k;
        if (n < N) {
          s[k] = fmaf(ai[n], s[k], ki[n] * vv);
          acc = fmaf(s[k], qi[n], acc);
        }
      }
      const float sum = group_sum<LANES>(acc);
      if (part == 0 && p < P) out[(size_t)(r0 + t0 + i) * ld_out + h * P + p] = sum * q_scale;
    }
    __syncthreads();  // the buffer is staged again at the next turn
  }
#pragma unroll
  for (int k = 0; k < RN; ++k) {
    const int n = part + LANES * k;
    if (p < P && n < N) mine[(size_t)p * N + n] = s[k];
  }
}

// ---------------------------------------------------------------------------------------------
// Generalised delta rule with a decay and a removal rate per key channel: per head, with the
// raw decay z, the raw removal rate y (plus its bias) and the unit key u = k / sqrt(k . k + 1e-6),
//   w = exp(-decay_rate * sigmoid(z)),   a = sigmoid(y + y_bias),
//   S <- diag(w) S - (a * u) (u^T S) + k v^T   (both terms read the old S),
//   out = S^T r,                                S: [N x P].
// A column of S never meets another: u^T S is one number per column, formed from the old
// column before it is overwritten (one exchange among the column's lanes), and the answer is a
// second one. proj rows hold r at 0, k at k_offset, y at a_offset (heads x N each) and v at
// v_offset (heads x P); z rows hold heads x N raw decays. State of a slot: S as [heads][P][N].
// The decays, the rates times the key and the key's inverse length are formed in shared
// memory once per chunk, in fp32.
template <int RN, int LANES>
__global__ void __launch_bounds__(SCAN_COLS * LANES)
delta_scan_kernel(const float* __restrict__ proj, int ld_proj, int k_offset, int v_offset,
                  int a_offset, const float* __restrict__ a_bias, const float* __restrict__ z,
                  int ld_z, float decay_rate, float* __restrict__ state, long long state_stride,
                  const int* __restrict__ row_start, const int* __restrict__ state_slot,
                  float* __restrict__ out, int ld_out, int heads, int N, int P, int chunk,
                  int vec) {
  extern __shared__ __align__(16) float scan_smem[];
  const int stage_floats = chunk * (4 * N + SCAN_COLS + 4);
  pdl_launch_dependents();
  const int h = blockIdx.x, b = blockIdx.y, p0 = blockIdx.z * SCAN_COLS;
  const int col = threadIdx.x / LANES, part = threadIdx.x % LANES;
  const int p = p0 + col;
  const int r0 = row_start[b], rows = row_start[b + 1] - r0;
  if (state_slot[b] < 0) return;  // a row of padding (a graph's bucket): no request, no state
  float* mine = state + (size_t)state_slot[b] * state_stride + (size_t)h * N * P;
  pdl_wait_for(proj, z, mine);
  float s[RN];
#pragma unroll
  for (int k = 0; k < RN; ++k) {
    const int n = part + LANES * k;
    s[k] = (p < P && n < N) ? mine[(size_t)p * N + n] : 0.f;
  }
  const int chunks = (rows + chunk - 1) / chunk;
  auto stage = [&](int c) {
    float* at = scan_smem + (size_t)(c % SCAN_STAGES) * stage_floats;
    const int t0 = c * chunk, count = min(chunk, rows - t0);
    const float* first = proj + (size_t)(r0 + t0) * ld_proj;
    stage_tile(at, first + h * N, ld_proj, count, N, vec);                                  // r
    stage_tile(at + (size_t)chunk * N, first + k_offset + h * N, ld_proj, count, N, vec);   // k
    stage_tile(at + (size_t)2 * chunk * N, z + (size_t)(r0 + t0) * ld_z + h * N, ld_z, count, N,
               vec);                                                                        // z
    stage_tile(at + (size_t)3 * chunk * N, first + a_offset + h * N, ld_proj, count, N, vec);  // y
    stage_columns(at + (size_t)4 * chunk * N, first + v_offset + h * P, ld_proj, count, p0, P,
                  vec);                                                                     // v
    copy_commit();
  };
  for (int c = 0; c < SCAN_STAGES - 1; ++c) {
    if (c < chunks) stage(c); else copy_commit();
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (int c = 0; c < chunks; ++c) {
    if (c + SCAN_STAGES - 1 < chunks) stage(c + SCAN_STAGES - 1); else copy_commit();
    copy_wait<SCAN_STAGES - 1>();
    __syncthreads();
    float* r_s = scan_smem + (size_t)(c % SCAN_STAGES) * stage_floats;
    float* k_s = r_s + (size_t)chunk * N;
    float* w_s = k_s + (size_t)chunk * N;   // raw decays, then the factors
    float* au_s = w_s + (size_t)chunk * N;  // raw rates, then rate * unit key
    float* v_s = au_s + (size_t)chunk * N;
    float* inv_s = v_s + (size_t)chunk * SCAN_COLS;  // 1 / length of each row's key
    const int t0 = c * chunk, count = min(chunk, rows - t0);
    for (int i = warp; i < count; i += warps) {  // a warp per row: the key's length, then
      float ss = 0.f;                            // the row's factors
      for (int n = lane; n < N; n += 32) ss = fmaf(k_s[i * N + n], k_s[i * N + n], ss);
      const float inv = 1.f / sqrtf(group_sum<32>(ss) + 1e-6f);
      if (lane == 0) inv_s[i] = inv;
      for (int n = lane; n < N; n += 32) {
        const int at = i * N + n;
        w_s[at] = expf(-decay_rate / (1.f + expf(-w_s[at])));
        const float rate = 1.f / (1.f + expf(-(au_s[at] + a_bias[h * N + n])));
        au_s[at] = rate * k_s[at] * inv;
      }
    }
    __syncthreads();
#pragma unroll 2
    for (int i = 0; i < count; ++i) {
      const float vv = v_s[i * SCAN_COLS + col];
      const float* ri = r_s + (size_t)i * N;
      const float* ki = k_s + (size_t)i * N;
      const float* wi = w_s + (size_t)i * N;
      const float* ai = au_s + (size_t)i * N;
      float seen = 0.f;  // k . (old column); times the inverse length: u . (old column)
#pragma unroll
      for (int k = 0; k < RN; ++k) {
        const int n = part + LANES * k;
        if (n < N) seen = fmaf(ki[n], s[k], seen);
      }
      seen = group_sum<LANES>(seen) * inv_s[i];
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < RN; ++k) {
        const int n = part + LANES * k;
        if (n < N) {
          s[k] = fmaf(wi[n], s[k], fmaf(ki[n], vv, -ai[n] * seen));
          acc = fmaf(s[k], ri[n], acc);
        }
      }
      const float sum = group_sum<LANES>(acc);
      if (part == 0 && p < P) out[(size_t)(r0 + t0 + i) * ld_out + h * P + p] = sum;
    }
    __syncthreads();  // the buffer is staged again at the next turn
  }
#pragma unroll
  for (int k = 0; k < RN; ++k) {
    const int n = part + LANES * k;
    if (p < P && n < N) mine[(size_t)p * N + n] = s[k];
  }
}

// rows of a chunk (at most 32: a warp scans a chunk's gates), and the ring's bytes: up to
// 68 KB, which a kernel has to be allowed once (allow_smem)
inline int scan_chunk(int n) { return n <= 64 ? 32 : (n <= 128 ? 16 : (n <= 256 ? 8 : 4)); }
inline size_t scan_smem_bytes(int chunk, int n) {
  return (size_t)SCAN_STAGES * chunk * (2 * n + SCAN_COLS + 4) * sizeof(float);
}
template <typename K> inline void allow_smem(K kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
}
// 16-byte copies when every staged address is a multiple of 16 bytes, else 4-byte ones
inline int scan_vec(const float* base, long long ld, int n, int P,
                    std::initializer_list<long long> offsets) {
  bool ok = ((uintptr_t)base % 16) == 0 && ld % 4 == 0 && n % 4 == 0 && P % 4 == 0;
  for (long long o : offsets) ok = ok && o % 4 == 0;
  return ok ? 4 : 1;
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

AYK_API int ayk_scan_columns() { return ayk::SCAN_COLS; }

// `in`: the step's rows, column 0 = channel 0 (a column range of the projection output);
// `state`: the first of (taps - 1) x channels kept inputs of slot 0; slots are state_stride
// floats apart. The convolution, then the update of the kept inputs: two launches.
AYK_API int ayk_causal_conv_silu(const float* in, int ld_in, const float* w, const float* bias,
                                 float* state, long long state_stride, const int* request_of_row,
                                 const int* row_start, const int* state_slot, float* out,
                                 int ld_out, int rows, int requests, int channels, int taps,
                                 void* stream) {
  using namespace ayk;
  if (rows == 0 || channels == 0) return AYK_OK;
  if (rows < 0 || requests < 1 || channels < 0 || taps < 1 || in == nullptr || w == nullptr ||
      state == nullptr || request_of_row == nullptr || row_start == nullptr ||
      state_slot == nullptr || out == nullptr || ld_in < channels || ld_out < channels ||
      requests > 65535) {
    return AYK_BAD_ARGUMENT;
  }
  const int threads = 128, tiles = (channels + threads - 1) / threads;
  if (taps > CONV_MAX_TAPS || tiles > 65535) return AYK_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  const int status = launch_kernel(causal_conv_silu_kernel, dim3(rows, tiles), dim3(threads), 0,
                                   s, 1, in, ld_in, w, bias, (const float*)state, state_stride,
                                   request_of_row, row_start, state_slot, out, ld_out, channels,
                                   taps);
  if (status != AYK_OK || taps == 1) return status;
  return launch_kernel(conv_state_update_kernel, dim3(tiles, requests), dim3(threads), 0, s, 1,
                       in, ld_in, state, state_stride, row_start, state_slot, channels, taps);
}

AYK_API int ayk_mamba2_scan(const float* xbc, int ld_xbc, const float* dt_raw, int ld_dt,
                            const float* dt_bias, const float* a_log, const float* skip,
                            float* state, long long state_stride, const int* row_start,
                            const int* state_slot, float* y, int ld_y, int requests, int heads,
                            int groups, int N, int P, void* stream) {
  using namespace ayk;
  if (requests == 0) return AYK_OK;
  if (requests < 0 || heads < 1 || groups < 1 || heads % groups || N < 1 || P < 1 ||
      xbc == nullptr || dt_raw == nullptr || dt_bias == nullptr || a_log == nullptr ||
      state == nullptr || row_start == nullptr || state_slot == nullptr || y == nullptr ||
      ld_xbc < heads * P + 2 * groups * N || ld_dt < heads || ld_y < heads * P ||
      requests > 65535) {
    return AYK_BAD_ARGUMENT;
  }
  if (N > SCAN_MAX_N || (P + SCAN_COLS - 1) / SCAN_COLS > 65535) return AYK_TOO_LARGE;
  const int chunk = scan_chunk(N);
  const size_t smem = scan_smem_bytes(chunk, N);
  const int vec = scan_vec(xbc, ld_xbc, N, P, {(long long)heads * P});
  const dim3 grid(heads, requests, (P + SCAN_COLS - 1) / SCAN_COLS);
#define AYK_MAMBA(RN, LANES, CP)                                                                  \
  {                                                                                            \
    static const bool allowed = (allow_smem(mamba2_scan_kernel<RN, LANES, CP>), true);         \
    (void)allowed;                                                                             \
    return launch_kernel(mamba2_scan_kernel<RN, LANES, CP>, grid, dim3(SCAN_COLS / CP * LANES),   \
                         smem,                                                                 \
                         (cudaStream_t)stream, 1, xbc, ld_xbc, dt_raw, ld_dt, dt_bias, a_log,  \
                         skip, state, state_stride, row_start, state_slot, y, ld_y, heads,     \
                         groups, N, P, chunk, vec);                                            \
  }
  if (N <= 8) AYK_MAMBA(1, 8, 1);
  if (N <= 16) AYK_MAMBA(2, 8, 1);
  if (N <= 32) AYK_MAMBA(4, 8, 1);
  if (N <= 64) AYK_MAMBA(4, 16, 1);
  if (N <= 128) AYK_MAMBA(4, 32, 1);
  if (N <= 256) AYK_MAMBA(8, 32, 1);
  AYK_MAMBA(16, 32, 1);
#undef AYK_MAMBA
}

AYK_API int ayk_mlstm_scan(const float* proj, int ld_proj, int k_offset, int v_offset,
                           int i_offset, int f_offset, const float* gate_bias, float cap,
                           float* state, long long state_stride, const int* row_start,
                           const int* state_slot, float* out, int ld_out, int requests, int heads,
                           int dim, int P, void* stream) {
  using namespace ayk;
  if (requests == 0) return AYK_OK;
  const int tiles = (P + SCAN_COLS - 1) / SCAN_COLS;
  if (requests < 0 || heads < 1 || dim < 1 || P < 1 || proj == nullptr || state == nullptr ||
      row_start == nullptr || state_slot == nullptr || out == nullptr || !(cap > 0.f) ||
      ld_out < heads * P || requests > 65535 ||
      state_stride < (long long)heads * dim * P + (long long)heads * tiles * (dim + 1)) {
    return AYK_BAD_ARGUMENT;
  }
  if (dim > SCAN_MAX_N || tiles > 65535) return AYK_TOO_LARGE;
  const int chunk = scan_chunk(dim);
  const size_t smem = scan_smem_bytes(chunk, dim);
  const int vec = scan_vec(proj, ld_proj, dim, P, {k_offset, v_offset});
  const dim3 grid(heads, requests, tiles);
#define AYK_MLSTM(RN, LANES, CP)                                                                  \
  {                                                                                            \
    static const bool allowed = (allow_smem(mlstm_scan_kernel<RN, LANES, CP>), true);          \
    (void)allowed;                                                                             \
    return launch_kernel(mlstm_scan_kernel<RN, LANES, CP>, grid, dim3(SCAN_COLS / CP * LANES),    \
                         smem,                                                                 \
                         (cudaStream_t)stream, 1, proj, ld_proj, k_offset, v_offset, i_offset, \
                         f_offset, gate_bias, cap, state, state_stride, row_start, state_slot, \
                         out, ld_out, heads, dim, P, chunk, vec);                              \
  }
  if (dim <= 8) AYK_MLSTM(1, 8, 1);
  if (dim <= 16) AYK_MLSTM(2, 8, 1);
  if (dim <= 32) AYK_MLSTM(4, 8, 1);
  if (dim <= 64) AYK_MLSTM(4, 16, 1);
  if (dim <= 128) AYK_MLSTM(4, 32, 1);
  if (dim <= 256) AYK_MLSTM(8, 32, 1);
  AYK_MLSTM(16, 32, 1);
#undef AYK_MLSTM
}

// rows of a chunk of the gated-linear-attention scan (three staged tiles of N entries a row)
static inline int gla_chunk(int n) { return n <= 32 ? 32 : (n <= 64 ? 16 : (n <= 128 ? 8 : 4)); }

AYK_API int ayk_gla_scan(const float* proj, int ld_proj, int k_offset, int v_offset,
                         const float* z, int ld_z, float tau, float q_scale, float* state,
                         long long state_stride, const int* row_start, const int* state_slot,
                         float* out, int ld_out, int requests, int heads, int N, int P,
                         void* stream) {
  using namespace ayk;
  if (requests == 0) return AYK_OK;
  const int tiles = (P + SCAN_COLS - 1) / SCAN_COLS;
  if (requests < 0 || heads < 1 || N < 1 || P < 1 || proj == nullptr || z == nullptr ||
      state == nullptr || row_start == nullptr || state_slot == nullptr || out == nullptr ||
      !(tau > 0.f) || ld_out < heads * P || ld_z < heads * N || requests > 65535 ||
      ld_proj < max(k_offset + heads * N, v_offset + heads * P) ||
      state_stride < (long long)heads * N * P) {
    return AYK_BAD_ARGUMENT;
  }
  if (N > SCAN_MAX_N || tiles > 65535) return AYK_TOO_LARGE;
  const int chunk = gla_chunk(N);
  const size_t smem = (size_t)SCAN_STAGES * chunk * (3 * N + SCAN_COLS) * sizeof(float);
  int vec = scan_vec(proj, ld_proj, N, P, {k_offset, v_offset});
  if (((uintptr_t)z % 16) != 0 || ld_z % 4 != 0) vec = 1;
  const dim3 grid(heads, requests, tiles);
#define AYK_GLA(RN, LANES)                                                                     \
  {                                                                                            \
    static const bool allowed =                                                                \
        (cudaFuncSetAttribute(gla_scan_kernel<RN, LANES>,                                      \
                              cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024), true); \
    (void)allowed;                                                                             \
    return launch_kernel(gla_scan_kernel<RN, LANES>, grid, dim3(SCAN_COLS * LANES), smem,      \
                         (cudaStream_t)stream, 1, proj, ld_proj, k_offset, v_offset, z, ld_z,  \
                         1.f / tau, q_scale, state, state_stride, row_start, state_slot, out,  \
                         ld_out, heads, N, P, chunk, vec);                                     \
  }
  if (N <= 8) AYK_GLA(1, 8);
  if (N <= 16) AYK_GLA(2, 8);
  if (N <= 32) AYK_GLA(4, 8);
  if (N <= 64) AYK_GLA(4, 16);
  if (N <= 128) AYK_GLA(4, 32);
  if (N <= 256) AYK_GLA(8, 32);
  AYK_GLA(16, 32);
#undef AYK_GLA
}

// rows of a chunk of the delta-rule scan (four staged tiles of N entries a row)
static inline int delta_chunk(int n) { return n <= 32 ? 32 : (n <= 64 ? 16 : (n <= 128 ? 8 : 4)); }

// See delta_scan_kernel. `a_bias`: heads x N floats. decay_rate: the factor on sigmoid(z) in
// the decay's exponent.
AYK_API int ayk_delta_scan(const float* proj, int ld_proj, int k_offset, int v_offset,
                           int a_offset, const float* a_bias, const float* z, int ld_z,
                           float decay_rate, float* state, long long state_stride,
                           const int* row_start, const int* state_slot, float* out, int ld_out,
                           int requests, int heads, int N, int P, void* stream) {
  using namespace ayk;
  if (requests == 0) return AYK_OK;
  const int tiles = (P + SCAN_COLS - 1) / SCAN_COLS;
  if (requests < 0 || heads < 1 || N < 1 || P < 1 || proj == nullptr || z == nullptr ||
      a_bias == nullptr || state == nullptr || row_start == nullptr || state_slot == nullptr ||
      out == nullptr || !(decay_rate >= 0.f) || ld_out < heads * P || ld_z < heads * N ||
      requests > 65535 || k_offset < 0 || v_offset < 0 || a_offset < 0 ||
      ld_proj < max(max(k_offset, a_offset) + heads * N, v_offset + heads * P) ||
      state_stride < (long long)heads * N * P) {
    return AYK_BAD_ARGUMENT;
  }
  if (N > SCAN_MAX_N || tiles > 65535) return AYK_TOO_LARGE;
  const int chunk = delta_chunk(N);
  const size_t smem = (size_t)SCAN_STAGES * chunk * (4 * N + SCAN_COLS + 4) * sizeof(float);
  int vec = scan_vec(proj, ld_proj, N, P, {k_offset, v_offset, a_offset});
  if (((uintptr_t)z % 16) != 0 || ld_z % 4 != 0) vec = 1;
  const dim3 grid(heads, requests, tiles);
#define AYK_DELTA(RN, LANES)                                                                   \
  {                                                                                            \
    static const bool allowed =                                                                \
        (cudaFuncSetAttribute(delta_scan_kernel<RN, LANES>,                                    \
                              cudaFuncAttributeMaxDynamicSharedMemorySize, 144 * 1024), true); \
    (void)allowed;                                                                             \
    return launch_kernel(delta_scan_kernel<RN, LANES>, grid, dim3(SCAN_COLS * LANES), smem,    \
                         (cudaStream_t)stream, 1, proj, ld_proj, k_offset, v_offset, a_offset, \
                         a_bias, z, ld_z, decay_rate, state, state_stride, row_start,          \
                         state_slot, out, ld_out, heads, N, P, chunk, vec);                    \
  }
  if (N <= 8) AYK_DELTA(1, 8);
  if (N <= 16) AYK_DELTA(2, 8);
  if (N <= 32) AYK_DELTA(4, 8);
  if (N <= 64) AYK_DELTA(4, 16);
  if (N <= 128) AYK_DELTA(4, 32);
  if (N <= 256) AYK_DELTA(8, 32);
  AYK_DELTA(16, 32);
#undef AYK_DELTA
}
