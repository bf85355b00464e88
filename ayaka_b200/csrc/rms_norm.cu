// Root-mean-square norms over fp32 rows: y = x * rsqrt(mean(x^2) + eps) * (offset + w), the
// mean taken over each of `groups` equal parts of the row on its own. `offset` is 0 for a
// plain weight and 1 for a weight stored as its deviation from one. `rows` may gather (output
// row i normalises input row rows[i]: the final norm runs on the wanted rows only).
//
// A gate may ride along (fp32, same row and column as x):
//   GATE_SILU_BEFORE: x is first multiplied by silu(gate), then normalised (the gated norm of a
//     state-space layer: the gate comes before the norm);
//   GATE_SIGMOID_AFTER: the normalised, weighted value is multiplied by sigmoid(gate) (the
//     output gate of a matrix-memory layer);
//   GATE_SILU_AFTER: the normalised, weighted value is multiplied by silu(gate) (the output
//     gate of a gated-linear-attention layer).
// `weight_period` > 0: the weight has that many entries and repeats along the row (one weight
// shared by every head).
//
// norm_sum: several fp32 rows of the same width, each normalised over the whole width with a
// weight of its own, are averaged, multiplied element by element by an optional scale and
// added to (or written into) an fp32 row: the join of mixers that run side by side.
// Everything in fp32, rounded once to the output type. Any width.
#include "common.cuh"

namespace ayk {

enum GateMode : int { GATE_NONE = 0, GATE_SILU_BEFORE = 1, GATE_SIGMOID_AFTER = 2,
                      GATE_SILU_AFTER = 3 };

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

template <typename TOut>
__global__ void rms_norm_kernel(const float* __restrict__ x, int ld_x,
                                const int* __restrict__ rows, const float* __restrict__ weight,
                                float weight_offset, float eps, int group_width,
                                const float* __restrict__ gate, int ld_gate, int gate_mode,
                                TOut* __restrict__ out, int ld_out, int weight_period) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int r = blockIdx.x, g = blockIdx.y;
  const int row = rows != nullptr ? rows[r] : r;
  pdl_wait_for(x, gate);
  const float* src = x + (size_t)row * ld_x + (size_t)g * group_width;
  const float* gt = gate != nullptr ? gate + (size_t)row * ld_gate + (size_t)g * group_width
                                    : nullptr;
  float s = 0.f;
  for (int c = threadIdx.x; c < group_width; c += blockDim.x) {
    float v = src[c];
    if (gate_mode == GATE_SILU_BEFORE) {
      const float z = gt[c];
      v *= z * sigmoid_f(z);
    }
    s += v * v;
  }
  const float inv = 1.f / sqrtf(block_sum(s, scratch) / (float)group_width + eps);
  const float* w = weight_period > 0 ? weight : weight + (size_t)g * group_width;
  const int w_first = weight_period > 0 ? (int)(((size_t)g * group_width) % weight_period) : 0;
  TOut* dst = out + (size_t)r * ld_out + (size_t)g * group_width;
  for (int c = threadIdx.x; c < group_width; c += blockDim.x) {
    float v = src[c];
    if (gate_mode == GATE_SILU_BEFORE) {
      const float z = gt[c];
      v *= z * sigmoid_f(z);
    }
    v = v * inv * (weight_offset + w[weight_period > 0 ? (w_first + c) % weight_period : c]);
    if (gate_mode == GATE_SIGMOID_AFTER) v *= sigmoid_f(gt[c]);
    if (gate_mode == GATE_SILU_AFTER) {
      const float z = gt[c];
      v *= z * sigmoid_f(z);
    }
    stf(dst + c, v);
  }
}

// dst[r][c] (+)= scale[c] * x[r][c]
__global__ void scale_add_kernel(const float* __restrict__ x, int ld_x,
                                 const float* __restrict__ scale, float* __restrict__ dst,
                                 int ld_dst, int width, int accumulate) {
  pdl_launch_dependents();
  const int r = blockIdx.x;
  pdl_wait_for(x, dst);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = x[(size_t)r * ld_x + c] * scale[c];
    float* to = dst + (size_t)r * ld_dst + c;
    *to = accumulate ? *to + v : v;
  }
}

template <typename TOut>
int rms_norm(const float* x, int ld_x, const int* rows, const float* weight, float weight_offset,
             float eps, int groups, const float* gate, int ld_gate, int gate_mode, void* out,
             int ld_out, int n, int width, int weight_period, cudaStream_t stream) {
  if (n == 0) return AYK_OK;
  if (n < 0 || width < 1 || groups < 1 || width % groups || ld_x < width || ld_out < width ||
      !(eps > 0.f) || weight == nullptr || gate_mode < GATE_NONE ||
      gate_mode > GATE_SILU_AFTER || ((gate_mode != GATE_NONE) != (gate != nullptr)) ||
      (gate != nullptr && ld_gate < width) || weight_period < 0) {
    return AYK_BAD_ARGUMENT;
  }
  const int group_width = width / groups;
  const int threads = group_width >= 2048 ? 512 : (group_width >= 512 ? 256 : 128);
  return launch_kernel(rms_norm_kernel<TOut>, dim3(n, groups), dim3(threads), 0, stream, 1, x,
                       ld_x, rows, weight, weight_offset, eps, group_width, gate, ld_gate,
                       gate_mode, (TOut*)out, ld_out, weight_period);
}

constexpr int SUM_MAX_BRANCHES = 4;
struct Branches {
  const float* x[SUM_MAX_BRANCHES];
  const float* weight[SUM_MAX_BRANCHES];
  int ld[SUM_MAX_BRANCHES];
};

// dst[r][c] (+)= scale[c] * factor * sum_b x_b[r][c] * rsqrt(mean_c(x_b[r]^2) + eps) * w_b[c]
__global__ void norm_sum_kernel(Branches in, int count, float eps, float factor,
                                const float* __restrict__ scale, float* __restrict__ dst,
                                int ld_dst, int width, int accumulate) {
  __shared__ float scratch[SUM_MAX_BRANCHES][32];
  pdl_launch_dependents();
  const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  pdl_wait_for(dst);
  // the branches' sums of squares side by side, through one exchange
  float inv[SUM_MAX_BRANCHES];
#pragma unroll
  for (int b = 0; b < SUM_MAX_BRANCHES; ++b) {
    float s = 0.f;
    if (b < count) {
      const float* src = in.x[b] + (size_t)r * in.ld[b];
      for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = src[c];
        s += v * v;
      }
      s = warp_sum(s);
      if (lane == 0) scratch[b][warp] = s;
    }
  }
  __syncthreads();
#pragma unroll
  for (int b = 0; b < SUM_MAX_BRANCHES; ++b) {
    inv[b] = 0.f;
    if (b < count) {
      float s = 0.f;
      for (int w = 0; w < warps; ++w) s += scratch[b][w];
      inv[b] = 1.f / sqrtf(s / (float)width + eps);
    }
  }
  float* to = dst + (size_t)r * ld_dst;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float sum = 0.f;
#pragma unroll
    for (int b = 0; b < SUM_MAX_BRANCHES; ++b) {
      if (b < count) sum += in.x[b][(size_t)r * in.ld[b] + c] * inv[b] * in.weight[b][c];
    }
    sum *= factor;
    if (scale != nullptr) sum *= scale[c];
    to[c] = accumulate ? to[c] + sum : sum;
  }
}

// dst[r][c] += factor * x[r][c] * rsqrt(mean_c(x[r]^2) + eps) * (offset + w[c]), and, when
// `copy` is given, copy[r][c] = the new dst[r][c] in the compute type: a sublayer's normed
// result joins the fp32 residual stream and the next sublayer's input leaves the same pass.
// When `next_out` is given, also next_out[r][c] = v[c] * rsqrt(mean_c(v^2) + next_eps) *
// (next_offset + next_weight[c]) with v the new dst[r]: the norm in front of the next sublayer,
// from the row that is in registers anyway (one more sum over the row, no launch of its own).
template <typename TOut>
__global__ void norm_add_kernel(const float* __restrict__ x, int ld_x,
                                const float* __restrict__ weight, float offset, float eps,
                                float factor, float* __restrict__ dst, int ld_dst,
                                TOut* __restrict__ copy, int ld_copy, int width,
                                const float* __restrict__ next_weight, float next_offset,
                                float next_eps, TOut* __restrict__ next_out, int ld_next) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int r = blockIdx.x;
  // A row of up to NA_KEEP entries a thread stays in registers: the weights are fetched before
  // the kernel ahead has finished, the branch and the stream's row in one trip to memory, and
  // nothing is read twice. The sums run in the same order as in the loops below.
  constexpr int NA_KEEP = 8;
  if (width <= NA_KEEP * (int)blockDim.x) {
    float ws[NA_KEEP], xs[NA_KEEP], ds[NA_KEEP];
#pragma unroll
    for (int i = 0; i < NA_KEEP; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      ws[i] = c < width ? offset + weight[c] : 0.f;
    }
    pdl_wait_for(x, dst);
    const float* src = x + (size_t)r * ld_x;
    float* to = dst + (size_t)r * ld_dst;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NA_KEEP; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      xs[i] = c < width ? src[c] : 0.f;
      ds[i] = c < width ? to[c] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < NA_KEEP; ++i) s += xs[i] * xs[i];
    const float inv = factor / sqrtf(block_sum(s, scratch) / (float)width + eps);
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NA_KEEP; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < width) {
        const float v = ds[i] + xs[i] * inv * ws[i];
        to[c] = v;
        if (copy != nullptr) stf(copy + (size_t)r * ld_copy + c, v);
        ds[i] = v;
        s2 += v * v;
      }
    }
    if (next_out != nullptr) {
      const float inv2 = 1.f / sqrtf(block_sum(s2, scratch) / (float)width + next_eps);
#pragma unroll
      for (int i = 0; i < NA_KEEP; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < width) {
          stf(next_out + (size_t)r * ld_next + c, ds[i] * inv2 * (next_offset + next_weight[c]));
        }
      }
    }
    return;
  }
  pdl_wait_for(x, dst);
  const float* src = x + (size_t)r * ld_x;
  float s = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) s += src[c] * src[c];
  const float inv = factor / sqrtf(block_sum(s, scratch) / (float)width + eps);
  float* to = dst + (size_t)r * ld_dst;
  float s2 = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to[c] + src[c] * inv * (offset + weight[c]);
    to[c] = v;
    if (copy != nullptr) stf(copy + (size_t)r * ld_copy + c, v);
    s2 += v * v;
  }
  if (next_out != nullptr) {  // (a thread reads back what it wrote itself)
    const float inv2 = 1.f / sqrtf(block_sum(s2, scratch) / (float)width + next_eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      stf(next_out + (size_t)r * ld_next + c, to[c] * inv2 * (next_offset + next_weight[c]));
    }
  }
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// out_type: 0 = float32, 1 = bfloat16.
AYK_API int ayk_rms_norm(const float* x, int ld_x, const int* rows, const float* weight,
                         float weight_offset, float eps, int groups, const float* gate,
                         int ld_gate, int gate_mode, void* out, int ld_out, int n, int width,
                         int out_type, int weight_period, void* stream) {
  if (out_type == 0) {
    return ayk::rms_norm<float>(x, ld_x, rows, weight, weight_offset, eps, groups, gate, ld_gate,
                                gate_mode, out, ld_out, n, width, weight_period,
                                (cudaStream_t)stream);
  }
  if (out_type == 1) {
    return ayk::rms_norm<__nv_bfloat16>(x, ld_x, rows, weight, weight_offset, eps, groups, gate,
                                        ld_gate, gate_mode, out, ld_out, n, width, weight_period,
                                        (cudaStream_t)stream);
  }
  return AYK_BAD_ARGUMENT;
}

// `count` rows x[b] (fp32, leading dimension ld[b]) with weights w[b]; `scale` may be null.
AYK_API int ayk_norm_sum(const float* const* x, const int* ld, const float* const* weight,
                         int count, float eps, float factor, const float* scale, float* dst,
                         int ld_dst, int n, int width, int accumulate, void* stream) {
  using namespace ayk;
  if (n == 0) return AYK_OK;
  if (n < 0 || width < 1 || count < 1 || x == nullptr || ld == nullptr || weight == nullptr ||
      dst == nullptr || ld_dst < width || !(eps > 0.f)) {
    return AYK_BAD_ARGUMENT;
  }
  if (count > SUM_MAX_BRANCHES) return AYK_TOO_LARGE;
  Branches in = {};
  for (int b = 0; b < count; ++b) {
    if (x[b] == nullptr || weight[b] == nullptr || ld[b] < width) return AYK_BAD_ARGUMENT;
    in.x[b] = x[b];
    in.weight[b] = weight[b];
    in.ld[b] = ld[b];
  }
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  return launch_kernel(norm_sum_kernel, dim3(n), dim3(threads), 0, (cudaStream_t)stream, 1, in,
                       count, eps, factor, scale, dst, ld_dst, width, accumulate);
}

AYK_API int ayk_scale_add(const float* x, int ld_x, const float* scale, float* dst, int ld_dst,
                          int n, int width, int accumulate, void* stream) {
  using namespace ayk;
  if (n == 0) return AYK_OK;
  if (n < 0 || width < 1 || x == nullptr || scale == nullptr || dst == nullptr ||
      ld_x < width || ld_dst < width) {
    return AYK_BAD_ARGUMENT;
  }
  return launch_kernel(scale_add_kernel, dim3(n), dim3(width >= 512 ? 256 : 128), 0,
                       (cudaStream_t)stream, 1, x, ld_x, scale, dst, ld_dst, width, accumulate);
}

// copy_type: 0 = float32, 1 = bfloat16, of `copy` and of `next_out` (ignored when both are
// null). `next_out` with `next_weight`: the following norm's output (see norm_add_kernel).
AYK_API int ayk_norm_add_next(const float* x, int ld_x, const float* weight, float offset,
                              float eps, float factor, float* dst, int ld_dst, void* copy,
                              int ld_copy, int copy_type, const float* next_weight,
                              float next_offset, float next_eps, void* next_out, int ld_next,
                              int n, int width, void* stream) {
  using namespace ayk;
  if (n == 0) return AYK_OK;
  if (n < 0 || width < 1 || x == nullptr || weight == nullptr || dst == nullptr ||
      ld_x < width || ld_dst < width || (copy != nullptr && ld_copy < width) || !(eps > 0.f) ||
      (next_out != nullptr && (next_weight == nullptr || ld_next < width ||
                               !(next_eps > 0.f)))) {
    return AYK_BAD_ARGUMENT;
  }
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  const bool typed = copy != nullptr || next_out != nullptr;
  if (typed && copy_type == 1) {
    return launch_kernel(norm_add_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0,
                         (cudaStream_t)stream, 1, x, ld_x, weight, offset, eps, factor, dst,
                         ld_dst, (__nv_bfloat16*)copy, ld_copy, width, next_weight, next_offset,
                         next_eps, (__nv_bfloat16*)next_out, ld_next);
  }
  if (typed && copy_type != 0) return AYK_BAD_ARGUMENT;
  return launch_kernel(norm_add_kernel<float>, dim3(n), dim3(threads), 0, (cudaStream_t)stream,
                       1, x, ld_x, weight, offset, eps, factor, dst, ld_dst, (float*)copy,
                       ld_copy, width, next_weight, next_offset, next_eps, (float*)next_out,
                       ld_next);
}

AYK_API int ayk_norm_add(const float* x, int ld_x, const float* weight, float offset, float eps,
                         float factor, float* dst, int ld_dst, void* copy, int ld_copy,
                         int copy_type, int n, int width, void* stream) {
  return ayk_norm_add_next(x, ld_x, weight, offset, eps, factor, dst, ld_dst, copy, ld_copy,
                           copy_type, nullptr, 0.f, 1.f, nullptr, 0, n, width, stream);
}
