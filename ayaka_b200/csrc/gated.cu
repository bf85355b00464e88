// Element-wise pieces of gated layers, fp32 arithmetic:
//   cast:  out[r][c] = x[r][c] in the compute type (a sublayer that reads the fp32 residual
//          stream itself, with no norm in front of it, gets its matrix operand this way);
//   unit:  out[r][c] = act(gate[r][c]) * other[r][c], act = silu or the tanh GELU, where
//          `other` is either a second fp32 matrix (the up half of a gated feed-forward) or a
//          row of a table picked by an index per row, from column `col` on (an embedding of
//          the row's token that gates a projection of the residual stream);
//   unary: out[r][c] = act(x[r][c] + bias[c]), act = tanh, or a quadratic-exponential unit
//          with two learned numbers (p, q): for z > 0, softplus(p) z^2 + z / 2; for z <= 0,
//          (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2.
#include "common.cuh"

namespace ayk {

enum GateAct : int { GATE_SILU = 0, GATE_GELU_TANH = 1 };

// The tanh GELU 0.5 z (1 + tanh(t)), t = sqrt(2 / pi) (z + 0.044715 z^3), written as
// z / (1 + exp(-2 t)): the same function without the sum 1 + tanh(t), which for negative z
// cancels to a few digits in fp32. A gate is a factor: where all gates of a row are small,
// what follows (a norm over the gated row's projection) keeps their relative error.
__device__ __forceinline__ float gelu_tanh_ratio(float z) {
  const float t = 0.7978845608028654f * (z + 0.044715f * z * z * z);
  return z / (1.f + expf(-2.f * t));
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, int ld_x, T* __restrict__ out,
                                 int ld_out, int rows, int width) {
  pdl_launch_dependents();
  pdl_wait_for(x);
  const long long total = (long long)rows * width;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / width), c = (int)(i % width);
    stf(out + (size_t)r * ld_out + c, x[(size_t)r * ld_x + c]);
  }
}

template <typename T, typename TTable>
__global__ void gated_unit_kernel(const float* __restrict__ gate, int ld_gate,
                                  const float* __restrict__ other, int ld_other,
                                  const TTable* __restrict__ table, int ld_table,
                                  const int* __restrict__ index, int table_rows, int col, int act,
                                  T* __restrict__ out, int ld_out, int rows, int width) {
  pdl_launch_dependents();
  pdl_wait_for(gate, other);
  const long long total = (long long)rows * width;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / width), c = (int)(i % width);
    const float g = gate[(size_t)r * ld_gate + c];
    const float a = act == GATE_GELU_TANH ? gelu_tanh_ratio(g) : g / (1.f + expf(-g));
    float b = 0.f;
    if (other != nullptr) {
      b = other[(size_t)r * ld_other + c];
    } else {
      const int t = index[r];
      // (an index outside the table was already reported by the embedding; read nothing)
      if (t >= 0 && t < table_rows) b = ldf(table + (size_t)t * ld_table + col + c);
    }
    stf(out + (size_t)r * ld_out + c, a * b);
  }
}

enum UnaryAct : int { UNARY_TANH = 0, UNARY_XIELU = 1 };

__device__ __forceinline__ float softplus_of(float z) {  // log(1 + e^z), exact for any z
  return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
}

template <typename T>
__global__ void unary_rows_kernel(const float* __restrict__ x, int ld_x,
                                  const float* __restrict__ bias, int act,
                                  const float* __restrict__ numbers, T* __restrict__ out,
                                  int ld_out, int rows, int width) {
  pdl_launch_dependents();
  float up = 0.f, down = 0.f;
  if (act == UNARY_XIELU) {  // (parameters: written once, when the model was loaded)
    up = softplus_of(numbers[0]);
    down = 0.5f + softplus_of(numbers[1]);
  }
  pdl_wait_for(x);
  const long long total = (long long)rows * width;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / width), c = (int)(i % width);
    float z = x[(size_t)r * ld_x + c];
    if (bias != nullptr) z += bias[c];
    float y;
    if (act == UNARY_TANH) {
      y = tanhf(z);
    } else {
      y = z > 0.f ? fmaf(up * z, z, 0.5f * z) : fmaf(down, expm1f(z) - z, 0.5f * z);
    }
    stf(out + (size_t)r * ld_out + c, y);
  }
}

inline int blocks_for(long long total, int threads) {
  const long long want = (total + threads - 1) / threads;
  const long long most = (long long)sm_count() * 16;
  return (int)(want < most ? (want < 1 ? 1 : want) : most);
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// out_type: 0 = float32, 1 = bfloat16.
AYK_API int ayk_cast_rows(const float* x, int ld_x, void* out, int ld_out, int rows, int width,
                          int out_type, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || width < 1 || x == nullptr || out == nullptr || ld_x < width ||
      ld_out < width) {
    return AYK_BAD_ARGUMENT;
  }
  const int threads = 256, blocks = blocks_for((long long)rows * width, threads);
  cudaStream_t s = (cudaStream_t)stream;
  if (out_type == 0) {
    return launch_kernel(cast_rows_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, x, ld_x,
                         (float*)out, ld_out, rows, width);
  }
  if (out_type == 1) {
    return launch_kernel(cast_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, 1,
                         x, ld_x, (__nv_bfloat16*)out, ld_out, rows, width);
  }
  return AYK_BAD_ARGUMENT;
}

// Either `other` (fp32) or `table` with `index` (int32 per row) is given. type: 0 = float32,
// 1 = bfloat16, of `out` and of `table`.
AYK_API int ayk_gated_unit(const float* gate, int ld_gate, const float* other, int ld_other,
                           const void* table, int ld_table, const int* index, int table_rows,
                           int col, int act, void* out, int ld_out, int rows, int width, int type,
                           void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || width < 1 || gate == nullptr || out == nullptr || ld_gate < width ||
      ld_out < width || (act != GATE_SILU && act != GATE_GELU_TANH) ||
      (other == nullptr) == (table == nullptr) || (other != nullptr && ld_other < width) ||
      (table != nullptr && (index == nullptr || col < 0 || ld_table < col + width ||
                            table_rows < 1))) {
    return AYK_BAD_ARGUMENT;
  }
  const int threads = 256, blocks = blocks_for((long long)rows * width, threads);
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return launch_kernel(gated_unit_kernel<float, float>, dim3(blocks), dim3(threads), 0, s, 1,
                         gate, ld_gate, other, ld_other, (const float*)table, ld_table, index,
                         table_rows, col, act, (float*)out, ld_out, rows, width);
  }
  if (type == 1) {
    return launch_kernel(gated_unit_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks),
                         dim3(threads), 0, s, 1, gate, ld_gate, other, ld_other,
                         (const __nv_bfloat16*)table, ld_table, index, table_rows, col, act,
                         (__nv_bfloat16*)out, ld_out, rows, width);
  }
  return AYK_BAD_ARGUMENT;
}

// act: 0 = tanh, 1 = the quadratic-exponential unit with `numbers` = (p, q). `bias` may be
// null. out_type: 0 = float32, 1 = bfloat16.
AYK_API int ayk_unary_rows(const float* x, int ld_x, const float* bias, int act,
                           const float* numbers, void* out, int ld_out, int rows, int width,
                           int out_type, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || width < 1 || x == nullptr || out == nullptr || ld_x < width ||
      ld_out < width || (act != UNARY_TANH && act != UNARY_XIELU) ||
      (act == UNARY_XIELU && numbers == nullptr)) {
    return AYK_BAD_ARGUMENT;
  }
  const int threads = 256, blocks = blocks_for((long long)rows * width, threads);
  cudaStream_t s = (cudaStream_t)stream;
  if (out_type == 0) {
    return launch_kernel(unary_rows_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, x, ld_x,
                         bias, act, numbers, (float*)out, ld_out, rows, width);
  }
  if (out_type == 1) {
    return launch_kernel(unary_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, 1,
                         x, ld_x, bias, act, numbers, (__nv_bfloat16*)out, ld_out, rows, width);
  }
  return AYK_BAD_ARGUMENT;
}
