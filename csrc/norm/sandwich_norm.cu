// RMS norms with per-coordinate weights around an fp32 residual stream ("sandwich" layout: every sublayer is normed
// on its way in and on its way out), for bf16 or fp32 activations:
//
//   llmctl_embed_positions   : x[t] = table[token[t]] + pos_table[position[t]]        (learned absolute positions)
//   llmctl_rmsnorm_rows      : out[r] = w * x[rows[r]] / sqrt(mean(x[rows[r]]^2) + eps) for all or selected rows
//   llmctl_sandwich_residual : x += wb * y / sqrt(mean(y^2) + eps), and in the same pass, when w_next is given,
//                              out = w_next * x / sqrt(mean(x^2) + eps) for the next sublayer (also unrounded in fp32
//                              when out32 is given: a router reads that)
//
// The stream, the sums and the weights are fp32 whatever the activation type; only `y` (a GEMM's output) and `out`
// (a GEMM's input) have the activation type.  One CTA per row.
// Reference: none (the reference has no model code; reference llmctl/runtime/engine.py:119-140 loads HF models).
#include "../common/dtype.cuh"

namespace llmctl {

template <typename T>
__global__ void __launch_bounds__(256)
embed_positions_kernel(const long long* __restrict__ tokens, const int* __restrict__ positions, const T* __restrict__ table,
                       const T* __restrict__ pos_table, float* __restrict__ x, int cols) {
  const long long row = blockIdx.x;
  const T* a = table + tokens[row] * cols;
  const T* b = pos_table + static_cast<long long>(positions[row]) * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) x[row * cols + c] = to_f32(a[c]) + to_f32(b[c]);
}

template <typename To>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const float* __restrict__ x, const long long* __restrict__ rows, const float* __restrict__ w,
                    To* __restrict__ out, int cols, float eps) {
  __shared__ float red[32];
  const long long src = rows ? rows[blockIdx.x] : blockIdx.x;
  const float* xr = x + src * cols;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) ss += xr[c] * xr[c];
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / static_cast<float>(cols) + eps);
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    out[static_cast<long long>(blockIdx.x) * cols + c] = from_f32<To>(xr[c] * r * w[c]);
}

template <typename Ty, typename To>
__global__ void __launch_bounds__(256)
sandwich_residual_kernel(const Ty* __restrict__ y, long long ldy, float* __restrict__ x, const float* __restrict__ wb,
                         const float* __restrict__ w_next, To* __restrict__ out, float* __restrict__ out32, int cols, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const Ty* yr = y + row * ldy;
  float* xr = x + row * cols;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = to_f32(yr[c]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / static_cast<float>(cols) + eps);
  float sx = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {       // every thread re-reads only what it wrote itself
    const float v = xr[c] + to_f32(yr[c]) * r * wb[c];
    xr[c] = v;
    sx += v * v;
  }
  if (!w_next) return;
  sx = block_sum(sx, red);
  const float r2 = 1.f / sqrtf(sx / static_cast<float>(cols) + eps);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = xr[c] * r2 * w_next[c];
    out[row * cols + c] = from_f32<To>(v);
    if (out32) out32[row * cols + c] = v;
  }
}

}  // namespace llmctl

using namespace llmctl;

LLMCTL_API int llmctl_embed_positions(const long long* tokens, const int* positions, const void* table, const void* pos_table,
                                      int is_fp32, float* x, int rows, int cols, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(cols > 0 && rows >= 0);
  if (rows == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (embed_positions_kernel<T><<<rows, 256, 0, (cudaStream_t)stream>>>(
      tokens, positions, (const T*)table, (const T*)pos_table, x, cols)));
  LLMCTL_RETURN_LAST();
}

// x: fp32 [*, cols]; rows: int64 [n_out] or null (then rows 0..n_out-1); w: fp32 [cols]; out: [n_out, cols].
LLMCTL_API int llmctl_rmsnorm_rows(const float* x, const long long* rows, const float* w, void* out, int out_fp32, int n_out,
                                   int cols, float eps, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(cols > 0 && n_out >= 0);
  if (n_out == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(out_fp32, T, (rmsnorm_rows_kernel<T><<<n_out, 256, 0, (cudaStream_t)stream>>>(x, rows, w, (T*)out, cols, eps)));
  LLMCTL_RETURN_LAST();
}

// y: [rows, cols] (fp32 if y_fp32 else bf16, row stride ldy); x: fp32 [rows, cols] updated in place; wb, w_next: fp32
// [cols]; out: [rows, cols] (fp32 if out_fp32 else bf16), written when w_next is not null; out32: optional fp32 copy of out
// before rounding.
LLMCTL_API int llmctl_sandwich_residual(const void* y, int y_fp32, long long ldy, float* x, const float* wb, const float* w_next,
                                        void* out, int out_fp32, float* out32, int rows, int cols, float eps, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(cols > 0 && rows >= 0 && ldy >= cols && (w_next == nullptr || out != nullptr));
  if (rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (y_fp32 && out_fp32)
    sandwich_residual_kernel<float, float><<<rows, 256, 0, s>>>((const float*)y, ldy, x, wb, w_next, (float*)out, out32, cols, eps);
  else if (y_fp32)
    sandwich_residual_kernel<float, __nv_bfloat16><<<rows, 256, 0, s>>>((const float*)y, ldy, x, wb, w_next, (__nv_bfloat16*)out, out32, cols, eps);
  else if (out_fp32)
    sandwich_residual_kernel<__nv_bfloat16, float><<<rows, 256, 0, s>>>((const __nv_bfloat16*)y, ldy, x, wb, w_next, (float*)out, out32, cols, eps);
  else
    sandwich_residual_kernel<__nv_bfloat16, __nv_bfloat16><<<rows, 256, 0, s>>>((const __nv_bfloat16*)y, ldy, x, wb, w_next, (__nv_bfloat16*)out, out32, cols, eps);
  LLMCTL_RETURN_LAST();
}
