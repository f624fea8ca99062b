// RMS norms of the post-norm residual layout, for bf16 or fp32 activations:
//
//   llmctl_postnorm_residual : x += g * y / sqrt(mean(y^2) + eps)   (the sublayer OUTPUT is normed, with a single
//                              gain g for all coordinates); x is the fp32 residual stream, which is also written
//                              out in the activation type for the next matrix product.
//   llmctl_scalar_rmsnorm    : out[r] = g * x[rows[r]] / sqrt(mean(x[rows[r]]^2) + eps) for a list of rows of the
//                              fp32 stream (final norm before the output head, only where logits are wanted).
//
// Sums and the residual are fp32 whatever the activation type.  One CTA per row.
// Reference: none (the reference has no model code; reference llmctl/runtime/engine.py:119-140 loads HF models).
#include "../common/dtype.cuh"

namespace llmctl {

template <typename Ty, typename Tx>
__global__ void __launch_bounds__(256)
postnorm_residual_kernel(const Ty* __restrict__ y, long long ldy, float* __restrict__ x, Tx* __restrict__ x_act,
                         const float* __restrict__ gain, int cols, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const Ty* yr = y + row * ldy;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = to_f32(yr[c]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = gain[0] / sqrtf(ss / static_cast<float>(cols) + eps);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = x[row * cols + c] + to_f32(yr[c]) * r;
    x[row * cols + c] = v;
    if (x_act) x_act[row * cols + c] = from_f32<Tx>(v);
  }
}

template <typename To>
__global__ void __launch_bounds__(256)
scalar_rmsnorm_kernel(const float* __restrict__ x, const long long* __restrict__ rows, To* __restrict__ out,
                      const float* __restrict__ gain, int cols, float eps) {
  __shared__ float red[32];
  const long long src = rows ? rows[blockIdx.x] : blockIdx.x;
  const float* xr = x + src * cols;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) ss += xr[c] * xr[c];
  ss = block_sum(ss, red);
  const float r = gain[0] / sqrtf(ss / static_cast<float>(cols) + eps);
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    out[static_cast<long long>(blockIdx.x) * cols + c] = from_f32<To>(xr[c] * r);
}

// x[t] = table[token[t]] * scale, in fp32 and in the activation type.
template <typename T>
__global__ void __launch_bounds__(256)
embed_scale_kernel(const long long* __restrict__ tokens, const T* __restrict__ table, float scale,
                   float* __restrict__ x, T* __restrict__ x_act, int cols) {
  const long long row = blockIdx.x;
  const T* src = table + tokens[row] * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = to_f32(src[c]) * scale;
    x[row * cols + c] = v;
    if (x_act) x_act[row * cols + c] = from_f32<T>(v);
  }
}

// v <- cap * tanh(v / cap), fp32 in place.
__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ v, long long n, float cap) {
  const float inv = 1.f / cap;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    v[i] = cap * tanhf(v[i] * inv);
}

}  // namespace llmctl

using namespace llmctl;

// y: [rows, cols] (fp32 if y_fp32 else bf16, row stride ldy); x: fp32 [rows, cols] updated in place;
// x_act: optional copy of the new x (fp32 if act_fp32 else bf16); gain: one fp32 number on the device.
LLMCTL_API int llmctl_postnorm_residual(const void* y, int y_fp32, long long ldy, float* x, void* x_act, int act_fp32,
                                        const float* gain, int rows, int cols, float eps, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(cols > 0 && rows >= 0 && ldy >= cols);
  if (rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (y_fp32 && act_fp32)
    postnorm_residual_kernel<float, float><<<rows, 256, 0, s>>>((const float*)y, ldy, x, (float*)x_act, gain, cols, eps);
  else if (y_fp32)
    postnorm_residual_kernel<float, __nv_bfloat16><<<rows, 256, 0, s>>>((const float*)y, ldy, x, (__nv_bfloat16*)x_act, gain, cols, eps);
  else if (act_fp32)
    postnorm_residual_kernel<__nv_bfloat16, float><<<rows, 256, 0, s>>>((const __nv_bfloat16*)y, ldy, x, (float*)x_act, gain, cols, eps);
  else
    postnorm_residual_kernel<__nv_bfloat16, __nv_bfloat16><<<rows, 256, 0, s>>>((const __nv_bfloat16*)y, ldy, x, (__nv_bfloat16*)x_act, gain, cols, eps);
  LLMCTL_RETURN_LAST();
}

LLMCTL_API int llmctl_scalar_rmsnorm(const float* x, const long long* rows, void* out, int out_fp32, const float* gain,
                                     int n_out, int cols, float eps, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(cols > 0 && n_out >= 0);
  if (n_out == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(out_fp32, T, (scalar_rmsnorm_kernel<T><<<n_out, 256, 0, (cudaStream_t)stream>>>(x, rows, (T*)out, gain, cols, eps)));
  LLMCTL_RETURN_LAST();
}

LLMCTL_API int llmctl_embed_scale(const long long* tokens, const void* table, int is_fp32, float scale, float* x,
                                  void* x_act, int rows, int cols, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(cols > 0 && rows >= 0);
  if (rows == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (embed_scale_kernel<T><<<rows, 256, 0, (cudaStream_t)stream>>>(tokens, (const T*)table, scale, x, (T*)x_act, cols)));
  LLMCTL_RETURN_LAST();
}

LLMCTL_API int llmctl_softcap(float* v, long long n, float cap, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(cap > 0.f);
  if (n == 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > kNumSMs * 8) blocks = kNumSMs * 8;
  softcap_kernel<<<static_cast<int>(blocks), 256, 0, (cudaStream_t)stream>>>(v, n, cap);
  LLMCTL_RETURN_LAST();
}
