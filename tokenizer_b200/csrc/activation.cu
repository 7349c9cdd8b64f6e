// Activations and gates that work on whole rows.
//
// PolyNorm: act[t,:] = a N(z) + b N(z^2) + c N(z^3) + e for a token's vector z, powers taken
// element by element, N(v) = v / sqrt(mean(v^2) + eps) over the vector.  The three mean squares
// and the result are 32-bit; the four numbers come from a small tensor on the device.
//
// Gated residual: delta[t,c] = (sum_s y[s,t,c] + bias[c]) * sigmoid(pre[t,c]): a sublayer's
// output (possibly float32 partial sums of a product cut along k, possibly still lacking its
// bias) times the gate whose pre-activation a projection of the sublayer's input produced.
// The result is float32: it is what the residual stream adds.
#include "common.cuh"

template <typename TI, typename TO>
__global__ void __launch_bounds__(1024)
poly_norm_kernel(const TI* __restrict__ z, int ld, const float* __restrict__ coeff,
                 TO* __restrict__ out, int n, float eps) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const float a = coeff[0], b = coeff[1], c = coeff[2], e = coeff[3];     // weights: no wait needed
  pdl_wait();
  pdl_launch();
  const TI* row = z + (size_t)t * ld;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = to_float(row[i]);
    const float v2 = v * v;
    s2 += v2;
    s4 += v2 * v2;
    s6 += v2 * v2 * v2;
  }
  s2 = block_sum(s2, scratch);
  s4 = block_sum(s4, scratch);
  s6 = block_sum(s6, scratch);
  const float inv_n = 1.0f / (float)n;
  const float r1 = a / sqrtf(s2 * inv_n + eps);
  const float r2 = b / sqrtf(s4 * inv_n + eps);
  const float r3 = c / sqrtf(s6 * inv_n + eps);
  TO* dst = out + (size_t)t * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = to_float(row[i]);
    dst[i] = from_float<TO>(v * r1 + v * v * r2 + v * v * v * r3 + e);
  }
}

TOKB200_API int tokb200_poly_norm(const void* z, int z_dtype, int ld, const float* coeff, void* out,
                                  int out_dtype, int n_rows, int n, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (n <= 0 || ld < n) return TOKB200_BAD_SIZE;
  int threads = 128;
  while (threads < 1024 && n > threads * 4) threads *= 2;
#define LAUNCH(TI, TO)                                                                          \
  return launch_dependent(poly_norm_kernel<TI, TO>, dim3(n_rows), dim3(threads), 0, stream,     \
                          (const TI*)z, ld, coeff, (TO*)out, n, eps)
  if (z_dtype == TOKB200_F32 && out_dtype == TOKB200_F32) LAUNCH(float, float);
  if (z_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16) LAUNCH(float, __nv_bfloat16);
  if (z_dtype == TOKB200_BF16 && out_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (z_dtype == TOKB200_BF16 && out_dtype == TOKB200_F32) LAUNCH(__nv_bfloat16, float);
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}

template <typename TY, typename TP>
__global__ void __launch_bounds__(256)
gated_delta_kernel(const TY* __restrict__ y, int n_partials, size_t partial_stride,
                   const float* __restrict__ bias, const TP* __restrict__ pre, int ld_pre,
                   float* __restrict__ delta, int n_rows, int hidden) {
  pdl_wait();
  pdl_launch();
  const size_t total = (size_t)n_rows * hidden;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / hidden), c = (int)(i % hidden);
    float v = 0.f;
    for (int s = 0; s < n_partials; ++s) v += to_float(y[(size_t)s * partial_stride + i]);
    if (bias) v += bias[c];
    const float g = to_float(pre[(size_t)t * ld_pre + c]);
    delta[i] = v / (1.0f + expf(-g));
  }
}

TOKB200_API int tokb200_gated_delta(const void* y, int y_dtype, int n_partials, long long partial_stride,
                                    const float* bias, const void* pre, int pre_dtype, int ld_pre,
                                    float* delta, int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (hidden <= 0 || ld_pre < hidden || n_partials < 1) return TOKB200_BAD_SIZE;
  const size_t total = (size_t)n_rows * hidden;
  const unsigned blocks = (unsigned)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
#define LAUNCH(TY, TP)                                                                         \
  return launch_dependent(gated_delta_kernel<TY, TP>, dim3(blocks), dim3(256), 0, stream,      \
                          (const TY*)y, n_partials, (size_t)partial_stride, bias, (const TP*)pre, \
                          ld_pre, delta, n_rows, hidden)
  if (y_dtype == TOKB200_F32 && pre_dtype == TOKB200_F32) LAUNCH(float, float);
  if (y_dtype == TOKB200_BF16 && pre_dtype == TOKB200_F32) LAUNCH(__nv_bfloat16, float);
  if (y_dtype == TOKB200_BF16 && pre_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (y_dtype == TOKB200_F32 && pre_dtype == TOKB200_BF16) LAUNCH(float, __nv_bfloat16);
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}
