// Layer norm with gain and bias, y = (x - mean) / sqrt(var + eps) * gain + bias (var: the mean of
// the squared deviations, taken in a second pass over the row), and the residual stream's steps
// of a layer that norms its sublayers' outputs as well as their inputs:
//
//   layer_norm          out = LN(x) (optionally of gathered rows)
//   post_norm_add       x += LN_post(y);  optionally out = LN_next(x): the norm on a sublayer's output,
//                       the residual add and the norm in front of the next sublayer in one pass
//   scaled_sum          out = s1 y1 + s2 y2
//   stream_inject       x += other + vector: what a pass of a looped stack adds before its first layer
//
// y is a sum of up to two scaled terms (two mixers side by side), each [T, H] in float32 or
// bfloat16 or float32 partial sums [S, T, H] of a product cut along k, added in index order.
// One block a row; a thread keeps up to LN_PER_THREAD elements in registers between the passes
// (wider rows are read again).  Statistics and the stream are 32-bit.
#include "common.cuh"

#define LN_PER_THREAD 8

struct LnTerm {
  const void* y;       // null: no term
  int bf16;            // the term's elements are bfloat16 (else float32)
  int n_partials;
  long long stride;    // elements between partial sums
  float scale;
};

__device__ __forceinline__ float ln_term(const LnTerm& t, size_t at) {
  if (t.y == nullptr) return 0.f;
  float v = 0.f;
  if (t.bf16) {
    v = __bfloat162float(((const __nv_bfloat16*)t.y)[at]);
  } else {
    const float* y = (const float*)t.y;
    for (int s = 0; s < t.n_partials; ++s) v += y[(size_t)s * t.stride + at];
  }
  return v * t.scale;
}

// mean and 1 / sqrt(var + eps) of the row's n values, which the caller hands over through `get`
template <typename F>
__device__ __forceinline__ void ln_statistics(F get, int n, float eps, float* scratch, float& mean, float& inv) {
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += get(i);
  mean = block_sum(s, scratch) / (float)n;
  float q = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float d = get(i) - mean;
    q += d * d;
  }
  inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)n + eps);
}

template <typename TO>
__global__ void __launch_bounds__(1024)
layer_norm_kernel(const float* __restrict__ x, const float* __restrict__ gain, const float* __restrict__ bias,
                  TO* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * hidden;
  TO* o = out + (size_t)r * hidden;
  const bool kept = hidden <= LN_PER_THREAD * (int)blockDim.x;
  float v[LN_PER_THREAD];
#pragma unroll
  for (int e = 0; e < LN_PER_THREAD; ++e) {
    const int i = threadIdx.x + e * blockDim.x;
    v[e] = (kept && i < hidden) ? xr[i] : 0.f;
  }
  float mean, inv;
  if (kept) {
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) s += v[e];
    mean = block_sum(s, scratch) / (float)hidden;
    float q = 0.f;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      const float d = i < hidden ? v[e] - mean : 0.f;
      q += d * d;
    }
    inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)hidden + eps);
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      if (i < hidden) o[i] = from_float<TO>((v[e] - mean) * inv * gain[i] + bias[i]);
    }
  } else {
    ln_statistics([&](int i) { return xr[i]; }, hidden, eps, scratch, mean, inv);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      o[i] = from_float<TO>((xr[i] - mean) * inv * gain[i] + bias[i]);
  }
}

template <typename TO>
__global__ void __launch_bounds__(1024)
post_norm_add_kernel(float* __restrict__ x, LnTerm t1, LnTerm t2, const float* __restrict__ gain,
                     const float* __restrict__ bias, float eps, const float* __restrict__ next_gain,
                     const float* __restrict__ next_bias, float next_eps, TO* __restrict__ out, int hidden) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const size_t base = (size_t)r * hidden;
  float* xr = x + base;
  const bool kept = hidden <= LN_PER_THREAD * (int)blockDim.x;
  if (kept) {
    float v[LN_PER_THREAD], xv[LN_PER_THREAD];
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      v[e] = i < hidden ? ln_term(t1, base + i) + ln_term(t2, base + i) : 0.f;
      xv[e] = i < hidden ? xr[i] : 0.f;
      s += v[e];
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float q = 0.f;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      const float d = i < hidden ? v[e] - mean : 0.f;
      q += d * d;
    }
    const float inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)hidden + eps);
    s = 0.f;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      if (i < hidden) {
        xv[e] += (v[e] - mean) * inv * gain[i] + bias[i];
        xr[i] = xv[e];
        s += xv[e];
      }
    }
    if (out == nullptr) return;
    const float mean2 = block_sum(s, scratch) / (float)hidden;
    q = 0.f;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      const float d = i < hidden ? xv[e] - mean2 : 0.f;
      q += d * d;
    }
    const float inv2 = 1.0f / sqrtf(block_sum(q, scratch) / (float)hidden + next_eps);
    TO* o = out + base;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      if (i < hidden) o[i] = from_float<TO>((xv[e] - mean2) * inv2 * next_gain[i] + next_bias[i]);
    }
    return;
  }
  float mean, inv;
  ln_statistics([&](int i) { return ln_term(t1, base + i) + ln_term(t2, base + i); }, hidden, eps, scratch, mean, inv);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    xr[i] += (ln_term(t1, base + i) + ln_term(t2, base + i) - mean) * inv * gain[i] + bias[i];
  if (out == nullptr) return;
  __syncthreads();
  ln_statistics([&](int i) { return xr[i]; }, hidden, next_eps, scratch, mean, inv);
  TO* o = out + base;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_float<TO>((xr[i] - mean) * inv * next_gain[i] + next_bias[i]);
}

__global__ void scaled_sum_kernel(LnTerm t1, LnTerm t2, float* __restrict__ out, size_t n) {
  pdl_wait();
  pdl_launch();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = ln_term(t1, i) + ln_term(t2, i);
}

// x[t, :] += other[t, :] (where given) + vector[:] (where given)
__global__ void stream_inject_kernel(float* __restrict__ x, const float* __restrict__ other,
                                     const float* __restrict__ vector, int hidden, size_t n) {
  pdl_wait();
  pdl_launch();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    x[i] += (other ? other[i] : 0.f) + (vector ? vector[i % hidden] : 0.f);
}

static inline int ln_threads(int hidden) {
  int threads = 128;   // rows of up to 4 elements a thread at first, 8 in the widest block
  while (threads < 1024 && hidden > threads * 4) threads *= 2;
  return threads;
}

static inline LnTerm ln_make_term(const void* y, int dtype, int n_partials, long long stride, float scale) {
  LnTerm t;
  t.y = y;
  t.bf16 = dtype == TOKB200_BF16;
  t.n_partials = n_partials;
  t.stride = stride;
  t.scale = scale;
  return t;
}

TOKB200_API int tokb200_layer_norm(const float* x, const float* gain, const float* bias, void* out, int out_dtype,
                                   const int* rows, int n_rows, int hidden, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (hidden <= 0) return TOKB200_BAD_SIZE;
  const int threads = ln_threads(hidden);
  if (out_dtype == TOKB200_F32)
    return launch_dependent(layer_norm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, gain, bias,
                            (float*)out, rows, hidden, eps);
  if (out_dtype == TOKB200_BF16)
    return launch_dependent(layer_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, gain,
                            bias, (__nv_bfloat16*)out, rows, hidden, eps);
  return TOKB200_BAD_DTYPE;
}

// y2 may be null (one term).  out may be null (no norm behind the add).
TOKB200_API int tokb200_post_norm_add(float* x, const void* y1, int y1_dtype, int y1_partials, long long y1_stride,
                                      float y1_scale, const void* y2, int y2_dtype, int y2_partials,
                                      long long y2_stride, float y2_scale, const float* gain, const float* bias,
                                      float eps, const float* next_gain, const float* next_bias, float next_eps,
                                      void* out, int out_dtype, int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (hidden <= 0 || y1 == nullptr || y1_partials < 1 || (y2 && y2_partials < 1)) return TOKB200_BAD_SIZE;
  if ((y1_dtype == TOKB200_BF16 && y1_partials != 1) || (y2 && y2_dtype == TOKB200_BF16 && y2_partials != 1))
    return TOKB200_BAD_DTYPE;
  const LnTerm t1 = ln_make_term(y1, y1_dtype, y1_partials, y1_stride, y1_scale);
  const LnTerm t2 = ln_make_term(y2, y2_dtype, y2_partials, y2_stride, y2_scale);
  const int threads = ln_threads(hidden);
  if (out == nullptr || out_dtype == TOKB200_F32)
    return launch_dependent(post_norm_add_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, t1, t2, gain,
                            bias, eps, next_gain, next_bias, next_eps, (float*)out, hidden);
  if (out_dtype == TOKB200_BF16)
    return launch_dependent(post_norm_add_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, t1, t2,
                            gain, bias, eps, next_gain, next_bias, next_eps, (__nv_bfloat16*)out, hidden);
  return TOKB200_BAD_DTYPE;
}

TOKB200_API int tokb200_scaled_sum(const void* y1, int y1_dtype, int y1_partials, long long y1_stride, float y1_scale,
                                   const void* y2, int y2_dtype, int y2_partials, long long y2_stride,
                                   float y2_scale, float* out, long long n, cudaStream_t stream) {
  if (n <= 0) return TOKB200_OK;
  if (y1 == nullptr || y1_partials < 1 || (y2 && y2_partials < 1)) return TOKB200_BAD_SIZE;
  const LnTerm t1 = ln_make_term(y1, y1_dtype, y1_partials, y1_stride, y1_scale);
  const LnTerm t2 = ln_make_term(y2, y2_dtype, y2_partials, y2_stride, y2_scale);
  const long long blocks = (n + 255) / 256;
  return launch_dependent(scaled_sum_kernel, dim3((unsigned)(blocks < 4096 ? blocks : 4096)), dim3(256), 0, stream,
                          t1, t2, out, (size_t)n);
}

TOKB200_API int tokb200_stream_inject(float* x, const float* other, const float* vector, int n_rows, int hidden,
                                      cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (hidden <= 0) return TOKB200_BAD_SIZE;
  const long long n = (long long)n_rows * hidden, blocks = (n + 255) / 256;
  return launch_dependent(stream_inject_kernel, dim3((unsigned)(blocks < 4096 ? blocks : 4096)), dim3(256), 0, stream,
                          x, other, vector, hidden, (size_t)n);
}
