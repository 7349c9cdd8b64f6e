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

// The three sums of a block in one pass over shared memory.
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float (*scratch)[33]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
  if (lane == 0) { scratch[0][warp] = a; scratch[1][warp] = b; scratch[2][warp] = c; }
  __syncthreads();
  if (warp < 3) {
    float v = lane < warps ? scratch[warp][lane] : 0.f;
    v = warp_sum(v);
    if (lane == 0) scratch[warp][32] = v;
  }
  __syncthreads();
  a = scratch[0][32]; b = scratch[1][32]; c = scratch[2][32];
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(1024)
poly_norm_kernel(const TI* __restrict__ z, const float* __restrict__ bias, int ld,
                 const float* __restrict__ coeff, TO* __restrict__ out, int n, float eps) {
  __shared__ float scratch[3][33];
  const int t = blockIdx.x;
  const float a = coeff[0], b = coeff[1], c = coeff[2], e = coeff[3];     // weights: no wait needed
  pdl_wait();
  pdl_launch();
  const TI* row = z + (size_t)t * ld;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = to_float(row[i]) + (bias ? bias[i] : 0.f);
    const float v2 = v * v;
    s2 += v2;
    s4 += v2 * v2;
    s6 += v2 * v2 * v2;
  }
  block_sum3(s2, s4, s6, scratch);
  const float inv_n = 1.0f / (float)n;
  const float r1 = a / sqrtf(s2 * inv_n + eps);
  const float r2 = b / sqrtf(s4 * inv_n + eps);
  const float r3 = c / sqrtf(s6 * inv_n + eps);
  TO* dst = out + (size_t)t * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = to_float(row[i]) + (bias ? bias[i] : 0.f);
    dst[i] = from_float<TO>(v * r1 + v * v * r2 + v * v * v * r3 + e);
  }
}

// float32 rows of a multiple of 4 lanes, 16-byte aligned, up to 8 x 4 values a thread kept in
// registers between the sums and the result: the row is read once, in 16-byte loads
#define POLY_VEC_MAX 8
__global__ void __launch_bounds__(256)
poly_norm_rows_kernel(const float* __restrict__ z, const float* __restrict__ bias, int ld,
                      const float* __restrict__ coeff, __nv_bfloat16* __restrict__ out, int n, float eps) {
  __shared__ float scratch[3][33];
  const int t = blockIdx.x;
  const float a = coeff[0], b = coeff[1], c = coeff[2], e = coeff[3];
  pdl_wait();
  pdl_launch();
  const float4* row = reinterpret_cast<const float4*>(z + (size_t)t * ld);
  const int n4 = n / 4;
  float4 v[POLY_VEC_MAX];
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
#pragma unroll
  for (int k = 0; k < POLY_VEC_MAX; ++k) {
    const int i = threadIdx.x + k * 256;
    v[k] = i < n4 ? __ldg(row + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias && i < n4) {
      const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias) + i);
      v[k].x += b4.x; v[k].y += b4.y; v[k].z += b4.z; v[k].w += b4.w;
    }
    const float x[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float v2 = x[j] * x[j];
      s2 += v2;
      s4 += v2 * v2;
      s6 += v2 * v2 * v2;
    }
  }
  block_sum3(s2, s4, s6, scratch);
  const float inv_n = 1.0f / (float)n;
  const float r1 = a / sqrtf(s2 * inv_n + eps);
  const float r2 = b / sqrtf(s4 * inv_n + eps);
  const float r3 = c / sqrtf(s6 * inv_n + eps);
  uint2* dst = reinterpret_cast<uint2*>(out + (size_t)t * n);
#pragma unroll
  for (int k = 0; k < POLY_VEC_MAX; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      const float x[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
      float y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = x[j] * r1 + x[j] * x[j] * r2 + x[j] * x[j] * x[j] * r3 + e;
      __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
      uint2 packed;
      packed.x = *reinterpret_cast<unsigned*>(&lo);
      packed.y = *reinterpret_cast<unsigned*>(&hi);
      dst[i] = packed;
    }
  }
}

// z + bias (one float32 a lane, or none: the bias of the product that made z) is the activation's input
TOKB200_API int tokb200_poly_norm(const void* z, int z_dtype, const float* bias, int ld, const float* coeff, void* out,
                                  int out_dtype, int n_rows, int n, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (n <= 0 || ld < n) return TOKB200_BAD_SIZE;
  if (z_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16 && n % 4 == 0 && ld % 4 == 0 &&
      n <= 4 * 256 * POLY_VEC_MAX && (((uintptr_t)z & 15) | ((uintptr_t)bias & 15) | ((uintptr_t)out & 7)) == 0)
    return launch_dependent(poly_norm_rows_kernel, dim3(n_rows), dim3(256), 0, stream, (const float*)z, bias, ld,
                            coeff, (__nv_bfloat16*)out, n, eps);
  int threads = 128;
  while (threads < 1024 && n > threads * 4) threads *= 2;
#define LAUNCH(TI, TO)                                                                          \
  return launch_dependent(poly_norm_kernel<TI, TO>, dim3(n_rows), dim3(threads), 0, stream,     \
                          (const TI*)z, bias, ld, coeff, (TO*)out, n, eps)
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
                   const float* __restrict__ bias, const TP* __restrict__ pre,
                   const float* __restrict__ pre_bias, int ld_pre,
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
    const float g = to_float(pre[(size_t)t * ld_pre + c]) + (pre_bias ? pre_bias[c] : 0.f);
    delta[i] = v / (1.0f + expf(-g));
  }
}

// float32 partial sums or a bfloat16 product, a float32 gate, 4 lanes a thread in 16-byte loads
template <typename TY>
__global__ void __launch_bounds__(256)
gated_delta_vec_kernel(const TY* __restrict__ y, int n_partials, size_t partial_stride,
                       const float* __restrict__ bias, const float* __restrict__ pre,
                       const float* __restrict__ pre_bias, int ld_pre,
                       float* __restrict__ delta, int n_rows, int hidden) {
  pdl_wait();
  pdl_launch();
  const int quads = hidden / 4;
  const size_t total = (size_t)n_rows * quads;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / quads), c = (int)(i % quads) * 4;
    const size_t at = (size_t)t * hidden + c;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < n_partials; ++s) {
      if constexpr (sizeof(TY) == 4) {
        const float4 p = *reinterpret_cast<const float4*>(y + (size_t)s * partial_stride + at);
        v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
      } else {
        const uint2 p = *reinterpret_cast<const uint2*>(y + (size_t)s * partial_stride + at);
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&p.x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&p.y);
        v[0] += __low2float(lo); v[1] += __high2float(lo); v[2] += __low2float(hi); v[3] += __high2float(hi);
      }
    }
    if (bias) {
      const float4 b = *reinterpret_cast<const float4*>(bias + c);
      v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
    }
    float4 g = *reinterpret_cast<const float4*>(pre + (size_t)t * ld_pre + c);
    if (pre_bias) {
      const float4 b = *reinterpret_cast<const float4*>(pre_bias + c);
      g.x += b.x; g.y += b.y; g.z += b.z; g.w += b.w;
    }
    float4 o;
    o.x = v[0] / (1.0f + expf(-g.x));
    o.y = v[1] / (1.0f + expf(-g.y));
    o.z = v[2] / (1.0f + expf(-g.z));
    o.w = v[3] / (1.0f + expf(-g.w));
    *reinterpret_cast<float4*>(delta + at) = o;
  }
}

TOKB200_API int tokb200_gated_delta(const void* y, int y_dtype, int n_partials, long long partial_stride,
                                    const float* bias, const void* pre, int pre_dtype, const float* pre_bias,
                                    int ld_pre, float* delta, int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (hidden <= 0 || ld_pre < hidden || n_partials < 1) return TOKB200_BAD_SIZE;
  const size_t total = (size_t)n_rows * hidden;
  if (pre_dtype == TOKB200_F32 && hidden % 4 == 0 && ld_pre % 4 == 0 && partial_stride % 4 == 0 &&
      (((uintptr_t)y | (uintptr_t)bias | (uintptr_t)pre | (uintptr_t)pre_bias | (uintptr_t)delta) & 15) == 0) {
    const size_t quads = total / 4;
    const unsigned vec_blocks = (unsigned)((quads + 255) / 256 > 148 * 16 ? 148 * 16 : (quads + 255) / 256);
    if (y_dtype == TOKB200_F32)
      return launch_dependent(gated_delta_vec_kernel<float>, dim3(vec_blocks), dim3(256), 0, stream, (const float*)y,
                              n_partials, (size_t)partial_stride, bias, (const float*)pre, pre_bias, ld_pre, delta, n_rows,
                              hidden);
    if (y_dtype == TOKB200_BF16)
      return launch_dependent(gated_delta_vec_kernel<__nv_bfloat16>, dim3(vec_blocks), dim3(256), 0, stream,
                              (const __nv_bfloat16*)y, n_partials, (size_t)partial_stride, bias, (const float*)pre,
                              pre_bias, ld_pre, delta, n_rows, hidden);
  }
  const unsigned blocks = (unsigned)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
#define LAUNCH(TY, TP)                                                                         \
  return launch_dependent(gated_delta_kernel<TY, TP>, dim3(blocks), dim3(256), 0, stream,      \
                          (const TY*)y, n_partials, (size_t)partial_stride, bias, (const TP*)pre, \
                          pre_bias, ld_pre, delta, n_rows, hidden)
  if (y_dtype == TOKB200_F32 && pre_dtype == TOKB200_F32) LAUNCH(float, float);
  if (y_dtype == TOKB200_BF16 && pre_dtype == TOKB200_F32) LAUNCH(__nv_bfloat16, float);
  if (y_dtype == TOKB200_BF16 && pre_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (y_dtype == TOKB200_F32 && pre_dtype == TOKB200_BF16) LAUNCH(float, __nv_bfloat16);
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}

// ---- the gate, the residual add and the norm that follows, in one pass over the row ----
// x[t,:] += (sum_s y[s,t,:] + bias) * sigmoid(pre[t,:] + pre_bias);  out[t,:] = x / sqrt(mean(x^2) + eps) * gain.
// A block a row; a thread keeps up to GN_KEEP of its lanes' new values in registers between the sum
// of squares and the result (rows beyond 256 * GN_KEEP lanes read the rest back from x).
#define GN_KEEP 16
template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
gated_add_rms_norm_kernel(float* __restrict__ x, const TY* __restrict__ y, int n_partials, size_t partial_stride,
                          const float* __restrict__ bias, const float* __restrict__ pre,
                          const float* __restrict__ pre_bias, int ld_pre, const float* __restrict__ gain,
                          float eps, TO* __restrict__ out, int hidden) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  pdl_wait();
  pdl_launch();
  float* row = x + (size_t)t * hidden;
  const float* gate = pre + (size_t)t * ld_pre;
  float kept[GN_KEEP];
  float sq = 0.f;
#pragma unroll
  for (int k = 0; k < GN_KEEP; ++k) {
    const int c = threadIdx.x + k * 256;
    kept[k] = 0.f;
    if (c < hidden) {
      float v = 0.f;
      for (int s = 0; s < n_partials; ++s) v += to_float(y[(size_t)s * partial_stride + (size_t)t * hidden + c]);
      if (bias) v += bias[c];
      const float g = gate[c] + (pre_bias ? pre_bias[c] : 0.f);
      const float now = row[c] + v / (1.0f + expf(-g));
      row[c] = now;
      kept[k] = now;
      sq += now * now;
    }
  }
  for (int c = threadIdx.x + GN_KEEP * 256; c < hidden; c += 256) {
    float v = 0.f;
    for (int s = 0; s < n_partials; ++s) v += to_float(y[(size_t)s * partial_stride + (size_t)t * hidden + c]);
    if (bias) v += bias[c];
    const float g = gate[c] + (pre_bias ? pre_bias[c] : 0.f);
    const float now = row[c] + v / (1.0f + expf(-g));
    row[c] = now;
    sq += now * now;
  }
  sq = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(sq / (float)hidden + eps);
  TO* dst = out + (size_t)t * hidden;
#pragma unroll
  for (int k = 0; k < GN_KEEP; ++k) {
    const int c = threadIdx.x + k * 256;
    if (c < hidden) dst[c] = from_float<TO>(kept[k] * inv * gain[c]);
  }
  for (int c = threadIdx.x + GN_KEEP * 256; c < hidden; c += 256) dst[c] = from_float<TO>(row[c] * inv * gain[c]);
}

// The same in 16-byte pieces: rows of a multiple of 4 lanes up to 256 * 4 * GN_QUADS, every pointer
// 16-byte aligned.  All of a piece's loads (the planes of y, x, the gate) are independent and issued
// together; the new values stay in registers for the result.
#define GN_QUADS 8
__device__ __forceinline__ float4 gn_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 gn_load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
gated_add_rms_norm_vec_kernel(float* __restrict__ x, const TY* __restrict__ y, int n_partials, size_t partial_stride,
                              const float* __restrict__ bias, const float* __restrict__ pre,
                              const float* __restrict__ pre_bias, int ld_pre, const float* __restrict__ gain,
                              float eps, TO* __restrict__ out, int hidden) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int quads = hidden / 4;
  pdl_wait();
  pdl_launch();
  float* row = x + (size_t)t * hidden;
  const float* gate = pre + (size_t)t * ld_pre;
  const TY* y_row = y + (size_t)t * hidden;
  float4 kept[GN_QUADS];
  float sq = 0.f;
#pragma unroll
  for (int k = 0; k < GN_QUADS; ++k) {
    const int c = (threadIdx.x + k * 256) * 4;
    kept[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < hidden) {
      float4 v = gn_load4(y_row + c);
#pragma unroll 8
      for (int s = 1; s < n_partials; ++s) {
        const float4 p = gn_load4(y_row + (size_t)s * partial_stride + c);
        v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
      }
      float4 g = gn_load4(gate + c);
      const float4 old = gn_load4(row + c);
      if (bias) { const float4 b = gn_load4(bias + c); v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w; }
      if (pre_bias) { const float4 b = gn_load4(pre_bias + c); g.x += b.x; g.y += b.y; g.z += b.z; g.w += b.w; }
      float4 now;
      now.x = old.x + v.x / (1.0f + expf(-g.x));
      now.y = old.y + v.y / (1.0f + expf(-g.y));
      now.z = old.z + v.z / (1.0f + expf(-g.z));
      now.w = old.w + v.w / (1.0f + expf(-g.w));
      *reinterpret_cast<float4*>(row + c) = now;
      kept[k] = now;
      sq += now.x * now.x + now.y * now.y + now.z * now.z + now.w * now.w;
    }
  }
  sq = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(sq / (float)hidden + eps);
  TO* dst = out + (size_t)t * hidden;
#pragma unroll
  for (int k = 0; k < GN_QUADS; ++k) {
    const int c = (threadIdx.x + k * 256) * 4;
    if (c < hidden) {
      const float4 w = gn_load4(gain + c);
      const float r0 = kept[k].x * inv * w.x, r1 = kept[k].y * inv * w.y;
      const float r2 = kept[k].z * inv * w.z, r3 = kept[k].w * inv * w.w;
      if constexpr (sizeof(TO) == 4) {
        *reinterpret_cast<float4*>(dst + c) = make_float4(r0, r1, r2, r3);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
        uint2 packed;
        packed.x = *reinterpret_cast<unsigned*>(&lo);
        packed.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(dst + c) = packed;
      }
    }
  }
  (void)quads;
}

TOKB200_API int tokb200_gated_add_rms_norm(float* x, const void* y, int y_dtype, int n_partials,
                                           long long partial_stride, const float* bias, const void* pre,
                                           int pre_dtype, const float* pre_bias, int ld_pre, const float* gain,
                                           float eps, void* out, int out_dtype, int n_rows, int hidden,
                                           cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (hidden <= 0 || ld_pre < hidden || n_partials < 1) return TOKB200_BAD_SIZE;
  if (pre_dtype != TOKB200_F32) return TOKB200_BAD_DTYPE;
  if (hidden % 4 == 0 && hidden <= 256 * 4 * GN_QUADS && ld_pre % 4 == 0 && partial_stride % 4 == 0 &&
      (((uintptr_t)x | (uintptr_t)y | (uintptr_t)bias | (uintptr_t)pre | (uintptr_t)pre_bias | (uintptr_t)gain |
        (uintptr_t)out) & 15) == 0) {
#define LAUNCH_VEC(TY, TO)                                                                              \
  return launch_dependent(gated_add_rms_norm_vec_kernel<TY, TO>, dim3(n_rows), dim3(256), 0, stream, x, \
                          (const TY*)y, n_partials, (size_t)partial_stride, bias, (const float*)pre,    \
                          pre_bias, ld_pre, gain, eps, (TO*)out, hidden)
    if (y_dtype == TOKB200_F32 && out_dtype == TOKB200_F32) LAUNCH_VEC(float, float);
    if (y_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16) LAUNCH_VEC(float, __nv_bfloat16);
    if (y_dtype == TOKB200_BF16 && out_dtype == TOKB200_BF16) LAUNCH_VEC(__nv_bfloat16, __nv_bfloat16);
    if (y_dtype == TOKB200_BF16 && out_dtype == TOKB200_F32) LAUNCH_VEC(__nv_bfloat16, float);
#undef LAUNCH_VEC
  }
#define LAUNCH(TY, TO)                                                                                  \
  return launch_dependent(gated_add_rms_norm_kernel<TY, TO>, dim3(n_rows), dim3(256), 0, stream, x,     \
                          (const TY*)y, n_partials, (size_t)partial_stride, bias, (const float*)pre,    \
                          pre_bias, ld_pre, gain, eps, (TO*)out, hidden)
  if (y_dtype == TOKB200_F32 && out_dtype == TOKB200_F32) LAUNCH(float, float);
  if (y_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16) LAUNCH(float, __nv_bfloat16);
  if (y_dtype == TOKB200_BF16 && out_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (y_dtype == TOKB200_BF16 && out_dtype == TOKB200_F32) LAUNCH(__nv_bfloat16, float);
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}
