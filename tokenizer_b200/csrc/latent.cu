// The small kernels around attention over a cached latent.
//
// latent_prepare: one projection's output row holds, side by side, a query latent (q_rank
// lanes), a key/value latent (kv_rank lanes) and a key part that carries the position (rot_dim
// lanes, possibly none).  Per token: the query latent is RMS-normed with its gain and written
// out dense; the key/value latent is RMS-normed with its gain and written to the token's cache
// row; the positional key part is rotated at the token's position and written behind it in the
// same cache row.  Norm statistics, angles, sines and cosines are 32-bit.
//
// rotate_interleaved: rotary encoding with lane 2i paired with lane 2i + 1, on `dims` lanes
// starting at `lane0` of every head's vector, in place; angle = position * inv_freq[i].
#include "common.cuh"

// a warp a token: the row's two sums by shuffles, no barrier; the second pass over the row hits L1
#define LAT_WARPS 8
template <typename TI, typename TO>
__global__ void __launch_bounds__(LAT_WARPS * 32)
latent_prepare_kernel(const TI* __restrict__ proj, int ld, int q_at, int q_rank, int c_at,
                      int kv_rank, int rot_dim, int rot_dims, const float* __restrict__ q_gain,
                      const float* __restrict__ c_gain, float eps,
                      const float* __restrict__ inv_freq, const int* __restrict__ pos,
                      const int* __restrict__ row_req, const int* __restrict__ slot,
                      TO* __restrict__ q_latent, TO* __restrict__ pool, int pool_row, int n_rows) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * LAT_WARPS + (threadIdx.x >> 5);
  const bool have = t < n_rows;
  const int r = have ? row_req[t] : -1;
  const int p = have ? pos[t] : 0;
  const int where = (have && slot) ? slot[t] : -1;
  pdl_wait();
  pdl_launch();
  if (r < 0) return;
  const TI* row = proj + (size_t)t * ld;
  float sq = 0.f, sc = 0.f;
  for (int i = lane; i < q_rank; i += 32) {
    const float v = to_float(row[q_at + i]);
    sq += v * v;
  }
  for (int i = lane; i < kv_rank; i += 32) {
    const float v = to_float(row[c_at + i]);
    sc += v * v;
  }
  sq = warp_sum(sq);
  sc = warp_sum(sc);
  const float inv_q = 1.0f / sqrtf(sq / (float)q_rank + eps);
  const float inv_c = 1.0f / sqrtf(sc / (float)kv_rank + eps);
  TO* q_dst = q_latent + (size_t)t * q_rank;
  for (int i = lane; i < q_rank; i += 32)
    q_dst[i] = from_float<TO>(to_float(row[q_at + i]) * inv_q * q_gain[i]);
  if (where < 0) return;
  TO* c_dst = pool + (size_t)where * pool_row;
  for (int i = lane; i < kv_rank; i += 32)
    c_dst[i] = from_float<TO>(to_float(row[c_at + i]) * inv_c * c_gain[i]);
  const TI* k_rot = row + c_at + kv_rank;
  for (int i = lane; i < rot_dim; i += 32) {
    float value = to_float(k_rot[i]);
    if (i < rot_dims) {          // lane 2j pairs with lane 2j + 1; the lanes behind rot_dims pass
      float s, c;
      sincosf((float)p * inv_freq[i >> 1], &s, &c);
      const float other = to_float(k_rot[i ^ 1]);
      value = (i & 1) ? value * c + other * s : value * c - other * s;
    }
    c_dst[kv_rank + i] = from_float<TO>(value);
  }
}

TOKB200_API int tokb200_latent_prepare(const void* proj, int proj_dtype, int ld, int q_at, int q_rank,
                                       int c_at, int kv_rank, int rot_dim, int rot_dims,
                                       const float* q_gain, const float* c_gain, float eps,
                                       const float* inv_freq, const int* pos, const int* row_req,
                                       const int* slot, void* q_latent, void* pool, int pool_row,
                                       int out_dtype, int n_rows, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (q_rank <= 0 || kv_rank <= 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1) ||
      pool_row < kv_rank + rot_dim || q_at + q_rank > ld || c_at + kv_rank + rot_dim > ld)
    return TOKB200_BAD_SIZE;
#define LAUNCH(TI, TO)                                                                           \
  return launch_dependent(latent_prepare_kernel<TI, TO>, dim3((n_rows + LAT_WARPS - 1) / LAT_WARPS),  \
                          dim3(LAT_WARPS * 32), 0, stream,                                        \
                          (const TI*)proj, ld, q_at, q_rank, c_at, kv_rank, rot_dim, rot_dims,   \
                          q_gain, c_gain, eps, inv_freq, pos, row_req, slot, (TO*)q_latent,      \
                          (TO*)pool, pool_row, n_rows)
  if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_F32) LAUNCH(float, float);
  if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16) LAUNCH(float, __nv_bfloat16);
  if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}

// x: [rows, heads, head_row]; pairs (lane0 + 2i, lane0 + 2i + 1), i < dims / 2, are rotated
template <typename T>
__global__ void __launch_bounds__(256)
rotate_interleaved_kernel(T* __restrict__ x, int heads, int head_row, int lane0, int dims,
                          const float* __restrict__ inv_freq, const int* __restrict__ pos,
                          const int* __restrict__ row_req, int n_rows) {
  pdl_wait();
  pdl_launch();
  const int half = dims / 2;
  const size_t total = (size_t)n_rows * heads * half;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int pair = (int)(i % half);
    const size_t th = i / half;
    const int t = (int)(th / heads);
    if (row_req[t] < 0) continue;
    float s, c;
    sincosf((float)pos[t] * inv_freq[pair], &s, &c);
    T* at = x + th * head_row + lane0 + 2 * pair;
    const float u = to_float(at[0]), v = to_float(at[1]);
    at[0] = from_float<T>(u * c - v * s);
    at[1] = from_float<T>(v * c + u * s);
  }
}

// bfloat16, 8 lanes (four pairs, 16 bytes) a thread: for rotated ranges that start and end on 16 bytes
__global__ void __launch_bounds__(256)
rotate_interleaved_vec_kernel(__nv_bfloat16* __restrict__ x, int heads, int head_row, int lane0, int dims,
                              const float* __restrict__ inv_freq, const int* __restrict__ pos,
                              const int* __restrict__ row_req, int n_rows) {
  pdl_wait();
  pdl_launch();
  const int pieces = dims / 8;
  const size_t total = (size_t)n_rows * heads * pieces;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int piece = (int)(i % pieces);
    const size_t th = i / pieces;
    const int t = (int)(th / heads);
    if (row_req[t] < 0) continue;
    const float p = (float)pos[t];
    uint4* at = reinterpret_cast<uint4*>(x + th * head_row + lane0 + 8 * piece);
    uint4 v = *at;
    __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float s, c;
      sincosf(p * inv_freq[4 * piece + k], &s, &c);
      const float u = __low2float(pairs[k]), w = __high2float(pairs[k]);
      pairs[k] = __floats2bfloat162_rn(u * c - w * s, w * c + u * s);
    }
    *at = v;
  }
}

TOKB200_API int tokb200_rotate_interleaved(void* x, int dtype, int heads, int head_row, int lane0, int dims,
                                           const float* inv_freq, const int* pos, const int* row_req,
                                           int n_rows, cudaStream_t stream) {
  if (n_rows <= 0 || dims <= 0) return TOKB200_OK;
  if (heads <= 0 || (dims & 1) || lane0 < 0 || lane0 + dims > head_row) return TOKB200_BAD_SIZE;
  if (dtype == TOKB200_BF16 && dims % 8 == 0 && lane0 % 8 == 0 && head_row % 8 == 0 && ((uintptr_t)x & 15) == 0) {
    const size_t pieces = (size_t)n_rows * heads * (dims / 8);
    const unsigned vec_blocks = (unsigned)((pieces + 255) / 256 > 148 * 16 ? 148 * 16 : (pieces + 255) / 256);
    return launch_dependent(rotate_interleaved_vec_kernel, dim3(vec_blocks), dim3(256), 0, stream, (__nv_bfloat16*)x,
                            heads, head_row, lane0, dims, inv_freq, pos, row_req, n_rows);
  }
  const size_t total = (size_t)n_rows * heads * (dims / 2);
  const unsigned blocks = (unsigned)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
  if (dtype == TOKB200_F32)
    return launch_dependent(rotate_interleaved_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x,
                            heads, head_row, lane0, dims, inv_freq, pos, row_req, n_rows);
  if (dtype == TOKB200_BF16)
    return launch_dependent(rotate_interleaved_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                            (__nv_bfloat16*)x, heads, head_row, lane0, dims, inv_freq, pos, row_req, n_rows);
  return TOKB200_BAD_DTYPE;
}
