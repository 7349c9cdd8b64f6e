// Gated linear recurrences over the rows of a step, with the state carried per request.
//
// minGRU: per channel c and token t
//     z = sigmoid(zp[t,c]),  cand = u >= 0 ? u + 1/2 : sigmoid(u)   (u = up[t,c]),
//     S_t = (1 - z) S_(t-1) + z cand,      y[t,c] = S_t * silu(g[t,c]),
// where zp, up and g are three column ranges of one projection's output (the projection adds
// the biases).  The state S is float32 [slots, width]; a request's rows are consecutive
// (q_start[r] .. q_start[r+1]) and its state lives in slot state_slot[r]: read before the
// request's first row of the step, written back after its last.  Gates, candidate, state and
// the product with silu(g) are 32-bit whatever the type of the projection's output.
//
// A step's rows of one request are taken in runs of TY * K tokens: thread (x, y) of a block owns
// one of the block's channels and K consecutive tokens; it folds them into one affine map
// S -> P S + B, the maps of the block's TY threads of a channel are chained through shared
// memory, and every thread then walks its K tokens again from the state it was handed, out of
// registers.  Every input is read once.  A block owns 32 channels (128 bytes of every row) and
// 8 runs where channels and requests give several blocks a multiprocessor, 32 runs where a lone
// long prompt leaves few blocks, which must then keep many loads in flight each.  A step of
// single tokens runs one thread a channel.
#include "common.cuh"

#define REC_MAX_X 32
#define REC_MAX_TY 32

// FAST (where the outputs are bfloat16): the exponential and the division by the hardware's
// approximations, exact to about 2 ulp of float32, far below the output's rounding; the float32
// path keeps the library's expf and the IEEE division.  Three sigmoids a token and channel make
// this kernel bound by them otherwise (8,192 tokens x 4,096 channels: 290 us against 72 us for
// its bytes).
template <bool FAST>
__device__ __forceinline__ float rec_sigmoid(float v) {
  if (FAST) return __fdividef(1.0f, 1.0f + __expf(-v));
  return 1.0f / (1.0f + expf(-v));
}

template <typename TI, typename TO, int K>
__global__ void __launch_bounds__(REC_MAX_X * REC_MAX_TY)
min_gru_scan_kernel(const TI* __restrict__ proj, const float* __restrict__ bias, int ld, int z_at, int u_at,
                    int g_at, int width,
                    float* __restrict__ state, const int* __restrict__ q_start,
                    const int* __restrict__ state_slot, TO* __restrict__ out) {
  __shared__ float p_s[REC_MAX_TY][REC_MAX_X + 1];
  __shared__ float b_s[REC_MAX_TY][REC_MAX_X + 1];
  __shared__ float carry_s[REC_MAX_X];
  constexpr bool FAST = sizeof(TO) == 2;
  const int x = threadIdx.x, y = threadIdx.y, ty = blockDim.y;
  const int c = blockIdx.x * blockDim.x + x;
  const int r = blockIdx.y;
  const bool live = c < width;
  // the projection's biases (one float32 a column of the product, or none): weights, read before the wait
  const float bz = (bias && live) ? bias[z_at + c] : 0.f;
  const float bu = (bias && live) ? bias[u_at + c] : 0.f;
  const float bg = (bias && live) ? bias[g_at + c] : 0.f;
  // the spans and slots were written before the predecessor started
  const int first = q_start[r], last = q_start[r + 1];
  const int slot = state_slot[r];
  pdl_wait();
  pdl_launch();
  if (first >= last || slot < 0) return;
  if (y == 0) carry_s[x] = live ? state[(size_t)slot * width + c] : 0.f;
  __syncthreads();
  for (int t0 = first; t0 < last; t0 += ty * K) {
    const int mine = t0 + y * K;
    // all of the run's loads first (3 K independent loads a thread in flight), then the arithmetic,
    // in place: a = 1 - z, b = z * candidate, gate = silu(g)
    float a[K], b[K], gate[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int t = mine + k;
      const bool on = live && t < last;
      const TI* row = proj + (size_t)(on ? t : first) * ld;
      a[k] = on ? to_float(row[z_at + c]) : 0.f;
      b[k] = on ? to_float(row[u_at + c]) : 0.f;
      gate[k] = on ? to_float(row[g_at + c]) : 0.f;
    }
    float p = 1.f, acc = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int t = mine + k;
      if (live && t < last) {
        const float z = rec_sigmoid<FAST>(a[k] + bz);
        const float u = b[k] + bu;
        const float g = gate[k] + bg;
        const float cand = u >= 0.f ? u + 0.5f : rec_sigmoid<FAST>(u);
        a[k] = 1.0f - z;
        b[k] = z * cand;
        gate[k] = g * rec_sigmoid<FAST>(g);
      } else {
        a[k] = 1.f; b[k] = 0.f; gate[k] = 0.f;
      }
      acc = a[k] * acc + b[k];
      p *= a[k];
    }
    float s = carry_s[x];
    if (ty > 1) {
      p_s[y][x] = p;
      b_s[y][x] = acc;
      __syncthreads();
      for (int i = 0; i < y; ++i) s = p_s[i][x] * s + b_s[i][x];
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int t = mine + k;
      s = a[k] * s + b[k];
      if (live && t < last) out[(size_t)t * width + c] = from_float<TO>(s * gate[k]);
    }
    if (ty > 1) __syncthreads();       // every thread has read the carry and the maps
    if (y == ty - 1) carry_s[x] = s;
    if (ty > 1) __syncthreads();
  }
  if (y == ty - 1 && live) state[(size_t)slot * width + c] = carry_s[x];
}

// proj: [rows, ld] (float32 or bfloat16) with the three column ranges starting at z_at, u_at,
// g_at, each `width` wide; out: [rows, width] dense.  `longest`: the most rows a request brings
// to the step (chooses the shape of a block).
TOKB200_API int tokb200_min_gru_scan(const void* proj, int proj_dtype, const float* bias, int ld, int z_at, int u_at,
                                     int g_at, int width, float* state, const int* q_start,
                                     const int* state_slot, int n_requests, int longest, void* out,
                                     int out_dtype, cudaStream_t stream) {
  if (n_requests <= 0 || longest <= 0) return TOKB200_OK;
  if (width <= 0 || ld < width || n_requests > 65535) return TOKB200_BAD_SIZE;
  const bool single = longest == 1;
  // a block owns 32 channels (128 bytes of every row).  Where channels and requests give two blocks
  // a multiprocessor and more, 8 runs (256 threads, several blocks a multiprocessor); else 32 runs
  // (1,024 threads), so that the few blocks of a lone long prompt keep enough loads in flight
  const int cx = REC_MAX_X;
  int ty = 1;
  if (!single) {
    ty = (long long)((width + 31) / 32) * n_requests >= 2 * 148 ? 8 : REC_MAX_TY;
    while (ty > 1 && (ty / 2) * 8 >= longest) ty /= 2;     // no more runs than the longest request fills
  }
  dim3 grid((width + cx - 1) / cx, n_requests);
  dim3 block(cx, ty);
#define LAUNCH(TI, TO)                                                                              \
  return single ? launch_dependent(min_gru_scan_kernel<TI, TO, 1>, grid, block, 0, stream,         \
                                   (const TI*)proj, bias, ld, z_at, u_at, g_at, width, state, q_start,  \
                                   state_slot, (TO*)out)                                            \
                : launch_dependent(min_gru_scan_kernel<TI, TO, 8>, grid, block, 0, stream,         \
                                   (const TI*)proj, bias, ld, z_at, u_at, g_at, width, state, q_start,  \
                                   state_slot, (TO*)out)
  if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_F32) LAUNCH(float, float);
  if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16) LAUNCH(float, __nv_bfloat16);
  if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_F32) LAUNCH(__nv_bfloat16, float);
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}
