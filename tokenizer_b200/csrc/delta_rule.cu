// The gated delta rule: a linear recurrence over a matrix state per head,
//     S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q        (S: dim x vdim, float32)
// with q and k unit vectors per head (q also times dim^(-1/2)), beta in (0, 1) and a decay g in
// (0, 1) per head and token, all of it 32-bit.  In front of it q, k and v pass a short causal
// convolution over time, channel by channel, and silu; behind it every head's o is divided by its
// root mean square, scaled by a gain and by silu of a gate projection.
//
// Per request the state slot holds, in float32: the heads' matrices TRANSPOSED and padded,
// [heads, vdim, dim_padded] (a thread owns consecutive rows of one column, so that its share is
// contiguous and a warp's loads coalesce), and behind them the convolution's last taps - 1 inputs,
// [taps - 1, channels], oldest first.  A request's rows of a step are consecutive
// (q_start[r] .. q_start[r + 1]); its state is read before its first row and written after its last.
//
//   gdn_prepare      a block a token: convolution (from the step's rows and, for a request's first
//                    rows, from the kept inputs), silu, unit vectors, beta and the decay
//   gdn_conv_state   the kept inputs move on (a thread a request and channel, after gdn_prepare)
//   gdn_scan         the recurrence: the columns of S are independent, so thread (column j, part p)
//                    keeps DPL rows of column j in registers; the P parts of a column add their
//                    shares of S^T k and S^T q (both of the matrix before the token's write: the
//                    read-out after it is g S^T q + (k . q) u) in one round of shuffles, one half of
//                    the lanes gathering one sum, the other half the other.  Tokens are staged through
//                    shared memory in runs by a warp of its own (cp.async), a run ahead of the warps
//                    that compute; a token's operands are in registers before the token before it is done
//   gdn_out_norm     a warp a (token, head): o / rms(o) * gain * scale * silu(gate)
#include "common.cuh"

#define GDN_MAX_TAPS 16
#define GDN_THREADS 256

__device__ __forceinline__ float gdn_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float gdn_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// proj: the stacked input product [T, ld]; columns qkv_at .. + channels are q (groups * dim), k
// (groups * dim), v (heads * vdim); b_at .. + heads and a_at .. + heads the projections behind
// beta and the decay.
template <typename TI>
__global__ void __launch_bounds__(GDN_THREADS)
gdn_prepare_kernel(const TI* __restrict__ proj, int ld, int qkv_at, int b_at, int a_at, int groups, int heads,
                   int dim, int vdim, int taps, const float* __restrict__ conv_w, const float* __restrict__ a_log,
                   const float* __restrict__ dt_bias, const float* __restrict__ state, long long state_stride,
                   int conv_off, const int* __restrict__ row_req, const int* __restrict__ q_start,
                   const int* __restrict__ state_slot, float q_scale, float* __restrict__ qkv_out,
                   float* __restrict__ bg_out) {
  extern __shared__ float gdn_vals[];      // channels, then 2 groups scales
  const int t = blockIdx.x;
  const int channels = 2 * groups * dim + heads * vdim;
  const int r = row_req[t];
  pdl_wait();
  pdl_launch();
  if (r < 0) return;
  const int at = t - q_start[r];                      // the row's place in its request's portion
  const float* kept = state + (size_t)state_slot[r] * state_stride + conv_off;
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;                  // tap j weighs the input `back` tokens ago
      const float in = back <= at ? to_float(proj[(size_t)(t - back) * ld + qkv_at + c])
                                  : kept[(size_t)(taps - 1 - (back - at)) * channels + c];
      acc += conv_w[(size_t)c * taps + j] * in;
    }
    gdn_vals[c] = acc * gdn_sigmoid(acc);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  float* out = qkv_out + (size_t)t * channels;
  float* scales = gdn_vals + channels;
  for (int h = warp; h < 2 * groups; h += warps) {   // q heads, then k heads
    float ss = 0.f;
    for (int l = lane; l < dim; l += 32) ss += gdn_vals[h * dim + l] * gdn_vals[h * dim + l];
    ss = warp_sum(ss);
    const float inv = (1.0f / sqrtf(ss + 1e-6f)) * (h < groups ? q_scale : 1.0f);
    for (int l = lane; l < dim; l += 32) out[h * dim + l] = gdn_vals[h * dim + l] * inv;
    if (lane == 0) scales[h] = inv;
  }
  __syncthreads();
  // q . k of every group, as the recurrence's read-out wants it (of the scaled unit vectors)
  for (int g = warp; g < groups; g += warps) {
    float dot = 0.f;
    for (int l = lane; l < dim; l += 32) dot = fmaf(gdn_vals[g * dim + l], gdn_vals[(groups + g) * dim + l], dot);
    dot = warp_sum(dot);
    if (lane == 0) bg_out[(size_t)t * (2 * heads + groups) + 2 * heads + g] = dot * scales[g] * scales[groups + g];
  }
  for (int c = 2 * groups * dim + threadIdx.x; c < channels; c += blockDim.x) out[c] = gdn_vals[c];
  for (int h = threadIdx.x; h < heads; h += blockDim.x) {
    const float b = to_float(proj[(size_t)t * ld + b_at + h]);
    const float a = to_float(proj[(size_t)t * ld + a_at + h]) + dt_bias[h];
    bg_out[(size_t)t * (2 * heads + groups) + h] = gdn_sigmoid(b);
    bg_out[(size_t)t * (2 * heads + groups) + heads + h] = expf(-expf(a_log[h]) * gdn_softplus(a));
  }
}

template <typename TI>
__global__ void gdn_conv_state_kernel(const TI* __restrict__ proj, int ld, int qkv_at, int channels, int taps,
                                      float* __restrict__ state, long long state_stride, int conv_off,
                                      const int* __restrict__ q_start, const int* __restrict__ state_slot) {
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int first = q_start[r], n = q_start[r + 1] - first;
  pdl_wait();
  pdl_launch();
  if (n <= 0 || c >= channels) return;
  float* kept = state + (size_t)state_slot[r] * state_stride + conv_off;
  float old[GDN_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < GDN_MAX_TAPS; ++j) old[j] = j < taps - 1 ? kept[(size_t)j * channels + c] : 0.f;
  // the last taps - 1 of (kept inputs, then the step's n inputs)
#pragma unroll
  for (int j = 0; j < GDN_MAX_TAPS; ++j) {
    if (j < taps - 1) {
      const int at = n + j;
      float v = 0.f;
      if (at >= taps - 1) {
        v = to_float(proj[(size_t)(first + at - (taps - 1)) * ld + qkv_at + c]);
      } else {
#pragma unroll
        for (int i = 0; i < GDN_MAX_TAPS; ++i) v = i == at ? old[i] : v;
      }
      kept[(size_t)j * channels + c] = v;
    }
  }
}

__device__ __forceinline__ void gdn_copy4(float* dst, const float* src) {
  const unsigned to = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(to), "l"(src) : "memory");
}

// qkv: [T, channels] as gdn_prepare wrote it; bg: [T, 2 heads + groups] (beta, the decay, q . k).
// Block: `cols` columns of one head of one request, P parts a column (cols * P = GDN_SCAN_THREADS
// threads that compute) and one more warp that only stages tokens.  Part p of a column owns the rows of
// the 4-row pieces p, P + p, 2 P + p, ...: the P parts of a column then read P neighbouring 16-byte
// pieces of k, of q and of the kept matrix at a time.
#define GDN_SCAN_THREADS 128

template <int DPL>
struct GdnToken {
  float k[DPL], q[DPL], v, beta, decay, kq;
};

template <int DPL>
__device__ __forceinline__ void gdn_fetch(GdnToken<DPL>& t, const float* k_mine, const float* q_mine,
                                          const float* v_mine, const float* b_s, int tok, int dim_p, int cols,
                                          int piece, int run) {
#pragma unroll
  for (int e = 0; e < DPL; e += 4) {
    const float4 a = *reinterpret_cast<const float4*>(k_mine + tok * dim_p + (e >> 2) * piece);
    const float4 b = *reinterpret_cast<const float4*>(q_mine + tok * dim_p + (e >> 2) * piece);
    t.k[e] = a.x; t.k[e + 1] = a.y; t.k[e + 2] = a.z; t.k[e + 3] = a.w;
    t.q[e] = b.x; t.q[e + 1] = b.y; t.q[e + 2] = b.z; t.q[e + 3] = b.w;
  }
  t.v = v_mine[tok * cols];
  t.beta = b_s[tok];
  t.decay = b_s[run + tok];
  t.kq = b_s[2 * run + tok];
}

__device__ __forceinline__ void gdn_copy16(float* dst, const float* src) {
  const unsigned to = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to), "l"(src) : "memory");
}

template <int DPL>
__global__ void __launch_bounds__(GDN_SCAN_THREADS + 32)
gdn_scan_kernel(const float* __restrict__ qkv, const float* __restrict__ bg, int channels, int groups, int heads,
                int dim, int vdim, int P, int cols, int run, float* __restrict__ state, long long state_stride,
                const int* __restrict__ q_start, const int* __restrict__ state_slot, float* __restrict__ o_out) {
  extern __shared__ __align__(16) float gdn_stage[];
  const int dim_p = P * DPL;
  const int r = blockIdx.z, h = blockIdx.y;
  const int col0 = blockIdx.x * cols;
  const int first = q_start[r], last = q_start[r + 1];
  pdl_wait();
  pdl_launch();
  if (first >= last) return;
  // a buffer: k [run][dim_p], q [run][dim_p], v [run][cols], beta [run], decay [run], k . q [run]
  const int per = (run * (2 * dim_p + cols + 3) + 3) / 4 * 4;     // whole 16 bytes: the rows are read as float4
  for (int i = threadIdx.x; i < 2 * per; i += blockDim.x) gdn_stage[i] = 0.f;   // the padded lanes stay zero
  __syncthreads();
  const int g = h / (heads / groups);
  const int k_col = (groups + g) * dim, q_col = g * dim, v_col = 2 * groups * dim + h * vdim + col0;
  const int n_cols = min(cols, vdim - col0);
  const int n_runs = (last - first + run - 1) / run;
  const int n_bg = 2 * heads + groups;

  if (threadIdx.x >= GDN_SCAN_THREADS) {
    // ---- the staging warp: run c + 1 lands while the others work through run c ----
    const int lane = threadIdx.x - GDN_SCAN_THREADS;
    // 16-byte copies where every row piece starts on 16 bytes
    const bool wide = dim % 4 == 0 && channels % 4 == 0 && k_col % 4 == 0 && q_col % 4 == 0 &&
                      (((uintptr_t)qkv) & 15) == 0;
    for (int c = 0; c <= n_runs; ++c) {
      if (c < n_runs) {
        float* k_s = gdn_stage + (size_t)(c & 1) * per;
        float* q_s = k_s + run * dim_p;
        float* v_s = q_s + run * dim_p;
        float* b_s = v_s + run * cols;
        const int t0 = first + c * run;
        const int n = min(run, last - t0);
        if (wide) {
          const int quads = dim >> 2;
          for (int i = lane; i < n * quads; i += 32) {
            const int tok = i / quads, l = (i - tok * quads) * 4;
            const float* row = qkv + (size_t)(t0 + tok) * channels;
            gdn_copy16(&k_s[tok * dim_p + l], row + k_col + l);
            gdn_copy16(&q_s[tok * dim_p + l], row + q_col + l);
          }
        } else {
          for (int i = lane; i < n * dim; i += 32) {
            const int tok = i / dim, l = i - tok * dim;
            const float* row = qkv + (size_t)(t0 + tok) * channels;
            gdn_copy4(&k_s[tok * dim_p + l], row + k_col + l);
            gdn_copy4(&q_s[tok * dim_p + l], row + q_col + l);
          }
        }
        for (int i = lane; i < n * n_cols; i += 32) {
          const int tok = i / n_cols, l = i - tok * n_cols;
          gdn_copy4(&v_s[tok * cols + l], qkv + (size_t)(t0 + tok) * channels + v_col + l);
        }
        for (int tok = lane; tok < n; tok += 32) {
          const float* row = bg + (size_t)(t0 + tok) * n_bg;
          gdn_copy4(&b_s[tok], row + h);
          gdn_copy4(&b_s[run + tok], row + heads + h);
          gdn_copy4(&b_s[2 * run + tok], row + 2 * heads + g);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      __syncthreads();      // run c is in place; everybody is done with run c - 1
    }
    return;
  }

  const int part = threadIdx.x % P, col = threadIdx.x / P;
  const int j = col0 + col;
  const bool live = j < vdim;
  const int piece = P * 4;
  float S[DPL];
  float* mine = state + (size_t)state_slot[r] * state_stride + ((size_t)h * vdim + (live ? j : 0)) * dim_p + part * 4;
#pragma unroll
  for (int e = 0; e < DPL; e += 4) {
    const float4 v = live ? *reinterpret_cast<const float4*>(mine + (e >> 2) * piece) : make_float4(0.f, 0.f, 0.f, 0.f);
    S[e] = v.x; S[e + 1] = v.y; S[e + 2] = v.z; S[e + 3] = v.w;
  }
  const bool upper = P > 1 && (part & (P >> 1));     // which of the two sums this lane ends up with
  float* o_mine = o_out + (size_t)first * heads * vdim + h * vdim + j;
  const bool writes = live && part == (P >> 1);

  auto step = [&](const GdnToken<DPL>& t, int row) {
    // both read-outs from the matrix as it stands: S'^T q = g S^T q + (k . q) u
    float dk[2] = {0.f, 0.f}, dq[2] = {0.f, 0.f};
#pragma unroll
    for (int e = 0; e < DPL; e += 2) {
      dk[0] = fmaf(S[e], t.k[e], dk[0]);
      dk[1] = fmaf(S[e + 1], t.k[e + 1], dk[1]);
      dq[0] = fmaf(S[e], t.q[e], dq[0]);
      dq[1] = fmaf(S[e + 1], t.q[e + 1], dq[1]);
    }
    float dot = dk[0] + dk[1], read = dq[0] + dq[1];
    if (P > 1) {
      // the two sums over a column's P lanes in one round: the lower half of the lanes gathers
      // S^T k, the upper half S^T q (each hands the other sum over first)
      float keep = upper ? read : dot;
      keep += __shfl_xor_sync(0xffffffffu, upper ? dot : read, P >> 1);
      for (int o = P >> 2; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
      dot = keep;
      read = keep;
    }
    float u = t.beta * (t.v - t.decay * dot);              // right in the lower lanes
    if (P > 1) u = __shfl_sync(0xffffffffu, u, 0, P);
    const float out = fmaf(t.kq, u, t.decay * read);       // right in the upper lanes (all, where P is 1)
#pragma unroll
    for (int e = 0; e < DPL; ++e) S[e] = fmaf(t.k[e], u, t.decay * S[e]);
    if (writes) o_mine[(size_t)row * heads * vdim] = out;
  };

  __syncthreads();          // run 0 is in place
  for (int c = 0; c < n_runs; ++c) {
    const float* k_s = gdn_stage + (size_t)(c & 1) * per;
    const float* q_s = k_s + run * dim_p;
    const float* v_s = q_s + run * dim_p;
    const float* b_s = v_s + run * cols;
    const float* k_mine = k_s + part * 4, *q_mine = q_s + part * 4, *v_mine = v_s + col;
    const int n = min(run, last - first - c * run);
    // a token's operands are asked for before the sums of the token before it are waited for
    GdnToken<DPL> even, odd;
    gdn_fetch<DPL>(even, k_mine, q_mine, v_mine, b_s, 0, dim_p, cols, piece, run);
    for (int tok = 0; tok < n; tok += 2) {
      if (tok + 1 < n) gdn_fetch<DPL>(odd, k_mine, q_mine, v_mine, b_s, tok + 1, dim_p, cols, piece, run);
      step(even, c * run + tok);
      if (tok + 1 < n) {
        if (tok + 2 < n) gdn_fetch<DPL>(even, k_mine, q_mine, v_mine, b_s, tok + 2, dim_p, cols, piece, run);
        step(odd, c * run + tok + 1);
      }
    }
    __syncthreads();        // done with run c; run c + 1 is in place
  }
  if (live) {
#pragma unroll
    for (int e = 0; e < DPL; e += 4)
      *reinterpret_cast<float4*>(mine + (e >> 2) * piece) = make_float4(S[e], S[e + 1], S[e + 2], S[e + 3]);
  }
}

// ---- the chunk form, for heads of 65 to 128 lanes (16 rows a thread, 8 parts a column) ----
// Within a run of 16 tokens, with G_t the product of the run's decays up to token t and S0 the matrix
// before the run, the rule unrolls to
//     u_t = beta_t (v_t - G_t S0^T k_t - sum_{s<t} (G_t / G_s) (k_s . k_t) u_s)
//     o_t = G_t S0^T q_t + sum_{s<=t} (G_t / G_s) (k_s . q_t) u_s
//     S16 = G_15 S0 + sum_s (G_15 / G_s) k_s u_s^T
// column by column.  The 32 sums against S0 are independent of one another (no chain from token to
// token), their shares are added over a column's 8 lanes in one packed round that leaves lane p with
// tokens 2 p and 2 p + 1; the scalars (G_t / G_s) (k_s . k_t) and (G_t / G_s) (k_s . q_t) are the same for
// all columns and computed once a run by the block; what stays a chain is the triangular solve, one
// shuffle and a few operations a token.  All 32-bit; only the order of the sums differs from the
// token-by-token kernel.  Measured SLOWER than that kernel (0.75 against 0.62 ms for 2,048 tokens of 16
// heads of 128 x 128): with a column's rows spread over 8 lanes every warp reads all of k and q of every
// token from shared memory, here twice (the sums, the matrix's move) and once more for the scalars, and
// the block's shared-memory reads (about 5,400 cycles a run of 16 tokens) bound it.  Off unless asked for.
#define GDN_RUN 16

__device__ __forceinline__ void gdn_compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(GDN_SCAN_THREADS) : "memory"); }

__global__ void __launch_bounds__(GDN_SCAN_THREADS + 32)
gdn_scan_chunked_kernel(const float* __restrict__ qkv, const float* __restrict__ bg, int channels, int groups,
                        int heads, int dim, int vdim, float* __restrict__ state, long long state_stride,
                        const int* __restrict__ q_start, const int* __restrict__ state_slot,
                        float* __restrict__ o_out) {
  constexpr int DPL = 16, P = 8, dim_p = 128, cols = GDN_SCAN_THREADS / P, run = GDN_RUN;
  extern __shared__ __align__(16) float gdn_stage[];
  const int r = blockIdx.z, h = blockIdx.y;
  const int col0 = blockIdx.x * cols;
  const int first = q_start[r], last = q_start[r + 1];
  pdl_wait();
  pdl_launch();
  if (first >= last) return;
  constexpr int per = run * (2 * dim_p + cols + 3);                // a multiple of 4
  float* a_k = gdn_stage + 2 * per;      // [run][run]: (G_t / G_s) k_s . k_t below the diagonal, zero elsewhere
  float* b_q = a_k + run * run;          // [run][run]: (G_t / G_s) k_s . q_t on and below the diagonal
  float* g_c = b_q + run * run;          // [run]: G_t
  float* r_l = g_c + run;                // [run]: G_15 / G_s
  for (int i = threadIdx.x; i < 2 * per; i += blockDim.x) gdn_stage[i] = 0.f;
  __syncthreads();
  const int g = h / (heads / groups);
  const int k_col = (groups + g) * dim, q_col = g * dim, v_col = 2 * groups * dim + h * vdim + col0;
  const int n_cols = min(cols, vdim - col0);
  const int n_runs = (last - first + run - 1) / run;
  const int n_bg = 2 * heads + groups;

  if (threadIdx.x >= GDN_SCAN_THREADS) {
    // ---- the staging warp, a run ahead ----
    const int lane = threadIdx.x - GDN_SCAN_THREADS;
    const bool wide = dim % 4 == 0 && channels % 4 == 0 && k_col % 4 == 0 && q_col % 4 == 0 &&
                      (((uintptr_t)qkv) & 15) == 0;
    for (int c = 0; c <= n_runs; ++c) {
      if (c < n_runs) {
        float* k_s = gdn_stage + (size_t)(c & 1) * per;
        float* q_s = k_s + run * dim_p;
        float* v_s = q_s + run * dim_p;
        float* b_s = v_s + run * cols;
        const int t0 = first + c * run;
        const int n = min(run, last - t0);
        if (wide) {
          const int quads = dim >> 2;
          for (int i = lane; i < n * quads; i += 32) {
            const int tok = i / quads, l = (i - tok * quads) * 4;
            const float* row = qkv + (size_t)(t0 + tok) * channels;
            gdn_copy16(&k_s[tok * dim_p + l], row + k_col + l);
            gdn_copy16(&q_s[tok * dim_p + l], row + q_col + l);
          }
        } else {
          for (int i = lane; i < n * dim; i += 32) {
            const int tok = i / dim, l = i - tok * dim;
            const float* row = qkv + (size_t)(t0 + tok) * channels;
            gdn_copy4(&k_s[tok * dim_p + l], row + k_col + l);
            gdn_copy4(&q_s[tok * dim_p + l], row + q_col + l);
          }
        }
        for (int i = lane; i < n * n_cols; i += 32) {
          const int tok = i / n_cols, l = i - tok * n_cols;
          gdn_copy4(&v_s[tok * cols + l], qkv + (size_t)(t0 + tok) * channels + v_col + l);
        }
        for (int tok = lane; tok < run; tok += 32) {
          if (tok < n) {
            const float* row = bg + (size_t)(t0 + tok) * n_bg;
            gdn_copy4(&b_s[tok], row + h);
            gdn_copy4(&b_s[run + tok], row + heads + h);
          } else {                        // tokens the run does not have: they write nothing and keep the matrix
            b_s[tok] = 0.f;
            b_s[run + tok] = 1.f;
          }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      __syncthreads();      // run c is in place; everybody is done with run c - 1
    }
    return;
  }

  const int part = threadIdx.x % P, col = threadIdx.x / P;
  const int j = col0 + col;
  const bool live = j < vdim;
  constexpr int piece = P * 4;
  float S[DPL];
  float* mine = state + (size_t)state_slot[r] * state_stride + ((size_t)h * vdim + (live ? j : 0)) * dim_p + part * 4;
#pragma unroll
  for (int e = 0; e < DPL; e += 4) {
    const float4 v = live ? *reinterpret_cast<const float4*>(mine + (e >> 2) * piece) : make_float4(0.f, 0.f, 0.f, 0.f);
    S[e] = v.x; S[e + 1] = v.y; S[e + 2] = v.z; S[e + 3] = v.w;
  }
  __syncthreads();          // run 0 is in place
  for (int c = 0; c < n_runs; ++c) {
    const float* k_s = gdn_stage + (size_t)(c & 1) * per;
    const float* q_s = k_s + run * dim_p;
    const float* v_s = q_s + run * dim_p;
    const float* b_s = v_s + run * cols;
    const float* d_s = b_s + run;
    const int n = min(run, last - first - c * run);
    // ---- the run's scalars: 256 pairs (t, s) over the 128 threads; pair (t, s) is k_s . k_t below the
    // diagonal and k_t . q_s on and above it (stored transposed) ----
#pragma unroll
    for (int rep = 0; rep < 2; ++rep) {
      const int idx = threadIdx.x + rep * GDN_SCAN_THREADS;
      const int t = idx >> 4, s = idx & 15;
      const bool lower = s < t;
      const float* a = k_s + (lower ? s : t) * dim_p;
      const float* b = lower ? k_s + t * dim_p : q_s + s * dim_p;
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
      if (t < n && s < n) {
        // every lane starts at another piece of its rows: the lanes' rows lie a whole number of banks apart
        for (int step = 0; step < dim_p / 4; ++step) {
          const int l = ((step + (int)threadIdx.x) & (dim_p / 4 - 1)) * 4;
          const float4 x = *reinterpret_cast<const float4*>(a + l), y = *reinterpret_cast<const float4*>(b + l);
          d0 = fmaf(x.x, y.x, d0); d1 = fmaf(x.y, y.y, d1); d2 = fmaf(x.z, y.z, d2); d3 = fmaf(x.w, y.w, d3);
        }
      }
      float ratio = 1.f;                                  // the decays between the two tokens
      const int lo = lower ? s : t, hi = lower ? t : s;
      for (int i = lo + 1; i <= hi; ++i) ratio *= d_s[i];
      const float value = ((d0 + d1) + (d2 + d3)) * ratio;
      if (lower) {
        a_k[t * run + s] = value;
        b_q[s * run + t] = 0.f;
      } else {
        b_q[s * run + t] = value;
        a_k[t * run + s] = 0.f;
      }
    }
    if (threadIdx.x < run) {
      float up = 1.f, down = 1.f;
      for (int i = 0; i <= threadIdx.x; ++i) up *= d_s[i];
      for (int i = threadIdx.x + 1; i < run; ++i) down *= d_s[i];
      g_c[threadIdx.x] = up;
      r_l[threadIdx.x] = down;
    }
    // ---- this thread's shares of S0^T k_t and S0^T q_t, t = 0 .. 15 ----
    float w[2 * GDN_RUN];
#pragma unroll
    for (int t = 0; t < run; ++t) {
      float dk = 0.f, dq = 0.f;
#pragma unroll
      for (int e = 0; e < DPL; e += 4) {
        const float4 x = *reinterpret_cast<const float4*>(k_s + t * dim_p + part * 4 + (e >> 2) * piece);
        const float4 y = *reinterpret_cast<const float4*>(q_s + t * dim_p + part * 4 + (e >> 2) * piece);
        dk = fmaf(S[e], x.x, dk); dk = fmaf(S[e + 1], x.y, dk); dk = fmaf(S[e + 2], x.z, dk); dk = fmaf(S[e + 3], x.w, dk);
        dq = fmaf(S[e], y.x, dq); dq = fmaf(S[e + 1], y.y, dq); dq = fmaf(S[e + 2], y.z, dq); dq = fmaf(S[e + 3], y.w, dq);
      }
      w[2 * t] = dk;
      w[2 * t + 1] = dq;
    }
    // ---- one packed round over the column's 8 lanes: lane p ends with w[4 p .. 4 p + 3], the sums of
    // tokens 2 p and 2 p + 1 ----
    {
      const bool hi4 = part & 4, hi2 = part & 2, hi1 = part & 1;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float got = __shfl_xor_sync(0xffffffffu, hi4 ? w[i] : w[i + 16], 4);
        w[i] = (hi4 ? w[i + 16] : w[i]) + got;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float got = __shfl_xor_sync(0xffffffffu, hi2 ? w[i] : w[i + 8], 2);
        w[i] = (hi2 ? w[i + 8] : w[i]) + got;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float got = __shfl_xor_sync(0xffffffffu, hi1 ? w[i] : w[i + 4], 1);
        w[i] = (hi1 ? w[i + 4] : w[i]) + got;
      }
    }
    gdn_compute_sync();       // the run's scalars are in place
    // ---- the solve, token by token: the lane that owns token s computes u_s and hands it to the others ----
    const int t_a = 2 * part, t_b = 2 * part + 1;
    const float base_a = v_s[t_a * cols + col] - g_c[t_a] * w[0], base_b = v_s[t_b * cols + col] - g_c[t_b] * w[2];
    const float beta_a = b_s[t_a], beta_b = b_s[t_b];
    float corr_a = 0.f, corr_b = 0.f;                     // sum_{s<t} a_k[t][s] u_s
    float out_a = g_c[t_a] * w[1], out_b = g_c[t_b] * w[3];
    float u[GDN_RUN];
#pragma unroll
    for (int s = 0; s < run; ++s) {
      const float mine_u = (s & 1) ? beta_b * (base_b - corr_b) : beta_a * (base_a - corr_a);
      u[s] = __shfl_sync(0xffffffffu, mine_u, s >> 1, P);
      corr_a = fmaf(a_k[t_a * run + s], u[s], corr_a);
      corr_b = fmaf(a_k[t_b * run + s], u[s], corr_b);
      out_a = fmaf(b_q[t_a * run + s], u[s], out_a);
      out_b = fmaf(b_q[t_b * run + s], u[s], out_b);
    }
    if (live) {
      float* o_row = o_out + (size_t)(first + c * run) * heads * vdim + h * vdim + j;
      if (t_a < n) o_row[(size_t)t_a * heads * vdim] = out_a;
      if (t_b < n) o_row[(size_t)t_b * heads * vdim] = out_b;
    }
    // ---- the matrix moves on by the whole run ----
    const float g_all = g_c[run - 1];
#pragma unroll
    for (int e = 0; e < DPL; ++e) S[e] *= g_all;
#pragma unroll
    for (int s = 0; s < run; ++s) {
      const float scaled = u[s] * r_l[s];
#pragma unroll
      for (int e = 0; e < DPL; e += 4) {
        const float4 x = *reinterpret_cast<const float4*>(k_s + s * dim_p + part * 4 + (e >> 2) * piece);
        S[e] = fmaf(x.x, scaled, S[e]); S[e + 1] = fmaf(x.y, scaled, S[e + 1]);
        S[e + 2] = fmaf(x.z, scaled, S[e + 2]); S[e + 3] = fmaf(x.w, scaled, S[e + 3]);
      }
    }
    __syncthreads();        // done with run c (and with its scalars); run c + 1 is in place
  }
  if (live) {
#pragma unroll
    for (int e = 0; e < DPL; e += 4)
      *reinterpret_cast<float4*>(mine + (e >> 2) * piece) = make_float4(S[e], S[e + 1], S[e + 2], S[e + 3]);
  }
}

// ---- a step of single tokens: convolution, unit vectors, the recurrence's one token and the output
// norm and gate in ONE kernel, a block a (row, head) with all of the head's columns (vdim * P threads).
// The kept inputs are read here and moved on by gdn_conv_state, launched behind.
template <int DPL, typename TI, typename TO>
__global__ void __launch_bounds__(1024)
gdn_step_kernel(const TI* __restrict__ proj, int ld, int qkv_at, int b_at, int a_at, int g_at, int groups, int heads,
                int dim, int vdim, int taps, int P, const float* __restrict__ conv_w, const float* __restrict__ a_log,
                const float* __restrict__ dt_bias, const float* __restrict__ gain, float out_scale, float eps,
                float q_scale, float* __restrict__ state, long long state_stride, int conv_off,
                const int* __restrict__ row_req, const int* __restrict__ state_slot, TO* __restrict__ out) {
  extern __shared__ __align__(16) float gdn_one[];      // q [dim_p], k [dim_p], v [vdim], o [vdim], 8 scalars
  __shared__ float scratch[33];
  const int dim_p = P * DPL;
  const int t = blockIdx.x, h = blockIdx.y;
  const int r = row_req[t];
  pdl_wait();
  pdl_launch();
  if (r < 0) return;
  float* q_s = gdn_one;
  float* k_s = q_s + dim_p;
  float* v_s = k_s + dim_p;
  float* o_s = v_s + vdim;
  float* misc = o_s + vdim;            // q scale, k scale, q . k, beta, decay
  const int g = h / (heads / groups);
  const int channels = 2 * groups * dim + heads * vdim;
  const int slot = state_slot[r];
  const float* kept = state + (size_t)slot * state_stride + conv_off;
  const TI* row = proj + (size_t)t * ld;
  // the head's 2 dim + vdim channels: the newest tap on this row, the others on the kept inputs
  for (int i = threadIdx.x; i < 2 * dim_p + vdim; i += blockDim.x) {
    const int which = i < dim_p ? 0 : i < 2 * dim_p ? 1 : 2;
    const int l = i - which * dim_p;
    float value = 0.f;
    if (which == 2 || l < dim) {
      const int c = which == 0 ? g * dim + l : which == 1 ? (groups + g) * dim + l : 2 * groups * dim + h * vdim + l;
      float acc = conv_w[(size_t)c * taps + taps - 1] * to_float(row[qkv_at + c]);
      for (int j = 0; j + 1 < taps; ++j) acc = fmaf(conv_w[(size_t)c * taps + j], kept[(size_t)j * channels + c], acc);
      value = acc * gdn_sigmoid(acc);
    }
    gdn_one[i] = value;                 // q, k (zeros behind dim), v lie one behind the other
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < 3) {
    const float* a = warp == 1 ? k_s : q_s;
    const float* b = warp == 0 ? q_s : k_s;
    float sum = 0.f;
    for (int l = lane; l < dim; l += 32) sum = fmaf(a[l], b[l], sum);
    sum = warp_sum(sum);
    if (lane == 0) misc[warp] = warp == 2 ? sum : 1.0f / sqrtf(sum + 1e-6f);     // 0: |q|, 1: |k|, 2: q . k (raw)
  } else if (warp == 3 && lane == 0) {
    misc[3] = gdn_sigmoid(to_float(row[b_at + h]));
    misc[4] = expf(-expf(a_log[h]) * gdn_softplus(to_float(row[a_at + h]) + dt_bias[h]));
  }
  __syncthreads();
  const float q_unit = misc[0] * q_scale, k_unit = misc[1];
  const float kq = misc[2] * q_unit * k_unit, beta = misc[3], decay = misc[4];
  const int part = threadIdx.x % P, j = threadIdx.x / P;          // every thread has a column: vdim * P threads
  const int piece = P * 4;
  float* mine = state + (size_t)slot * state_stride + ((size_t)h * vdim + j) * dim_p + part * 4;
  float dk[2] = {0.f, 0.f}, dq[2] = {0.f, 0.f};
  float S[DPL], kk[DPL];
#pragma unroll
  for (int e = 0; e < DPL; e += 4) {
    const float4 m = *reinterpret_cast<const float4*>(mine + (e >> 2) * piece);
    const float4 a = *reinterpret_cast<const float4*>(k_s + part * 4 + (e >> 2) * piece);
    const float4 b = *reinterpret_cast<const float4*>(q_s + part * 4 + (e >> 2) * piece);
    S[e] = m.x; S[e + 1] = m.y; S[e + 2] = m.z; S[e + 3] = m.w;
    kk[e] = a.x * k_unit; kk[e + 1] = a.y * k_unit; kk[e + 2] = a.z * k_unit; kk[e + 3] = a.w * k_unit;
    dk[0] = fmaf(S[e], kk[e], dk[0]);
    dk[1] = fmaf(S[e + 1], kk[e + 1], dk[1]);
    dk[0] = fmaf(S[e + 2], kk[e + 2], dk[0]);
    dk[1] = fmaf(S[e + 3], kk[e + 3], dk[1]);
    dq[0] = fmaf(S[e], b.x * q_unit, dq[0]);
    dq[1] = fmaf(S[e + 1], b.y * q_unit, dq[1]);
    dq[0] = fmaf(S[e + 2], b.z * q_unit, dq[0]);
    dq[1] = fmaf(S[e + 3], b.w * q_unit, dq[1]);
  }
  float dot = dk[0] + dk[1], read = dq[0] + dq[1];
  const bool upper = P > 1 && (part & (P >> 1));
  if (P > 1) {
    float keep = upper ? read : dot;
    keep += __shfl_xor_sync(0xffffffffu, upper ? dot : read, P >> 1);
    for (int o = P >> 2; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
    dot = keep;
    read = keep;
  }
  float u = beta * (v_s[j] - decay * dot);
  if (P > 1) u = __shfl_sync(0xffffffffu, u, 0, P);
#pragma unroll
  for (int e = 0; e < DPL; e += 4)
    *reinterpret_cast<float4*>(mine + (e >> 2) * piece) =
        make_float4(fmaf(kk[e], u, decay * S[e]), fmaf(kk[e + 1], u, decay * S[e + 1]),
                    fmaf(kk[e + 2], u, decay * S[e + 2]), fmaf(kk[e + 3], u, decay * S[e + 3]));
  const float mine_out = fmaf(kq, u, decay * read);
  if (part == (P >> 1)) o_s[j] = mine_out;
  const float ss = block_sum(part == (P >> 1) ? mine_out * mine_out : 0.f, scratch);     // publishes o_s too
  const float inv = (1.0f / sqrtf(ss / (float)vdim + eps)) * out_scale;
  for (int l = threadIdx.x; l < vdim; l += blockDim.x) {
    const float z = to_float(row[g_at + h * vdim + l]);
    out[((size_t)t * heads + h) * vdim + l] = from_float<TO>(o_s[l] * inv * gain[l] * (z * gdn_sigmoid(z)));
  }
}

template <typename TG, typename TO>
__global__ void gdn_out_norm_kernel(const float* __restrict__ o, const TG* __restrict__ gate, int ld, int g_at,
                                    const float* __restrict__ gain, float scale, float eps, TO* __restrict__ out,
                                    int n_rows, int heads, int vdim, const int* __restrict__ row_req) {
  pdl_wait();
  pdl_launch();
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (unit >= n_rows * heads) return;
  const int t = unit / heads, h = unit % heads;
  if (row_req[t] < 0) return;
  const float* row = o + ((size_t)t * heads + h) * vdim;
  const TG* gates = gate + (size_t)t * ld + g_at + h * vdim;
  TO* y = out + ((size_t)t * heads + h) * vdim;
  if (vdim == 128 && sizeof(TG) == 4 && ((((uintptr_t)row) | ((uintptr_t)gates) | ((uintptr_t)gain)) & 15) == 0 &&
      (((uintptr_t)y) & 7) == 0) {
    // a head of 128 lanes: four consecutive lanes a thread, every operand in one 16-byte load
    const float4 v = *reinterpret_cast<const float4*>(row + lane * 4);
    const float4 z = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(gates) + lane * 4);
    const float4 w = *reinterpret_cast<const float4*>(gain + lane * 4);
    const float ss4 = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
    const float inv4 = (1.0f / sqrtf(ss4 / 128.0f + eps)) * scale;
    y[lane * 4] = from_float<TO>(v.x * inv4 * w.x * (z.x * gdn_sigmoid(z.x)));
    y[lane * 4 + 1] = from_float<TO>(v.y * inv4 * w.y * (z.y * gdn_sigmoid(z.y)));
    y[lane * 4 + 2] = from_float<TO>(v.z * inv4 * w.z * (z.z * gdn_sigmoid(z.z)));
    y[lane * 4 + 3] = from_float<TO>(v.w * inv4 * w.w * (z.w * gdn_sigmoid(z.w)));
    return;
  }
  float ss = 0.f;
  for (int l = lane; l < vdim; l += 32) ss += row[l] * row[l];
  ss = warp_sum(ss);
  const float inv = (1.0f / sqrtf(ss / (float)vdim + eps)) * scale;
  for (int l = lane; l < vdim; l += 32) {
    const float z = to_float(gates[l]);
    y[l] = from_float<TO>(row[l] * inv * gain[l] * (z * gdn_sigmoid(z)));
  }
}

// ---- launchers -----------------------------------------------------------------------------------
// Rows a thread keeps of its column: 8 for heads of up to 32 lanes, 16 up to 128, 32 beyond; and the
// parts of a column (a power of two).
static inline int gdn_rows(int dim) {
  static const int forced = [] {                     // TOKB200_GDN_ROWS=8|16|32: another split, for measurements
    const char* v = getenv("TOKB200_GDN_ROWS");
    const int n = v ? atoi(v) : 0;
    return (n == 8 || n == 16 || n == 32) ? n : 0;
  }();
  if (forced && (dim + forced - 1) / forced <= 32) return forced;
  return dim <= 32 ? 8 : dim <= 128 ? 16 : 32;
}
static inline int gdn_parts(int dim, int dpl) {
  int p = 1;
  while (p * dpl < dim) p <<= 1;
  return p;
}

// Rows of a head's padded state column.
TOKB200_API int tokb200_gdn_padded_dim(int dim) {
  if (dim <= 0 || dim > 1024) return 0;
  return gdn_parts(dim, gdn_rows(dim)) * gdn_rows(dim);
}

static inline int gdn_conv_state(const void* proj, int proj_dtype, int ld, int qkv_at, int channels, int taps,
                                 float* state, long long state_stride, int conv_off, const int* q_start,
                                 const int* state_slot, int n_requests, cudaStream_t stream) {
  if (taps == 1) return TOKB200_OK;
  dim3 grid((channels + 127) / 128, n_requests);
  if (proj_dtype == TOKB200_F32)
    return launch_dependent(gdn_conv_state_kernel<float>, grid, dim3(128), 0, stream, (const float*)proj, ld, qkv_at,
                            channels, taps, state, state_stride, conv_off, q_start, state_slot);
  return launch_dependent(gdn_conv_state_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream,
                          (const __nv_bfloat16*)proj, ld, qkv_at, channels, taps, state, state_stride, conv_off,
                          q_start, state_slot);
}

TOKB200_API int tokb200_gdn_prepare(const void* proj, int proj_dtype, int ld, int qkv_at, int b_at, int a_at,
                                    int groups, int heads, int dim, int vdim, int taps, const float* conv_w,
                                    const float* a_log, const float* dt_bias, float* state, long long state_stride,
                                    int conv_off, const int* row_req, const int* q_start, const int* state_slot,
                                    int n_rows, int n_requests, float* qkv_out, float* bg_out, cudaStream_t stream) {
  if (n_rows <= 0 || n_requests <= 0) return TOKB200_OK;
  if (groups <= 0 || heads <= 0 || heads % groups || dim <= 0 || vdim <= 0 || taps < 1 || taps > GDN_MAX_TAPS ||
      n_requests > 65535)
    return TOKB200_BAD_SIZE;
  const int channels = 2 * groups * dim + heads * vdim;
  const size_t smem = (size_t)(channels + 2 * groups) * sizeof(float);
  if (smem > 48 * 1024) return TOKB200_BAD_SIZE;
  const float q_scale = 1.0f / sqrtf((float)dim);
  int status;
  if (proj_dtype == TOKB200_F32)
    status = launch_dependent(gdn_prepare_kernel<float>, dim3(n_rows), dim3(GDN_THREADS), smem, stream,
                              (const float*)proj, ld, qkv_at, b_at, a_at, groups, heads, dim, vdim, taps, conv_w, a_log,
                              dt_bias, (const float*)state, state_stride, conv_off, row_req, q_start, state_slot,
                              q_scale, qkv_out, bg_out);
  else if (proj_dtype == TOKB200_BF16)
    status = launch_dependent(gdn_prepare_kernel<__nv_bfloat16>, dim3(n_rows), dim3(GDN_THREADS), smem, stream,
                              (const __nv_bfloat16*)proj, ld, qkv_at, b_at, a_at, groups, heads, dim, vdim, taps,
                              conv_w, a_log, dt_bias, (const float*)state, state_stride, conv_off, row_req, q_start,
                              state_slot, q_scale, qkv_out, bg_out);
  else
    return TOKB200_BAD_DTYPE;
  if (status != TOKB200_OK) return status;
  return gdn_conv_state(proj, proj_dtype, ld, qkv_at, channels, taps, state, state_stride, conv_off, q_start, state_slot,
                        n_requests, stream);
}

// Whether a step of single tokens can run as one kernel: a block holds all of a head's columns.
TOKB200_API int tokb200_gdn_step_supported(int dim, int vdim) {
  if (dim <= 0 || dim > 1024 || vdim <= 0) return 0;
  const int dpl = gdn_rows(dim), P = gdn_parts(dim, dpl);
  const int threads = vdim * P;
  return threads <= 1024 && threads % 32 == 0 && threads >= 128;
}

// One token a request (row t belongs to request row_req[t], whose state lies in state_slot[row_req[t]]).
TOKB200_API int tokb200_gdn_step(const void* proj, int proj_dtype, int ld, int qkv_at, int b_at, int a_at, int g_at,
                                 int groups, int heads, int dim, int vdim, int taps, const float* conv_w,
                                 const float* a_log, const float* dt_bias, const float* gain, float out_scale, float eps,
                                 float* state, long long state_stride, int conv_off, const int* row_req,
                                 const int* q_start, const int* state_slot, int n_rows, int n_requests, void* out,
                                 int out_dtype, cudaStream_t stream) {
  if (n_rows <= 0 || n_requests <= 0) return TOKB200_OK;
  if (groups <= 0 || heads <= 0 || heads % groups || taps < 1 || taps > GDN_MAX_TAPS || heads > 65535 ||
      !tokb200_gdn_step_supported(dim, vdim))
    return TOKB200_BAD_SIZE;
  if (((uintptr_t)state & 15) || state_stride % 4) return TOKB200_BAD_ALIGNMENT;
  const int channels = 2 * groups * dim + heads * vdim;
  const int dpl = gdn_rows(dim), P = gdn_parts(dim, dpl);
  const size_t smem = (size_t)(2 * P * dpl + 2 * vdim + 8) * sizeof(float);
  const float q_scale = 1.0f / sqrtf((float)dim);
  dim3 grid(n_rows, heads), block(vdim * P);
  int status = TOKB200_BAD_DTYPE;
#define LAUNCH(D, TI, TO)                                                                                            \
  status = launch_dependent(gdn_step_kernel<D, TI, TO>, grid, block, smem, stream, (const TI*)proj, ld, qkv_at, b_at, \
                            a_at, g_at, groups, heads, dim, vdim, taps, P, conv_w, a_log, dt_bias, gain, out_scale,  \
                            eps, q_scale, state, state_stride, conv_off, row_req, state_slot, (TO*)out)
#define BY_ROWS(TI, TO)            \
  if (dpl == 8) LAUNCH(8, TI, TO); \
  else if (dpl == 16) LAUNCH(16, TI, TO); \
  else LAUNCH(32, TI, TO)
  if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_F32) { BY_ROWS(float, float); }
  else if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16) { BY_ROWS(float, __nv_bfloat16); }
  else if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_BF16) { BY_ROWS(__nv_bfloat16, __nv_bfloat16); }
  else if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_F32) { BY_ROWS(__nv_bfloat16, float); }
#undef BY_ROWS
#undef LAUNCH
  if (status != TOKB200_OK) return status;
  return gdn_conv_state(proj, proj_dtype, ld, qkv_at, channels, taps, state, state_stride, conv_off, q_start, state_slot,
                        n_requests, stream);
}

TOKB200_API int tokb200_gdn_scan(const float* qkv, const float* bg, int groups, int heads, int dim, int vdim,
                                 float* state, long long state_stride, const int* q_start, const int* state_slot,
                                 int n_requests, int longest, int chunks, float* o_out, cudaStream_t stream) {
  if (n_requests <= 0) return TOKB200_OK;
  if (groups <= 0 || heads <= 0 || heads % groups || dim <= 0 || dim > 1024 || vdim <= 0 || heads > 65535 ||
      n_requests > 65535)
    return TOKB200_BAD_SIZE;
  if (((uintptr_t)state & 15) || state_stride % 4) return TOKB200_BAD_ALIGNMENT;
  const int channels = 2 * groups * dim + heads * vdim;
  const int dpl = gdn_rows(dim);
  const int P = gdn_parts(dim, dpl);
  const int cols = GDN_SCAN_THREADS / P;
  const int dim_p = P * dpl;
  // tokens a run: what two buffers of 48 KB together hold, at most 16
  int run = (48 * 1024 / 2 / (int)sizeof(float) - 4) / (2 * dim_p + cols + 3);
  run = run > 16 ? 16 : run;
  if (run < 1) return TOKB200_BAD_SIZE;
  const size_t smem = (size_t)2 * ((run * (2 * dim_p + cols + 3) + 3) / 4 * 4) * sizeof(float);
  dim3 grid((vdim + cols - 1) / cols, heads, n_requests);
  if (chunks && dpl == 16 && P == 8 && longest >= 2 * GDN_RUN) {
    // asked for: portions of 32 tokens and more of heads of 65 to 128 lanes in the chunk form
    constexpr int per = GDN_RUN * (2 * 128 + GDN_SCAN_THREADS / 8 + 3);
    const size_t bytes = (size_t)(2 * per + 2 * GDN_RUN * GDN_RUN + 2 * GDN_RUN) * sizeof(float);
    return launch_dependent(gdn_scan_chunked_kernel, grid, dim3(GDN_SCAN_THREADS + 32), bytes, stream, qkv, bg, channels,
                            groups, heads, dim, vdim, state, state_stride, q_start, state_slot, o_out);
  }
#define LAUNCH(D)                                                                                               \
  return launch_dependent(gdn_scan_kernel<D>, grid, dim3(GDN_SCAN_THREADS + 32), smem, stream, qkv, bg, channels, \
                          groups, heads, dim, vdim, P, cols, run, state, state_stride, q_start, state_slot, o_out)
  if (dpl == 8) LAUNCH(8);
  if (dpl == 16) LAUNCH(16);
  LAUNCH(32);
#undef LAUNCH
}

TOKB200_API int tokb200_gdn_out_norm(const float* o, const void* gate, int gate_dtype, int ld, int g_at,
                                     const float* gain, float scale, float eps, void* out, int out_dtype, int n_rows,
                                     int heads, int vdim, const int* row_req, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (heads <= 0 || vdim <= 0) return TOKB200_BAD_SIZE;
  const long long units = (long long)n_rows * heads;
  dim3 grid((unsigned)((units + 7) / 8)), block(256);
#define LAUNCH(TG, TO)                                                                                       \
  return launch_dependent(gdn_out_norm_kernel<TG, TO>, grid, block, 0, stream, o, (const TG*)gate, ld, g_at, \
                          gain, scale, eps, (TO*)out, n_rows, heads, vdim, row_req)
  if (gate_dtype == TOKB200_F32 && out_dtype == TOKB200_F32) LAUNCH(float, float);
  if (gate_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16) LAUNCH(float, __nv_bfloat16);
  if (gate_dtype == TOKB200_BF16 && out_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (gate_dtype == TOKB200_BF16 && out_dtype == TOKB200_F32) LAUNCH(__nv_bfloat16, float);
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}
