// Short causal convolutions over time, one filter a channel, across the steps of a sequence.
//
//   y_t[c] = bias[c] + sum_{j < taps} w[c, j] * u_{t - taps + 1 + j}[c]        (u = 0 before position 0)
//
// The step's tokens are packed one sequence after another.  A sequence's last taps - 1 inputs are kept
// per slot ("state": float [taps - 1, C], oldest first, zero for a fresh slot), so a token whose
// predecessors came in earlier steps finds them there.  Which of a token's predecessors lie in this step
// is read off the tokens' slots (a slot appears once a step): rows m - 1, m - 2, ... with the same slot.
// The sum runs from the oldest tap to the newest whatever the cut, and the state holds the inputs as they
// were stored (a bf16 value widened to float is exact), so a position's result does not depend on how the
// sequence was cut into steps.  The state is written by a second kernel, after every reader of the old one.
//
// rl_qkv_prepare fuses, for an attention layer: the convolution of the projected queries, keys and values,
// an RMS norm of every query and key head (one weight vector for all heads), the rotary encoding (half-split
// pairs over the first `rot` dimensions, cos and sin times `magnitude`) and the write of keys and values
// into the paged cache.  Each of the four is optional.
#include <math.h>

#include "common.cuh"

#define CONV_MAX_TAPS 8
#define CONV_THREADS 256

// how many of rows m - 1, m - 2, ... (at most taps - 1) belong to row m's sequence.  The slots are loaded
// independently of one another (no load waits for the one before it), then counted while the run lasts.
__device__ __forceinline__ int conv_rows_back(const int* __restrict__ slot_of_token, int m, int taps) {
  const int slot = slot_of_token[m];
  int same[CONV_MAX_TAPS - 1];
#pragma unroll
  for (int d = 1; d < CONV_MAX_TAPS; ++d) same[d - 1] = (d < taps && m - d >= 0) ? (slot_of_token[m - d] == slot) : 0;
  int n = 0, run = 1;
#pragma unroll
  for (int d = 1; d < CONV_MAX_TAPS; ++d) { run &= same[d - 1]; n += run; }
  return n;
}

// the input `dist` positions before row m's (dist >= 0), channel c; n = conv_rows_back
template <typename T>
__device__ __forceinline__ float conv_input(const T* __restrict__ u, int ldu, const float* __restrict__ st, int C, int taps,
                                            int m, int n, int dist, int c) {
  if (dist <= n) return rl_ld(u + (size_t)(m - dist) * ldu + c);
  return st[(size_t)(taps - 2 - (dist - n - 1)) * C + c];
}

template <typename T>
__device__ __forceinline__ float conv_at(const T* __restrict__ u, int ldu, const float* __restrict__ w, const float* __restrict__ st,
                                         int C, int taps, int m, int n, int c, float acc) {
  if (taps == 4 && ((uintptr_t)w & 15) == 0) {        // the usual four taps: the channel's filter as one 16-byte load
    const float4 f = *reinterpret_cast<const float4*>(w + (size_t)c * 4);
    acc = fmaf(f.x, conv_input(u, ldu, st, C, 4, m, n, 3, c), acc);
    acc = fmaf(f.y, conv_input(u, ldu, st, C, 4, m, n, 2, c), acc);
    acc = fmaf(f.z, conv_input(u, ldu, st, C, 4, m, n, 1, c), acc);
    return fmaf(f.w, conv_input(u, ldu, st, C, 4, m, n, 0, c), acc);
  }
  for (int dist = taps - 1; dist >= 0; --dist)
    acc = fmaf(w[(size_t)c * taps + taps - 1 - dist], conv_input(u, ldu, st, C, taps, m, n, dist, c), acc);
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(CONV_THREADS)
short_conv_kernel(const T* __restrict__ u, int ldu, const float* __restrict__ w, const float* __restrict__ bias, int act, int C,
                  int taps, const int* __restrict__ slot_of_token, const float* __restrict__ state, long long state_stride,
                  T* __restrict__ out, int ldo) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
  if (c >= C) return;
  const int n = conv_rows_back(slot_of_token, m, taps);
  const float* st = state + (size_t)slot_of_token[m] * state_stride;
  float acc = conv_at(u, ldu, w, st, C, taps, m, n, c, bias ? bias[c] : 0.f);
  if (act == 1) acc = acc / (1.0f + expf(-acc));
  rl_st(out + (size_t)m * ldo + c, acc);
}

template <typename T>
__global__ void __launch_bounds__(CONV_THREADS)
short_conv_state_kernel(const T* __restrict__ u, int ldu, int C, int taps, const int* __restrict__ cu_seqlens,
                        const int* __restrict__ seq_slots, float* __restrict__ state, long long state_stride) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int b = blockIdx.x;
  const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
  if (c >= C) return;
  const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1], nq = hi - lo;
  float* st = state + (size_t)seq_slots[b] * state_stride;
  float nv[CONV_MAX_TAPS - 1];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
    if (j < taps - 1) {
      // entry j will hold the input of position (length after the step) - (taps - 1) + j
      const int row = hi - (taps - 1) + j;
      nv[j] = row >= lo ? rl_ld(u + (size_t)row * ldu + c) : st[(size_t)(j + nq) * C + c];
    }
  }
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
    if (j < taps - 1) st[(size_t)j * C + c] = nv[j];
}

#define PREP_WARPS 8
#define PREP_MAX_W 256

template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32)
qkv_prepare_kernel(const T* __restrict__ u, int ldu, T* __restrict__ q_out, int ldq, const float* __restrict__ conv_w, int taps,
                   const float* __restrict__ state, long long state_stride, const float* __restrict__ q_norm,
                   const float* __restrict__ k_norm, float eps, const int* __restrict__ positions,
                   const int* __restrict__ slot_of_token, const int* __restrict__ page_table, int max_pages,
                   const float* __restrict__ inv_freq, int rot, float magnitude, int H, int G, int hd, int vd,
                   T* __restrict__ k_pool, T* __restrict__ v_pool) {
  constexpr int NE = PREP_MAX_W / 32;
  __shared__ float s_val[PREP_WARPS][PREP_MAX_W];
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hs = blockIdx.y * PREP_WARPS + warp;          // head slot: [0, H) queries, [H, H + G) keys, then G values
  if (hs >= H + 2 * G) return;
  const bool is_q = hs < H, is_v = hs >= H + G;
  const int width = is_v ? vd : hd;
  const int col0 = is_v ? (H + G) * hd + (hs - H - G) * vd : hs * hd;
  const int C = (H + G) * hd + G * vd;
  const int pos = positions[m];
  const int slot = slot_of_token[m];
  int n = 0;
  const float* st = nullptr;
  if (conv_w) {
    n = conv_rows_back(slot_of_token, m, taps);
    st = state + (size_t)slot * state_stride;
  }
  float val[NE];
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < NE; ++e) {
    const int i = lane + 32 * e;
    val[e] = 0.f;
    if (i < width) {
      val[e] = conv_w ? conv_at(u, ldu, conv_w, st, C, taps, m, n, col0 + i, 0.f) : rl_ld(u + (size_t)m * ldu + col0 + i);
      ss = fmaf(val[e], val[e], ss);
    }
  }
  const float* nw = is_v ? nullptr : is_q ? q_norm : k_norm;
  if (nw) {
    const float r = 1.0f / sqrtf(rl_warp_sum(ss) / (float)hd + eps);
#pragma unroll
    for (int e = 0; e < NE; ++e) {
      const int i = lane + 32 * e;
      if (i < width) val[e] = val[e] * r * nw[i];
    }
  }
  if (!is_v && rot > 0) {
    const int half = rot / 2;
#pragma unroll
    for (int e = 0; e < NE; ++e) {
      const int i = lane + 32 * e;
      if (i < width) s_val[warp][i] = val[e];
    }
    __syncwarp();
#pragma unroll
    for (int e = 0; e < NE; ++e) {
      const int i = lane + 32 * e;
      if (i < rot) {
        const bool first = i < half;
        const float other = s_val[warp][first ? i + half : i - half];
        float sn, cs;
        sincosf((float)pos * inv_freq[first ? i : i - half], &sn, &cs);
        sn *= magnitude;
        cs *= magnitude;
        val[e] = first ? val[e] * cs - other * sn : val[e] * cs + other * sn;
      }
    }
  }
  T* dst;
  if (is_q) {
    dst = q_out + (size_t)m * ldq + (size_t)hs * hd;
  } else {
    if (k_pool == nullptr) return;
    const int page = page_table[(size_t)slot * max_pages + pos / RL_PAGE];
    dst = is_v ? v_pool + (((size_t)page * G + (hs - H - G)) * RL_PAGE + pos % RL_PAGE) * vd
               : k_pool + (((size_t)page * G + (hs - H)) * RL_PAGE + pos % RL_PAGE) * hd;
  }
#pragma unroll
  for (int e = 0; e < NE; ++e) {
    const int i = lane + 32 * e;
    if (i < width) rl_st(dst + i, val[e]);
  }
}

// u [M, ldu] (channels [0, C)), w float [C, taps], bias float [C] or null, act 0 none / 1 silu,
// state float [slots, state_stride] (this convolution's [taps - 1, C] at the given pointer), out [M, ldo].
extern "C" int rl_short_conv(const void* u, int ldu, int dtype, const float* w, const float* bias, int act, int channels,
                             int taps, const int* slot_of_token, const float* state, long long state_stride, void* out, int ldo,
                             int num_tokens, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && channels > 0, "rl_short_conv: bad sizes");
  RL_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "rl_short_conv: %d taps outside [1, %d]", taps, CONV_MAX_TAPS);
  RL_REQUIRE(ldu >= channels && ldo >= channels, "rl_short_conv: row strides too small");
  RL_REQUIRE(act == 0 || act == 1, "rl_short_conv: unknown activation %d", act);
  if (num_tokens == 0) return RL_OK;
  const dim3 grid(num_tokens, (channels + CONV_THREADS - 1) / CONV_THREADS);
  if (dtype == RL_F32)
    rl_launch_pdl(short_conv_kernel<float>, grid, CONV_THREADS, 0, stream, (const float*)u, ldu, w, bias, act, channels, taps,
                  slot_of_token, state, state_stride, (float*)out, ldo);
  else if (dtype == RL_BF16)
    rl_launch_pdl(short_conv_kernel<__nv_bfloat16>, grid, CONV_THREADS, 0, stream, (const __nv_bfloat16*)u, ldu, w, bias, act,
                  channels, taps, slot_of_token, state, state_stride, (__nv_bfloat16*)out, ldo);
  else
    RL_REQUIRE(false, "rl_short_conv: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_short_conv");
  return RL_OK;
}

// After the step's convolutions have run: the state takes the sequence's last taps - 1 inputs.
extern "C" int rl_short_conv_state(const void* u, int ldu, int dtype, int channels, int taps, const int* cu_seqlens,
                                   const int* seq_slots, int num_seqs, float* state, long long state_stride, cudaStream_t stream) {
  RL_REQUIRE(num_seqs >= 0 && channels > 0 && ldu >= channels, "rl_short_conv_state: bad sizes");
  RL_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "rl_short_conv_state: %d taps outside [1, %d]", taps, CONV_MAX_TAPS);
  if (num_seqs == 0 || taps == 1) return RL_OK;
  const dim3 grid(num_seqs, (channels + CONV_THREADS - 1) / CONV_THREADS);
  if (dtype == RL_F32)
    rl_launch_pdl(short_conv_state_kernel<float>, grid, CONV_THREADS, 0, stream, (const float*)u, ldu, channels, taps, cu_seqlens,
                  seq_slots, state, state_stride);
  else if (dtype == RL_BF16)
    rl_launch_pdl(short_conv_state_kernel<__nv_bfloat16>, grid, CONV_THREADS, 0, stream, (const __nv_bfloat16*)u, ldu, channels,
                  taps, cu_seqlens, seq_slots, state, state_stride);
  else
    RL_REQUIRE(false, "rl_short_conv_state: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_short_conv_state");
  return RL_OK;
}

// u: [M, ldu] holding H query heads and G key heads of head_dim, then G value heads of value_dim, as the
// projection left them.  Queries go to q_out [M, ldq]; keys and values to the pools
// ([pages, G, RL_PAGE, head_dim] and [pages, G, RL_PAGE, value_dim]; both null: nothing is cached).
// conv_w (float [C, taps], may be null), q_norm / k_norm (float [head_dim], may be null), rotary width `rot`
// (even, <= head_dim, may be 0) with inv_freq [rot / 2].
extern "C" int rl_qkv_prepare(const void* u, int ldu, void* q_out, int ldq, int dtype, const float* conv_w, int taps,
                              const float* state, long long state_stride, const float* q_norm, const float* k_norm, float eps,
                              const int* positions, const int* slot_of_token, const int* page_table, int max_pages,
                              const float* inv_freq, int rotary_dim, float magnitude, int num_tokens, int num_heads,
                              int num_kv_heads, int head_dim, int value_dim, void* k_pool, void* v_pool, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && num_heads > 0 && num_kv_heads > 0, "rl_qkv_prepare: bad sizes");
  RL_REQUIRE(head_dim > 0 && head_dim <= PREP_MAX_W && value_dim > 0 && value_dim <= PREP_MAX_W,
             "rl_qkv_prepare: head widths %d, %d outside (0, %d]", head_dim, value_dim, PREP_MAX_W);
  RL_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0, "rl_qkv_prepare: rotary width %d must be even and <= %d",
             rotary_dim, head_dim);
  RL_REQUIRE(conv_w == nullptr || (taps >= 1 && taps <= CONV_MAX_TAPS && (taps == 1 || state != nullptr)), "rl_qkv_prepare: %d taps outside [1, %d], or no state",
             taps, CONV_MAX_TAPS);
  RL_REQUIRE(ldu >= (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim && ldq >= num_heads * head_dim,
             "rl_qkv_prepare: row strides too small");
  RL_REQUIRE((k_pool == nullptr) == (v_pool == nullptr), "rl_qkv_prepare: give both cache pools or none");
  if (num_tokens == 0) return RL_OK;
  const dim3 grid(num_tokens, (num_heads + 2 * num_kv_heads + PREP_WARPS - 1) / PREP_WARPS);
  if (dtype == RL_F32)
    rl_launch_pdl(qkv_prepare_kernel<float>, grid, PREP_WARPS * 32, 0, stream, (const float*)u, ldu, (float*)q_out, ldq, conv_w, taps,
                  state, state_stride, q_norm, k_norm, eps, positions, slot_of_token, page_table, max_pages, inv_freq, rotary_dim,
                  magnitude, num_heads, num_kv_heads, head_dim, value_dim, (float*)k_pool, (float*)v_pool);
  else if (dtype == RL_BF16)
    rl_launch_pdl(qkv_prepare_kernel<__nv_bfloat16>, grid, PREP_WARPS * 32, 0, stream, (const __nv_bfloat16*)u, ldu,
                  (__nv_bfloat16*)q_out, ldq, conv_w, taps, state, state_stride, q_norm, k_norm, eps, positions, slot_of_token,
                  page_table, max_pages, inv_freq, rotary_dim, magnitude, num_heads, num_kv_heads, head_dim, value_dim,
                  (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool);
  else
    RL_REQUIRE(false, "rl_qkv_prepare: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_qkv_prepare");
  return RL_OK;
}
