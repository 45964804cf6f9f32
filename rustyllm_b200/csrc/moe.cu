// Mixture of experts on the CUDA cores: router, and the chosen experts' gated feed-forward
// per (token, choice).  Float or bf16 storage, 32-bit accumulation.
//
//   router : z = Wr h + b (32-bit), the `top` largest logits chosen (ties: the lower index),
//            weights = softmax over the chosen logits only
//   expert : y_e = Wdown_e (silu(Wgate_e h) * (Wup_e h))
//   output : residual += sum_c weight_c * y_{e_c}     (choices in the order of falling logits)
//
// Every token is computed by itself, its sums in an order that its own sizes fix, so a token's
// result does not depend on the batch.  Weights: gate_up [E, 2, F, d] (an expert's gate rows,
// then its up rows), down [E, d, F].
#include <math.h>

#include "common.cuh"

#define MOE_THREADS 256
#define MOE_MAX_TOP 32

// ------------------------------------------------------------------ router
// One block a token; warp w takes experts w, w + 8, ...; then warp 0 selects.
template <typename T>
__global__ void __launch_bounds__(MOE_THREADS)
moe_route_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ wr, const float* __restrict__ bias,
                 int d, int E, int top, int* __restrict__ ids, float* __restrict__ weights) {
  extern __shared__ float s_logit[];     // [E]
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* xr = x + (size_t)m * ldx;
  for (int e = warp; e < E; e += MOE_THREADS / 32) {
    const T* w = wr + (size_t)e * d;
    float part = 0.f;
    for (int i = lane; i < d; i += 32) part = fmaf(rl_ld(xr + i), rl_ld(w + i), part);
    part = rl_warp_sum(part);
    if (lane == 0) s_logit[e] = part + (bias ? bias[e] : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  float chosen = 0.f, first = 0.f, denom = 0.f;      // lane c keeps choice c's logit
  int chosen_id = 0;
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float z = s_logit[e];
      if (z > best) { best = z; at = e; }            // ascending e: the lower index wins a tie
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = 0;                    // all logits NaN or -inf: still a valid index
    if (c == 0) first = best;
    if (lane == c) { chosen = best; chosen_id = at; }
    __syncwarp();
    if (lane == 0) s_logit[at] = -INFINITY;
    __syncwarp();
  }
  const float e_c = lane < top ? expf(chosen - first) : 0.f;
  denom = rl_warp_sum(e_c);
  if (lane < top) {
    ids[(size_t)m * top + lane] = chosen_id;
    weights[(size_t)m * top + lane] = e_c / denom;
  }
}

extern "C" int rl_moe_route(const void* x, int ldx, const void* router, const float* bias, int dtype, int num_tokens,
                            int hidden, int num_experts, int top, int* ids, float* weights, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && hidden > 0 && num_experts > 0, "rl_moe_route: bad sizes M=%d d=%d E=%d", num_tokens, hidden, num_experts);
  RL_REQUIRE(top > 0 && top <= num_experts && top <= MOE_MAX_TOP, "rl_moe_route: top %d must lie in [1, min(%d, %d)]", top, num_experts, MOE_MAX_TOP);
  RL_REQUIRE(num_experts <= 8192, "rl_moe_route: at most 8192 experts");
  if (num_tokens == 0) return RL_OK;
  const size_t smem = (size_t)num_experts * sizeof(float);
  if (dtype == RL_F32)
    rl_launch_pdl(moe_route_kernel<float>, num_tokens, MOE_THREADS, smem, stream, (const float*)x, ldx, (const float*)router, bias,
                  hidden, num_experts, top, ids, weights);
  else if (dtype == RL_BF16)
    rl_launch_pdl(moe_route_kernel<__nv_bfloat16>, num_tokens, MOE_THREADS, smem, stream, (const __nv_bfloat16*)x, ldx,
                  (const __nv_bfloat16*)router, bias, hidden, num_experts, top, ids, weights);
  else
    RL_REQUIRE(false, "rl_moe_route: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_moe_route");
  return RL_OK;
}

// ------------------------------------------------------------------ gate and up of the chosen experts
// grid (row blocks of F, M * top); the token's input in shared memory; a warp a row of the expert.
template <typename T>
__global__ void __launch_bounds__(MOE_THREADS)
moe_gate_up_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ wgu, const int* __restrict__ ids,
                   int d, int F, int top, T* __restrict__ h) {
  extern __shared__ float s_x[];          // [d]
  rl_pdl_trigger();
  rl_pdl_wait();
  const int pair = blockIdx.y, m = pair / top;
  const int e = ids[pair];
  const T* xr = x + (size_t)m * ldx;
  for (int i = threadIdx.x; i < d; i += MOE_THREADS) s_x[i] = rl_ld(xr + i);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * (MOE_THREADS / 32) + warp;
  if (r >= F) return;
  const T* wg = wgu + ((size_t)e * 2 * F + r) * d;
  const T* wu = wg + (size_t)F * d;
  float g = 0.f, u = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float xv = s_x[i];
    g = fmaf(xv, rl_ld(wg + i), g);
    u = fmaf(xv, rl_ld(wu + i), u);
  }
  g = rl_warp_sum(g);
  u = rl_warp_sum(u);
  if (lane == 0) rl_st(h + (size_t)pair * F + r, g / (1.0f + expf(-g)) * u);
}

// ------------------------------------------------------------------ down of the chosen experts, weighted, into the residual
// grid (row blocks of d, M); a warp an output element; choices summed in their order.
template <typename T>
__global__ void __launch_bounds__(MOE_THREADS)
moe_down_kernel(const T* __restrict__ h, const T* __restrict__ wd, const int* __restrict__ ids,
                const float* __restrict__ weights, int d, int F, int top, float* __restrict__ residual) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * (MOE_THREADS / 32) + warp;
  if (r >= d) return;
  float y = 0.f;
  for (int c = 0; c < top; ++c) {
    const int e = ids[(size_t)m * top + c];
    const T* w = wd + ((size_t)e * d + r) * F;
    const T* hr = h + ((size_t)m * top + c) * F;
    float part = 0.f;
    for (int i = lane; i < F; i += 32) part = fmaf(rl_ld(hr + i), rl_ld(w + i), part);
    part = rl_warp_sum(part);
    y = fmaf(weights[(size_t)m * top + c], part, y);
  }
  if (lane == 0) residual[(size_t)m * d + r] += y;
}

// x [M, ldx]; gate_up [E, 2, F, d]; down [E, d, F]; ids, weights [M, top] (from rl_moe_route);
// h [M * top, F] scratch in the same dtype; residual [M, d] float, added into.
extern "C" int rl_moe_experts(const void* x, int ldx, const void* gate_up, const void* down, int dtype, const int* ids,
                              const float* weights, int num_tokens, int hidden, int expert_ff, int num_experts, int top,
                              void* h, float* residual, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && hidden > 0 && expert_ff > 0 && num_experts > 0 && top > 0,
             "rl_moe_experts: bad sizes M=%d d=%d F=%d E=%d top=%d", num_tokens, hidden, expert_ff, num_experts, top);
  RL_REQUIRE((long long)num_tokens * top <= 65535LL * 1024, "rl_moe_experts: too many (token, choice) pairs for one launch");
  RL_REQUIRE(hidden <= 48 * 1024 / 4, "rl_moe_experts: hidden size %d above %d", hidden, 48 * 1024 / 4);
  if (num_tokens == 0) return RL_OK;
  const int per = MOE_THREADS / 32;
  // grid.y is limited to 65535: pairs beyond that run as further launches
  for (long long p0 = 0; p0 < (long long)num_tokens * top; p0 += 65535LL / top * top) {
    const long long n = ((long long)num_tokens * top - p0) < 65535LL / top * top ? ((long long)num_tokens * top - p0) : 65535LL / top * top;
    const int m0 = (int)(p0 / top), mt = (int)(n / top);
    dim3 g1((expert_ff + per - 1) / per, (unsigned)n), g2((hidden + per - 1) / per, (unsigned)mt);
    const size_t smem = (size_t)hidden * sizeof(float);
    if (dtype == RL_F32) {
      rl_launch_pdl(moe_gate_up_kernel<float>, g1, MOE_THREADS, smem, stream, (const float*)x + (size_t)m0 * ldx, ldx, (const float*)gate_up,
                    ids + p0, hidden, expert_ff, top, (float*)h + (size_t)p0 * expert_ff);
      rl_launch_pdl(moe_down_kernel<float>, g2, MOE_THREADS, 0, stream, (const float*)h + (size_t)p0 * expert_ff, (const float*)down,
                    ids + p0, weights + p0, hidden, expert_ff, top, residual + (size_t)m0 * hidden);
    } else if (dtype == RL_BF16) {
      rl_launch_pdl(moe_gate_up_kernel<__nv_bfloat16>, g1, MOE_THREADS, smem, stream, (const __nv_bfloat16*)x + (size_t)m0 * ldx, ldx,
                    (const __nv_bfloat16*)gate_up, ids + p0, hidden, expert_ff, top, (__nv_bfloat16*)h + (size_t)p0 * expert_ff);
      rl_launch_pdl(moe_down_kernel<__nv_bfloat16>, g2, MOE_THREADS, 0, stream, (const __nv_bfloat16*)h + (size_t)p0 * expert_ff,
                    (const __nv_bfloat16*)down, ids + p0, weights + p0, hidden, expert_ff, top, residual + (size_t)m0 * hidden);
    } else {
      RL_REQUIRE(false, "rl_moe_experts: unknown dtype %d", dtype);
    }
    RL_LAUNCH_CHECK("rl_moe_experts");
  }
  return RL_OK;
}
