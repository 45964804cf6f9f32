// Linear recurrences with a matrix state per head, carried from step to step:
//
//   S_t = a_t S_{t-1} + b_t k_t v_t^T          (S: dk x dv, float, zero for a fresh sequence)
//   o_t = S_t^T q_t (+ skip_h v_t)
//
// mode 0: a_t = decay[h], b_t = 1 (linear attention with a fixed decay a head);
// mode 1: dt = softplus(dt_raw[t, h] + dt_bias[h]), a_t = exp(-exp(rate[h]) dt), b_t = dt (a selective
//         state space: q = C, k = B, v = x, skip = D).
// Query and key heads may be shared by `hpg` consecutive heads (head h reads group h / hpg).  With act = 1
// q, k and v pass through silu as they are loaded.  Everything behind the loads is 32-bit.
//
// A block owns SCAN_COLS columns of one head's state of one sequence and walks the sequence's tokens of
// the step in order; SCAN_R neighbouring lanes share a column (lane r holds rows r, r + SCAN_R, ...) and
// add their parts of q . S[:, col] by shuffles.  Tokens are staged SCAN_TILE at a time in shared memory.
// The order of every sum is fixed by the sizes alone, so a position's output does not depend on how the
// sequence was cut into steps or on the batch.  State layout per slot: [H, dv, dk].
#include <math.h>

#include "common.cuh"

#define SCAN_R 8
#define SCAN_COLS 16
#define SCAN_TILE 16
#define SCAN_MAX_DK 256

__device__ __forceinline__ float scan_silu(float z) { return z / (1.0f + expf(-z)); }

template <typename T, int NPT>
__global__ void __launch_bounds__(SCAN_R * SCAN_COLS)
linear_scan_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ k, int ldk, const T* __restrict__ v, int ldv,
                   const T* __restrict__ dt_raw, int lddt, const float* __restrict__ dt_bias, const float* __restrict__ rate,
                   const float* __restrict__ skip, int mode, int act, const int* __restrict__ cu_seqlens,
                   const int* __restrict__ seq_slots, float* __restrict__ state, long long state_stride,
                   float* __restrict__ out, int ldo, int H, int hpg, int dk, int dv) {
  __shared__ float s_q[SCAN_TILE][NPT * SCAN_R], s_k[SCAN_TILE][NPT * SCAN_R];
  __shared__ float s_v[SCAN_TILE][SCAN_COLS], s_a[SCAN_TILE], s_b[SCAN_TILE];
  rl_pdl_trigger();
  rl_pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, r = tid % SCAN_R, c = tid / SCAN_R;
  const int col = blockIdx.z * SCAN_COLS + c;
  const bool live = col < dv;
  const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1];
  float* st = state + (size_t)seq_slots[b] * state_stride + ((size_t)h * dv + (live ? col : 0)) * dk;
  float S[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = r + SCAN_R * i;
    S[i] = (live && n < dk) ? st[n] : 0.f;
  }
  const int qk0 = (h / hpg) * dk;
  const float skip_h = skip ? skip[h] : 0.f;
  for (int t0 = lo; t0 < hi; t0 += SCAN_TILE) {
    const int nt = min(SCAN_TILE, hi - t0);
    __syncthreads();
    for (int idx = tid; idx < nt * dk; idx += SCAN_R * SCAN_COLS) {
      const int tt = idx / dk, n = idx % dk;
      float qv = rl_ld(q + (size_t)(t0 + tt) * ldq + qk0 + n), kv = rl_ld(k + (size_t)(t0 + tt) * ldk + qk0 + n);
      if (act) { qv = scan_silu(qv); kv = scan_silu(kv); }
      s_q[tt][n] = qv;
      s_k[tt][n] = kv;
    }
    for (int idx = tid; idx < nt * SCAN_COLS; idx += SCAN_R * SCAN_COLS) {
      const int tt = idx / SCAN_COLS, cc = blockIdx.z * SCAN_COLS + idx % SCAN_COLS;
      float vv = cc < dv ? rl_ld(v + (size_t)(t0 + tt) * ldv + (size_t)h * dv + cc) : 0.f;
      if (act) vv = scan_silu(vv);
      s_v[tt][idx % SCAN_COLS] = vv;
    }
    if (tid < nt) {
      if (mode == 0) {
        s_a[tid] = rate[h];
        s_b[tid] = 1.0f;
      } else {
        const float z = rl_ld(dt_raw + (size_t)(t0 + tid) * lddt + h) + dt_bias[h];
        const float dt = z > 20.0f ? z : log1pf(expf(z));
        s_a[tid] = expf(-expf(rate[h]) * dt);
        s_b[tid] = dt;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float a = s_a[tt], vv = s_v[tt][c], bv = s_b[tt] * vv;
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        const int n = r + SCAN_R * i;
        if (n < dk) {
          S[i] = fmaf(a, S[i], bv * s_k[tt][n]);
          part = fmaf(S[i], s_q[tt][n], part);
        }
      }
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      part += __shfl_xor_sync(0xffffffffu, part, 4);
      if (r == 0 && live) out[(size_t)(t0 + tt) * ldo + (size_t)h * dv + col] = part + skip_h * vv;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = r + SCAN_R * i;
      if (n < dk) st[n] = S[i];
    }
  }
}

template <typename T>
static int scan_launch(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const void* dt_raw, int lddt,
                       const float* dt_bias, const float* rate, const float* skip, int mode, int act, const int* cu_seqlens,
                       const int* seq_slots, int num_seqs, float* state, long long state_stride, float* out, int ldo, int H,
                       int hpg, int dk, int dv, cudaStream_t stream) {
  const dim3 grid(num_seqs, H, (dv + SCAN_COLS - 1) / SCAN_COLS);
  const int threads = SCAN_R * SCAN_COLS;
#define SCAN_GO(NPT)                                                                                                        \
  rl_launch_pdl(linear_scan_kernel<T, NPT>, grid, threads, 0, stream, (const T*)q, ldq, (const T*)k, ldk, (const T*)v, ldv, \
                (const T*)dt_raw, lddt, dt_bias, rate, skip, mode, act, cu_seqlens, seq_slots, state, state_stride, out, ldo, H, hpg, dk, dv)
  if (dk <= 4 * SCAN_R) SCAN_GO(4);
  else if (dk <= 8 * SCAN_R) SCAN_GO(8);
  else if (dk <= 16 * SCAN_R) SCAN_GO(16);
  else SCAN_GO(32);
#undef SCAN_GO
  return 0;
}

// q, k: [M, ld] with group g at columns [g * dk, (g + 1) * dk); v: [M, ldv] with head h at [h * dv, (h + 1) * dv);
// dt_raw [M, lddt] (mode 1; same dtype); dt_bias, rate, skip: float [H] (skip may be null; rate is the decay itself
// in mode 0 and the logarithm of the decay rate in mode 1).  state: float, this recurrence's [H, dv, dk] of slot s
// at state + s * state_stride.  out: float [M, ldo].
extern "C" int rl_linear_scan(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const void* dt_raw,
                              int lddt, int dtype, const float* dt_bias, const float* rate, const float* skip, int mode, int act,
                              const int* cu_seqlens, const int* seq_slots, int num_seqs, float* state, long long state_stride,
                              float* out, int ldo, int num_heads, int heads_per_group, int dk, int dv, cudaStream_t stream) {
  RL_REQUIRE(num_seqs >= 0 && num_heads > 0 && heads_per_group > 0 && num_heads % heads_per_group == 0, "rl_linear_scan: bad sizes");
  RL_REQUIRE(dk > 0 && dk <= SCAN_MAX_DK && dv > 0, "rl_linear_scan: dk %d outside (0, %d] or dv %d", dk, SCAN_MAX_DK, dv);
  RL_REQUIRE(mode == 0 || (mode == 1 && dt_raw != nullptr && dt_bias != nullptr), "rl_linear_scan: mode %d, or no step sizes", mode);
  RL_REQUIRE(rate != nullptr && state != nullptr, "rl_linear_scan: no decay or no state");
  RL_REQUIRE(num_heads <= 65535, "rl_linear_scan: more than 65,535 heads");
  if (num_seqs == 0) return RL_OK;
  if (dtype == RL_F32)
    scan_launch<float>(q, ldq, k, ldk, v, ldv, dt_raw, lddt, dt_bias, rate, skip, mode, act, cu_seqlens, seq_slots, num_seqs, state,
                       state_stride, out, ldo, num_heads, heads_per_group, dk, dv, stream);
  else if (dtype == RL_BF16)
    scan_launch<__nv_bfloat16>(q, ldq, k, ldk, v, ldv, dt_raw, lddt, dt_bias, rate, skip, mode, act, cu_seqlens, seq_slots, num_seqs,
                               state, state_stride, out, ldo, num_heads, heads_per_group, dk, dv, stream);
  else
    RL_REQUIRE(false, "rl_linear_scan: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_linear_scan");
  return RL_OK;
}
