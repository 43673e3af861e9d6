// The gated delta rule, a recurrence with a matrix state per head, for prompts, portions of prompts and single
// tokens alike.  All arithmetic is float32.  Per head h (query/key head j = h / (H / G)) with state S [d, e]:
//
//   q_t = u_q / sqrt(sum(u_q^2) + unit_eps) * d^-1/2,  k_t = u_k / sqrt(sum(u_k^2) + unit_eps)     (unit vectors)
//   beta_t = sigmoid(b_t),  g_t = exp(-exp(A_log_h) softplus(a_t + dt_bias_h))
//   S <- g_t S;  w = beta_t (v_t - S^T k_t);  S <- S + k_t w^T;  o_t = S^T q_t                 (the read-out sees the write)
//
// u_q, u_k, v are columns of `conv` (the projections after their short convolution and activation), b and a columns
// of `raw` (the projection as it left the product).  The state of a sequence lives at state[slot][state_off ...] as
// [H][d][e], is read at the start of a step and written back at its end.
//
// A block owns one (sequence, head, 16 value columns); eight lanes share a column, each with every eighth row of it
// in registers (up to 32 rows: d <= 256).  With a = S_old^T k and c = S_old^T q of the state before the token,
// w = beta (v - g a) and o = g c + (k . q) w: both sums over the column are taken before the update, in one round
// of shuffles.  Tokens are staged in chunks through a ring of two shared-memory buffers (cp.async), normed there by
// a warp per token, then walked one after another without a barrier.
#include <math_constants.h>
#include <stdio.h>

#include "common.cuh"

namespace {

constexpr int THREADS = 128;
constexpr int LANES = 8;             // lanes that share a column
constexpr int CT = THREADS / LANES;  // columns of a block

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int RMAX, int CH>
__global__ void __launch_bounds__(THREADS) delta_rule_kernel(
    const float* __restrict__ conv, int ldc, int q_col, int k_col, int v_col, const float* __restrict__ raw, int ld,
    int b_col, int a_col, const float* __restrict__ A_log, const float* __restrict__ dt_bias, float unit_eps,
    float* __restrict__ out, float* __restrict__ state, long long slot_stride, long long state_off,
    const int* __restrict__ q_start, const int* __restrict__ seq_slot, int H, int G, int d, int e) {
  constexpr int DP = RMAX * LANES;                       // rows as staged: zeros behind the d that exist
  constexpr int ROW = 2 * DP + CT + 4;                   // q, k, v tile, (a -> g), (b -> beta), k . q, unused
  __shared__ __align__(16) float stage[2][CH][ROW];
  jb::pdl_launch_dependents();
  const int seq = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * CT;
  const int j = h / (H / G);
  const int p = threadIdx.x & (LANES - 1), c = c0 + (threadIdx.x >> 3);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool has_col = c < e;
  for (int i = threadIdx.x; i < 2 * CH * ROW; i += THREADS) (&stage[0][0][0])[i] = 0.0f;
  const float neg_rate = -expf(A_log[h]), bias = dt_bias[h];
  jb::pdl_wait();
  const int t0 = q_start[seq], n_tok = q_start[seq + 1] - t0;
  float* S_g = state + (size_t)seq_slot[seq] * slot_stride + state_off + (size_t)h * d * e;
  float S[RMAX];
#pragma unroll
  for (int i = 0; i < RMAX; ++i) {
    const int r = p + LANES * i;
    S[i] = (has_col && r < d) ? S_g[(size_t)r * e + c] : 0.0f;
  }
  __syncthreads();                                       // the zeros are in place before the first copies land
  auto issue = [&](int chunk, int buf) {
    const int first = chunk * CH, n = min(CH, n_tok - first);
    for (int i = threadIdx.x; i < n * (2 * d + CT + 2); i += THREADS) {
      const int tt = i / (2 * d + CT + 2), x = i % (2 * d + CT + 2);
      const size_t t = (size_t)(t0 + first + tt);
      float* row = stage[buf][tt];
      if (x < d) cp_async4(row + x, conv + t * ldc + q_col + (size_t)j * d + x);
      else if (x < 2 * d) cp_async4(row + DP + x - d, conv + t * ldc + k_col + (size_t)j * d + x - d);
      else if (x < 2 * d + CT) {
        const int cc = x - 2 * d;
        if (c0 + cc < e) cp_async4(row + 2 * DP + cc, conv + t * ldc + v_col + (size_t)h * e + c0 + cc);
      } else if (x == 2 * d + CT) cp_async4(row + 2 * DP + CT, raw + t * ld + a_col + h);
      else cp_async4(row + 2 * DP + CT + 1, raw + t * ld + b_col + h);
    }
  };
  const int n_chunks = (n_tok + CH - 1) / CH;
  const float q_mult = rsqrtf((float)d);
  if (n_chunks > 0) issue(0, 0);
  cp_async_commit();
  for (int chunk = 0; chunk < n_chunks; ++chunk) {
    const int buf = chunk & 1;
    const int first = chunk * CH, n = min(CH, n_tok - first);
    cp_async_wait_all();
    __syncthreads();                                     // this chunk has landed; the chunk before is done with
    if (chunk + 1 < n_chunks) issue(chunk + 1, buf ^ 1);
    cp_async_commit();
    for (int tt = warp; tt < n; tt += THREADS / 32) {    // a warp norms a token's q and k and makes its gates
      float* row = stage[buf][tt];
      float sq = 0.0f, sk = 0.0f, qk = 0.0f;
      for (int x = lane; x < d; x += 32) {
        const float a = row[x], b = row[DP + x];
        sq = fmaf(a, a, sq);
        sk = fmaf(b, b, sk);
        qk = fmaf(a, b, qk);
      }
      sq = jb::warp_sum(sq);
      sk = jb::warp_sum(sk);
      qk = jb::warp_sum(qk);
      const float iq = q_mult / sqrtf(sq + unit_eps), ik = 1.0f / sqrtf(sk + unit_eps);
      for (int x = lane; x < d; x += 32) {
        row[x] *= iq;
        row[DP + x] *= ik;
      }
      if (lane == 0) {
        const float z = row[2 * DP + CT] + bias;
        const float sp = z > 20.0f ? z : log1pf(expf(z));
        row[2 * DP + CT] = expf(neg_rate * sp);
        row[2 * DP + CT + 1] = 1.0f / (1.0f + expf(-row[2 * DP + CT + 1]));
        row[2 * DP + CT + 2] = qk * iq * ik;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float* row = stage[buf][tt];
      float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
#pragma unroll
      for (int i = 0; i < RMAX; i += 2) {
        a0 = fmaf(S[i], row[DP + p + LANES * i], a0);
        b0 = fmaf(S[i], row[p + LANES * i], b0);
        a1 = fmaf(S[i + 1], row[DP + p + LANES * (i + 1)], a1);
        b1 = fmaf(S[i + 1], row[p + LANES * (i + 1)], b1);
      }
      float a = a0 + a1, b = b0 + b1;
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
      }
      const float g = row[2 * DP + CT], beta = row[2 * DP + CT + 1], kq = row[2 * DP + CT + 2];
      const float w = beta * (row[2 * DP + (threadIdx.x >> 3)] - g * a);
#pragma unroll
      for (int i = 0; i < RMAX; ++i) S[i] = fmaf(row[DP + p + LANES * i], w, g * S[i]);
      if (p == 0 && has_col) out[((size_t)(t0 + first + tt) * H + h) * e + c] = fmaf(kq, w, g * b);
    }
  }
  if (has_col) {
#pragma unroll
    for (int i = 0; i < RMAX; ++i) {
      const int r = p + LANES * i;
      if (r < d) S_g[(size_t)r * e + c] = S[i];
    }
  }
}

}  // namespace

// conv: float32 [T, ldc], queries at q_col ([G][d]), keys at k_col ([G][d]), values at v_col ([H][e]); raw: float32
// [T, ld], beta's argument at b_col ([H]), the decay's at a_col ([H]); A_log, dt_bias: float32 [H]; out: float32
// [T, H e]; state: per slot slot_stride floats, the recurrence's [H][d][e] at state_off.
JB_EXPORT int jb_delta_rule(const float* conv, int ldc, int q_col, int k_col, int v_col, const float* raw, int ld,
                            int b_col, int a_col, const float* A_log, const float* dt_bias, float unit_eps, float* out,
                            float* state, long long slot_stride, long long state_off, const int* q_start,
                            const int* seq_slot, int n_seqs, int H, int G, int d, int e, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  JB_REFUSE(d < 1 || d > 256 || e < 1, "delta_rule: key size %d is outside [1, 256]", d);
  JB_REFUSE(G < 1 || H % G != 0, "delta_rule: %d heads are not a multiple of %d key heads", H, G);
  jb::Launch cfg(dim3((e + CT - 1) / CT, H, n_seqs), dim3(THREADS), 0, stream);
  cudaError_t err;
#define JB_LAUNCH_DR(RMAX, CH)                                                                                       \
  err = cudaLaunchKernelEx(&cfg.c, delta_rule_kernel<RMAX, CH>, conv, ldc, q_col, k_col, v_col, raw, ld, b_col, a_col, \
                           A_log, dt_bias, unit_eps, out, state, slot_stride, state_off, q_start, seq_slot, H, G, d, e)
  if (d <= 64) JB_LAUNCH_DR(8, 16);
  else if (d <= 128) JB_LAUNCH_DR(16, 16);
  else JB_LAUNCH_DR(32, 8);
#undef JB_LAUNCH_DR
  return (int)err;
}
