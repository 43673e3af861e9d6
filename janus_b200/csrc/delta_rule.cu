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
// A block owns one (sequence, head, 16 value columns).  Four of its warps walk the recurrence: eight lanes share a
// column, each with a run of RMAX rows of it in registers (d <= 8 RMAX).  With a = S_old^T k and c = S_old^T q of
// the state before the token, w = beta (v - g a) and o = g c + (k . q) w: both sums over the column are taken before
// the update, in one round of shuffles.  The other four warps stage the chunk of tokens that comes next into the
// second of two shared-memory buffers meanwhile: a warp per token reads q and k, makes them unit vectors in
// registers and writes them laid out as the walking lanes read them (a lane's run of rows as float4s, runs padded
// so that the eight lanes meet eight different groups of banks), with the token's gates behind them.
#include <math_constants.h>
#include <stdio.h>

#include "common.cuh"

namespace {

constexpr int WALKERS = 128;         // threads that walk the recurrence
constexpr int THREADS = 256;         // and as many that stage the next tokens
constexpr int LANES = 8;             // lanes that share a column
constexpr int CT = WALKERS / LANES;  // columns of a block

template <int RMAX, int CH>
__global__ void __launch_bounds__(THREADS) delta_rule_kernel(
    const float* __restrict__ conv, int ldc, int q_col, int k_col, int v_col, const float* __restrict__ raw, int ld,
    int b_col, int a_col, const float* __restrict__ A_log, const float* __restrict__ dt_bias, float unit_eps,
    float* __restrict__ out, float* __restrict__ state, long long slot_stride, long long state_off,
    const int* __restrict__ q_start, const int* __restrict__ seq_slot, int H, int G, int d, int e) {
  constexpr int SEG = RMAX + 4;                          // a lane's run of rows and its padding
  constexpr int DP = LANES * SEG;                        // q (or k) of a token as staged
  constexpr int ROW = 2 * DP + CT + 4;                   // q, k, v tile, g, beta, k . q, unused
  constexpr int JMAX = RMAX * LANES / 32;                // numbers of q (or k) a staging lane holds
  constexpr int PER_WARP = CH / 4;                       // tokens of a chunk that one staging warp takes
  static_assert(RMAX % 4 == 0 && CH % 4 == 0, "runs are read as float4s; four warps share a chunk");
  __shared__ __align__(16) float stage[2][CH][ROW];
  jb::pdl_launch_dependents();
  const int seq = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * CT;
  const int j = h / (H / G);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool walker = threadIdx.x < WALKERS;
  const int p = threadIdx.x & (LANES - 1), c = c0 + ((threadIdx.x & (WALKERS - 1)) >> 3);
  const bool has_col = walker && c < e;
  for (int i = threadIdx.x; i < 2 * CH * ROW; i += THREADS) (&stage[0][0][0])[i] = 0.0f;   // rows behind d stay zero
  const float neg_rate = -expf(A_log[h]), bias = dt_bias[h];
  const float q_mult = rsqrtf((float)d);
  jb::pdl_wait();
  const int t0 = q_start[seq], n_tok = q_start[seq + 1] - t0;
  float* S_g = state + (size_t)seq_slot[seq] * slot_stride + state_off + (size_t)h * d * e;
  float S[RMAX];
#pragma unroll
  for (int i = 0; i < RMAX; ++i) {
    const int r = p * RMAX + i;
    S[i] = (has_col && r < d) ? S_g[(size_t)r * e + c] : 0.0f;
  }
  __syncthreads();                                       // the zeros are in place before the first tokens land

  // a staging warp brings its tokens of a chunk: loads first, for all of them, then the sums and the stores
  auto bring = [&](int chunk, int buf) {
    const int first = chunk * CH, n = min(CH, n_tok - first);
    const int sw = warp - WALKERS / 32;
    float qv[PER_WARP][JMAX], kv[PER_WARP][JMAX], vv[PER_WARP], av[PER_WARP], bv[PER_WARP];
#pragma unroll
    for (int u = 0; u < PER_WARP; ++u) {
      const int tt = sw + 4 * u;
      const size_t t = (size_t)(t0 + first + min(tt, n - 1));
      const float* qs = conv + t * ldc + q_col + (size_t)j * d;
      const float* ks = conv + t * ldc + k_col + (size_t)j * d;
#pragma unroll
      for (int x = 0; x < JMAX; ++x) {
        const int r = lane + 32 * x;
        qv[u][x] = r < d ? qs[r] : 0.0f;
        kv[u][x] = r < d ? ks[r] : 0.0f;
      }
      vv[u] = (lane < CT && c0 + lane < e) ? conv[t * ldc + v_col + (size_t)h * e + c0 + lane] : 0.0f;
      av[u] = raw[t * ld + a_col + h];
      bv[u] = raw[t * ld + b_col + h];
    }
#pragma unroll
    for (int u = 0; u < PER_WARP; ++u) {
      const int tt = sw + 4 * u;
      if (tt >= n) break;
      float sq = 0.0f, sk = 0.0f, qk = 0.0f;
#pragma unroll
      for (int x = 0; x < JMAX; ++x) {
        sq = fmaf(qv[u][x], qv[u][x], sq);
        sk = fmaf(kv[u][x], kv[u][x], sk);
        qk = fmaf(qv[u][x], kv[u][x], qk);
      }
      sq = jb::warp_sum(sq);
      sk = jb::warp_sum(sk);
      qk = jb::warp_sum(qk);
      const float iq = q_mult / sqrtf(sq + unit_eps), ik = 1.0f / sqrtf(sk + unit_eps);
      float* row = stage[buf][tt];
#pragma unroll
      for (int x = 0; x < JMAX; ++x) {
        const int r = lane + 32 * x;
        if (r < d) {
          const int at = (r / RMAX) * SEG + r % RMAX;
          row[at] = qv[u][x] * iq;
          row[DP + at] = kv[u][x] * ik;
        }
      }
      if (lane < CT) row[2 * DP + lane] = vv[u];
      if (lane == 0) {
        const float z = av[u] + bias;
        const float sp = z > 20.0f ? z : log1pf(expf(z));
        row[2 * DP + CT] = expf(neg_rate * sp);
        row[2 * DP + CT + 1] = 1.0f / (1.0f + expf(-bv[u]));
        row[2 * DP + CT + 2] = qk * iq * ik;
      }
    }
  };

  const int n_chunks = (n_tok + CH - 1) / CH;
  if (!walker && n_chunks > 0) bring(0, 0);
  __syncthreads();
  for (int chunk = 0; chunk < n_chunks; ++chunk) {
    const int buf = chunk & 1;
    if (!walker) {
      if (chunk + 1 < n_chunks) bring(chunk + 1, buf ^ 1);
    } else {
      const int first = chunk * CH, n = min(CH, n_tok - first);
      for (int tt = 0; tt < n; ++tt) {
        const float* row = stage[buf][tt];
        const float4* q4 = reinterpret_cast<const float4*>(row + p * SEG);
        const float4* k4 = reinterpret_cast<const float4*>(row + DP + p * SEG);
        float kr[RMAX];
        float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
#pragma unroll
        for (int i = 0; i < RMAX; i += 4) {
          const float4 kk = k4[i >> 2], qq = q4[i >> 2];
          kr[i] = kk.x, kr[i + 1] = kk.y, kr[i + 2] = kk.z, kr[i + 3] = kk.w;
          a0 = fmaf(S[i], kk.x, a0);
          a1 = fmaf(S[i + 1], kk.y, a1);
          a0 = fmaf(S[i + 2], kk.z, a0);
          a1 = fmaf(S[i + 3], kk.w, a1);
          b0 = fmaf(S[i], qq.x, b0);
          b1 = fmaf(S[i + 1], qq.y, b1);
          b0 = fmaf(S[i + 2], qq.z, b0);
          b1 = fmaf(S[i + 3], qq.w, b1);
        }
        float a = a0 + a1, b = b0 + b1;
#pragma unroll
        for (int o = 1; o < LANES; o <<= 1) {
          a += __shfl_xor_sync(0xffffffffu, a, o);
          b += __shfl_xor_sync(0xffffffffu, b, o);
        }
        const float g = row[2 * DP + CT], beta = row[2 * DP + CT + 1], kq = row[2 * DP + CT + 2];
        const float w = beta * (row[2 * DP + ((threadIdx.x & (WALKERS - 1)) >> 3)] - g * a);
#pragma unroll
        for (int i = 0; i < RMAX; ++i) S[i] = fmaf(kr[i], w, g * S[i]);
        if (p == 0 && has_col) out[((size_t)(t0 + first + tt) * H + h) * e + c] = fmaf(kq, w, g * b);
      }
    }
    __syncthreads();                                     // the next chunk is staged; this one is done with
  }
  if (has_col) {
#pragma unroll
    for (int i = 0; i < RMAX; ++i) {
      const int r = p * RMAX + i;
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
  else JB_LAUNCH_DR(32, 8);   // 8 RMAX rows hold d; a chunk's two buffers stay within the static shared memory
#undef JB_LAUNCH_DR
  return (int)err;
}
