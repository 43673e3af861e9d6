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
// the update, in one round of shuffles.  Tokens are walked two at a time: with S the state before the pair, all four
// sums S^T k1, S^T q1, S^T k2, S^T q2 are taken in one pass and one round of shuffles, and the second token's follow
// from them, since the state between the two is g1 S + k1 w1^T:
//   a2 = g1 (S^T k2) + (k1 . k2) w1,   c2 = g1 (S^T q2) + (k1 . q2) w1,   S <- g1 g2 S + k1 (g2 w1)^T + k2 w2^T,
// which halves the chain of dependent instructions a token.  The other four warps stage the chunk of tokens that
// comes next into the second of two shared-memory buffers meanwhile: a warp per pair of tokens reads q and k, makes
// them unit vectors in registers and writes them laid out as the walking lanes read them (a lane's run of rows as
// float4s, runs padded so that the eight lanes meet eight different groups of banks), with the token's gates and
// the products k . q, k1 . k2, k1 . q2 behind them.
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
  constexpr int ROW = 2 * DP + CT + 8;                   // q, k, v tile, g, beta, k . q, k' . k, k' . q (k' of the token before), unused
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
      const int tt = 2 * (sw + 4 * (u >> 1)) + (u & 1);  // a warp takes both tokens of a pair
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
    float ik_before = 0.0f;
#pragma unroll
    for (int u = 0; u < PER_WARP; ++u) {
      const int tt = 2 * (sw + 4 * (u >> 1)) + (u & 1);
      if (tt >= n) break;
      float sq = 0.0f, sk = 0.0f, qk = 0.0f, kk = 0.0f, kq = 0.0f;
#pragma unroll
      for (int x = 0; x < JMAX; ++x) {
        sq = fmaf(qv[u][x], qv[u][x], sq);
        sk = fmaf(kv[u][x], kv[u][x], sk);
        qk = fmaf(qv[u][x], kv[u][x], qk);
        if (u & 1) {
          kk = fmaf(kv[u - (u & 1)][x], kv[u][x], kk);
          kq = fmaf(kv[u - (u & 1)][x], qv[u][x], kq);
        }
      }
      sq = jb::warp_sum(sq);
      sk = jb::warp_sum(sk);
      qk = jb::warp_sum(qk);
      if (u & 1) {
        kk = jb::warp_sum(kk);
        kq = jb::warp_sum(kq);
      }
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
        row[2 * DP + CT + 3] = kk * ik_before * ik;
        row[2 * DP + CT + 4] = kq * ik_before * iq;
      }
      ik_before = ik;
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
      const int col = (threadIdx.x & (WALKERS - 1)) >> 3;
      int tt = 0;
      for (; tt + 1 < n; tt += 2) {                      // two tokens from one pass over the state
        const float* r1 = stage[buf][tt];
        const float* r2 = stage[buf][tt + 1];
        const float4* q1 = reinterpret_cast<const float4*>(r1 + p * SEG);
        const float4* k1 = reinterpret_cast<const float4*>(r1 + DP + p * SEG);
        const float4* q2 = reinterpret_cast<const float4*>(r2 + p * SEG);
        const float4* k2 = reinterpret_cast<const float4*>(r2 + DP + p * SEG);
        float kr1[RMAX], kr2[RMAX];
        float a1 = 0.0f, c1 = 0.0f, a2 = 0.0f, c2 = 0.0f, a1b = 0.0f, c1b = 0.0f, a2b = 0.0f, c2b = 0.0f;
#pragma unroll
        for (int i = 0; i < RMAX; i += 4) {
          const float4 ka = k1[i >> 2], qa = q1[i >> 2], kb = k2[i >> 2], qb = q2[i >> 2];
          kr1[i] = ka.x, kr1[i + 1] = ka.y, kr1[i + 2] = ka.z, kr1[i + 3] = ka.w;
          kr2[i] = kb.x, kr2[i + 1] = kb.y, kr2[i + 2] = kb.z, kr2[i + 3] = kb.w;
          a1 = fmaf(S[i], ka.x, a1), a1b = fmaf(S[i + 1], ka.y, a1b);
          a1 = fmaf(S[i + 2], ka.z, a1), a1b = fmaf(S[i + 3], ka.w, a1b);
          c1 = fmaf(S[i], qa.x, c1), c1b = fmaf(S[i + 1], qa.y, c1b);
          c1 = fmaf(S[i + 2], qa.z, c1), c1b = fmaf(S[i + 3], qa.w, c1b);
          a2 = fmaf(S[i], kb.x, a2), a2b = fmaf(S[i + 1], kb.y, a2b);
          a2 = fmaf(S[i + 2], kb.z, a2), a2b = fmaf(S[i + 3], kb.w, a2b);
          c2 = fmaf(S[i], qb.x, c2), c2b = fmaf(S[i + 1], qb.y, c2b);
          c2 = fmaf(S[i + 2], qb.z, c2), c2b = fmaf(S[i + 3], qb.w, c2b);
        }
        a1 += a1b, c1 += c1b, a2 += a2b, c2 += c2b;
#pragma unroll
        for (int o = 1; o < LANES; o <<= 1) {
          a1 += __shfl_xor_sync(0xffffffffu, a1, o);
          c1 += __shfl_xor_sync(0xffffffffu, c1, o);
          a2 += __shfl_xor_sync(0xffffffffu, a2, o);
          c2 += __shfl_xor_sync(0xffffffffu, c2, o);
        }
        const float g1 = r1[2 * DP + CT], beta1 = r1[2 * DP + CT + 1], kq1 = r1[2 * DP + CT + 2];
        const float g2 = r2[2 * DP + CT], beta2 = r2[2 * DP + CT + 1], kq2 = r2[2 * DP + CT + 2];
        const float k1k2 = r2[2 * DP + CT + 3], k1q2 = r2[2 * DP + CT + 4];
        const float w1 = beta1 * (r1[2 * DP + col] - g1 * a1);
        const float w2 = beta2 * (r2[2 * DP + col] - g2 * fmaf(k1k2, w1, g1 * a2));
        const float gg = g1 * g2, w1g = g2 * w1;
#pragma unroll
        for (int i = 0; i < RMAX; ++i) S[i] = fmaf(kr2[i], w2, fmaf(kr1[i], w1g, gg * S[i]));
        if (p == 0 && has_col) {
          float* dst = out + ((size_t)(t0 + first + tt) * H + h) * e + c;
          dst[0] = fmaf(kq1, w1, g1 * c1);
          dst[(size_t)H * e] = fmaf(kq2, w2, g2 * fmaf(k1q2, w1, g1 * c2));
        }
      }
      for (; tt < n; ++tt) {                             // a token left over
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
        const float w = beta * (row[2 * DP + col] - g * a);
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
