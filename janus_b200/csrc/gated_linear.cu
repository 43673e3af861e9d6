// Linear attention whose state decays by gates that depend on the token: a matrix state per head that is a linear
// recurrence once the gates are known,
//
//   S_t = diag(a_t) S_(t-1) + b_t k_t v_t^T,      o_t = S_t^T (q_t q_scale)       (S: [d, e] float32 per sequence)
//
// in two forms that share the walk over the tokens:
//   decay per key channel (gated linear attention): a_t is a vector of d decays, b_t = 1;
//   exponential gates with a running maximum (the matrix memory of xLSTM): a_t = keep_t and b_t = take_t are one
//   number per head and token, a normalizer n_t = keep_t n_(t-1) + take_t k_t walks along, and the walk also leaves
//   max(|n_t . q_t|, exp(-m_t)) + 1e-6, the number that o_t is to be divided by.
//
// gla_decay:   a_t = sigmoid(z)^(1/tau), z = A2 low_t + bias, from the low-rank projection's float32 output low_t.
// exp_gates:   with the log gates i_t = cap tanh((zi + bi) / cap), f_t = logsigmoid(cap tanh((zf + bf) / cap)) and the
//              running maximum m_t = max(f_t + m_(t-1), i_t):  keep_t = exp(f_t + m_(t-1) - m_t), take_t = exp(i_t - m_t).
//              m is a max-plus recurrence, so a block cuts a sequence's tokens into one run per thread, composes each
//              run into (sum of f, what the maximum would be from minus infinity), chains the runs, and walks again.
// gated_linear_scan: a block owns one (sequence or segment, head, block of EB value columns); a thread owns two value
//              columns and a quarter of the rows of S in registers and walks the tokens in order (chunks of CT tokens
//              come into shared memory by asynchronous copies, the next chunk while the current one is walked); the
//              four partial sums of o meet by shuffles in a fixed order.  The
//              normalizer is a column of its own that the block's first warp carries.  The state is read from and
//              written back to the sequence's slot, so prompts, portions of prompts and single tokens are the same code.
//
// Long prompts run in segments of `seg_len` tokens so that the segments of one sequence run side by side: (1) every
// segment but a sequence's last computes the state it would reach from zero, and the product of its decays,
// (2) a prefix pass turns these into every segment's starting state, start_(s+1) = P_s start_s + local_s,
// (3) every segment walks its tokens again from its starting state and writes the outputs; the last one leaves the
// sequence's state.
#include <math_constants.h>
#include <stdio.h>

#include "common.cuh"

namespace {

constexpr int PARTS = 4;      // threads that share a value column (each a quarter of the rows)
constexpr int EB = 64;        // value columns a block owns, two a thread
constexpr int CT = 8;         // tokens staged at a time, in each of two buffers
constexpr int THREADS = EB / 2 * PARTS;
constexpr float DEN_FLOOR = 1e-6f;

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

// ---------------------------------------------------------------------------------------------------------------
// alpha[t][c] = exp(logsigmoid(bias[c] + sum_j a2t[j][c] low[t][j]) inv_tau); TB tokens a block, CPT channels a thread
// ---------------------------------------------------------------------------------------------------------------
constexpr int TB = 16;          // tokens a block
constexpr int CPT = 2;          // channels a thread
// The low-rank rows of the block's tokens lie in shared memory, padded with zeros to whole float4s: a thread reads four
// numbers of a token's row with one load (all lanes the same address), and every weight it fetched serves TB tokens.
__global__ void __launch_bounds__(128) gla_decay_kernel(const float* __restrict__ proj, int ld, int low_col, int rank,
                                                        const float* __restrict__ a2t, const float* __restrict__ bias,
                                                        float inv_tau, float* __restrict__ alpha, int C, int T) {
  extern __shared__ __align__(16) float low_s[];               // [TB][rank4]
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int rank4 = (rank + 3) & ~3;
  const int t0 = blockIdx.x * TB, n = min(TB, T - t0);
  for (int i = threadIdx.x; i < TB * rank4; i += blockDim.x) {
    const int u = i / rank4, j = i % rank4;
    low_s[i] = (u < n && j < rank) ? proj[(size_t)(t0 + u) * ld + low_col + j] : 0.0f;
  }
  __syncthreads();
  for (int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * CPT; c0 < C; c0 += gridDim.y * blockDim.x * CPT) {
    float z[CPT][TB];
#pragma unroll
    for (int q = 0; q < CPT; ++q) {
      const float b = c0 + q < C ? bias[c0 + q] : 0.0f;
#pragma unroll
      for (int u = 0; u < TB; ++u) z[q][u] = b;
    }
    for (int j = 0; j < rank4; j += 4) {
      float w[CPT][4];
#pragma unroll
      for (int q = 0; q < CPT; ++q)
#pragma unroll
        for (int i = 0; i < 4; ++i) w[q][i] = (j + i < rank && c0 + q < C) ? a2t[(size_t)(j + i) * C + c0 + q] : 0.0f;
#pragma unroll
      for (int u = 0; u < TB; ++u) {
        const float4 l = *reinterpret_cast<const float4*>(low_s + u * rank4 + j);
#pragma unroll
        for (int q = 0; q < CPT; ++q)
          z[q][u] = fmaf(w[q][3], l.w, fmaf(w[q][2], l.z, fmaf(w[q][1], l.y, fmaf(w[q][0], l.x, z[q][u]))));
      }
    }
#pragma unroll
    for (int u = 0; u < TB; ++u) {
      if (u < n) {
#pragma unroll
        for (int q = 0; q < CPT; ++q)
          if (c0 + q < C) alpha[(size_t)(t0 + u) * C + c0 + q] = expf(log_sigmoid(z[q][u]) * inv_tau);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// gates[t][h] = (keep, take, exp(-m_t), 0); the running maximum of a sequence lives at state[slot][m_off + h]
// ---------------------------------------------------------------------------------------------------------------
constexpr int GT = 256;
__global__ void __launch_bounds__(GT) exp_gates_kernel(const float* __restrict__ proj, int ld, int i_col, int f_col,
                                                       const float* __restrict__ bi, const float* __restrict__ bf,
                                                       float cap, float4* __restrict__ gates, float* __restrict__ state,
                                                       long long state_ld, long long m_off,
                                                       const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                                                       int H) {
  __shared__ float sum_s[GT], top_s[GT], start_s[GT];
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int seq = blockIdx.x, h = blockIdx.y;
  const int s0 = q_start[seq], n = q_start[seq + 1] - s0;
  if (n <= 0) return;
  const int per = (n + GT - 1) / GT;
  const int a = s0 + min(n, (int)threadIdx.x * per), b = s0 + min(n, ((int)threadIdx.x + 1) * per);
  const float bias_i = bi[h], bias_f = bf[h];
  // a run of tokens as one step of the maximum: m -> max(sum + m, top)
  float sum = 0.0f, top = -CUDART_INF_F;
  for (int t = a; t < b; ++t) {
    const float* row = proj + (size_t)t * ld;
    const float gi = cap * tanhf((row[i_col + h] + bias_i) / cap);
    const float gf = log_sigmoid(cap * tanhf((row[f_col + h] + bias_f) / cap));
    gates[(size_t)t * H + h] = make_float4(gi, gf, 0.0f, 0.0f);
    top = fmaxf(top + gf, gi);
    sum += gf;
  }
  sum_s[threadIdx.x] = sum;
  top_s[threadIdx.x] = top;
  __syncthreads();
  float* m_state = state + (size_t)seq_slot[seq] * state_ld + m_off + h;
  if (threadIdx.x == 0) {
    float m = *m_state;
    const int runs = min(GT, (n + per - 1) / per);
    for (int j = 0; j < runs; ++j) {
      start_s[j] = m;
      m = fmaxf(sum_s[j] + m, top_s[j]);
    }
    *m_state = m;
  }
  __syncthreads();
  if (a >= b) return;
  float m = start_s[threadIdx.x];
  for (int t = a; t < b; ++t) {
    const float4 g = gates[(size_t)t * H + h];
    const float m_new = fmaxf(g.y + m, g.x);
    gates[(size_t)t * H + h] = make_float4(expf(g.y + m - m_new), expf(g.x - m_new), expf(-m_new), 0.0f);
    m = m_new;
  }
}

enum { WHOLE = 0, LOCAL = 1, FROM_START = 3 };

// Asynchronous copies global -> shared; with `in` false nothing is read and the destination is filled with zeros.
__device__ __forceinline__ void copy_async_16(float* dst, const float* src, bool in) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int n = in ? 16 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void copy_async_4(float* dst, const float* src, bool in) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int n = in ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copy_async_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

constexpr int VEC_QK = 1, VEC_V = 2;   // which rows of a token are whole, aligned 16-byte vectors in global memory

// RMAX: rows of S a thread holds (a multiple of 4, 4 RMAX >= d); shared rows are padded to 4 RMAX with zeros.
// SCALAR: one decay and one input scale per head and token (`dec` is the float4 gates [T][H]); else `dec` holds a decay
// per key channel, [T][dec_ld] with head h at column h d.  NORM: the normalizer column and the divisor (SCALAR only).
// State of a head, in the slot and in the segments' scratch alike: [d][e] floats of S, then with NORM [d] of n.
// The tokens' rows come into shared memory by asynchronous copies, CT tokens at a time into one of two buffers: the
// next chunk is on its way while the current one is walked.  The copies are plain, so the query's scale multiplies
// the sums and the input's scale the values where they are used.
template <int RMAX, int PHASE, bool SCALAR, bool NORM>
__global__ void __launch_bounds__(THREADS, RMAX <= 32 ? 4 : 2) gated_linear_scan_kernel(
    const float* __restrict__ proj, int ld, int q_col, int k_col, int v_col, float q_scale,
    const float* __restrict__ dec, int dec_ld, float* __restrict__ out, float* __restrict__ den,
    float* __restrict__ state, long long state_ld, const int* __restrict__ q_start, const int* __restrict__ seq_slot,
    int H, int d, int e, int seg_len, int tiles_per_seq, float* __restrict__ scratch, int vec) {
  constexpr int phase = PHASE;
  constexpr int DP = PARTS * RMAX;         // padded rows
  // a part's rows start four floats after the part before ends: the four parts of a column read their 16 bytes
  // from different banks
  constexpr int PS = RMAX + 4;             // floats from part to part
  constexpr int TS = PARTS * PS;           // floats from token to token
  constexpr int BUF = (SCALAR ? 2 : 3) * CT * TS + CT * EB + CT * 4;   // floats of one buffer
  extern __shared__ __align__(16) float smem[];          // twice: q [CT][TS], k [CT][TS], v [CT][EB], gates [CT][4], a [CT][TS]
  jb::pdl_launch_dependents();
  const int seq = blockIdx.x / tiles_per_seq, seg = blockIdx.x % tiles_per_seq;
  const int h = blockIdx.y, e0 = blockIdx.z * EB;
  const int part = threadIdx.x % PARTS, col = threadIdx.x / PARTS;
  const bool carries_n = NORM && threadIdx.x < 32;        // the first warp, every lane alike; its first column's lanes write
  const int j0 = e0 + 2 * col, j1 = j0 + 1;
  const int ex = e + (NORM ? 1 : 0);
  jb::pdl_wait();
  const int s0 = q_start[seq], q_len = q_start[seq + 1] - s0;
  if ((long long)seg * seg_len >= q_len) return;
  const int t0 = s0 + seg * seg_len, t1 = min(s0 + q_len, t0 + seg_len);
  const bool last = t1 == s0 + q_len;
  if (phase == LOCAL && last) return;              // nobody needs the last segment's state from zero
  float* st = state + (size_t)seq_slot[seq] * state_ld + (size_t)h * d * ex;
  float* sc = scratch ? scratch + (((size_t)blockIdx.x * H + h) * d) * ex : nullptr;
  const float* init = phase == WHOLE ? st : phase == FROM_START ? sc : nullptr;

  // the rows of the tokens [c0, c0 + n) on their way into buffer `b`
  auto stage = [&](int b, int c0) {
    const int n = min(CT, t1 - c0);
    float* q_b = smem + b * BUF;
    float* k_b = q_b + CT * TS;
    float* v_b = k_b + CT * TS;
    float* g_b = v_b + CT * EB;
    float* a_b = g_b + CT * 4;
    if (SCALAR && threadIdx.x < n * 4)
      copy_async_4(g_b + threadIdx.x, dec + ((size_t)(c0 + (threadIdx.x >> 2)) * H + h) * 4 + (threadIdx.x & 3), true);
    if (vec & VEC_QK) {
      for (int idx = threadIdx.x; idx < n * (DP / 4); idx += THREADS) {
        const int tt = idx / (DP / 4), r = (idx % (DP / 4)) * 4;
        const bool in = r < d;                     // d is a multiple of 4 here: a group is inside or outside as a whole
        const size_t row = (size_t)(c0 + tt), at_col = (size_t)h * d + (in ? r : 0);
        const int at = tt * TS + (r / RMAX) * PS + r % RMAX;
        if (phase != LOCAL) copy_async_16(q_b + at, proj + row * ld + q_col + at_col, in);
        copy_async_16(k_b + at, proj + row * ld + k_col + at_col, in);
        if (!SCALAR) copy_async_16(a_b + at, dec + row * dec_ld + at_col, in);
      }
    } else {
      for (int idx = threadIdx.x; idx < n * DP; idx += THREADS) {
        const int tt = idx / DP, r = idx % DP;
        const bool in = r < d;
        const size_t row = (size_t)(c0 + tt), at_col = (size_t)h * d + (in ? r : 0);
        const int at = tt * TS + (r / RMAX) * PS + r % RMAX;
        if (phase != LOCAL) copy_async_4(q_b + at, proj + row * ld + q_col + at_col, in);
        copy_async_4(k_b + at, proj + row * ld + k_col + at_col, in);
        if (!SCALAR) copy_async_4(a_b + at, dec + row * dec_ld + at_col, in);
      }
    }
    if (vec & VEC_V) {
      for (int idx = threadIdx.x; idx < n * (EB / 4); idx += THREADS) {
        const int tt = idx / (EB / 4), c = (idx % (EB / 4)) * 4;
        const bool in = e0 + c < e;                // e is a multiple of 4 here
        copy_async_16(v_b + tt * EB + c, proj + (size_t)(c0 + tt) * ld + v_col + (size_t)h * e + (in ? e0 + c : 0), in);
      }
    } else {
      for (int idx = threadIdx.x; idx < n * EB; idx += THREADS) {
        const int tt = idx / EB, c = idx % EB;
        const bool in = e0 + c < e;
        copy_async_4(v_b + tt * EB + c, proj + (size_t)(c0 + tt) * ld + v_col + (size_t)h * e + (in ? e0 + c : 0), in);
      }
    }
  };

  stage(0, t0);
  copy_async_commit();
  float S0[RMAX], S1[RMAX], Sn[NORM ? RMAX : 1];
#pragma unroll
  for (int i = 0; i < RMAX; ++i) {
    const int r = part * RMAX + i;
    S0[i] = (init && r < d && j0 < e) ? init[(size_t)r * e + j0] : 0.0f;
    S1[i] = (init && r < d && j1 < e) ? init[(size_t)r * e + j1] : 0.0f;
    if constexpr (NORM) Sn[i] = (init && carries_n && r < d) ? init[(size_t)d * e + r] : 0.0f;
  }
  int b = 0;
  for (int c0 = t0; c0 < t1; c0 += CT, b ^= 1) {
    const int n = min(CT, t1 - c0);
    if (c0 + CT < t1) stage(b ^ 1, c0 + CT);
    copy_async_commit();                           // an empty group behind the last chunk
    copy_async_wait_all_but_one();                 // this chunk's copies have landed
    __syncthreads();
    const float* q_s = smem + b * BUF;
    const float* k_s = q_s + CT * TS;
    const float* v_s = k_s + CT * TS;
    const float* g_s = v_s + CT * EB;
    const float* a_s = g_s + CT * 4;
    for (int tt = 0; tt < n; ++tt) {
      float2 v = *reinterpret_cast<const float2*>(v_s + tt * EB + 2 * col);
      const float4* qr = reinterpret_cast<const float4*>(q_s + tt * TS + part * PS);
      const float4* kr = reinterpret_cast<const float4*>(k_s + tt * TS + part * PS);
      const float4* ar = reinterpret_cast<const float4*>(a_s + tt * TS + part * PS);
      const float keep = SCALAR ? g_s[tt * 4] : 0.0f, take = SCALAR ? g_s[tt * 4 + 1] : 0.0f;
      if (SCALAR) {
        // the input's scale goes onto the values: take (k v^T) = k (take v)^T
        v.x *= take;
        v.y *= take;
      }
      float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f, b0 = 0.0f, b1 = 0.0f, b2 = 0.0f, b3 = 0.0f;
      float n0 = 0.0f, n1 = 0.0f;
#pragma unroll
      for (int i = 0; i < RMAX / 4; ++i) {
        const float4 k4 = kr[i];
        float4 a4;
        if (SCALAR) a4 = make_float4(keep, keep, keep, keep);
        else a4 = ar[i];
        S0[4 * i] = fmaf(a4.x, S0[4 * i], k4.x * v.x);
        S0[4 * i + 1] = fmaf(a4.y, S0[4 * i + 1], k4.y * v.x);
        S0[4 * i + 2] = fmaf(a4.z, S0[4 * i + 2], k4.z * v.x);
        S0[4 * i + 3] = fmaf(a4.w, S0[4 * i + 3], k4.w * v.x);
        S1[4 * i] = fmaf(a4.x, S1[4 * i], k4.x * v.y);
        S1[4 * i + 1] = fmaf(a4.y, S1[4 * i + 1], k4.y * v.y);
        S1[4 * i + 2] = fmaf(a4.z, S1[4 * i + 2], k4.z * v.y);
        S1[4 * i + 3] = fmaf(a4.w, S1[4 * i + 3], k4.w * v.y);
        if constexpr (NORM) if (carries_n) {
          Sn[4 * i] = fmaf(keep, Sn[4 * i], k4.x * take);
          Sn[4 * i + 1] = fmaf(keep, Sn[4 * i + 1], k4.y * take);
          Sn[4 * i + 2] = fmaf(keep, Sn[4 * i + 2], k4.z * take);
          Sn[4 * i + 3] = fmaf(keep, Sn[4 * i + 3], k4.w * take);
        }
        if (phase != LOCAL) {
          const float4 q4 = qr[i];
          a0 = fmaf(S0[4 * i], q4.x, a0);
          a1 = fmaf(S0[4 * i + 1], q4.y, a1);
          a2 = fmaf(S0[4 * i + 2], q4.z, a2);
          a3 = fmaf(S0[4 * i + 3], q4.w, a3);
          b0 = fmaf(S1[4 * i], q4.x, b0);
          b1 = fmaf(S1[4 * i + 1], q4.y, b1);
          b2 = fmaf(S1[4 * i + 2], q4.z, b2);
          b3 = fmaf(S1[4 * i + 3], q4.w, b3);
          if constexpr (NORM) if (carries_n) {
            n0 = fmaf(Sn[4 * i], q4.x, n0);
            n1 = fmaf(Sn[4 * i + 1], q4.y, n1);
            n0 = fmaf(Sn[4 * i + 2], q4.z, n0);
            n1 = fmaf(Sn[4 * i + 3], q4.w, n1);
          }
        }
      }
      if (phase != LOCAL) {
        float acc0 = (a0 + a1) + (a2 + a3), acc1 = (b0 + b1) + (b2 + b3);
        // the four parts of a column are neighbouring lanes: part 0 + 1, 2 + 3, then the two sums
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
        if (part == 0) {
          float* orow = out + (size_t)(c0 + tt) * H * e + (size_t)h * e;
          if (j0 < e) orow[j0] = acc0 * q_scale;
          if (j1 < e) orow[j1] = acc1 * q_scale;
        }
        if constexpr (NORM) if (carries_n) {
          float nq = n0 + n1;
          nq += __shfl_xor_sync(0xffffffffu, nq, 1);
          nq += __shfl_xor_sync(0xffffffffu, nq, 2);
          if (threadIdx.x == 0 && blockIdx.z == 0)
            den[(size_t)(c0 + tt) * H + h] = fmaxf(fabsf(nq * q_scale), g_s[tt * 4 + 2]) + DEN_FLOOR;
        }
      }
    }
    __syncthreads();                               // the buffer is free for the chunk after the next
  }
  float* dst = phase == LOCAL ? sc : (last ? st : nullptr);
  if (dst == nullptr) return;
#pragma unroll
  for (int i = 0; i < RMAX; ++i) {
    const int r = part * RMAX + i;
    if (r < d && j0 < e) dst[(size_t)r * e + j0] = S0[i];
    if (r < d && j1 < e) dst[(size_t)r * e + j1] = S1[i];
    if constexpr (NORM) if (threadIdx.x < PARTS && blockIdx.z == 0 && r < d) dst[(size_t)d * e + r] = Sn[i];
  }
}

// seg_decay[block][h][r] = the product of the decays of the segment's tokens (r = 0 alone with one decay a head)
template <bool SCALAR>
__global__ void segment_decay_kernel(const float* __restrict__ dec, int dec_ld, float* __restrict__ seg_decay,
                                     const int* __restrict__ q_start, int H, int d, int seg_len, int tiles_per_seq) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int seq = blockIdx.x / tiles_per_seq, seg = blockIdx.x % tiles_per_seq, h = blockIdx.y;
  const int s0 = q_start[seq], q_len = q_start[seq + 1] - s0;
  if ((long long)seg * seg_len >= q_len) return;
  const int t0 = s0 + seg * seg_len, t1 = min(s0 + q_len, t0 + seg_len);
  const int rows = SCALAR ? 1 : d;
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    float p = 1.0f;
    for (int t = t0; t < t1; ++t)
      p *= SCALAR ? dec[((size_t)t * H + h) * 4] : dec[(size_t)t * dec_ld + h * d + r];
    seg_decay[((size_t)blockIdx.x * H + h) * rows + r] = p;
  }
}

// scratch[seq][seg] holds segment seg's state from zero; afterwards it holds the state the segment starts from
template <bool SCALAR>
__global__ void gated_linear_prefix_kernel(float* __restrict__ scratch, const float* __restrict__ state,
                                           long long state_ld, const float* __restrict__ seg_decay,
                                           const int* __restrict__ q_start, const int* __restrict__ seq_slot, int H,
                                           int d, int e, int ex, int seg_len, int tiles_per_seq) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int seq = blockIdx.x;
  const size_t per = (size_t)H * d * ex;
  const size_t idx = (size_t)blockIdx.y * blockDim.x + threadIdx.x;
  if (idx >= per) return;
  const int h = (int)(idx / ((size_t)d * ex));
  const int rem = (int)(idx % ((size_t)d * ex));
  const int r = rem < d * e ? rem / e : rem - d * e;
  const int rows = SCALAR ? 1 : d;
  const int q_len = q_start[seq + 1] - q_start[seq];
  const int n_seg = (q_len + seg_len - 1) / seg_len;
  float S = state[(size_t)seq_slot[seq] * state_ld + idx];
  float* p = scratch + (size_t)seq * tiles_per_seq * per + idx;
  const float* pd = seg_decay + ((size_t)seq * tiles_per_seq * H + h) * rows + (SCALAR ? 0 : r);
  for (int s = 0; s + 1 < n_seg; ++s) {
    const float local = p[(size_t)s * per];
    p[(size_t)s * per] = S;
    S = fmaf(pd[(size_t)s * H * rows], S, local);
  }
  if (n_seg > 0) p[(size_t)(n_seg - 1) * per] = S;
}

}  // namespace

// proj: float32 [T, ld] with the low-rank projection's output at columns [low_col, low_col + rank); a2t: float32
// [rank][C], the second matrix transposed; bias [C]; alpha: float32 [T, C].
JB_EXPORT int jb_gla_decay(const float* proj, int ld, int low_col, int rank, const float* a2t, const float* bias,
                           float inv_tau, float* alpha, int C, int T, cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t smem = (size_t)TB * ((rank + 3) & ~3) * sizeof(float);
  JB_REFUSE(rank < 1 || smem > 48 * 1024, "gla_decay: a rank of %d", rank);
  const int per_block = 128 * CPT;
  const int by = (C + per_block - 1) / per_block < 64 ? (C + per_block - 1) / per_block : 64;
  jb::Launch cfg(dim3((T + TB - 1) / TB, by), dim3(128), smem, stream);
  return (int)cudaLaunchKernelEx(&cfg.c, gla_decay_kernel, proj, ld, low_col, rank, a2t, bias, inv_tau, alpha, C, T);
}

// proj: float32 [T, ld] with the gates' arguments at columns i_col + h and f_col + h; gates: float4 [T][H], written;
// state: float32 rows of state_ld floats, a sequence's running maxima at m_off + h of its slot's row.
JB_EXPORT int jb_exp_gates(const float* proj, int ld, int i_col, int f_col, const float* bi, const float* bf, float cap,
                           float* gates, float* state, long long state_ld, long long m_off, const int* q_start,
                           const int* seq_slot, int n_seqs, int H, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  JB_REFUSE(((uintptr_t)gates & 15) != 0, "exp_gates: the gates must be 16-byte aligned");
  jb::Launch cfg(dim3(n_seqs, H), dim3(GT), 0, stream);
  return (int)cudaLaunchKernelEx(&cfg.c, exp_gates_kernel, proj, ld, i_col, f_col, bi, bf, cap, (float4*)gates, state,
                                 state_ld, m_off, q_start, seq_slot, H);
}

namespace {
template <int RMAX, int PHASE, bool SCALAR, bool NORM>
cudaError_t launch_scan(dim3 grid, size_t smem, cudaStream_t stream, const float* proj, int ld, int q_col, int k_col,
                        int v_col, float q_scale, const float* dec, int dec_ld, float* out, float* den, float* state,
                        long long state_ld, const int* q_start, const int* seq_slot, int H, int d, int e, int seg,
                        int tiles, float* scratch, int vec) {
  auto k = gated_linear_scan_kernel<RMAX, PHASE, SCALAR, NORM>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
  }
  jb::Launch cfg(grid, dim3(THREADS), smem, stream);
  return cudaLaunchKernelEx(&cfg.c, k, proj, ld, q_col, k_col, v_col, q_scale, dec, dec_ld, out, den, state, state_ld,
                            q_start, seq_slot, H, d, e, seg, tiles, scratch, vec);
}

template <int PHASE, bool SCALAR, bool NORM, typename... A>
cudaError_t launch_scan_r(int rmax, A... a) {
  if (rmax == 8) return launch_scan<8, PHASE, SCALAR, NORM>(a...);
  if (rmax == 16) return launch_scan<16, PHASE, SCALAR, NORM>(a...);
  if (rmax == 32) return launch_scan<32, PHASE, SCALAR, NORM>(a...);
  return launch_scan<64, PHASE, SCALAR, NORM>(a...);
}

template <bool SCALAR, bool NORM>
int scan_all(const float* proj, int ld, int q_col, int k_col, int v_col, float q_scale, const float* dec, int dec_ld,
             float* out, float* den, float* state, long long state_ld, const int* q_start, const int* seq_slot,
             int n_seqs, int H, int d, int e, int max_q_len, int seg_len, float* scratch, float* seg_decay,
             cudaStream_t stream) {
  const int rmax = d <= 32 ? 8 : d <= 64 ? 16 : d <= 128 ? 32 : 64;
  const int ts = PARTS * (rmax + 4);
  const size_t smem = 2 * (size_t)((SCALAR ? 2 : 3) * CT * ts + CT * EB + CT * 4) * sizeof(float);   // two buffers
  // rows that are whole 16-byte vectors at aligned addresses are copied 16 bytes at a time
  const bool base16 = ((uintptr_t)proj & 15) == 0 && ld % 4 == 0;
  const bool dec16 = SCALAR || (((uintptr_t)dec & 15) == 0 && dec_ld % 4 == 0);
  const int vec = (base16 && dec16 && d % 4 == 0 && q_col % 4 == 0 && k_col % 4 == 0 ? VEC_QK : 0) |
                  (base16 && e % 4 == 0 && v_col % 4 == 0 ? VEC_V : 0);
  const bool segmented = seg_len > 0;
  const int tiles = segmented ? (max_q_len + seg_len - 1) / seg_len : 1;
  const int seg = segmented ? seg_len : 0x40000000;
  const int ex = e + (NORM ? 1 : 0);
  const dim3 grid(n_seqs * tiles, H, (e + EB - 1) / EB);
  cudaError_t err;
  if (!segmented) {
    err = launch_scan_r<WHOLE, SCALAR, NORM>(rmax, grid, smem, stream, proj, ld, q_col, k_col, v_col, q_scale, dec,
                                             dec_ld, out, den, state, state_ld, q_start, seq_slot, H, d, e, seg, tiles,
                                             scratch, vec);
    return (int)err;
  }
  err = launch_scan_r<LOCAL, SCALAR, NORM>(rmax, grid, smem, stream, proj, ld, q_col, k_col, v_col, q_scale, dec, dec_ld,
                                           out, den, state, state_ld, q_start, seq_slot, H, d, e, seg, tiles, scratch,
                                           vec);
  if (err != cudaSuccess) return (int)err;
  {
    jb::Launch cfg(dim3(n_seqs * tiles, H), dim3(SCALAR ? 32 : (d <= 64 ? 64 : d <= 128 ? 128 : 256)), 0, stream);
    err = cudaLaunchKernelEx(&cfg.c, segment_decay_kernel<SCALAR>, dec, dec_ld, seg_decay, q_start, H, d, seg_len, tiles);
    if (err != cudaSuccess) return (int)err;
  }
  {
    const size_t per = (size_t)H * d * ex;
    jb::Launch cfg(dim3(n_seqs, (unsigned)((per + 255) / 256)), dim3(256), 0, stream);
    err = cudaLaunchKernelEx(&cfg.c, gated_linear_prefix_kernel<SCALAR>, scratch, (const float*)state, state_ld,
                             (const float*)seg_decay, q_start, seq_slot, H, d, e, ex, seg_len, tiles);
    if (err != cudaSuccess) return (int)err;
  }
  err = launch_scan_r<FROM_START, SCALAR, NORM>(rmax, grid, smem, stream, proj, ld, q_col, k_col, v_col, q_scale, dec,
                                                dec_ld, out, den, state, state_ld, q_start, seq_slot, H, d, e, seg,
                                                tiles, scratch, vec);
  return (int)err;
}
}  // namespace

// proj: float32 [T, ld], the projections: q at column q_col ([H][d]), k at k_col ([H][d]), v at v_col ([H][e]);
// scalar = 0: dec is float32 [T, dec_ld] with a decay per key channel (head h at column h d), no normalizer;
// scalar = 1: dec is the float4 gates [T][H] that jb_exp_gates left, the normalizer walks along and den (float32
// [T, H]) gets the divisors.  out: float32 [T, H e].  state: float32 rows of state_ld floats, a slot's heads one
// after another, each [d][e] (scalar = 1: then [d] of the normalizer).  seg_len > 0 with scratch (float32, n_seqs *
// ceil(max_q_len / seg_len) * H * d * (e + scalar)) and seg_decay (n_seqs * tiles * H * (scalar ? 1 : d)) runs the
// passes over segments; seg_len = 0 walks every sequence in one block per column block.
JB_EXPORT int jb_gated_linear_scan(const float* proj, int ld, int q_col, int k_col, int v_col, float q_scale,
                                   const float* dec, int dec_ld, int scalar, float* out, float* den, float* state,
                                   long long state_ld, const int* q_start, const int* seq_slot, int n_seqs, int H, int d,
                                   int e, int max_q_len, int seg_len, float* scratch, float* seg_decay,
                                   cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  JB_REFUSE(d < 1 || d > 256 || e < 1, "gated_linear_scan: key size %d is outside [1, 256]", d);
  JB_REFUSE(seg_len > 0 && (scratch == nullptr || seg_decay == nullptr), "gated_linear_scan: segments need scratch");
  JB_REFUSE(scalar && den == nullptr, "gated_linear_scan: the normalizer needs a place for the divisors");
  if (scalar)
    return scan_all<true, true>(proj, ld, q_col, k_col, v_col, q_scale, dec, dec_ld, out, den, state, state_ld, q_start,
                                seq_slot, n_seqs, H, d, e, max_q_len, seg_len, scratch, seg_decay, stream);
  return scan_all<false, false>(proj, ld, q_col, k_col, v_col, q_scale, dec, dec_ld, out, den, state, state_ld, q_start,
                                seq_slot, n_seqs, H, d, e, max_q_len, seg_len, scratch, seg_decay, stream);
}
