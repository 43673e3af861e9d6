// A feed-forward made of experts of which every token uses a few: the router's choice, the experts' products for
// steps of few tokens (every chosen expert's rows are streamed once for up to four tokens that chose it, float32 sums), and the
// bookkeeping around the tensor-core products of steps with many tokens (rows gathered expert by expert, results
// added back token by token).
//
//   scores s = sigmoid(z) of the router's float32 logits z [T, E]; a token's `top` experts are those with the largest
//   scores (the lower index wins a tie); its weights are those scores, as they are.
//   out[t] += sum over the chosen e of  Wd_e ( act(Wg_e x) * (Wu_e x) ),  x = s_e h[t]        (the weight is on the input)
//   or, with the weight on the output,  out[t] += sum over the chosen e of  s_e Wd_e ( act(Wg_e h[t]) * (Wu_e h[t]) ).
//   Scores may also be the softmax over all experts, and the choice may be limited to the best groups of neighbours.
//
// Experts' weights: gate and up [E][F][W], down [E][W][F], row-major, float32 or bfloat16.
#include <math_constants.h>
#include <stdio.h>

#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int MAX_TOP = 16;

// one warp per token.  softmax = 0: a score is the logit's sigmoid; 1: the softmax over all experts.  groups > 0: the
// experts form `groups` equal groups of neighbours, a group's score is its largest score, and only experts of the
// `keep` groups with the largest scores can be chosen (the lower group wins a tie).
__global__ void route_topk_kernel(const float* __restrict__ logits, int ld, int E, int top, int* __restrict__ sel_e,
                                  float* __restrict__ sel_w, int T, int softmax, int groups, int keep) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const float* z = logits + (size_t)t * ld;
  float z_max = 0.0f, z_sum = 1.0f;
  if (softmax) {
    z_max = -CUDART_INF_F;
    for (int e = lane; e < E; e += 32) z_max = fmaxf(z_max, z[e]);
    z_max = jb::warp_max(z_max);
    z_sum = 0.0f;
    for (int e = lane; e < E; e += 32) z_sum += expf(z[e] - z_max);
    z_sum = jb::warp_sum(z_sum);
  }
  unsigned long long kept = ~0ull;               // bit g: experts of group g can be chosen
  const int per_group = groups > 0 ? E / groups : E;
  if (groups > 0) {
    kept = 0ull;
    for (int k = 0; k < keep; ++k) {
      float best = -CUDART_INF_F;
      int arg = 0x7fffffff;
      for (int e = lane; e < E; e += 32) {
        const int g = e / per_group;
        const float v = z[e];                    // scores keep the order of the logits
        if (!((kept >> g) & 1ull) && (v > best || (v == best && g < arg))) {
          best = v;
          arg = g;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) {
          best = ob;
          arg = oa;
        }
      }
      if (arg < groups) kept |= 1ull << arg;
    }
  }
  int picked[MAX_TOP];
  for (int k = 0; k < top; ++k) {
    float best = -CUDART_INF_F;
    int arg = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool taken = groups > 0 && !((kept >> (e / per_group)) & 1ull);
      for (int q = 0; q < k; ++q) taken |= picked[q] == e;
      const float v = z[e];            // the sigmoid and the softmax keep the order of the logits
      if (!taken && (v > best || (v == best && e < arg))) {
        best = v;
        arg = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) {
        best = ob;
        arg = oa;
      }
    }
    picked[k] = arg;
    if (lane == 0) {
      sel_e[(size_t)t * top + k] = arg;
      sel_w[(size_t)t * top + k] = softmax ? expf(best - z_max) / z_sum : 1.0f / (1.0f + expf(-best));
    }
  }
}

template <typename TW> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&v)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  }
  __device__ static void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec<bf16> {
  static constexpr int N = 8;
  __device__ static void load(const bf16* p, float (&v)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static void store(bf16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <typename T> __host__ __device__ bool aligned16(const T* p) { return ((uintptr_t)p & 15) == 0; }

constexpr int GU_WARPS = 8, GU_ROWS = 2;   // rows of gate (and of up) per warp

// The pairs among [base, base + blockDim.x) that chose expert e, in list[0 .. n) (in no fixed order: every pair's
// result is computed by itself, so the order changes nothing).
__device__ __forceinline__ int pairs_of_expert(const int* __restrict__ sel_e, int n_pairs, int base, int e, int* list,
                                               int* count) {
  if (threadIdx.x == 0) *count = 0;
  __syncthreads();
  const int pr = base + threadIdx.x;
  if (pr < n_pairs && sel_e[pr] == e) list[atomicAdd(count, 1)] = pr;
  __syncthreads();
  return *count;
}

// act[pair][f] = gated(Wg_e[f] . x, Wu_e[f] . x) with x = weight[pair] * h[token of the pair].  A block owns rows of
// ONE expert (blockIdx.y) and serves every pair that chose it, PB pairs at a time: the expert's rows come from
// memory once however many of the step's tokens chose it, and not at all when none did.
template <typename TW, typename TX, bool VEC, int PB>
__global__ void __launch_bounds__(GU_WARPS * 32) expert_gate_up_kernel(
    const TX* __restrict__ h, const int* __restrict__ sel_e, const float* __restrict__ sel_w, int top, int n_pairs,
    const TW* __restrict__ w_gate, const TW* __restrict__ w_up, float* __restrict__ act, int W, int F, jb::Gate gate,
    int weigh_input) {
  extern __shared__ __align__(16) float x_s[];           // [PB][W]
  __shared__ int list[GU_WARPS * 32];
  __shared__ int count;
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int e = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f0 = (blockIdx.x * GU_WARPS + warp) * GU_ROWS;
  const TW* g_rows = w_gate + ((size_t)e * F + min(f0, F - 1)) * W;
  const TW* u_rows = w_up + ((size_t)e * F + min(f0, F - 1)) * W;
  for (int base = 0; base < n_pairs; base += blockDim.x) {
    const int n = pairs_of_expert(sel_e, n_pairs, base, e, list, &count);
    for (int g0 = 0; g0 < n; g0 += PB) {
      const int nb = min(PB, n - g0);
      for (int b = 0; b < nb; ++b) {
        const int pair = list[g0 + b];
        const float s = weigh_input ? sel_w[pair] : 1.0f;
        const TX* src = h + (size_t)(pair / top) * W;
        for (int i = threadIdx.x; i < W; i += blockDim.x) x_s[(size_t)b * W + i] = s * jb::to_f32(src[i]);
      }
      __syncthreads();
      if (f0 < F) {
        float ag[GU_ROWS][PB], au[GU_ROWS][PB];
#pragma unroll
        for (int r = 0; r < GU_ROWS; ++r)
#pragma unroll
          for (int b = 0; b < PB; ++b) ag[r][b] = au[r][b] = 0.0f;
        if (VEC) {
          constexpr int N = Vec<TW>::N;
          for (int i = lane * N; i < W; i += 32 * N) {
            float gv[GU_ROWS][N], uv[GU_ROWS][N];
#pragma unroll
            for (int r = 0; r < GU_ROWS; ++r) {
              const size_t off = (size_t)(f0 + r < F ? r : 0) * W + i;
              Vec<TW>::load(g_rows + off, gv[r]);
              Vec<TW>::load(u_rows + off, uv[r]);
            }
#pragma unroll
            for (int b = 0; b < PB; ++b) {
              if (b < nb) {
#pragma unroll
                for (int q = 0; q < N; ++q) {
                  const float x = x_s[(size_t)b * W + i + q];
#pragma unroll
                  for (int r = 0; r < GU_ROWS; ++r) {
                    ag[r][b] = fmaf(gv[r][q], x, ag[r][b]);
                    au[r][b] = fmaf(uv[r][q], x, au[r][b]);
                  }
                }
              }
            }
          }
        } else {
          for (int i = lane; i < W; i += 32) {
#pragma unroll
            for (int r = 0; r < GU_ROWS; ++r) {
              const size_t off = (size_t)(f0 + r < F ? r : 0) * W + i;
              const float g = jb::to_f32(g_rows[off]), u = jb::to_f32(u_rows[off]);
#pragma unroll
              for (int b = 0; b < PB; ++b) {
                if (b < nb) {
                  const float x = x_s[(size_t)b * W + i];
                  ag[r][b] = fmaf(g, x, ag[r][b]);
                  au[r][b] = fmaf(u, x, au[r][b]);
                }
              }
            }
          }
        }
#pragma unroll
        for (int r = 0; r < GU_ROWS; ++r)
#pragma unroll
          for (int b = 0; b < PB; ++b) {
            if (b < nb) {
              const float g = jb::warp_sum(ag[r][b]), u = jb::warp_sum(au[r][b]);
              if (lane == 0 && f0 + r < F) act[(size_t)list[g0 + b] * F + f0 + r] = jb::gated(g, u, gate);
            }
          }
      }
      __syncthreads();                                   // the rows of x are free for the next pairs
    }
  }
}

constexpr int DN_WARPS = 8, DN_ROWS = 4;

// out[token of the pair][c] += Wd_e[c] . act[pair] (times out_w[pair] if given), a block per (rows, expert) as above
template <typename TW, bool VEC, int PB>
__global__ void __launch_bounds__(DN_WARPS * 32) expert_down_kernel(
    const float* __restrict__ act, const int* __restrict__ sel_e, const float* __restrict__ out_w, int top, int n_pairs,
    const TW* __restrict__ w_down, float* __restrict__ out, int W, int F) {
  extern __shared__ __align__(16) float a_s[];           // [PB][F]
  __shared__ int list[DN_WARPS * 32];
  __shared__ int count;
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int e = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = (blockIdx.x * DN_WARPS + warp) * DN_ROWS;
  const TW* rows = w_down + ((size_t)e * W + min(c0, W - 1)) * F;
  for (int base = 0; base < n_pairs; base += blockDim.x) {
    const int n = pairs_of_expert(sel_e, n_pairs, base, e, list, &count);
    for (int g0 = 0; g0 < n; g0 += PB) {
      const int nb = min(PB, n - g0);
      for (int b = 0; b < nb; ++b) {
        const float* src = act + (size_t)list[g0 + b] * F;
        for (int i = threadIdx.x; i < F; i += blockDim.x) a_s[(size_t)b * F + i] = src[i];
      }
      __syncthreads();
      if (c0 < W) {
        float acc[DN_ROWS][PB];
#pragma unroll
        for (int r = 0; r < DN_ROWS; ++r)
#pragma unroll
          for (int b = 0; b < PB; ++b) acc[r][b] = 0.0f;
        if (VEC) {
          constexpr int N = Vec<TW>::N;
          for (int i = lane * N; i < F; i += 32 * N) {
            float wv[DN_ROWS][N];
#pragma unroll
            for (int r = 0; r < DN_ROWS; ++r) Vec<TW>::load(rows + (size_t)(c0 + r < W ? r : 0) * F + i, wv[r]);
#pragma unroll
            for (int b = 0; b < PB; ++b) {
              if (b < nb) {
#pragma unroll
                for (int q = 0; q < N; ++q) {
                  const float a = a_s[(size_t)b * F + i + q];
#pragma unroll
                  for (int r = 0; r < DN_ROWS; ++r) acc[r][b] = fmaf(wv[r][q], a, acc[r][b]);
                }
              }
            }
          }
        } else {
          for (int i = lane; i < F; i += 32) {
#pragma unroll
            for (int r = 0; r < DN_ROWS; ++r) {
              const float wgt = jb::to_f32(rows[(size_t)(c0 + r < W ? r : 0) * F + i]);
#pragma unroll
              for (int b = 0; b < PB; ++b)
                if (b < nb) acc[r][b] = fmaf(wgt, a_s[(size_t)b * F + i], acc[r][b]);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < DN_ROWS; ++r)
#pragma unroll
          for (int b = 0; b < PB; ++b) {
            if (b < nb) {
              float v = jb::warp_sum(acc[r][b]);
              if (out_w != nullptr) v *= out_w[list[g0 + b]];      // the pair's weight, on the expert's output
              if (lane == 0 && c0 + r < W) {
                float* dst = out + (size_t)(list[g0 + b] / top) * W + c0 + r;
                if (top == 1) *dst += v;                   // the token's only pair: nobody else adds here
                else atomicAdd(dst, v);
              }
            }
          }
      }
      __syncthreads();
    }
  }
}

constexpr int PLAN_THREADS = 1024, PLAN_MAX_EXPERTS = 1024;

// Sorts the (token, choice) pairs by expert and lists the tiles of the two grouped products, in one block, so that
// the host never learns the router's choice.  order[place] = pair and where[pair] = place, an expert's pairs next
// to each other (in no fixed order inside an expert: a row's result does not depend on its place).  A table holds
// its count of items in [0] and item i as (t0, t_end, wf0, f0) at [4 + 4 i]: rows [t0, t_end) of the sorted pairs,
// weight rows from wf0 on in the stack of the experts' matrices, output columns from f0 on.  Tiles are 256 rows;
// `gu` tiles are 128 features of F wide, `dn` tiles 256 features of W.  Inside an expert the row tiles run fastest,
// so CTAs that run side by side share a weight tile.
__global__ void __launch_bounds__(PLAN_THREADS) expert_plan_kernel(const int* __restrict__ sel_e, int n_pairs, int E,
                                                                   int F, int W, int* __restrict__ order,
                                                                   int* __restrict__ where, int* __restrict__ gu,
                                                                   int* __restrict__ dn) {
  __shared__ int count[PLAN_MAX_EXPERTS], start[PLAN_MAX_EXPERTS], cursor[PLAN_MAX_EXPERTS], tiles_before[PLAN_MAX_EXPERTS];
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&count[sel_e[i]], 1);
  __syncthreads();
  const int gu_per = (F + 127) / 128, dn_per = (W + 255) / 256;
  if (threadIdx.x == 0) {
    int rows = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = cursor[e] = rows;
      tiles_before[e] = tiles;
      rows += count[e];
      tiles += (count[e] + 255) / 256;
    }
    gu[0] = tiles * gu_per;
    dn[0] = tiles * dn_per;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int place = atomicAdd(&cursor[sel_e[i]], 1);
    order[place] = i;
    where[i] = place;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int n_tt = (count[e] + 255) / 256, end = start[e] + count[e];
    int4* g = reinterpret_cast<int4*>(gu + 4) + (size_t)tiles_before[e] * gu_per;
    for (int ft = 0; ft < gu_per; ++ft)
      for (int tt = 0; tt < n_tt; ++tt) g[ft * n_tt + tt] = make_int4(start[e] + tt * 256, end, e * F + ft * 128, ft * 128);
    int4* d = reinterpret_cast<int4*>(dn + 4) + (size_t)tiles_before[e] * dn_per;
    for (int ft = 0; ft < dn_per; ++ft)
      for (int tt = 0; tt < n_tt; ++tt) d[ft * n_tt + tt] = make_int4(start[e] + tt * 256, end, e * W + ft * 256, ft * 256);
  }
}

// rows[i] = weight[order[i]] * h[order[i] / top] (no weights: the row itself) in the products' dtype: the pairs (token, choice) in the order the
// experts' products take them
template <typename TX>
__global__ void expert_gather_kernel(const TX* __restrict__ h, const int* __restrict__ order,
                                     const float* __restrict__ sel_w, int top, TX* __restrict__ rows, int W) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int pair = order[blockIdx.x];
  const float s = sel_w != nullptr ? sel_w[pair] : 1.0f;
  const TX* src = h + (size_t)(pair / top) * W;
  TX* dst = rows + (size_t)blockIdx.x * W;
  constexpr int N = Vec<TX>::N;
  if (W % N == 0 && aligned16(h) && aligned16(rows)) {          // 16 bytes a thread
    for (int i = threadIdx.x * N; i < W; i += blockDim.x * N) {
      float v[N];
      Vec<TX>::load(src + i, v);
#pragma unroll
      for (int q = 0; q < N; ++q) v[q] *= s;
      Vec<TX>::store(dst + i, v);
    }
    return;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] = jb::from_f32<TX>(s * jb::to_f32(src[i]));
}

// out[t] += sum over k of results[where[t * top + k]] (times out_w[t * top + k] if given)
__global__ void expert_scatter_kernel(const float* __restrict__ results, const int* __restrict__ where,
                                      const float* __restrict__ out_w, int top, float* __restrict__ out, int W) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x;
  if (W % 4 == 0 && aligned16(results) && aligned16(out)) {     // 16 bytes a thread
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      for (int k = 0; k < top; ++k) {
        const float4 r = *reinterpret_cast<const float4*>(results + (size_t)where[(size_t)t * top + k] * W + i);
        const float s = out_w != nullptr ? out_w[(size_t)t * top + k] : 1.0f;
        v.x = fmaf(s, r.x, v.x), v.y = fmaf(s, r.y, v.y), v.z = fmaf(s, r.z, v.z), v.w = fmaf(s, r.w, v.w);
      }
      float4* o = reinterpret_cast<float4*>(out + (size_t)t * W + i);
      float4 a = *o;
      a.x += v.x, a.y += v.y, a.z += v.z, a.w += v.w;
      *o = a;
    }
    return;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = 0.0f;
    for (int k = 0; k < top; ++k)
      v = fmaf(out_w != nullptr ? out_w[(size_t)t * top + k] : 1.0f, results[(size_t)where[(size_t)t * top + k] * W + i], v);
    out[(size_t)t * W + i] += v;
  }
}


}  // namespace

JB_EXPORT int jb_route_topk(const float* logits, int ld, int E, int top, int* sel_e, float* sel_w, int T, int softmax,
                            int groups, int keep, cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(top < 1 || top > MAX_TOP || top > E, "route_topk: %d of %d experts (at most %d a token)", top, E, MAX_TOP);
  JB_REFUSE(groups < 0 || groups > 64 || (groups > 0 && (E % groups != 0 || keep < 1 || keep > groups ||
                                                          keep * (E / groups) < top)),
            "route_topk: %d groups of which %d are kept do not fit %d experts and %d a token", groups, keep, E, top);
  jb::Launch cfg(dim3((T + 3) / 4), dim3(128), 0, stream);
  return (int)cudaLaunchKernelEx(&cfg.c, route_topk_kernel, logits, ld, E, top, sel_e, sel_w, T, softmax, groups, keep);
}

// h: [T, W] in x_dtype; the experts' weights ([E] of them) in w_dtype; act: float32 scratch [T top, F]; out: float32
// [T, W], added to.  weight_on_output: a pair's weight multiplies its expert's output instead of its input.
JB_EXPORT int jb_experts_few_tokens(const void* h, int x_dtype, const int* sel_e, const float* sel_w, int top,
                                    const void* w_gate, const void* w_up, const void* w_down, int w_dtype, float* act,
                                    float* out, int T, int W, int F, int E, float gate_limit, float gate_alpha,
                                    int weight_on_output, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int pairs = T * top;
  JB_REFUSE(E < 1 || E > 65535, "experts: %d experts", E);
  JB_REFUSE((size_t)max(W, F) * sizeof(float) > 96 * 1024, "experts: rows of %d floats do not fit shared memory", max(W, F));
  // pairs served at once by a block: as many rows of x (or of act) as fit 96 KB of shared memory, four at most
  const int pb = (size_t)max(W, F) * sizeof(float) * 4 <= 96 * 1024 ? 4 : (size_t)max(W, F) * sizeof(float) * 2 <= 96 * 1024 ? 2 : 1;
  const size_t smem1 = (size_t)pb * W * sizeof(float), smem2 = (size_t)pb * F * sizeof(float);
  const jb::Gate gate{gate_limit, gate_alpha};
  jb::Launch c1(dim3((F + GU_WARPS * GU_ROWS - 1) / (GU_WARPS * GU_ROWS), E), dim3(GU_WARPS * 32), smem1, stream);
  jb::Launch c2(dim3((W + DN_WARPS * DN_ROWS - 1) / (DN_WARPS * DN_ROWS), E), dim3(DN_WARPS * 32), smem2, stream);
  cudaError_t e;
#define JB_LAUNCH_GU(TW, TX, V, PB)                                                                                   \
  do {                                                                                                                \
    auto k = expert_gate_up_kernel<TW, TX, V, PB>;                                                                    \
    if (smem1 > 48 * 1024) e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);      \
    if (e == cudaSuccess)                                                                                             \
      e = cudaLaunchKernelEx(&c1.c, k, (const TX*)h, sel_e, sel_w, top, pairs, (const TW*)w_gate, (const TW*)w_up,    \
                             act, W, F, gate, weight_on_output ? 0 : 1);                                              \
  } while (0)
#define JB_LAUNCH_DN(TW, V, PB)                                                                                       \
  do {                                                                                                                \
    auto k = expert_down_kernel<TW, V, PB>;                                                                           \
    if (smem2 > 48 * 1024) e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);      \
    if (e == cudaSuccess)                                                                                             \
      e = cudaLaunchKernelEx(&c2.c, k, (const float*)act, sel_e, weight_on_output ? sel_w : (const float*)nullptr,   \
                             top, pairs, (const TW*)w_down, out, W, F);                                               \
  } while (0)
#define JB_LAUNCH_EX(TW, TX)                                                                                          \
  do {                                                                                                                \
    const bool v1 = W % Vec<TW>::N == 0 && aligned16((const TW*)w_gate) && aligned16((const TW*)w_up);                \
    const bool v2 = F % Vec<TW>::N == 0 && aligned16((const TW*)w_down);                                              \
    e = cudaSuccess;                                                                                                  \
    if (v1 && pb == 4) JB_LAUNCH_GU(TW, TX, true, 4);                                                                 \
    else if (v1 && pb == 2) JB_LAUNCH_GU(TW, TX, true, 2);                                                            \
    else if (v1) JB_LAUNCH_GU(TW, TX, true, 1);                                                                       \
    else if (pb == 4) JB_LAUNCH_GU(TW, TX, false, 4);                                                                 \
    else if (pb == 2) JB_LAUNCH_GU(TW, TX, false, 2);                                                                 \
    else JB_LAUNCH_GU(TW, TX, false, 1);                                                                              \
    if (e != cudaSuccess) return (int)e;                                                                              \
    if (v2 && pb == 4) JB_LAUNCH_DN(TW, true, 4);                                                                     \
    else if (v2 && pb == 2) JB_LAUNCH_DN(TW, true, 2);                                                                \
    else if (v2) JB_LAUNCH_DN(TW, true, 1);                                                                           \
    else if (pb == 4) JB_LAUNCH_DN(TW, false, 4);                                                                     \
    else if (pb == 2) JB_LAUNCH_DN(TW, false, 2);                                                                     \
    else JB_LAUNCH_DN(TW, false, 1);                                                                                  \
  } while (0)
  if (w_dtype == JB_F32 && x_dtype == JB_F32) JB_LAUNCH_EX(float, float);
  else if (w_dtype == JB_BF16 && x_dtype == JB_BF16) JB_LAUNCH_EX(bf16, bf16);
  else return JB_ERR_BAD_DTYPE;
#undef JB_LAUNCH_EX
#undef JB_LAUNCH_GU
#undef JB_LAUNCH_DN
  return (int)e;
}

// order, where: [pairs]; gu, dn: tables of the grouped products (4 ints and 4 more per item), see the kernel
JB_EXPORT int jb_expert_plan(const int* sel_e, int pairs, int E, int F, int W, int* order, int* where, int* gu, int* dn,
                             cudaStream_t stream) {
  if (pairs <= 0) return 0;
  JB_REFUSE(E < 1 || E > PLAN_MAX_EXPERTS, "expert_plan: %d experts (at most %d)", E, PLAN_MAX_EXPERTS);
  JB_REFUSE(((uintptr_t)gu | (uintptr_t)dn) & 15, "expert_plan: tables must be 16-byte aligned");
  jb::Launch cfg(dim3(1), dim3(PLAN_THREADS), 0, stream);
  return (int)cudaLaunchKernelEx(&cfg.c, expert_plan_kernel, sel_e, pairs, E, F, W, order, where, gu, dn);
}

// rows: [pairs, W] in dtype, row i = weight[order[i]] * h[order[i] / top]
JB_EXPORT int jb_expert_gather(const void* h, int dtype, const int* order, const float* sel_w, int top, void* rows,
                               int pairs, int W, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  jb::Launch cfg(dim3(pairs), dim3(W >= 1024 ? 256 : 128), 0, stream);
  cudaError_t e;
  if (dtype == JB_F32)
    e = cudaLaunchKernelEx(&cfg.c, expert_gather_kernel<float>, (const float*)h, order, sel_w, top, (float*)rows, W);
  else if (dtype == JB_BF16)
    e = cudaLaunchKernelEx(&cfg.c, expert_gather_kernel<bf16>, (const bf16*)h, order, sel_w, top, (bf16*)rows, W);
  else
    return JB_ERR_BAD_DTYPE;
  return (int)e;
}

// out[t] += sum_k out_w[t top + k] results[where[t top + k]] (out_w null: the plain sum); results float32 [pairs, W],
// out float32 [T, W]
JB_EXPORT int jb_expert_scatter(const float* results, const int* where, const float* out_w, int top, float* out, int T,
                                int W, cudaStream_t stream) {
  if (T <= 0) return 0;
  jb::Launch cfg(dim3(T), dim3(W >= 1024 ? 256 : 128), 0, stream);
  return (int)cudaLaunchKernelEx(&cfg.c, expert_scatter_kernel, results, where, out_w, top, out, W);
}
