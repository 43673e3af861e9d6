// What happens where a sublayer's output joins the residual stream and the next sublayer reads it, in one launch,
// for designs with a layer norm (or a root-mean-square norm), a per-feature scale on what joins the stream, and
// sublayers made of two branches.  All arithmetic is float32.  For one row r of the stream (width W):
//
//   y  = ya                                                     (a sublayer's output), or, with branch weights,
//   y  = mult ya / rms(ya) wa + mult_b yb / rms(yb) wb          rms(v) = sqrt(mean(v^2) + eps), or, with two
//   y  = mult ya + mult_b yb                                    branches and no branch weights, their weighted sum
//   r <- r + scale * y          (scale per feature, or 1)       ya and yb are set to zero afterwards
//   r <- r + extra              (another stream's row, e.g. the embedding's output that joins before a pass)
//   x  = (r - mean(r)) / sqrt(mean((r - mean(r))^2) + eps) gamma        (center = 1: layer norm, no bias)
//   x  = r / sqrt(mean(r^2) + eps) gamma                                (center = 0)
//
// Every step is optional: without ya the row is only read; without gamma nothing is normed; with row_index the
// rows of x are picked (x[i] = norm(r[row_index[i]])) and the stream is not written.  `clear`, `clear2`: float32
// buffers of whole 16-byte vectors that the launch sets to zero on the way.  One block per row; the row lives in
// shared memory between the passes.
#include <stdio.h>

#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void clear_slice(float4* buf, size_t n4) {
  if (buf == nullptr) return;
  const float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) buf[i] = z;
}

// V floats at a time (4: rows of whole, aligned 16-byte vectors; 1: any row)
template <int V> struct Vec;
template <> struct Vec<1> {
  float v[1];
  __device__ __forceinline__ void load(const float* p) { v[0] = *p; }
  __device__ __forceinline__ void store(float* p) const { *p = v[0]; }
};
template <> struct Vec<4> {
  float v[4];
  __device__ __forceinline__ void load(const float* p) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
  }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <int V> __device__ __forceinline__ void store_out(float* p, const Vec<V>& x) { x.store(p); }
__device__ __forceinline__ void store_out(bf16* p, const Vec<1>& x) { *p = __float2bfloat16(x.v[0]); }
__device__ __forceinline__ void store_out(bf16* p, const Vec<4>& x) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(x.v[0], x.v[1]), hi = __floats2bfloat162_rn(x.v[2], x.v[3]);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&lo);
  u.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TO, int V>
__global__ void join_norm_kernel(float* __restrict__ stream, float* __restrict__ ya, float* __restrict__ yb,
                                 const float* __restrict__ wa, const float* __restrict__ wb, float mult,
                                 float mult_b, const float* __restrict__ scale, const float* __restrict__ extra,
                                 const float* __restrict__ gamma, float eps, int center, TO* __restrict__ x_out,
                                 const int* __restrict__ row_index, int W, float4* __restrict__ clear, size_t clear_n4,
                                 float4* __restrict__ clear2, size_t clear2_n4) {
  extern __shared__ __align__(16) float row_s[];   // the row of the stream
  __shared__ float scratch[33];
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  clear_slice(clear, clear_n4);
  clear_slice(clear2, clear2_n4);
  const size_t src = row_index != nullptr ? (size_t)row_index[blockIdx.x] : (size_t)blockIdx.x;
  float* r = stream + src * W;
  float* pa = ya != nullptr ? ya + src * W : nullptr;
  float* pb = yb != nullptr ? yb + src * W : nullptr;
  const int first = threadIdx.x * V, step = blockDim.x * V;
  const bool branches = pa != nullptr && pb != nullptr;
  const bool normed = branches && wa != nullptr;
  float inv_a = 1.0f, inv_b = 1.0f;
  if (normed) {
    float sa = 0.0f, sb = 0.0f;
    for (int i = first; i < W; i += step) {
      Vec<V> a, b;
      a.load(pa + i);
      b.load(pb + i);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        sa = fmaf(a.v[j], a.v[j], sa);
        sb = fmaf(b.v[j], b.v[j], sb);
      }
    }
    sa = jb::block_sum(sa, scratch);
    sb = jb::block_sum(sb, scratch);
    inv_a = 1.0f / sqrtf(sa / (float)W + eps);
    inv_b = 1.0f / sqrtf(sb / (float)W + eps);
  }
  Vec<V> zero;
#pragma unroll
  for (int j = 0; j < V; ++j) zero.v[j] = 0.0f;
  float sum = 0.0f;
  for (int i = first; i < W; i += step) {
    Vec<V> v;
    v.load(r + i);
    if (pa != nullptr) {
      Vec<V> y;
      y.load(pa + i);
      zero.store(pa + i);
      if (branches) {
        Vec<V> b, ga, gb;
        b.load(pb + i);
        zero.store(pb + i);
        if (normed) {
          ga.load(wa + i);
          gb.load(wb + i);
#pragma unroll
          for (int j = 0; j < V; ++j)
            y.v[j] = mult * ((y.v[j] * inv_a) * ga.v[j]) + mult_b * ((b.v[j] * inv_b) * gb.v[j]);
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) y.v[j] = mult * y.v[j] + mult_b * b.v[j];
        }
      }
      if (scale != nullptr) {
        Vec<V> sc;
        sc.load(scale + i);
#pragma unroll
        for (int j = 0; j < V; ++j) v.v[j] = fmaf(sc.v[j], y.v[j], v.v[j]);
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) v.v[j] += y.v[j];
      }
    }
    if (extra != nullptr) {
      Vec<V> x;
      x.load(extra + src * W + i);
#pragma unroll
      for (int j = 0; j < V; ++j) v.v[j] += x.v[j];
    }
    if (pa != nullptr || extra != nullptr) v.store(r + i);
    v.store(row_s + i);
#pragma unroll
    for (int j = 0; j < V; ++j) sum += v.v[j];
  }
  if (x_out == nullptr) return;
  float mean = 0.0f;
  if (center) mean = jb::block_sum(sum, scratch) / (float)W;
  float sq = 0.0f;
  for (int i = first; i < W; i += step) {   // a thread reads back what it wrote itself
    Vec<V> v;
    v.load(row_s + i);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float d = v.v[j] - mean;
      sq = fmaf(d, d, sq);
    }
  }
  sq = jb::block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(sq / (float)W + eps);
  TO* x = x_out + (size_t)blockIdx.x * W;
  for (int i = first; i < W; i += step) {
    Vec<V> v, g;
    v.load(row_s + i);
    g.load(gamma + i);
#pragma unroll
    for (int j = 0; j < V; ++j) v.v[j] = ((v.v[j] - mean) * inv) * g.v[j];
    store_out(x + i, v);
  }
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * act(gate[t, h, :]), one warp per (token, head);
// weight [e] is shared by the heads (w_stride 0) or every head has its own (w_stride e); act: 0 = SiLU, 1 = sigmoid.
// With `denom` (float32 [T, heads]) o[t, h, :] is first divided by denom[t, h].
template <typename TO>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate, int ld_gate,
                                      const float* __restrict__ weight, int w_stride, const float* __restrict__ denom,
                                      float eps, int act, TO* __restrict__ out, long long items, int heads, int e) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const int lane = threadIdx.x & 31;
  const long long t = item / heads;
  const int h = (int)(item % heads);
  const float* row = o + (size_t)item * e;
  const float under = denom != nullptr ? 1.0f / denom[item] : 1.0f;
  float ss = 0.0f;
  for (int i = lane; i < e; i += 32) {
    const float v = row[i] * under;
    ss = fmaf(v, v, ss);
  }
  ss = jb::warp_sum(ss);
  const float inv = under / sqrtf(ss / (float)e + eps);
  const float* g = gate + (size_t)t * ld_gate + (size_t)h * e;
  const float* w = weight + (size_t)h * w_stride;
  for (int i = lane; i < e; i += 32) {
    const float z = g[i], s = 1.0f / (1.0f + expf(-z));
    out[(size_t)item * e + i] = jb::from_f32<TO>(((row[i] * inv) * w[i]) * (act == 0 ? z * s : s));
  }
}

// x[t, h, j] *= sigmoid(gate[t, h e + j]) for j < e, in place: x holds heads of `stored` >= e numbers (the columns
// behind e are left alone), the gate is float32 with rows of ld_gate floats.
template <typename TO>
__global__ void sigmoid_gate_kernel(TO* __restrict__ x, const float* __restrict__ gate, int ld_gate, int heads, int e,
                                    int stored, long long n) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(i % stored);
    if (j >= e) continue;
    const long long th = i / stored;
    const long long t = th / heads;
    const int h = (int)(th % heads);
    const float z = gate[(size_t)t * ld_gate + (size_t)h * e + j];
    x[i] = jb::from_f32<TO>(jb::to_f32(x[i]) / (1.0f + expf(-z)));
  }
}

// The same, four numbers a thread (e, stored and ld_gate multiples of 4, both pointers on 16-byte boundaries).
template <typename TO>
__global__ void sigmoid_gate_vec_kernel(TO* __restrict__ x, const float* __restrict__ gate, int ld_gate, int heads,
                                        int e, int stored, long long n4) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int per_head = stored >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(i % per_head) << 2;
    if (j >= e) continue;
    const long long th = i / per_head;
    const long long t = th / heads;
    const int h = (int)(th % heads);
    const float4 z = *reinterpret_cast<const float4*>(gate + (size_t)t * ld_gate + (size_t)h * e + j);
    Vec<4> v;
    if (sizeof(TO) == 4) {
      v.load(reinterpret_cast<const float*>(x) + i * 4);
    } else {
      const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(x) + i * 4);
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      v.v[0] = a.x, v.v[1] = a.y, v.v[2] = b.x, v.v[3] = b.y;
    }
    v.v[0] /= 1.0f + expf(-z.x);
    v.v[1] /= 1.0f + expf(-z.y);
    v.v[2] /= 1.0f + expf(-z.z);
    v.v[3] /= 1.0f + expf(-z.w);
    store_out(x + i * 4, v);
  }
}

}  // namespace

// stream: float32 [rows of the stream, W]; ya, yb: float32 of the stream's shape or null (yb without wa and wb: the
// weighted sum mult ya + mult_b yb joins the stream); wa, wb, scale, gamma: float32 [W]
// or null; extra: float32 of the stream's shape or null; x_out: [T, W] in out_dtype or null; row_index: int32 [T] or null.
JB_EXPORT int jb_join_norm(float* stream, float* ya, float* yb, const float* wa, const float* wb, float mult,
                           float mult_b, const float* scale, const float* extra, const float* gamma, float eps, int center,
                           void* x_out, int out_dtype, const int* row_index, int T, int W, float* clear,
                           long long clear_n, float* clear2, long long clear2_n, cudaStream_t stream_) {
  if (T <= 0) return 0;
  JB_REFUSE((clear != nullptr && ((clear_n & 3) != 0 || ((uintptr_t)clear & 15) != 0)) ||
                (clear2 != nullptr && ((clear2_n & 3) != 0 || ((uintptr_t)clear2 & 15) != 0)),
            "join_norm: a buffer to clear is not made of whole 16-byte vectors");
  JB_REFUSE((wa != nullptr) != (wb != nullptr) || (wa != nullptr && (ya == nullptr || yb == nullptr)) ||
                (yb != nullptr && ya == nullptr),
            "join_norm: two branches need two outputs, and two weights or none");
  JB_REFUSE(row_index != nullptr && (ya != nullptr || extra != nullptr), "join_norm: picked rows are only read");
  JB_REFUSE(x_out != nullptr && gamma == nullptr, "join_norm: a norm needs its weight");
  const size_t smem = (size_t)W * sizeof(float);
  JB_REFUSE(smem > 200 * 1024, "join_norm: a row of %d floats does not fit shared memory", W);
  // rows of whole 16-byte vectors at aligned addresses are read and written four floats at a time
  const uintptr_t all = (uintptr_t)stream | (uintptr_t)ya | (uintptr_t)yb | (uintptr_t)wa | (uintptr_t)wb |
                        (uintptr_t)scale | (uintptr_t)extra | (uintptr_t)gamma | (uintptr_t)x_out;
  const bool vec = W % 4 == 0 && (all & 15) == 0;
  const int per = vec ? 4 : 1;
  jb::Launch cfg(dim3(T), dim3(W >= 2048 * per ? 512 : W >= 512 * per ? 256 : 128), smem, stream_);
  cudaError_t e;
#define JB_LAUNCH_JN(TO, V)                                                                                        \
  do {                                                                                                             \
    if (smem > 48 * 1024) {                                                                                        \
      e = cudaFuncSetAttribute(join_norm_kernel<TO, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
      if (e != cudaSuccess) return (int)e;                                                                         \
    }                                                                                                              \
    e = cudaLaunchKernelEx(&cfg.c, join_norm_kernel<TO, V>, stream, ya, yb, wa, wb, mult, mult_b, scale, extra, gamma, eps, \
                           center, (TO*)x_out, row_index, W, (float4*)clear, clear ? (size_t)clear_n >> 2 : (size_t)0, \
                           (float4*)clear2, clear2 ? (size_t)clear2_n >> 2 : (size_t)0);                           \
  } while (0)
  if (out_dtype == JB_F32 && vec) JB_LAUNCH_JN(float, 4);
  else if (out_dtype == JB_F32) JB_LAUNCH_JN(float, 1);
  else if (out_dtype == JB_BF16 && vec) JB_LAUNCH_JN(bf16, 4);
  else if (out_dtype == JB_BF16) JB_LAUNCH_JN(bf16, 1);
  else return JB_ERR_BAD_DTYPE;
#undef JB_LAUNCH_JN
  return (int)e;
}

// o: float32 [T, heads e]; gate: float32 rows of ld_gate floats, head h at columns [h e, (h + 1) e); weight float32 [e].
JB_EXPORT int jb_head_norm_gate(const float* o, const float* gate, int ld_gate, const float* weight, int w_stride,
                                const float* denom, float eps, int act, void* out, int out_dtype, int T, int heads,
                                int e, cudaStream_t stream) {
  if (T <= 0) return 0;
  const long long items = (long long)T * heads;
  jb::Launch cfg(dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream);
  cudaError_t err;
  if (out_dtype == JB_F32)
    err = cudaLaunchKernelEx(&cfg.c, head_norm_gate_kernel<float>, o, gate, ld_gate, weight, w_stride, denom, eps, act, (float*)out, items,
                             heads, e);
  else if (out_dtype == JB_BF16)
    err = cudaLaunchKernelEx(&cfg.c, head_norm_gate_kernel<bf16>, o, gate, ld_gate, weight, w_stride, denom, eps, act, (bf16*)out, items,
                             heads, e);
  else
    return JB_ERR_BAD_DTYPE;
  return (int)err;
}

// x: [T, heads stored] in dtype; gate: float32 rows of ld_gate floats, head h at columns [h e, (h + 1) e).
JB_EXPORT int jb_sigmoid_gate(void* x, int dtype, const float* gate, int ld_gate, int T, int heads, int e, int stored,
                              cudaStream_t stream) {
  if (T <= 0 || heads <= 0) return 0;
  JB_REFUSE(stored < e, "sigmoid_gate: heads of %d cannot be stored in %d columns", e, stored);
  const long long n = (long long)T * heads * stored;
  if (e % 4 == 0 && stored % 4 == 0 && ld_gate % 4 == 0 && (reinterpret_cast<uintptr_t>(gate) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (dtype == JB_F32 || dtype == JB_BF16)) {
    const long long n4 = n >> 2;
    jb::Launch vcfg(dim3((unsigned)((n4 + 255) / 256 < 8192 ? (n4 + 255) / 256 : 8192)), dim3(256), 0, stream);
    if (dtype == JB_F32)
      return (int)cudaLaunchKernelEx(&vcfg.c, sigmoid_gate_vec_kernel<float>, (float*)x, gate, ld_gate, heads, e,
                                     stored, n4);
    return (int)cudaLaunchKernelEx(&vcfg.c, sigmoid_gate_vec_kernel<bf16>, (bf16*)x, gate, ld_gate, heads, e, stored,
                                   n4);
  }
  jb::Launch cfg(dim3((unsigned)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096)), dim3(256), 0, stream);
  cudaError_t err;
  if (dtype == JB_F32)
    err = cudaLaunchKernelEx(&cfg.c, sigmoid_gate_kernel<float>, (float*)x, gate, ld_gate, heads, e, stored, n);
  else if (dtype == JB_BF16)
    err = cudaLaunchKernelEx(&cfg.c, sigmoid_gate_kernel<bf16>, (bf16*)x, gate, ld_gate, heads, e, stored, n);
  else
    return JB_ERR_BAD_DTYPE;
  return (int)err;
}
