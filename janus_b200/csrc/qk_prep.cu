// What happens between the projections of an attention mixer and the attention kernel itself, for two mixers
// whose queries and keys are normed over the whole projection.  All arithmetic is float32; the projections are the
// products' float32 accumulators.
//
// qk_norm_rope_cache (attention whose values are its keys as projected):
//   q = proj[:, 0 : H d] + bq,  k = proj[:, H d : (H + G) d] + bk
//   v = k                                             (before norm and rotation; appended to the value pages)
//   q <- q / sqrt(mean(q^2) + eps) * wq               (one root mean square over all H d numbers), k likewise
//   the first `rot` dimensions of every head of q and k are turned in the pairing (i, i + rot/2) by the angle
//   of the token's position (cos and sin from a table [positions][rot/2][2]); the rest pass
//   q is written [T, H dp] in the engine dtype, k is appended to the key pages; dp >= d is the size a head is
//   stored with (a head size that the attention kernel does not take is stored as the next size it takes, the
//   extra columns zero: scores and sums do not change).
//
// latent_prep (latent attention, queries already multiplied into the latent space):
//   q = proj[:, 0 : Q] written [T, Q] in the engine dtype
//   c = proj[:, Q : Q + r] / sqrt(mean(.^2) + eps) * w, appended to the pages as the token's one key row
//
// Pages of one place: [page][kv_head][page_size][size]; dest[t] = page * page_size + row of token t.
// One block per token.
#include <stdio.h>

#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

template <typename TO>
__global__ void qk_norm_rope_cache_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bq,
                                          const float* __restrict__ bk, const float* __restrict__ wq,
                                          const float* __restrict__ wk, float eps, const float* __restrict__ table,
                                          int rot, const int* __restrict__ positions, TO* __restrict__ q_out,
                                          const int* __restrict__ dest, TO* __restrict__ k_cache,
                                          TO* __restrict__ v_cache, int H, int G, int d, int dp, int page_size,
                                          int write_kv) {
  extern __shared__ __align__(16) float row_s[];     // q [H d], then k [G d]
  __shared__ float scratch[33];
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x;
  const int QW = H * d, KW = write_kv ? G * d : 0;
  const float* pr = proj + (size_t)t * ld;
  size_t page = 0;
  int prow = 0;
  if (write_kv) {
    page = (size_t)(dest[t] / page_size);
    prow = dest[t] % page_size;
  }
  float sq = 0.0f, sk = 0.0f;
  for (int i = threadIdx.x; i < QW + KW; i += blockDim.x) {
    float v = pr[i];
    if (i < QW) {
      if (bq != nullptr) v += bq[i];
      sq += v * v;
    } else {
      const int c = i - QW;
      if (bk != nullptr) v += bk[c];
      sk += v * v;
      const int g = c / d, j = c % d;
      v_cache[((page * G + g) * page_size + prow) * dp + j] = jb::from_f32<TO>(v);
    }
    row_s[i] = v;
  }
  sq = jb::block_sum(sq, scratch);
  const float rq = sqrtf(sq / (float)QW + eps);
  float rk = 1.0f;
  if (write_kv) {
    sk = jb::block_sum(sk, scratch);
    rk = sqrtf(sk / (float)KW + eps);
  }
  const int half = rot >> 1;
  const float* cs = (table != nullptr && rot > 0) ? table + (size_t)positions[t] * half * 2 : nullptr;
  // a thread takes a number and, where it is rotated, writes both members of its pair
  for (int i = threadIdx.x; i < QW + KW; i += blockDim.x) {
    const bool is_q = i < QW;
    const int c = is_q ? i : i - QW;
    const int head = c / d, j = c % d;
    const float* w = is_q ? wq : wk;
    const float r = is_q ? rq : rk;
    TO* out = is_q ? q_out + ((size_t)t * H + head) * dp
                   : k_cache + ((page * G + head) * page_size + prow) * dp;
    if (cs != nullptr && j < rot) {
      if (j >= half) continue;                       // written by the thread of the pair's first member
      const float u = (row_s[i] / r) * w[c], v = (row_s[i + half] / r) * w[c + half];
      const float co = cs[2 * j], si = cs[2 * j + 1];
      out[j] = jb::from_f32<TO>(u * co - v * si);
      out[j + half] = jb::from_f32<TO>(v * co + u * si);
    } else {
      out[j] = jb::from_f32<TO>((row_s[i] / r) * w[c]);
    }
  }
  // heads stored wider than they are: the queries' extra columns are zero (those of the pages are never written)
  const int extra = dp - d;
  for (int i = threadIdx.x; i < H * extra; i += blockDim.x)
    q_out[((size_t)t * H + i / extra) * dp + d + i % extra] = jb::from_f32<TO>(0.0f);
}

template <typename TO>
__global__ void latent_prep_kernel(const float* __restrict__ proj, int ld, int Q, int r, int rp, const float* __restrict__ w,
                                   float eps, TO* __restrict__ q_out, const int* __restrict__ dest,
                                   TO* __restrict__ c_cache, int write_c) {
  __shared__ float scratch[33];
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x;
  const float* pr = proj + (size_t)t * ld;
  for (int i = threadIdx.x; i < Q; i += blockDim.x) q_out[(size_t)t * Q + i] = jb::from_f32<TO>(pr[i]);
  if (!write_c) return;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < r; i += blockDim.x) ss += pr[Q + i] * pr[Q + i];
  ss = jb::block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)r + eps);
  TO* out = c_cache + (size_t)dest[t] * rp;         // one key head: row dest[t] of [page * page_size][rp]
  for (int i = threadIdx.x; i < r; i += blockDim.x) out[i] = jb::from_f32<TO>((pr[Q + i] / rms) * w[i]);
}

// head_norm_rope_cache (grouped-query attention whose queries and keys are normed head by head):
//   q = proj[:, 0 : H d], k = proj[:, H d : (H + G) d], v = proj[:, (H + G) d : (H + G) d + G e]
//   every head of q and of k is divided by its own root mean square over d (eps inside the root) and multiplied by
//   wq (or wk), a weight of size d that all heads share (null: no norm, or with `unit` the division alone, which a
//   rotation commutes with: it keeps every pair's sum of squares); then the first `rot` dimensions are turned as
//   above, and q is multiplied by the query temperature 1 + temp_coef ln(floor((p + 1) / temp_every) + 1) of the
//   token's position p (temp_every 0: none).  q is written [T, H dp], k and v are appended to pages whose rows hold dp numbers (dp >= d, dp >= e; the
//   extra columns of q are zero, those of the pages are never written).  One block per token, a warp per head.
template <typename TO>
__global__ void head_norm_rope_cache_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ wq,
                                            const float* __restrict__ wk, float eps, const float* __restrict__ table,
                                            int rot, const int* __restrict__ positions, TO* __restrict__ q_out,
                                            const int* __restrict__ dest, TO* __restrict__ k_cache,
                                            TO* __restrict__ v_cache, int H, int G, int d, int e, int dp, int page_size,
                                            int write_kv, int unit, float temp_coef, int temp_every) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const float* pr = proj + (size_t)t * ld;
  size_t page = 0;
  int prow = 0;
  if (write_kv) {
    page = (size_t)(dest[t] / page_size);
    prow = dest[t] % page_size;
  }
  const int half = rot >> 1;
  const float* cs = (table != nullptr && rot > 0) ? table + (size_t)positions[t] * half * 2 : nullptr;
  const int n_heads = H + (write_kv ? 2 * G : 0);
  const float temp = temp_every > 0 ? 1.0f + temp_coef * logf((float)((positions[t] + 1) / temp_every) + 1.0f) : 1.0f;
  for (int head = warp; head < n_heads; head += warps) {
    if (head >= H + G) {                                // a value head: appended as projected
      const int g = head - H - G;
      const float* x = pr + (size_t)(H + G) * d + (size_t)g * e;
      TO* out = v_cache + ((page * G + g) * page_size + prow) * dp;
      for (int j = lane; j < e; j += 32) out[j] = jb::from_f32<TO>(x[j]);
      continue;
    }
    const bool is_q = head < H;
    const float* x = pr + (size_t)head * d;
    const float* w = is_q ? wq : wk;
    float inv = 1.0f;
    if (w != nullptr || unit) {
      float ss = 0.0f;
      for (int j = lane; j < d; j += 32) ss = fmaf(x[j], x[j], ss);
      ss = jb::warp_sum(ss);
      inv = 1.0f / sqrtf(ss / (float)d + eps);
    }
    if (is_q) inv *= temp;
    TO* out = is_q ? q_out + ((size_t)t * H + head) * dp
                   : k_cache + ((page * G + (head - H)) * page_size + prow) * dp;
    for (int j = lane; j < d; j += 32) {
      if (cs != nullptr && j < rot) {
        if (j >= half) continue;                        // written with the pair's first member
        const float u = (x[j] * inv) * (w ? w[j] : 1.0f), v = (x[j + half] * inv) * (w ? w[j + half] : 1.0f);
        const float co = cs[2 * j], si = cs[2 * j + 1];
        out[j] = jb::from_f32<TO>(u * co - v * si);
        out[j + half] = jb::from_f32<TO>(v * co + u * si);
      } else {
        out[j] = jb::from_f32<TO>((x[j] * inv) * (w ? w[j] : 1.0f));
      }
    }
    if (is_q)
      for (int j = d + lane; j < dp; j += 32) out[j] = jb::from_f32<TO>(0.0f);
  }
}

}  // namespace

// proj: float32 [T, ld]; bq [H d], bk [G d] (either may be null), wq [H d], wk [G d] float32; table: float32
// [positions][rot/2][2] or null (no rotation); q_out [T, H dp] and the pages (rows of dp) in out_dtype.  write_kv = 0: q only
// (a place that reads the keys and values another place wrote).
JB_EXPORT int jb_qk_norm_rope_cache(const float* proj, int ld, const float* bq, const float* bk, const float* wq,
                                    const float* wk, float eps, const float* table, int rot, const int* positions,
                                    void* q_out, int out_dtype, const int* dest, void* k_cache, void* v_cache, int T,
                                    int H, int G, int d, int dp, int page_size, int write_kv, cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(dp < d, "qk_norm_rope_cache: heads of %d cannot be stored in %d columns", d, dp);
  JB_REFUSE(rot < 0 || rot > d || (rot & 1), "qk_norm_rope_cache: %d rotated dimensions do not fit a head of %d", rot, d);
  JB_REFUSE(ld < (H + (write_kv ? G : 0)) * d, "qk_norm_rope_cache: rows of %d floats do not hold the projections", ld);
  const size_t smem = (size_t)(H + (write_kv ? G : 0)) * d * sizeof(float);
  JB_REFUSE(smem > 200 * 1024, "qk_norm_rope_cache: a token's projections (%zu bytes) do not fit shared memory", smem);
  jb::Launch cfg(dim3(T), dim3(256), smem, stream);
  cudaError_t e;
#define JB_LAUNCH_QK(TO)                                                                                               \
  do {                                                                                                                 \
    if (smem > 48 * 1024) {                                                                                            \
      e = cudaFuncSetAttribute(qk_norm_rope_cache_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                                             \
    }                                                                                                                  \
    e = cudaLaunchKernelEx(&cfg.c, qk_norm_rope_cache_kernel<TO>, proj, ld, bq, bk, wq, wk, eps, table, rot,           \
                           positions, (TO*)q_out, dest, (TO*)k_cache, (TO*)v_cache, H, G, d, dp, page_size, write_kv);\
  } while (0)
  if (out_dtype == JB_F32) JB_LAUNCH_QK(float);
  else if (out_dtype == JB_BF16) JB_LAUNCH_QK(bf16);
  else return JB_ERR_BAD_DTYPE;
#undef JB_LAUNCH_QK
  return (int)e;
}

// proj: float32 [T, ld] with the queries in columns [0, Q) and the latent projection in [Q, Q + r); w [r] float32;
// q_out [T, Q] and the pages ([page][1][page_size][rp], rp >= r the size a row is stored with, extra columns never
// written) in out_dtype.  write_c = 0: queries only.
JB_EXPORT int jb_latent_prep(const float* proj, int ld, int Q, int r, int rp, const float* w, float eps, void* q_out,
                             int out_dtype, const int* dest, void* c_cache, int T, int write_c, cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(ld < Q + (write_c ? r : 0) || rp < r, "latent_prep: rows of %d floats do not hold the projections", ld);
  jb::Launch cfg(dim3(T), dim3(256), 0, stream);
  cudaError_t e;
  if (out_dtype == JB_F32)
    e = cudaLaunchKernelEx(&cfg.c, latent_prep_kernel<float>, proj, ld, Q, r, rp, w, eps, (float*)q_out, dest,
                           (float*)c_cache, write_c);
  else if (out_dtype == JB_BF16)
    e = cudaLaunchKernelEx(&cfg.c, latent_prep_kernel<bf16>, proj, ld, Q, r, rp, w, eps, (bf16*)q_out, dest,
                           (bf16*)c_cache, write_c);
  else
    return JB_ERR_BAD_DTYPE;
  return (int)e;
}

// proj: float32 [T, ld] = [q: H d | k: G d | v: G e]; wq, wk: float32 [d] or null; table: float32 [positions][rot/2][2]
// or null; q_out [T, H dp] and the pages (rows of dp) in out_dtype.  write_kv = 0: q only.  unit = 1: heads are divided by
// their root mean square also without a weight.  temp_every > 0: the query temperature.
JB_EXPORT int jb_head_norm_rope_cache(const float* proj, int ld, const float* wq, const float* wk, float eps,
                                      const float* table, int rot, const int* positions, void* q_out, int out_dtype,
                                      const int* dest, void* k_cache, void* v_cache, int T, int H, int G, int d, int e,
                                      int dp, int page_size, int write_kv, int unit, float temp_coef, int temp_every,
                                      cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(dp < d || dp < e, "head_norm_rope_cache: heads of %d and %d cannot be stored in %d columns", d, e, dp);
  JB_REFUSE(rot < 0 || rot > d || (rot & 1), "head_norm_rope_cache: %d rotated dimensions do not fit a head of %d", rot, d);
  JB_REFUSE(ld < H * d + (write_kv ? G * (d + e) : 0), "head_norm_rope_cache: rows of %d floats do not hold the projections", ld);
  const int heads = H + (write_kv ? 2 * G : 0);
  jb::Launch cfg(dim3(T), dim3(heads >= 8 ? 256 : heads >= 4 ? 128 : 64), 0, stream);
  cudaError_t err;
  if (out_dtype == JB_F32)
    err = cudaLaunchKernelEx(&cfg.c, head_norm_rope_cache_kernel<float>, proj, ld, wq, wk, eps, table, rot, positions,
                             (float*)q_out, dest, (float*)k_cache, (float*)v_cache, H, G, d, e, dp, page_size, write_kv,
                             unit, temp_coef, temp_every);
  else if (out_dtype == JB_BF16)
    err = cudaLaunchKernelEx(&cfg.c, head_norm_rope_cache_kernel<bf16>, proj, ld, wq, wk, eps, table, rot, positions,
                             (bf16*)q_out, dest, (bf16*)k_cache, (bf16*)v_cache, H, G, d, e, dp, page_size, write_kv,
                             unit, temp_coef, temp_every);
  else
    return JB_ERR_BAD_DTYPE;
  return (int)err;
}
