// Attention over a cached latent: what surrounds the attention kernel.
//
// A token stores c = RMSNorm(first R numbers of its down-projection) * w and one rotated key part
// k_r of r numbers that all heads share.  Head h's key is [W_uk[h] c | k_r] and its value W_uv[h] c, so
//
//   score_h(i, j) = (q_h(i) . W_uk[h] c_j + q_r,h(i) . k_r(j)) * scale = ([W_uk[h]^T q_h(i) | q_r,h(i)] . [c_j | k_r(j)]) * scale
//   o_h(i) = W_uv[h] sum_j p_h(i, j) c_j
//
// which is attention of H query heads of R + r numbers over ONE key head [c | k_r] whose values are c:
// nothing per head is ever expanded for a cached token.  `latent_prep` makes the cache entry of each
// new token (norm, rotation, write into the paged key cache rows [c | k_r] and value cache rows c) and
// rotates the rotated part of every query head in place; `head_linear` is the small product per head
// that folds W_uk into the queries in front of the attention kernel and applies W_uv behind it.
// The attention itself is the package's kernel for keys and values of different sizes.
// Rotation of the first rd numbers of the rotated part: pairs (i, i + rd/2), or (2 i, 2 i + 1) where the model
// interleaves them; angle = position * freq[pair] in float32 (the caller's table: any scaling of the frequencies is
// already in it), cos and sin times one factor.  All arithmetic float32; T is the storage type of the cache.
#include "cache_layout.cuh"
#include "common.cuh"

namespace tb {

// Number i of a rotated part (r numbers of which the first rd are turned) at position pos.  Pairing: (i, i + rd / 2),
// or with `interleaved` (2 i, 2 i + 1); pair n turns by the angle pos * freq[n]; cos and sin carry the factor `mag`.
__device__ __forceinline__ float turned(const float* __restrict__ src, int i, int rd, int interleaved, float pos,
                                        const float* __restrict__ freq, float mag) {
  if (i >= rd) return src[i];
  const int half = rd >> 1;
  const bool first = interleaved ? !(i & 1) : i < half;
  const int pair = interleaved ? i >> 1 : (first ? i : i - half);
  const int other = interleaved ? i ^ 1 : (first ? i + half : i - half);
  const float a = pos * freq[pair];
  const float cs = cosf(a) * mag, sn = sinf(a) * mag;
  return first ? src[i] * cs - src[other] * sn : src[i] * cs + src[other] * sn;
}

// One block per token.  q_in float32 rows of H query heads of (d + r) numbers; kv_in float32 rows of the
// down-projection (R + r numbers).  q_out float32 [T, H, R + r]: the rotated query part is written to columns
// R .. R + r of each head (the first R columns are filled by head_linear).
template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ q_in, long long q_stride, const float* __restrict__ kv_in,
                                   long long kv_stride, const float* __restrict__ norm_w,
                                   const float* __restrict__ freq, const int* __restrict__ positions,
                                   const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                   float* __restrict__ q_out, int H, int d, int r, int rd, int R, int page_size, float eps,
                                   int write_kv, int interleaved, float mag) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float* row = q_in + (size_t)t * q_stride;
  const float pos = (float)positions[t];
  // the rotated part of every query head
  for (int e = threadIdx.x; e < H * r; e += blockDim.x) {
    const int h = e / r, i = e % r;
    q_out[((size_t)t * H + h) * (R + r) + R + i] = turned(row + (size_t)h * (d + r) + d, i, rd, interleaved, pos, freq, mag);
  }
  // the cache entry
  const float* kv = kv_in + (size_t)t * kv_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += blockDim.x) ss = fmaf(kv[i], kv[i], ss);
  ss = block_sum(ss, scratch);
  const int slot = (write_kv && slots) ? slots[t] : -1;
  if (slot < 0) return;
  const float inv = rsqrtf(ss / (float)R + eps);
  const int dk = R + r;
  T* ktile = k_cache + cache_tile(slot / page_size, 0, 1, page_size, dk);
  T* vtile = v_cache + cache_tile(slot / page_size, 0, 1, page_size, R);
  const int rr = slot % page_size;
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const T c = from_float<T>(kv[i] * inv * norm_w[i]);
    ktile[cache_offset<T>(rr, i, page_size, dk)] = c;
    vtile[cache_offset<T>(rr, i, page_size, R)] = c;
  }
  for (int i = threadIdx.x; i < r; i += blockDim.x)
    ktile[cache_offset<T>(rr, R + i, page_size, dk)] = from_float<T>(turned(kv + R, i, rd, interleaved, pos, freq, mag));
}

// out[t, h, n] = sum_k x[t, h, k] * W[h][n, k]  (or W[h][k, n] with `transposed`).  A block serves one head and
// HL_TOKENS tokens, so a weight is fetched once for all of them; a thread owns output columns n and keeps one sum
// per token.  x rows: x + t * x_stride + h * x_head; out rows: out + t * out_stride + h * out_head.  X, W: float or
// bfloat16; sums in float32 in ascending k for every (token, n), so a token's result does not depend on the batch.
constexpr int HL_TOKENS = 16;

template <typename X, typename W, typename O>
__global__ void __launch_bounds__(128)
head_linear_kernel(const X* __restrict__ x, long long x_stride, int x_head, const W* __restrict__ w, O* __restrict__ out,
                   long long out_stride, int out_head, int T_tokens, int N, int K, int transposed) {
  extern __shared__ float xs[];  // [K][HL_TOKENS]: the tokens of one k side by side
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * HL_TOKENS, h = blockIdx.y;
  const int nt = min(HL_TOKENS, T_tokens - t0);
  for (int e = threadIdx.x; e < HL_TOKENS * K; e += blockDim.x) {
    const int tt = e / K, k = e % K;
    xs[k * HL_TOKENS + tt] = tt < nt ? to_float(x[(size_t)(t0 + tt) * x_stride + (size_t)h * x_head + k]) : 0.f;
  }
  __syncthreads();
  const W* wh = w + (size_t)h * N * K;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    float acc[HL_TOKENS];
#pragma unroll
    for (int tt = 0; tt < HL_TOKENS; ++tt) acc[tt] = 0.f;
    const W* col = transposed ? wh + n : wh + (size_t)n * K;
    const size_t step = transposed ? N : 1;
    for (int k = 0; k < K; ++k) {
      const float wv = to_float(col[(size_t)k * step]);
      const float4* xv = reinterpret_cast<const float4*>(xs + k * HL_TOKENS);
#pragma unroll
      for (int q4 = 0; q4 < HL_TOKENS / 4; ++q4) {
        const float4 v = xv[q4];
        acc[4 * q4] = fmaf(v.x, wv, acc[4 * q4]);
        acc[4 * q4 + 1] = fmaf(v.y, wv, acc[4 * q4 + 1]);
        acc[4 * q4 + 2] = fmaf(v.z, wv, acc[4 * q4 + 2]);
        acc[4 * q4 + 3] = fmaf(v.w, wv, acc[4 * q4 + 3]);
      }
    }
#pragma unroll
    for (int tt = 0; tt < HL_TOKENS; ++tt)
      if (tt < nt) out[(size_t)(t0 + tt) * out_stride + (size_t)h * out_head + n] = from_float<O>(acc[tt]);
  }
}

// y[t, c] = o[t, c] * sigmoid(g[t, c / per]), rounded to T.  o float32, g float32 rows with stride g_stride (per = 1: a gate
// value per output; per = the value size of a head: one per head).
template <typename T>
__global__ void sigmoid_gate_kernel(const float* __restrict__ o, const float* __restrict__ g, int g_stride, T* __restrict__ y,
                                    long long total, int N, int per) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / N;
    const int c = (int)(i % N);
    const float gate = g ? 1.f / (1.f + expf(-g[(size_t)t * g_stride + c / per])) : 1.f;
    y[i] = from_float<T>(o[i] * gate);
  }
}

}  // namespace tb

extern "C" {

// q_in: rows of H heads of d + r numbers (row stride q_stride floats); kv_in: rows of R + r numbers (row stride kv_stride).
// interleaved: pairs (2 i, 2 i + 1) instead of (i, i + rd / 2); mag: factor on cos and sin.
int tb_latent_prep(void* stream, const float* q_in, long long q_stride, const float* kv_in, long long kv_stride, const float* norm_w,
                   const float* freq, const int* positions, const int* slots, void* k_cache, void* v_cache, float* q_out,
                   int T_tokens, int H, int d, int r, int rd, int R, int page_size, float eps, int write_kv, int interleaved, float mag,
                   int dtype) {
  if (T_tokens <= 0) return 0;
  if (H <= 0 || d <= 0 || r < 0 || rd < 0 || rd > r || (rd & 1) || R <= 0 || page_size <= 0 || (rd && !freq)) return TB_ERR_BAD_SIZE;
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::latent_prep_kernel<T>, dim3(T_tokens), dim3(128), 0, stream, q_in, q_stride, kv_in, kv_stride,
                                      norm_w, freq, positions, slots, (T*)k_cache, (T*)v_cache, q_out, H, d, r, rd, R, page_size, eps,
                                      write_kv, interleaved, mag));
}

// x_dtype / w_dtype / out_dtype: TB_F32 or TB_BF16 (x and out float32 with either weight type; x bfloat16 with bfloat16 weights).
int tb_head_linear(void* stream, const void* x, int x_dtype, long long x_stride, int x_head, const void* w, int w_dtype, void* out,
                   int out_dtype, long long out_stride, int out_head, int T_tokens, int H, int N, int K, int transposed) {
  if (T_tokens <= 0) return 0;
  if (H <= 0 || H > 65535 || N <= 0 || K <= 0 || K > 3456) return TB_ERR_BAD_SIZE;
  const dim3 grid((T_tokens + tb::HL_TOKENS - 1) / tb::HL_TOKENS, H), block(128);
  const size_t smem = (size_t)K * tb::HL_TOKENS * sizeof(float);
#define TB_HL(XX, WW, OO)                                                                                                           \
  do {                                                                                                                              \
    if (smem > 48 * 1024) {                                                                                                         \
      const cudaError_t e = cudaFuncSetAttribute(tb::head_linear_kernel<XX, WW, OO>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                                 (int)smem);                                                                        \
      if (e != cudaSuccess) return (int)e;                                                                                          \
    }                                                                                                                               \
    return tb::launch(tb::head_linear_kernel<XX, WW, OO>, grid, block, smem, stream, (const XX*)x, x_stride, x_head, (const WW*)w, \
                      (OO*)out, out_stride, out_head, T_tokens, N, K, transposed);                                                  \
  } while (0)
  using B = __nv_bfloat16;
  if (x_dtype == TB_F32 && w_dtype == TB_F32 && out_dtype == TB_F32) TB_HL(float, float, float);
  if (x_dtype == TB_F32 && w_dtype == TB_BF16 && out_dtype == TB_F32) TB_HL(float, B, float);
  if (x_dtype == TB_BF16 && w_dtype == TB_BF16 && out_dtype == TB_F32) TB_HL(B, B, float);
#undef TB_HL
  return TB_ERR_BAD_DTYPE;
}

int tb_sigmoid_gate(void* stream, const float* o, const float* g, int g_stride, void* y, int T_tokens, int N, int per, int dtype) {
  const long long total = (long long)T_tokens * N;
  if (total <= 0) return 0;
  if (per <= 0 || N % per) return TB_ERR_BAD_SIZE;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::sigmoid_gate_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, o, g, g_stride, (T*)y,
                                      total, N, per));
}

}  // extern "C"
